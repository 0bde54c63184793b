"""Autograd wrappers of the tensor-product / graph-message kernels.

The operator is trilinear in (features x, harmonics sh, gates g).  With A(x, sh, g; v) the first
adjoint (gradients of <v, F(x, sh, g)>), every higher derivative is again a sum of F and A calls with
one argument replaced by a tangent, so ``_TpForward`` and ``_TpAdjoint`` below are closed under
differentiation: when autograd is recording, their backward passes are written with the two
functions themselves.  That covers the reference's first adjoint, its mixed second derivatives
(ictc_o3/operators.py:57-158; ictc_o3/ops/rematerialized_message.py:138-214) and any higher order,
without a differentiable non-kernel expression.
"""
from __future__ import annotations

import torch

from .. import _lib
from ..autograd.adjoint_requirements import required_gradients
from .topology import Topology


# When set to a list, every launch appends (kernel name, start event, end event) recorded on the
# launching stream; used by bench.py to time kernels live and to count launches.
PROFILE = None


class _Timed:
    def __init__(self, name, device):
        self.name, self.device = name, device

    def __enter__(self):
        if PROFILE is not None:
            self.start = torch.cuda.Event(enable_timing=True)
            self.start.record(torch.cuda.current_stream(self.device))

    def __exit__(self, *exc):
        if PROFILE is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record(torch.cuda.current_stream(self.device))
            PROFILE.append((self.name, self.start, end))


class TpCall:
    """Bound, non-differentiable arguments of one tensor-product call."""

    def __init__(self, spec: int, channels: int, weight, mask, topology: Topology | None):
        self.spec, self.channels = spec, channels
        self.weight = weight      # [P,C] contiguous or None (unit base coefficients)
        self.mask = mask          # [E] contiguous or None
        self.topology = topology  # None: edge-owned rows
        self.nx, self.nh, self.np, self.no, _ = _lib.tp_spec_info(spec)

    # ---- raw launches -------------------------------------------------------------------
    def forward(self, x, sh, g):
        lib, dev, c = _lib.load(), x.device, self.channels
        topo = self.topology
        if topo is not None:
            rowptr, order = topo.by_dst()
        with _lib.on_device(dev), _Timed("edge_forward" if topo is None else "graph_forward", dev):
            if topo is None:
                e = x.shape[0]
                out = torch.empty(e, self.no * c, dtype=torch.float32, device=dev)
                _lib.check(lib.ictc_tp_edge_forward(self.spec, c, e, _lib.ptr(x), _lib.ptr(sh), _lib.ptr(self.weight),
                                                    _lib.ptr(g), _lib.ptr(self.mask), _lib.ptr(out),
                                                    _lib.stream(dev)), "ictc_tp_edge_forward")
            else:
                out = torch.empty(topo.num_nodes, self.no * c, dtype=torch.float32, device=dev)
                _lib.check(lib.ictc_tp_graph_forward(self.spec, c, topo.num_nodes, topo.num_edges, _lib.ptr(x),
                                                     _lib.ptr(sh), _lib.ptr(self.weight), _lib.ptr(g),
                                                     _lib.ptr(topo.src), rowptr.data_ptr(), _lib.ptr(order),
                                                     _lib.ptr(self.mask), _lib.ptr(out), _lib.stream(dev)),
                           "ictc_tp_graph_forward")
        return out

    def adjoint(self, x, sh, g, v, needed):
        lib, dev, c = _lib.load(), x.device, self.channels
        topo = self.topology
        e = sh.shape[0]
        dx = torch.empty_like(x) if needed[0] else None
        dsh = torch.empty_like(sh) if needed[1] else None
        dg = torch.empty_like(g) if needed[2] else None
        if not any(needed):
            return dx, dsh, dg
        if topo is not None:
            topo.by_src()
        with _lib.on_device(dev), _Timed("edge_adjoint" if topo is None else "graph_adjoint", dev):
            if topo is None:
                _lib.check(lib.ictc_tp_edge_adjoint(self.spec, c, e, _lib.ptr(x), _lib.ptr(sh), _lib.ptr(self.weight),
                                                    _lib.ptr(g), _lib.ptr(self.mask), _lib.ptr(v), _lib.ptr(dx),
                                                    _lib.ptr(dsh), _lib.ptr(dg), _lib.stream(dev)),
                           "ictc_tp_edge_adjoint")
            else:
                rowptr, order = topo.by_src()
                _lib.check(lib.ictc_tp_graph_adjoint(self.spec, c, topo.num_nodes, topo.num_edges, _lib.ptr(x),
                                                     _lib.ptr(sh), _lib.ptr(self.weight), _lib.ptr(g),
                                                     _lib.ptr(topo.dst), rowptr.data_ptr(), _lib.ptr(order),
                                                     _lib.ptr(self.mask), _lib.ptr(v), _lib.ptr(dx), _lib.ptr(dsh),
                                                     _lib.ptr(dg), _lib.stream(dev)), "ictc_tp_graph_adjoint")
        return dx, dsh, dg


def _add(a, b):
    if a is None:
        return b
    if b is None:
        return a
    return a + b


class _TpForward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, sh, g, call):
        ctx.call = call
        ctx.save_for_backward(x, sh, g)
        return call.forward(x, sh, g)

    @staticmethod
    def backward(ctx, grad):
        x, sh, g = ctx.saved_tensors
        needed = required_gradients((x, sh, g), ctx.needs_input_grad[:3])
        grad = grad.contiguous()
        if torch.is_grad_enabled():
            dx, dsh, dg = _TpAdjoint.apply(x, sh, g, grad, ctx.call, needed)
        else:
            dx, dsh, dg = ctx.call.adjoint(x, sh, g, grad, needed)
        return dx, dsh, dg, None


class _TpAdjoint(torch.autograd.Function):
    """(dx, dsh, dg) = A(x, sh, g; v); differentiable in x, sh, g and v."""

    @staticmethod
    def forward(ctx, x, sh, g, v, call, needed):
        ctx.set_materialize_grads(False)
        ctx.call, ctx.needed = call, tuple(needed)
        ctx.save_for_backward(x, sh, g, v)
        return call.adjoint(x, sh, g, v, needed)

    @staticmethod
    def backward(ctx, hx, hs, hg):
        x, sh, g, v = ctx.saved_tensors
        call = ctx.call
        need_x, need_s, need_g, need_v = required_gradients(
            (x, sh, g, v), (*ctx.needs_input_grad[:3], ctx.needs_input_grad[3]))
        hx = hx.contiguous() if hx is not None else None
        hs = hs.contiguous() if hs is not None else None
        hg = hg.contiguous() if hg is not None else None
        record = torch.is_grad_enabled()

        def adj(xa, sa, ga, needed):
            if not any(needed):
                return None, None, None
            if record:
                return _TpAdjoint.apply(xa, sa, ga, v, call, needed)
            return call.adjoint(xa, sa, ga, v, needed)

        def fwd(xa, sa, ga):
            return _TpForward.apply(xa, sa, ga, call) if record else call.forward(xa, sa, ga)

        big_x = big_s = big_g = big_v = None
        # L = <hx, dx> + <hs, dsh> + <hg, dg> = <v, F(hx,sh,g) + F(x,hs,g) + F(x,sh,hg)>
        if hx is not None:
            _, ds, dg = adj(hx, sh, g, (False, need_s, need_g))
            big_s, big_g = _add(big_s, ds), _add(big_g, dg)
        if hs is not None:
            dx, _, dg = adj(x, hs, g, (need_x, False, need_g))
            big_x, big_g = _add(big_x, dx), _add(big_g, dg)
        if hg is not None:
            dx, ds, _ = adj(x, sh, hg, (need_x, need_s, False))
            big_x, big_s = _add(big_x, dx), _add(big_s, ds)
        if need_v:
            if hx is not None:
                big_v = _add(big_v, fwd(hx, sh, g))
            if hs is not None:
                big_v = _add(big_v, fwd(x, hs, g))
            if hg is not None:
                big_v = _add(big_v, fwd(x, sh, hg))
        return big_x, big_s, big_g, big_v, None, None


def tensor_product(x, sh, g, call: TpCall):
    """out = F(x, sh, g): edge rows when ``call.topology`` is None, receiver rows otherwise."""
    return _TpForward.apply(x, sh, g, call)
