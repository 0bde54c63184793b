"""Public operators of the ICTC hot path on B200.

The names, argument meaning, accepted values and exception types are those of the reference's
``ictc_o3/operators.py`` (EdgeTensorProduct :161-340, PackedGraphMessage :343-409, GraphMessage :412-468,
direction_harmonics :471-490, channel_linear :609-628, normalized_silu :631-636), so a caller of the
reference can switch packages without touching its code.  The bodies are this build's own: every call ends in
``libictc_b200.so`` through the C ABI, CPU tensors are refused, and there is a single kernel path, so the
reference's schedule-selection arguments are validated and then have no further effect.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from . import tables

__all__ = [
    "EdgeTensorProduct", "GraphMessage", "PackedGraphMessage", "direction_harmonics",
    "create_symmetric_contraction", "configure_symmetric_contraction",
    "channel_linear", "normalized_silu", "convert_layout",
]


def strict_fp32():
    """Library GEMMs must not drop to TF32 behind the caller's back (ictc_o3/backends/k100/fp32_policy.py:6-11)."""
    if torch.backends.cuda.matmul.allow_tf32 or torch.get_float32_matmul_precision() != "highest":
        torch.set_float32_matmul_precision("highest")
        torch.backends.cuda.matmul.allow_tf32 = False
    if torch.backends.cudnn.allow_tf32:
        torch.backends.cudnn.allow_tf32 = False


# ------------------------------------------------------------------------------- argument checks
def _is_count(value, least):
    return isinstance(value, int) and not isinstance(value, bool) and value >= least


def _need_degree(value, name):
    if not _is_count(value, 0):
        raise ValueError(f"{name}: expected an integer degree >= 0, got {value!r}")


def _need_positive(value, name):
    if not _is_count(value, 1):
        raise ValueError(f"{name}: expected an integer >= 1, got {value!r}")


def _need_choice(value, allowed, name):
    if value not in allowed:
        raise ValueError(f"{name}: {value!r} is not one of {', '.join(map(repr, allowed))}")


def _need_eager(sample):
    """The kernels are plain eager launches: tracing, functorch transforms, fake tensors and autocast are
    refused (the reference has the same rule, ictc_o3/operators.py:24-32)."""
    strict_fp32()
    from torch._subclasses.fake_tensor import is_fake
    from torch.fx.experimental.proxy_tensor import get_proxy_mode
    traced = torch.compiler.is_compiling() or get_proxy_mode() is not None or is_fake(sample)
    if traced or torch._C._are_functorch_transforms_active() or torch.is_autocast_enabled(sample.device.type):
        raise ValueError("the tensor-product kernels run eagerly only: no compile/functorch tracing, no autocast")


def _need_tensor(value, shape, like, name):
    """``value`` must be an fp32 tensor of exactly ``shape`` on the device of ``like``."""
    shape = tuple(int(s) for s in shape)
    if not isinstance(value, torch.Tensor) or tuple(value.shape) != shape:
        got = tuple(value.shape) if isinstance(value, torch.Tensor) else type(value).__name__
        raise ValueError(f"{name}: expected a tensor of shape {shape}, got {got}")
    if value.dtype != torch.float32 or value.device != like.device:
        raise ValueError(f"{name}: expected float32 on {like.device}, got {value.dtype} on {value.device}")


def _need_tp(tp, input_lmax, edge_lmax, live_weight_ok=False):
    """Coverage test of a tensor-product module: right class, fp32 on CUDA, frozen base coefficients and a
    path list that stays inside the declared degrees."""
    from .basis.ictd_irreps import EdgeWeightedPathPreservingTensorProduct as TP
    _need_degree(input_lmax, "input_lmax")
    _need_degree(edge_lmax, "edge_lmax")
    if not isinstance(tp, TP):
        raise TypeError(f"expected an EdgeWeightedPathPreservingTensorProduct, got {type(tp).__name__}")
    w = tp.weight
    fp32 = w.dtype == torch.float32 and tp.internal_compute_dtype == torch.float32
    if not (w.is_cuda and fp32 and tp.channels >= 1 and tp.lmax >= 0):
        raise ValueError("the tensor product must live on a CUDA device and compute in float32 with >= 1 channel")
    if w.requires_grad and not live_weight_ok:
        raise ValueError("base coefficients of the tensor product still require grad: freeze them first")
    inside = all(l1 <= input_lmax and l2 <= edge_lmax for l1, l2, _ in tp.paths)
    if len(tp.paths) == 0 or not inside:
        raise ValueError("the path list is empty or uses a degree above input_lmax / edge_lmax")


def _need_index(value, count, like, name):
    ok = (isinstance(value, torch.Tensor) and value.dtype == torch.int64 and value.ndim == 1
          and value.numel() == count and value.device == like.device)
    if not ok:
        raise ValueError(f"{name}: expected an int64 vector of {count} node indices on {like.device}")


# ------------------------------------------------------------------------------- layout conversion
class _LayoutCopy(torch.autograd.Function):
    """mul_ir <-> ir_mul conversion of whole rows in one kernel (``ictc_layout_copy``); its adjoint is the
    opposite conversion, so the function is its own derivative up to the direction flag."""

    @staticmethod
    def forward(ctx, flat, channels, blocks, to_ir_mul):
        ctx.args = (channels, blocks, to_ir_mul)
        flat = flat.contiguous()
        out = torch.empty_like(flat)
        counts = (C.c_int * len(blocks))(*[b[0] for b in blocks])
        ms = (C.c_int * len(blocks))(*[b[1] for b in blocks])
        with _lib.on_device(flat.device):
            _lib.check(_lib.load().ictc_layout_copy(flat.shape[0], channels, len(blocks), counts, ms, _lib.ptr(flat),
                                                    _lib.ptr(out), int(to_ir_mul), _lib.stream(flat.device)),
                       "ictc_layout_copy")
        return out

    @staticmethod
    def backward(ctx, grad):
        channels, blocks, to_ir_mul = ctx.args
        return _LayoutCopy.apply(grad, channels, blocks, not to_ir_mul), None, None, None


def convert_layout(flat, channels, blocks, to_ir_mul):
    """Rows ``[rows, sum(count*C*m)]`` made of degree blocks ``blocks = ((count, m), ...)``: mul_ir (slot
    [C, m]) -> ir_mul (slot [m, C]) when ``to_ir_mul`` else the reverse.  Differentiable; CUDA fp32 only.
    Stands in for the reference's ``fused_pack`` copy kernel (ictc_o3/ops/message_layout.py:25-93)."""
    blocks = tuple((int(c), int(m)) for c, m in blocks)
    if flat.ndim != 2 or flat.shape[1] != sum(c * m for c, m in blocks) * channels:
        raise ValueError("convert_layout: row width does not match the block list")
    if not flat.is_cuda or flat.dtype != torch.float32:
        raise ValueError("convert_layout: expected a float32 CUDA tensor")
    return _LayoutCopy.apply(flat, int(channels), blocks, bool(to_ir_mul))


# ------------------------------------------------------------------------------- edge tensor product
class EdgeTensorProduct(torch.nn.Module):
    """Tensor product of per-edge feature rows with per-edge harmonics, one gate per (path, channel).

    Buffer contract of the reference (ictc_o3/operators.py:161-340): layout ``ir_mul`` keeps [component,
    channel] inside every degree block and path slot, ``mul_ir`` keeps [channel, component]; paths keep their
    own output slots; autograd of first, mixed second and higher order works; eager execution only.
    ``execution`` ('direct' / 'legacy') picks between K100 schedules in the reference and changes nothing here.
    """

    def __init__(self, tp, *, input_lmax, edge_lmax, layout="ir_mul", execution="direct", _allow_live_weight=False):
        super().__init__()
        _need_tp(tp, input_lmax, edge_lmax, _allow_live_weight)
        _need_choice(layout, ("ir_mul", "mul_ir"), "layout")
        _need_choice(execution, ("direct", "legacy"), "execution")
        top = max(path[2] for path in tp.paths)
        full = tables.natural_paths(input_lmax, edge_lmax, top)
        if full != [tuple(path) for path in tp.paths]:
            raise ValueError(f"kernels exist for complete natural-parity path sets only; input_lmax={input_lmax}, "
                             f"edge_lmax={edge_lmax} came with paths {list(tp.paths)}")
        self.tp, self.layout, self.execution = tp, layout, execution
        self.input_lmax, self.edge_lmax = input_lmax, edge_lmax
        self._allow_live_weight = _allow_live_weight
        self._spec = _lib.tp_spec(input_lmax, edge_lmax, top)
        self._unit_seen = None       # (weight version, all-ones?) of the last look at the base coefficients

    @classmethod
    def create(cls, *, input_lmax, edge_lmax, output_lmax=None, channels=64, layout="ir_mul", execution="direct",
               device="cuda"):
        """A fresh float32 operator over the full natural-parity path set with all base coefficients equal to
        one and frozen (ictc_o3/operators.py:190-215)."""
        from .basis.ictd_irreps import EdgeWeightedPathPreservingTensorProduct as TP
        _need_positive(channels, "channels")
        for name, value in (("input_lmax", input_lmax), ("edge_lmax", edge_lmax)):
            _need_degree(value, name)
        if output_lmax is None:
            output_lmax = input_lmax
        _need_degree(output_lmax, "output_lmax")
        if torch.device(device).type != "cuda":
            raise ValueError(f"device: the operator exists on CUDA devices only, got {device!r}")
        module = TP(channels=channels, lmax=max(input_lmax, edge_lmax, output_lmax),
                    allowed_paths=tables.natural_paths(input_lmax, edge_lmax, output_lmax), path_policy="full",
                    internal_compute_dtype=torch.float32).to(device=device, dtype=torch.float32)
        module.weight.requires_grad_(False)
        module.weight.fill_(1.0)
        return cls(module, input_lmax=input_lmax, edge_lmax=edge_lmax, layout=layout, execution=execution)

    # ---- sizes
    @property
    def paths(self):
        """(input degree, edge degree, output degree) per gate block, in gate order."""
        return tuple((int(a), int(b), int(c)) for a, b, c in self.tp.paths)

    @property
    def gate_width(self):
        return self.tp.channels * self.tp.num_paths

    def _slots(self, l):
        return int(self.tp.path_counts_by_l.get(l, 0))

    @property
    def output_width(self):
        return self.tp.channels * sum(self._slots(l) * (2 * l + 1) for l in range(self.tp.lmax + 1))

    def _in_blocks(self):
        return tuple((1, 2 * l + 1) for l in range(self.input_lmax + 1))

    def _out_blocks(self):
        return tuple((self._slots(l), 2 * l + 1) for l in range(self.tp.lmax + 1))

    def _weight(self):
        """Base coefficients for the kernel; None stands for "all one" (looked up once per weight update)."""
        w = self.tp.weight
        stamp = None if w.is_inference() else w._version
        if stamp is None or self._unit_seen is None or self._unit_seen[0] != stamp:
            self._unit_seen = (stamp, bool((w == 1).all().item()))
        return None if self._unit_seen[1] else w.detach().contiguous()

    # ---- dictionary <-> flat rows
    def pack_input(self, blocks):
        """{l: [rows, C, 2l+1]} -> flat rows in this operator's layout."""
        degrees = range(self.input_lmax + 1)
        if sorted(blocks) != list(degrees):
            raise ValueError(f"pack_input: need exactly the degrees 0..{self.input_lmax}, got {sorted(blocks)}")
        c, rows = self.tp.channels, blocks[0].shape[0]
        flat = []
        for l in degrees:
            _need_tensor(blocks[l], (rows, c, 2 * l + 1), self.tp.weight, f"blocks[{l}]")
            piece = blocks[l].permute(0, 2, 1) if self.layout == "ir_mul" else blocks[l]
            flat.append(piece.reshape(rows, -1))
        return torch.cat(flat, dim=1).contiguous()

    def unpack_output(self, output):
        """Flat output rows -> {l: [rows, slots_l * C, 2l+1]} (slot outer, channel inner)."""
        _need_tensor(output, (output.shape[0], self.output_width), self.tp.weight, "output")
        c, rows, start, result = self.tp.channels, output.shape[0], 0, {}
        for l in range(self.tp.lmax + 1):
            slots, m = self._slots(l), 2 * l + 1
            stop = start + slots * c * m
            piece = output[:, start:stop]
            if self.layout == "ir_mul":
                piece = piece.reshape(rows, slots, m, c).permute(0, 1, 3, 2)
            result[l] = piece.reshape(rows, slots * c, m)
            start = stop
        return result

    def forward(self, features, harmonics, gates):
        """features [E, C*(L_in+1)^2], harmonics [E, (L_edge+1)^2], gates [E, P*C] or [E, P, C]."""
        _need_tp(self.tp, self.input_lmax, self.edge_lmax, self._allow_live_weight)
        _need_eager(features)
        if features.ndim != 2:
            raise ValueError("features: expected flat rows [E, width]")
        c, rows, like = self.tp.channels, features.shape[0], self.tp.weight
        _need_tensor(features, (rows, c * (self.input_lmax + 1) ** 2), like, "features")
        _need_tensor(harmonics, (rows, (self.edge_lmax + 1) ** 2), like, "harmonics")
        gate_shape = (rows, self.tp.num_paths, c) if gates.ndim == 3 else (rows, self.gate_width)
        _need_tensor(gates, gate_shape, like, "gates")
        gates = gates.reshape(rows, self.gate_width)
        if rows == 0:       # keep the autograd link of all three operands on an empty result
            link = features[:, :1] * harmonics[:, :1] * gates[:, :1]
            return link.expand(0, self.output_width)
        from .ops.tensor_product import TpCall, tensor_product
        mul_ir = self.layout == "mul_ir"
        if mul_ir:
            features = convert_layout(features, c, self._in_blocks(), True)
        call = TpCall(self._spec, c, self._weight(), None, None)
        result = tensor_product(features.contiguous(), harmonics.contiguous(), gates.contiguous(), call)
        return convert_layout(result, c, self._out_blocks(), False) if mul_ir else result


# ------------------------------------------------------------------------------- graph messages
class PackedGraphMessage(torch.nn.Module):
    """Gather at the sender, tensor product, sum at the receiver, on packed ir_mul rows.

    Same call contract as the reference (ictc_o3/operators.py:343-409).  The receiver sum always walks a
    receiver CSR with one warp per row (no float atomics, bitwise repeatable), so ``reduction`` and the K100
    tuning arguments (``edge_chunk_size``, ``topology_backend``, ``csr_accumulator_limit``,
    ``csr_slice_search``, ``geometry_schedule``) are checked for validity and otherwise unused.
    """

    def __init__(self, tp, *, input_lmax, edge_lmax, cartesian_schedule='native', reduction='atomic',
                 edge_chunk_size=65536, topology_backend='native', csr_accumulator_limit=None,
                 csr_slice_search=False, geometry_schedule='auto'):
        super().__init__()
        _need_choice(cartesian_schedule, ("native",), "cartesian_schedule")
        _need_choice(reduction, ("atomic", "csr"), "reduction")
        _need_choice(topology_backend, ("native", "device"), "topology_backend")
        _need_choice(geometry_schedule, ("auto", "native", "streamed"), "geometry_schedule")
        _need_positive(edge_chunk_size, "edge_chunk_size")
        if csr_accumulator_limit is not None:
            _need_positive(csr_accumulator_limit, "csr_accumulator_limit")
        if not isinstance(csr_slice_search, bool):
            raise ValueError(f"csr_slice_search: expected True or False, got {csr_slice_search!r}")
        self.edge = EdgeTensorProduct(tp, input_lmax=input_lmax, edge_lmax=edge_lmax)
        self.cartesian_schedule, self.reduction, self.edge_chunk_size = cartesian_schedule, reduction, edge_chunk_size
        self._topology, self._topology_key = None, None

    @classmethod
    def create(cls, *, channels=64, input_lmax=3, edge_lmax=3, output_lmax=None, device='cuda', **kwargs):
        seed = EdgeTensorProduct.create(channels=channels, input_lmax=input_lmax, edge_lmax=edge_lmax,
                                        output_lmax=output_lmax, device=device)
        return cls(seed.tp, input_lmax=input_lmax, edge_lmax=edge_lmax, **kwargs)

    tp = property(lambda self: self.edge.tp)
    gate_width = property(lambda self: self.edge.gate_width)
    output_width = property(lambda self: self.edge.output_width)

    def topology(self, src, dst, num_nodes):
        """Receiver / sender CSR pair of the edge list; cached until the index tensors change."""
        from .ops.topology import Topology
        stamp = (num_nodes, src.numel(), src.data_ptr(), dst.data_ptr(), src._version, dst._version)
        if self._topology_key != stamp:
            self._topology, self._topology_key = Topology(src, dst, num_nodes), stamp
        return self._topology

    def forward(self, features, harmonics, gates, src, dst, mask=None):
        _need_eager(features)
        edge = self.edge
        _need_tp(edge.tp, edge.input_lmax, edge.edge_lmax)
        if features.ndim != 2:
            raise ValueError("features: expected packed node rows [N, width]")
        like, c = edge.tp.weight, edge.tp.channels
        nodes, edges = features.shape[0], src.numel()
        _need_tensor(features, (nodes, c * (edge.input_lmax + 1) ** 2), like, "features")
        _need_tensor(harmonics, (edges, (edge.edge_lmax + 1) ** 2), like, "harmonics")
        gate_shape = (edges, edge.tp.num_paths, c) if gates.ndim == 3 else (edges, edge.gate_width)
        _need_tensor(gates, gate_shape, like, "gates")
        _need_index(src, edges, features, "src")
        _need_index(dst, edges, features, "dst")
        if mask is not None:
            if not isinstance(mask, torch.Tensor) or mask.requires_grad or tuple(mask.shape) not in ((edges,), (edges, 1)):
                raise ValueError("mask: expected a constant tensor of shape [E] or [E, 1]")
            _need_tensor(mask, mask.shape, like, "mask")
            mask = mask.reshape(edges).contiguous()
        from .ops.tensor_product import TpCall, tensor_product
        call = TpCall(edge._spec, c, edge._weight(), mask, self.topology(src, dst, nodes))
        return tensor_product(features.contiguous(), harmonics.contiguous(),
                              gates.reshape(edges, edge.gate_width).contiguous(), call)


class GraphMessage(torch.nn.Module):
    """Graph message with dictionary input and output (ictc_o3/operators.py:412-468):
    features {l: [N, C, 2l+1]}, harmonics {l: [E, 1, 2l+1]}, gates [E, P*C] -> {l: [N, slots_l*C, 2l+1]}.

    ``layout`` says how the dictionaries become kernel rows: 'packed' uses tensor reshapes, 'fused_pack' and
    'canonical' use the one-launch conversion kernel (``convert_layout``); the kernels themselves always work
    on ir_mul rows.  ``reduction`` is validated only (the receiver-CSR sum is the one reduction here).
    """

    def __init__(self, tp, *, input_lmax, edge_lmax, layout="packed", edge_chunk_size=65536, reduction="auto",
                 cartesian_schedule="native"):
        super().__init__()
        _need_tp(tp, input_lmax, edge_lmax)
        _need_choice(layout, ("packed", "fused_pack", "canonical"), "layout")
        _need_choice(reduction, ("auto", "atomic", "csr"), "reduction")
        _need_choice(cartesian_schedule, ("native",), "cartesian_schedule")
        _need_positive(edge_chunk_size, "edge_chunk_size")
        self.tp, self.layout, self.edge_chunk_size = tp, layout, edge_chunk_size
        self.input_lmax, self.edge_lmax = input_lmax, edge_lmax
        self._packed = PackedGraphMessage(tp, input_lmax=input_lmax, edge_lmax=edge_lmax)

    def forward(self, features, harmonics, gates, src, dst, mask=None):
        _need_tp(self.tp, self.input_lmax, self.edge_lmax)
        in_degrees, edge_degrees = list(range(self.input_lmax + 1)), list(range(self.edge_lmax + 1))
        if sorted(features) != in_degrees or sorted(harmonics) != edge_degrees:
            raise ValueError("features / harmonics: the dictionaries must hold every declared degree and no other")
        _need_eager(features[0])
        like, c = self.tp.weight, self.tp.channels
        nodes, edges = features[0].shape[0], src.numel()
        for l in in_degrees:
            _need_tensor(features[l], (nodes, c, 2 * l + 1), like, f"features[{l}]")
        for l in edge_degrees:
            _need_tensor(harmonics[l], (edges, 1, 2 * l + 1), like, f"harmonics[{l}]")
        _need_tensor(gates, (edges, self.tp.num_paths * c), like, "gates")
        edge = self._packed.edge
        sh = torch.cat([harmonics[l].reshape(edges, -1) for l in edge_degrees], dim=1)
        if self.layout == "packed":
            x = torch.cat([features[l].permute(0, 2, 1).reshape(nodes, -1) for l in in_degrees], dim=1)
            return edge.unpack_output(self._packed(x, sh, gates, src, dst, mask))
        # one conversion kernel each way instead of per-degree transposes and concatenations
        x = convert_layout(torch.cat([features[l].reshape(nodes, -1) for l in in_degrees], dim=1), c,
                           edge._in_blocks(), True)
        out = convert_layout(self._packed(x, sh, gates, src, dst, mask), c, edge._out_blocks(), False)
        result, start = {}, 0
        for l in range(self.tp.lmax + 1):
            width = edge._slots(l) * c * (2 * l + 1)
            result[l] = out[:, start:start + width].reshape(nodes, edge._slots(l) * c, 2 * l + 1)
            start += width
        return result


# ------------------------------------------------------------------------------- harmonics
def direction_harmonics(directions, lmax, *, policy="auto"):
    """Component-normalised Cartesian harmonics of unit vectors [E, 3] on a CUDA device: a list with one
    [E, 2l+1] block per degree (ictc_o3/operators.py:471-490).  The caller normalises its displacement
    vectors and differentiates through that normalisation.  ``policy`` picks between implementations in the
    reference; there is one here."""
    _need_degree(lmax, "lmax")
    _need_choice(policy, ("auto", "generated", "reference"), "policy")
    if directions.ndim != 2 or directions.shape[-1] != 3:
        raise ValueError(f"directions: expected [E, 3], got {tuple(directions.shape)}")
    if directions.dtype != torch.float32 or not directions.is_cuda:
        raise ValueError("directions: expected a float32 CUDA tensor")
    if lmax > tables.TABLE_LMAX:
        raise ValueError(f"lmax: harmonics are compiled for degrees up to {tables.TABLE_LMAX}")
    from .ops.harmonics import harmonics_flat
    return list(torch.split(harmonics_flat(directions, lmax), [2 * l + 1 for l in range(lmax + 1)], dim=-1))


# ------------------------------------------------------------------------------- channel linear
def _packed_operand(weight, transpose):
    """``weight`` [rows, 64] in the shared-memory operand layout of the tensor-core kernels.  Packed on every
    call (one small launch): a cache keyed on storage addresses could hand back the packing of a freed tensor."""
    packed = torch.empty(2 * weight.numel(), dtype=torch.float32, device=weight.device)
    with _lib.on_device(weight.device):
        _lib.check(_lib.load().ictc_gate_pack_weights(weight.shape[0], weight.data_ptr(), transpose,
                                                      packed.data_ptr(), _lib.stream(weight.device)),
                   "ictc_gate_pack_weights")
    return packed


def _tc_eligible(rows, weight):
    cout, cin = weight.shape
    return (weight.is_cuda and weight.dtype == torch.float32 and rows.is_cuda and min(cout, cin) == 64
            and cout % 64 == 0 and cin % 64 == 0)


def _tc_matmul(rows, weight):
    """rows [R, Cin] @ weight[Cout, Cin]^T on the tcgen05 channel-linear kernel (three-term TF32 split)."""
    cout, cin = weight.shape
    rows = rows.contiguous()
    out = torch.empty(rows.shape[0], cout, dtype=torch.float32, device=rows.device)
    if rows.shape[0] == 0:
        return out
    w = weight.detach().contiguous()
    if cin == 64:
        packed, kc, nc = _packed_operand(w, 0), 1, cout // 64
    else:
        packed, kc, nc = _packed_operand(w.t().contiguous(), 1), cin // 64, 1
    with _lib.on_device(rows.device):
        _lib.check(_lib.load().ictc_channel_linear_tc(rows.shape[0], kc, nc, rows.data_ptr(), 1, cin, packed.data_ptr(),
                                                      out.data_ptr(), 1, cout, _lib.stream(rows.device)),
                   "ictc_channel_linear_tc")
    return out


def _tc_weight_grad(grad, rows):
    """grad^T @ rows = [Cout, Cin], contracted over the rows on the tcgen05 weight-gradient kernel
    (``ictc_weight_grad_tc``: split over the SMs, partial sums added in a fixed order).  The 64-wide side is the
    kernel's second operand; the wide side is covered in blocks of at most 768 columns."""
    cout, cin = grad.shape[1], rows.shape[1]
    if cin != 64:                         # the wide side has to be the first operand: dW^T = rows^T @ grad
        return _tc_weight_grad(rows, grad).t()
    grad, rows = grad.contiguous(), rows.contiguous()
    r = grad.shape[0]
    out = torch.empty(cout, 64, dtype=torch.float32, device=grad.device)
    lib = _lib.load()
    with _lib.on_device(grad.device):
        for start in range(0, cout, 768):
            width = min(768, cout - start)
            need = lib.ictc_weight_grad_workspace(r, width)
            work = torch.empty(max(need, 16) // 4, dtype=torch.float32, device=grad.device)
            _lib.check(lib.ictc_weight_grad_tc(r, width, grad.data_ptr() + 4 * start, cout, rows.data_ptr(), 64,
                                               out.data_ptr() + 4 * 64 * start, 64, work.data_ptr(),
                                               _lib.stream(grad.device)), "ictc_weight_grad_tc")
    return out


class _WeightGrad(torch.autograd.Function):
    """The weight gradient as a differentiable node (its own derivatives are plain products, on the library GEMM:
    they are only met by third-order differentiation)."""

    @staticmethod
    def forward(ctx, grad, rows):
        ctx.save_for_backward(grad, rows)
        return _tc_weight_grad(grad, rows)

    @staticmethod
    def backward(ctx, g):
        grad, rows = ctx.saved_tensors
        return (rows.mm(g.t()) if ctx.needs_input_grad[0] else None,
                grad.mm(g) if ctx.needs_input_grad[1] else None)


class _RowsTimesWeight(torch.autograd.Function):
    """y = rows @ weight^T on the tensor-core kernel.  The input gradient is the same kernel with the weight
    transposed (applied through this function, so it stays differentiable); the weight gradient is the
    row-contracted outer product on the tcgen05 weight-gradient kernel."""

    @staticmethod
    def forward(ctx, rows, weight):
        ctx.save_for_backward(rows, weight)
        return _tc_matmul(rows, weight)

    @staticmethod
    def backward(ctx, grad):
        rows, weight = ctx.saved_tensors
        grad = grad.contiguous()
        d_rows = _RowsTimesWeight.apply(grad, weight.t()) if ctx.needs_input_grad[0] else None
        d_weight = _WeightGrad.apply(grad, rows.contiguous()) if ctx.needs_input_grad[1] else None
        return d_rows, d_weight


def channel_linear(features, weight, bias=None):
    """One weight matrix shared by every angular component: [*, Cin, m] x [Cout, Cin] -> [*, Cout, m]
    (ictc_o3/operators.py:609-628).  A bias is allowed for scalar blocks (m = 1) only.  With a 64-wide side
    and the other side a multiple of 64 on CUDA fp32 the product runs on the tcgen05 kernel
    (``ictc_channel_linear_tc``); other shapes use the library's fp32 GEMM."""
    strict_fp32()
    if weight.ndim != 2 or features.ndim < 2 or features.shape[-2] != weight.shape[1]:
        raise ValueError("channel_linear: features must be [*, Cin, m] and weight [Cout, Cin] with matching Cin")
    if (features.dtype, features.device) != (weight.dtype, weight.device):
        raise ValueError("channel_linear: features and weight differ in dtype or device")
    cout, cin = weight.shape
    if bias is not None:
        if features.shape[-1] != 1:
            raise ValueError("channel_linear: a bias only makes sense for the scalar block (m = 1)")
        if tuple(bias.shape) != (cout,) or (bias.dtype, bias.device) != (weight.dtype, weight.device):
            raise ValueError("channel_linear: bias must be [Cout] with the weight's dtype and device")
    by_component = features.transpose(-2, -1)                       # [*, m, Cin]
    lead = by_component.shape[:-1]
    rows = by_component.reshape(-1, cin)
    if _tc_eligible(rows, weight):
        product = _RowsTimesWeight.apply(rows, weight)
        if bias is not None:
            product = product + bias
    else:
        product = torch.addmm(bias, rows, weight.t()) if bias is not None else rows.mm(weight.t())
    return product.reshape(*lead, cout).transpose(-2, -1)


def normalized_silu(features, scale=1.0):
    """SiLU followed by a constant factor (ictc_o3/operators.py:631-636)."""
    if isinstance(scale, bool) or not isinstance(scale, (int, float)):
        raise TypeError(f"scale: expected a plain number, got {type(scale).__name__}")
    return float(scale) * torch.nn.functional.silu(features)


def create_symmetric_contraction(**kwargs):
    from .symmetric_contraction import create_symmetric_contraction as impl
    return impl(**kwargs)


def configure_symmetric_contraction(module, **kwargs):
    from .symmetric_contraction import configure_symmetric_contraction as impl
    return impl(module, **kwargs)
