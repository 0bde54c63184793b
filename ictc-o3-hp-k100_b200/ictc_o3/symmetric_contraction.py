"""Per-species symmetric contraction (correlation <= 3, lmax 2) on the CUDA kernels of csrc/sc.cu.

Module and factory names follow the reference (ictc_o3/ops/symmetric_contraction.py:8-158,
ictc_o3/operators.py:493-606).  Parameter layout is the reference's: one contraction per output
degree with ``weights_max`` (order = correlation) and ``weights[0..]`` (lower orders, descending),
each [S, P, C] initialised ``randn / P`` (ictc_o3/ops/_mace_symmetric_contraction.py:153-156,200-205).

The U tensors are the reference's e3nn-free construction ``ictd_u_matrix_so3`` (shipped in the constant
tables).  The reference's default product backend builds U from e3nn Wigner-3j symbols instead; both
span the same equivariant polynomials but individual path columns differ, so a weight tensor trained
with one is not portable to the other.
"""
from __future__ import annotations

import torch
from torch import nn

from . import _lib
from . import tables
from .autograd.adjoint_requirements import required_gradients

_LMAX = 2


class _ScCall:
    def __init__(self, channels, target_lmax, num_species, species, ir_mul):
        self.c, self.lt, self.s, self.species, self.ir_mul = channels, target_lmax, num_species, species, int(ir_mul)
        self.nw = _lib.load().ictc_sc_num_weights(_LMAX, target_lmax)
        self.ny = (target_lmax + 1) ** 2

    def _scratch(self, n, dev):
        nbytes = int(_lib.load().ictc_sc_scratch_bytes(_LMAX, self.lt, self.c, n, self.s))
        return torch.empty(nbytes, dtype=torch.uint8, device=dev)

    def forward(self, x, bank):
        n, dev = x.shape[0], x.device
        y = torch.empty(n, self.ny * self.c, dtype=torch.float32, device=dev)
        with _lib.on_device(dev):
            _lib.check(_lib.load().ictc_sc_forward(_LMAX, self.lt, self.c, n, self.s, self.ir_mul, _lib.ptr(x),
                                                   _lib.ptr(self.species), _lib.ptr(bank), _lib.ptr(y),
                                                   _lib.stream(dev)), "ictc_sc_forward")
        return y

    def adjoint(self, x, bank, gy, needed):
        n, dev = x.shape[0], x.device
        gx = torch.empty_like(x) if needed[0] else None
        gw = torch.empty_like(bank) if needed[1] else None
        scratch = self._scratch(n, dev) if needed[1] else None
        with _lib.on_device(dev):
            _lib.check(_lib.load().ictc_sc_adjoint(_LMAX, self.lt, self.c, n, self.s, self.ir_mul, _lib.ptr(x),
                                                   _lib.ptr(self.species), _lib.ptr(bank), _lib.ptr(gy),
                                                   _lib.ptr(gx), _lib.ptr(gw), _lib.ptr(scratch),
                                                   _lib.stream(dev)), "ictc_sc_adjoint")
        return gx, gw

    def second(self, x, bank, gy, hx, hw, needed):
        n, dev = x.shape[0], x.device
        dx = torch.empty_like(x) if needed[0] else None
        dw = torch.empty_like(bank) if needed[1] else None
        dgy = torch.empty_like(gy) if needed[2] else None
        scratch = self._scratch(n, dev) if needed[1] else None
        with _lib.on_device(dev):
            _lib.check(_lib.load().ictc_sc_second(_LMAX, self.lt, self.c, n, self.s, self.ir_mul, _lib.ptr(x),
                                                  _lib.ptr(self.species), _lib.ptr(bank), _lib.ptr(gy),
                                                  _lib.ptr(hx), _lib.ptr(hw), _lib.ptr(dgy), _lib.ptr(dx),
                                                  _lib.ptr(dw), _lib.ptr(scratch), _lib.stream(dev)),
                       "ictc_sc_second")
        return dx, dw, dgy


class _ScForward(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bank, call):
        ctx.call = call
        ctx.save_for_backward(x, bank)
        return call.forward(x, bank)

    @staticmethod
    def backward(ctx, gy):
        x, bank = ctx.saved_tensors
        needed = required_gradients((x, bank), ctx.needs_input_grad[:2])
        gy = gy.contiguous()
        if torch.is_grad_enabled():
            gx, gw = _ScAdjoint.apply(x, bank, gy, ctx.call, needed)
        else:
            gx, gw = ctx.call.adjoint(x, bank, gy, needed)
        return gx, gw, None


class _ScAdjoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bank, gy, call, needed):
        ctx.set_materialize_grads(False)
        ctx.call = call
        ctx.save_for_backward(x, bank, gy)
        return call.adjoint(x, bank, gy, needed)

    @staticmethod
    def backward(ctx, hx, hw):
        if torch.is_grad_enabled():
            raise NotImplementedError("third derivatives of the symmetric contraction are not provided")
        x, bank, gy = ctx.saved_tensors
        needed = required_gradients((x, bank, gy), ctx.needs_input_grad[:3])
        if hx is None and hw is None:
            return None, None, None, None, None
        dx, dw, dgy = ctx.call.second(x, bank, gy, None if hx is None else hx.contiguous(),
                                      None if hw is None else hw.contiguous(), needed)
        return dx, dw, dgy, None, None


class _Contraction(nn.Module):
    """Weights of one output degree (reference: _mace_symmetric_contraction.py:86-205)."""

    def __init__(self, output_l, correlation, num_elements, channels):
        super().__init__()
        self.output_lmax, self.correlation = int(output_l), int(correlation)
        sizes = {nu: tables.sc_u_tensor(output_l, nu).shape[-1] for nu in range(1, correlation + 1)}
        self.weights_max = nn.Parameter(torch.randn(num_elements, sizes[correlation], channels) / sizes[correlation])
        self.weights = nn.ParameterList(
            [nn.Parameter(torch.randn(num_elements, sizes[nu], channels) / sizes[nu])
             for nu in range(correlation - 1, 0, -1)])

    def by_order(self):
        """[W_1, W_2, ..., W_corr]"""
        return list(reversed(list(self.weights))) + [self.weights_max]


class _Contractions(nn.Module):
    def __init__(self, contractions):
        super().__init__()
        self.contractions = nn.ModuleList(contractions)


class ICTDBridgeUSymmetricContractionSO3(nn.Module):
    """Symmetric contraction consuming and returning ICTC-basis flat features (mul_ir rows).

    forward(node_feats [N, 9*C], node_attrs, node_type_idx=None) -> [N, (target_lmax+1)^2 * C]
    (ictc_o3/ops/symmetric_contraction.py:98-147).  Species come from ``node_type_idx`` (int64 [N]) or,
    when absent, from the arg-max of the one-hot ``node_attrs``.
    """

    def __init__(self, *, num_elements, channels, lmax, target_lmax, correlation=3, use_reduced_cg=False):
        super().__init__()
        if lmax != _LMAX or target_lmax not in (0, _LMAX):
            raise ValueError("symmetric-contraction kernels are compiled for lmax 2 and target_lmax 0 or 2")
        if correlation not in (1, 2, 3):
            raise ValueError("correlation must be 1, 2 or 3")
        if use_reduced_cg:
            raise ValueError("reduced CG is not provided")
        self.channels, self.lmax, self.target_lmax = int(channels), int(lmax), int(target_lmax)
        self.num_elements, self.correlation, self.use_reduced_cg = int(num_elements), int(correlation), False
        self.symmetric_contractions = _Contractions(
            [_Contraction(l, correlation, num_elements, channels) for l in range(target_lmax + 1)])
        self.ir_mul = False

    def weight_bank(self):
        """[S, NW, C] in kernel order (l_out, nu = 1..3, p); orders above ``correlation`` are zero."""
        parts = []
        for l, contraction in enumerate(self.symmetric_contractions.contractions):
            ws = contraction.by_order()
            for nu in (1, 2, 3):
                if nu <= self.correlation:
                    parts.append(ws[nu - 1])
                else:
                    size = tables.sc_u_tensor(l, nu).shape[-1]
                    parts.append(ws[0].new_zeros(self.num_elements, size, self.channels))
        return torch.cat(parts, dim=1).contiguous()

    def forward(self, node_feats, node_attrs=None, node_type_idx=None):
        if not node_feats.is_cuda or node_feats.dtype != torch.float32:
            raise ValueError("Generated SC requires CUDA FP32")
        n = node_feats.shape[0]
        if node_feats.ndim != 2 or node_feats.shape[1] != 9 * self.channels:
            raise ValueError(f"node_feats must have shape [N, {9 * self.channels}]")
        if node_type_idx is None:
            if node_attrs is None:
                raise ValueError("node_attrs or node_type_idx is required")
            node_type_idx = node_attrs.argmax(-1)
        if node_type_idx.shape != (n,) or node_type_idx.device != node_feats.device or node_type_idx.dtype != torch.int64:
            raise ValueError("Species indices must be int64 [N] on the feature device")
        call = _ScCall(self.channels, self.target_lmax, self.num_elements, node_type_idx.contiguous(), self.ir_mul)
        return _ScForward.apply(node_feats.contiguous(), self.weight_bank(), call)


def create_symmetric_contraction(*, num_elements, lmax, target_lmax=None, channels=64, correlation=3,
                                 use_reduced_cg=False, device="cuda", policy="generated", high_l_policy="auto",
                                 training=False, reference_buffer_policy="auto", species_schedule="auto",
                                 inference_basis_fusion="auto"):
    """Create a parameterised trainable SC (ictc_o3/operators.py:493-526)."""
    from .operators import _need_degree, _need_positive, strict_fp32
    _need_degree(lmax, "lmax")
    _need_positive(channels, "channels")
    _need_positive(correlation, "correlation")
    if correlation > 3:
        raise ValueError(f"correlation: orders 1 to 3 are provided, got {correlation}")
    if not isinstance(use_reduced_cg, bool):
        raise TypeError(f"use_reduced_cg: expected True or False, got {type(use_reduced_cg).__name__}")
    if use_reduced_cg:
        raise ValueError("use_reduced_cg: this factory builds the full Clebsch-Gordan basis only")
    if target_lmax is None:
        target_lmax = lmax
    _need_degree(target_lmax, "target_lmax")
    _need_positive(num_elements, "num_elements")
    strict_fp32()
    module = ICTDBridgeUSymmetricContractionSO3(
        num_elements=num_elements, channels=channels, lmax=lmax, target_lmax=target_lmax,
        correlation=correlation, use_reduced_cg=use_reduced_cg).to(device=device, dtype=torch.float32)
    configure_symmetric_contraction(module, policy=policy, high_l_policy=high_l_policy, training=training,
                                    reference_buffer_policy=reference_buffer_policy,
                                    species_schedule=species_schedule, inference_basis_fusion=inference_basis_fusion)
    return module


def configure_symmetric_contraction(module, *, policy="auto", high_l_policy="auto", training=False,
                                    reference_buffer_policy="auto", species_schedule="auto",
                                    inference_basis_fusion="auto"):
    """Validate the reference's option set and report the selected plan (ictc_o3/operators.py:529-606).

    There is one kernel path here, so the K100 scheduling options only get validated."""
    from .operators import _need_choice
    if not isinstance(module, ICTDBridgeUSymmetricContractionSO3):
        raise TypeError(f"module: expected the bridge-U symmetric contraction, got {type(module).__name__}")
    _need_choice(policy, ("auto", "generated", "reference"), "policy")
    _need_choice(high_l_policy, ("auto", "off"), "high_l_policy")
    _need_choice(species_schedule, ("auto", "grouped", "indexed"), "species_schedule")
    _need_choice(reference_buffer_policy, ("auto", "device"), "reference_buffer_policy")
    if inference_basis_fusion != "auto" and not isinstance(inference_basis_fusion, bool):
        raise ValueError(f"inference_basis_fusion: expected 'auto', True or False, got {inference_basis_fusion!r}")
    if not isinstance(training, bool):
        raise TypeError(f"training: expected True or False, got {type(training).__name__}")
    weights = next(module.parameters())
    supported = weights.dtype == torch.float32 and weights.is_cuda
    if not supported and policy == "generated":
        raise ValueError("policy='generated' needs the module on a CUDA device in float32")
    return {"selected": "generated" if supported else "reference", "high_l_policy": high_l_policy,
            "species_schedule": species_schedule, "indexed_species_active": True,
            "inference_basis_fusion": inference_basis_fusion, "basis_fusion_active": False,
            "reference_buffer_policy": reference_buffer_policy, "sc_schedule": "circuit",
            "reasons": [] if supported else ["outside qualified standalone SC coverage"]}
