"""Direction harmonics with analytic first and second adjoints (kernels in csrc/harmonics.cu).

Autograd structure follows ictc_o3/ops/generated_direction_harmonics.py:123-158: value -> vjp ->
second-order kernel; third derivatives are not provided.
"""
from __future__ import annotations

import torch

from .. import _lib
from ..autograd.adjoint_requirements import required_gradients


def _forward_raw(n, lmax):
    lib, e = _lib.load(), n.shape[0]
    y = torch.empty(e, (lmax + 1) ** 2, dtype=torch.float32, device=n.device)
    with _lib.on_device(n.device):
        _lib.check(lib.ictc_harmonics_forward(lmax, e, _lib.ptr(n), _lib.ptr(y), _lib.stream(n.device)),
                   "ictc_harmonics_forward")
    return y


def _vjp_raw(n, gy, lmax):
    lib, e = _lib.load(), n.shape[0]
    dn = torch.empty_like(n)
    with _lib.on_device(n.device):
        _lib.check(lib.ictc_harmonics_vjp(lmax, e, _lib.ptr(n), _lib.ptr(gy), _lib.ptr(dn), _lib.stream(n.device)),
                   "ictc_harmonics_vjp")
    return dn


def _second_raw(n, gy, hn, lmax, needed):
    lib, e = _lib.load(), n.shape[0]
    dn2 = torch.empty_like(n) if needed[0] else None
    dgy = torch.empty_like(gy) if needed[1] else None
    with _lib.on_device(n.device):
        _lib.check(lib.ictc_harmonics_second(lmax, e, _lib.ptr(n), _lib.ptr(gy), _lib.ptr(hn), _lib.ptr(dn2),
                                             _lib.ptr(dgy), _lib.stream(n.device)), "ictc_harmonics_second")
    return dn2, dgy


class _HarmonicsVjp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, n, gy, lmax):
        ctx.lmax = lmax
        ctx.save_for_backward(n, gy)
        return _vjp_raw(n, gy, lmax)

    @staticmethod
    def backward(ctx, h):
        n, gy = ctx.saved_tensors
        if torch.is_grad_enabled():
            raise NotImplementedError("third derivatives of the direction harmonics are not provided")
        needed = required_gradients((n, gy), ctx.needs_input_grad[:2])
        dn2, dgy = _second_raw(n, gy, h.contiguous(), ctx.lmax, needed)
        return dn2, dgy, None


class _Harmonics(torch.autograd.Function):
    @staticmethod
    def forward(ctx, n, lmax):
        ctx.lmax = lmax
        ctx.save_for_backward(n)
        return _forward_raw(n, lmax)

    @staticmethod
    def backward(ctx, gy):
        (n,) = ctx.saved_tensors
        gy = gy.contiguous()
        if torch.is_grad_enabled():
            return _HarmonicsVjp.apply(n, gy, ctx.lmax), None
        return _vjp_raw(n, gy, ctx.lmax), None


def harmonics_flat(n: torch.Tensor, lmax: int) -> torch.Tensor:
    """[E,3] unit vectors -> [E,(lmax+1)^2]."""
    return _Harmonics.apply(n.contiguous(), int(lmax))
