"""Receiver- and sender-CSR of an edge list, built on the device by ``ictc_csr_build``.

Replaces the reference's ``topology(dst, N)`` helper (ictc_o3/backends/k100/generated_csr_forward.py:17-31).
The forward of the graph message reduces over receivers, the feature adjoint over senders, so one
edge list needs up to two CSRs; both are built lazily and cached on this object.
"""
from __future__ import annotations

import torch

from .. import _lib


def build_csr(keys: torch.Tensor, num_nodes: int, assume_sorted: bool | None = None):
    """Return ``(rowptr[N+1], order[E] or None)``; ``order`` is None when keys are already sorted.

    ``assume_sorted=None`` reads the device-side sortedness flag back (one host sync); True/False
    skips the read-back and trusts the caller.
    """
    lib = _lib.load()
    dev = keys.device
    e = keys.numel()
    rowptr = torch.empty(num_nodes + 1, dtype=torch.int64, device=dev)
    order = torch.empty(e, dtype=torch.int64, device=dev)
    flag = torch.empty(1, dtype=torch.int32, device=dev)
    scratch = torch.empty(int(lib.ictc_csr_scratch_bytes(num_nodes, e)), dtype=torch.uint8, device=dev)
    with _lib.on_device(dev):
        _lib.check(lib.ictc_csr_build(_lib.ptr(keys), num_nodes, e, rowptr.data_ptr(), _lib.ptr(order),
                                      flag.data_ptr(), scratch.data_ptr(), _lib.stream(dev)), "ictc_csr_build")
    if assume_sorted is None:
        state = int(flag.item())
        if state < 0:
            raise ValueError("edge index outside [0, num_nodes)")
        assume_sorted = state == 1
    return rowptr, (None if assume_sorted else order)


class Topology:
    """Edge list ``(src, dst)`` over ``num_nodes`` rows with cached CSRs."""

    def __init__(self, src: torch.Tensor, dst: torch.Tensor, num_nodes: int, dst_sorted: bool | None = None):
        self.src, self.dst, self.num_nodes = src.contiguous(), dst.contiguous(), int(num_nodes)
        self.num_edges = int(src.numel())
        self._dst_sorted = dst_sorted
        self._by_dst = None
        self._by_src = None

    def by_dst(self):
        if self._by_dst is None:
            self._by_dst = build_csr(self.dst, self.num_nodes, self._dst_sorted)
        return self._by_dst

    def by_src(self):
        if self._by_src is None:
            self._by_src = build_csr(self.src, self.num_nodes, None)
        return self._by_src
