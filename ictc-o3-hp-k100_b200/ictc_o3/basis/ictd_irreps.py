"""Minimal host-side mirror of the reference's tensor-product module classes.

Only what the hot path needs from ``ictc_o3/basis/ictd_irreps.py`` of the reference: the
path-preserving edge-weighted tensor product as a *parameter holder* (path list, per-(path,channel)
base coefficients, per-degree path slots).  All arithmetic runs in the CUDA kernels; the couplings
come from the frozen constant tables.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch
from torch import nn

from .. import tables


class EdgeWeightedPathPreservingTensorProduct(nn.Module):
    """Path-preserving ICTC tensor product (reference: ictc_o3/basis/ictd_irreps.py:2299-2391, 2681-2713).

    Attributes mirror the reference: ``channels``, ``lmax``, ``paths`` (natural-parity (l1,l2,l3) with
    l3 <= lmax), ``num_paths``, ``weight`` [P, C] (initialised N(0, 0.02^2) as in the reference),
    ``path_l3``, ``path_offset``, ``path_counts_by_l``, ``internal_compute_dtype``.
    """

    def __init__(self, channels: int, lmax: int, *, allowed_paths: List[Tuple[int, int, int]] | None = None,
                 path_policy: str = "full", internal_compute_dtype: torch.dtype | None = None):
        super().__init__()
        if path_policy != "full":
            raise ValueError("only path_policy='full' is provided")
        self.channels, self.lmax = int(channels), int(lmax)
        self.internal_compute_dtype = torch.float32 if internal_compute_dtype is None else internal_compute_dtype
        all_paths = [(l1, l2, l3) for l1 in range(self.lmax + 1) for l2 in range(self.lmax + 1)
                     for l3 in range(abs(l1 - l2), min(l1 + l2, self.lmax) + 1) if (l1 + l2 + l3) % 2 == 0]
        if allowed_paths is not None:
            allowed = {tuple(p) for p in allowed_paths}
            all_paths = [p for p in all_paths if p in allowed]
        self.paths = all_paths
        self.num_paths = len(self.paths)
        self.weight = nn.Parameter(torch.randn(self.num_paths, self.channels) * 0.02)
        if self.paths:
            in_l = max(p[0] for p in self.paths)
            ed_l = max(p[1] for p in self.paths)
            plan = tables.tp_plan(tuple(self.paths), in_l, ed_l, self.lmax)
            self.path_l3 = [p[2] for p in self.paths]
            self.path_offset = list(plan.path_offset)
            self.path_counts_by_l: Dict[int, int] = dict(plan.counts)
        else:
            self.path_l3, self.path_offset = [], []
            self.path_counts_by_l = {l: 0 for l in range(self.lmax + 1)}

    def forward(self, x1: Dict[int, torch.Tensor], x2: Dict[int, torch.Tensor], gates: torch.Tensor | None = None):
        """{l:[E,C,2l+1]} x {l:[E,1,2l+1]} -> {l3:[E,count*C,2l3+1]} through the CUDA kernels."""
        from ..operators import EdgeTensorProduct
        in_l, ed_l = max(x1), max(x2)
        rows = next(iter(x1.values())).shape[0]
        if gates is None:
            gates = next(iter(x1.values())).new_ones(rows, self.num_paths * self.channels)
        op = EdgeTensorProduct(self, input_lmax=in_l, edge_lmax=ed_l, layout="mul_ir", _allow_live_weight=True)
        flat = torch.cat([x1[l].reshape(rows, -1) for l in range(in_l + 1)], -1)
        sh = torch.cat([x2[l].reshape(rows, 2 * l + 1) for l in range(ed_l + 1)], -1)
        return op.unpack_output(op(flat, sh, gates))
