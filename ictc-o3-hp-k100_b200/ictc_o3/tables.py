"""Host-side constant tables of the ICTC Cartesian-harmonic basis and the TP path plan.

Everything numeric comes from ``constants/ictc_tables_lmax{L}.npz`` (derived from the reference's
frozen basis assets by ``constants/make_tables.py``).  This module restates, as plain Python:

* the natural-parity path list, the (l1,l2) grouping, per-degree path slots and the flat
  ``ir_mul`` / ``mul_ir`` offsets of the reference plan
  (reference: ictc_o3/basis/ictd_irreps.py:2315-2391,2692-2706; ictc_o3/ops/fused_message.py:423-489);
* the coupling normalisation  C_p = CG * sqrt(2*l3+1)/||CG||_F * 1/sqrt(#paths landing on l3)
  (ictd_irreps.py:116-157);
* the sparse list of non-zero couplings, keeping |c| > 1e-12 as the reference's projector plan does
  (ictc_o3/ops/bond_projection.py:63-71).
"""
from __future__ import annotations

import functools
import math
import os
from dataclasses import dataclass, field
from typing import Dict, List, Tuple

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
TABLE_LMAX = 2
COEFF_THRESHOLD = 1e-12


@functools.lru_cache(maxsize=None)
def raw_tables(lmax: int = TABLE_LMAX) -> Dict[str, np.ndarray]:
    path = os.path.join(_HERE, "constants", f"ictc_tables_lmax{lmax}.npz")
    with np.load(path) as data:
        return {k: np.array(data[k]) for k in data.files}


def natural_paths(input_lmax: int, edge_lmax: int, output_lmax: int) -> List[Tuple[int, int, int]]:
    """Path order of ``EdgeTensorProduct.create`` (ictc_o3/operators.py:206-207)."""
    return [(i, j, k) for i in range(input_lmax + 1) for j in range(edge_lmax + 1)
            for k in range(output_lmax + 1) if abs(i - j) <= k <= i + j and (i + j + k) % 2 == 0]


def normalized_cg(l1: int, l2: int, l3: int) -> np.ndarray:
    """Component-normalised coupling tensor [2l1+1, 2l2+1, 2l3+1] (float64)."""
    t = raw_tables()
    key = f"cg_{l1}{l2}{l3}"
    if key not in t:
        raise ValueError(f"coupling ({l1},{l2},{l3}) is outside the shipped tables (lmax {TABLE_LMAX})")
    c = t[key]
    norm = float(np.sqrt((c * c).sum()))
    return c * (math.sqrt(2 * l3 + 1) / norm) if norm > 1e-30 else c


@dataclass(frozen=True)
class TpPlan:
    """Offsets and sparse couplings of one path-preserving tensor product.

    Component indices are in units of one channel vector: feature component ``i`` lives at
    ``x[row, i*C + c]`` in ir_mul and at ``x[row, xoff(l)*C + c*(2l+1) + (i-xoff(l))]`` in mul_ir.
    """
    paths: Tuple[Tuple[int, int, int], ...]
    input_lmax: int
    edge_lmax: int
    lmax: int                                 # output degrees run 0..lmax
    path_offset: Tuple[int, ...]              # slot of path p inside its output degree
    counts: Dict[int, int]                    # paths per output degree
    scales: Tuple[float, ...]                 # 1/sqrt(#paths -> l3)
    x_off: Dict[int, int]                     # first component of input degree l
    o_off: Dict[int, int]                     # first component of output degree l
    nx: int
    nh: int
    no: int
    out_base: Tuple[int, ...]                 # first output component of path p
    nnz: Tuple[Tuple[int, int, int, int, float], ...] = field(repr=False)   # (i, j, k, p, coeff)

    @property
    def num_paths(self) -> int:
        return len(self.paths)

    def dense(self) -> np.ndarray:
        """Dense [nx, nh, no] coupling array (float64) — used by tests and the CPU oracle."""
        a = np.zeros((self.nx, self.nh, self.no))
        for i, j, k, _p, c in self.nnz:
            a[i, j, k] = c
        return a

    def out_path(self) -> List[int]:
        """Path index of every output component."""
        res = [0] * self.no
        for p, (_l1, _l2, l3) in enumerate(self.paths):
            for m in range(2 * l3 + 1):
                res[self.out_base[p] + m] = p
        return res


@functools.lru_cache(maxsize=None)
def tp_plan(paths: Tuple[Tuple[int, int, int], ...], input_lmax: int, edge_lmax: int, lmax: int) -> TpPlan:
    paths = tuple(tuple(int(v) for v in p) for p in paths)
    if not paths:
        raise ValueError("TP paths must be nonempty")
    # groups sorted by (l1,l2); slots are handed out in group iteration order (ictd_irreps.py:2694-2706)
    groups: Dict[Tuple[int, int], List[int]] = {}
    for p, (l1, l2, _l3) in enumerate(paths):
        groups.setdefault((l1, l2), []).append(p)
    counts = {l: 0 for l in range(lmax + 1)}
    path_offset = [0] * len(paths)
    for key in sorted(groups):
        for p in groups[key]:
            l3 = paths[p][2]
            path_offset[p] = counts[l3]
            counts[l3] += 1
    scales = tuple(1.0 / math.sqrt(counts[p[2]]) for p in paths)
    x_off, acc = {}, 0
    for l in range(input_lmax + 1):
        x_off[l] = acc
        acc += 2 * l + 1
    nx = acc
    o_off, acc = {}, 0
    for l in range(lmax + 1):
        o_off[l] = acc
        acc += counts[l] * (2 * l + 1)
    no = acc
    nh = (edge_lmax + 1) ** 2
    out_base = tuple(o_off[l3] + path_offset[p] * (2 * l3 + 1) for p, (_a, _b, l3) in enumerate(paths))
    nnz = []
    for p, (l1, l2, l3) in enumerate(paths):
        c = normalized_cg(l1, l2, l3) * scales[p]
        for i in range(2 * l1 + 1):
            for j in range(2 * l2 + 1):
                for m in range(2 * l3 + 1):
                    v = float(c[i, j, m])
                    if abs(v) > COEFF_THRESHOLD:
                        nnz.append((x_off[l1] + i, l2 * l2 + j, out_base[p] + m, p, v))
    return TpPlan(paths, input_lmax, edge_lmax, lmax, tuple(path_offset), counts, scales, x_off, o_off,
                  nx, nh, no, out_base, tuple(nnz))


def harmonic_terms(lmax: int):
    """Polynomial terms of the component-normalised direction harmonics.

    Returns ``terms[h] = [((a,b,c), coeff), ...]`` with ``Y[h] = sum coeff * x^a y^b z^c`` for the flat
    harmonic index ``h`` (degrees ascending).  Restates the term extraction of
    ictc_o3/ops/generated_direction_harmonics.py:60-66 (no coefficient threshold, exact zeros skipped).
    """
    if lmax > TABLE_LMAX:
        raise ValueError(f"direction harmonics are shipped up to lmax {TABLE_LMAX}")
    t = raw_tables()
    terms = [[((0, 0, 0), 1.0)]]
    for l in range(1, lmax + 1):
        exps, coef = t[f"harm_exps_{l}"], t[f"harm_coef_{l}"]
        for h in range(2 * l + 1):
            terms.append([(tuple(int(v) for v in exps[r]), float(coef[r, h]))
                          for r in range(exps.shape[0]) if coef[r, h] != 0.0])
    return terms


def sc_u_tensor(lout: int, nu: int) -> np.ndarray:
    """U tensor of the e3nn-free symmetric contraction (ictd_irreps.py:1535-1557), lmax 2, float64."""
    return raw_tables()[f"u_{lout}_{nu}"]
