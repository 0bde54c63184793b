"""Seeded synthetic systems with the shapes and value distributions of the benchmark configurations.

No dataset is involved anywhere: every input of the tests and of bench.py is drawn here.
Host-side helpers (numpy / scipy) build the *inputs*; they are never inside a timed region.
"""
from __future__ import annotations

import math

import numpy as np
import torch

SILU_SCALE = 1.6791767923989418


def uniform_box(num_atoms: int, density: float, seed: int):
    """Uniform random positions in a periodic cube of the given number density (atoms / A^3).

    Atoms are then ordered by spatial bin (bins of ~cutoff size, x-major) the way an MD code keeps
    its atoms sorted, so neighbouring rows are close in space."""
    rng = np.random.default_rng(seed)
    box = (num_atoms / density) ** (1.0 / 3.0)
    pos = rng.random((num_atoms, 3)) * box
    nb = max(1, int(box // 4.5))
    cell = np.minimum((pos / (box / nb)).astype(np.int64), nb - 1)
    key = (cell[:, 0] * nb + cell[:, 1]) * nb + cell[:, 2]
    order = np.argsort(key, kind="stable")
    return pos[order].astype(np.float32), np.array([box, box, box], dtype=np.float64)


def jittered_lattice(nx: int, ny: int, nz: int, spacing: float, sigma: float, seed: int):
    """Simple-cubic lattice with Gaussian jitter, H:C:O = 1:2:1 species, periodic box."""
    rng = np.random.default_rng(seed)
    grid = np.stack(np.meshgrid(np.arange(nx), np.arange(ny), np.arange(nz), indexing="ij"), -1).reshape(-1, 3)
    pos = (grid + 0.5) * spacing + rng.normal(0.0, sigma, size=(grid.shape[0], 3))
    box = np.array([nx, ny, nz], dtype=np.float64) * spacing
    pos = np.mod(pos, box)
    species = rng.permutation(np.resize(np.array([0, 1, 1, 2], dtype=np.int64), grid.shape[0]))
    return pos.astype(np.float32), box, species


def neighbor_list_host(pos: np.ndarray, box: np.ndarray, cutoff: float):
    """Full periodic neighbour list on the host: edge (src=j, dst=i) for every ordered pair with
    |r_j - r_i + S*box|^2 <= cutoff^2, sorted by (dst, src, shift) — the reference's canonical edge
    order (lammps_user_mfftorch/src/USER-MFFTORCH/pair_mff_torch_kokkos.cpp:767-785, 897-911).

    Distances are evaluated in float64 on the float32 positions.  Needs box >= 2*cutoff per axis
    (one image per pair).  Returns src, dst (int64) and shifts [E,3] (int64, lattice units) with
    edge_vec = pos[dst] - pos[src] + shifts*box.
    """
    from scipy.spatial import cKDTree
    p = np.mod(pos.astype(np.float64), box)
    p = np.where(p >= box, 0.0, p)
    tree = cKDTree(p, boxsize=box)
    pairs = tree.query_pairs(cutoff * (1 + 1e-9), output_type="ndarray")
    i, j = pairs[:, 0], pairs[:, 1]
    d = pos[i].astype(np.float64) - pos[j].astype(np.float64)          # vec for edge src=j,dst=i before shift
    shift = -np.round(d / box)
    d = d + shift * box
    keep = (d * d).sum(1) <= cutoff * cutoff
    i, j, shift = i[keep], j[keep], shift[keep].astype(np.int64)
    src = np.concatenate([j, i])
    dst = np.concatenate([i, j])
    shifts = np.concatenate([shift, -shift])
    order = np.lexsort((shifts[:, 2], shifts[:, 1], shifts[:, 0], src, dst))
    return src[order], dst[order], shifts[order]


def bessel_basis(r: torch.Tensor, cutoff: float, num_basis: int = 8, p: int = 5) -> torch.Tensor:
    """sqrt(2/rc) sin(n pi r/rc)/r times the polynomial cutoff envelope of order p
    (reference: mace_ictc/models/radial_basis.py:11-92)."""
    n = torch.arange(1, num_basis + 1, device=r.device, dtype=r.dtype)
    x = r.unsqueeze(-1)
    bessel = math.sqrt(2.0 / cutoff) * torch.sin(n * math.pi * x / cutoff) / x
    u = (r / cutoff).unsqueeze(-1)
    env = (1.0 - (p + 1.0) * (p + 2.0) / 2.0 * u ** p + p * (p + 2.0) * u ** (p + 1)
           - p * (p + 1.0) / 2.0 * u ** (p + 2))
    return bessel * env * (u < 1.0)


def random_radial_mlp(widths, seed: int, device):
    """Bias-free linears initialised N(0, 1/fan_in) (mace_ictc/models/mace/common.py:361-365)."""
    gen = torch.Generator().manual_seed(seed)
    return [(torch.randn(o, i, generator=gen) / math.sqrt(i)).to(device) for i, o in zip(widths[:-1], widths[1:])]


def radial_gates(basis: torch.Tensor, weights) -> torch.Tensor:
    h = basis
    for k, w in enumerate(weights):
        h = h @ w.t()
        if k + 1 < len(weights):
            h = torch.nn.functional.silu(h) * SILU_SCALE
    return h
