"""CPU oracle of the MACE-ICTC baseline model (fp64 by default).  TEST INFRASTRUCTURE ONLY.

A plain-torch restatement of the reference's model assembly, written against the oracle operators of
``ictc_oracle`` (dense coupling tensors, dense U tensors): backbone forward
(mace_ictc/models/mace/backbone.py:860-1246), interaction block (mace_ictc/models/mace/layers.py:1042-1368),
product block (mace_ictc/models/mace/products.py:792-841, recursion
ictc_o3/ops/_mace_symmetric_contraction.py:298-354), readouts (mace_ictc/models/mace/heads.py:12-27,
mace_ictc/models/pure_cartesian_ictd_layers.py:89-113), radial embedding (mace_ictc/models/radial_basis.py:11-92),
energy and forces (mace_ictc/hp/runtime.py:82-111).

Parity status: the reference model itself cannot be imported without e3nn / opt_einsum_fx, so this
restatement is pinned only through its parts (tensor product, harmonics and graph message against the
reference's golden vectors; U tensors from the reference's tables).  The product block's equivariant
linear is taken as x @ W / sqrt(C) per degree — "parity unpinned" for that normalisation.
It takes its weights from a state dict with the reference's parameter names.
"""
from __future__ import annotations

import math

import torch

from . import ictc_oracle as O


def _split(x, c, lmax):
    out, off = {}, 0
    for l in range(lmax + 1):
        w = c * (2 * l + 1)
        out[l] = x[:, off:off + w].reshape(-1, c, 2 * l + 1)
        off += w
    return out


def _merge(blocks, lmax):
    return torch.cat([blocks[l].reshape(blocks[l].shape[0], -1) for l in range(lmax + 1)], -1)


def radial_embedding(r, r_max, num_basis=8, p=5):
    w = math.pi / r_max * torch.linspace(1.0, float(num_basis), num_basis, dtype=r.dtype)
    emb = math.sqrt(2.0 / r_max) * torch.sin(r.unsqueeze(-1) * w) / r.clamp_min(1e-12).unsqueeze(-1)
    u = r / r_max
    env = (1.0 - ((p + 1.0) * (p + 2.0) / 2.0) * u ** p + p * (p + 2.0) * u ** (p + 1)
           - (p * (p + 1.0) / 2.0) * u ** (p + 2)) * (r < r_max).to(r.dtype)
    return emb * env.unsqueeze(-1)


class ModelOracle:
    def __init__(self, state_dict, *, channels, lmax, num_interactions, correlation, atomic_numbers, cutoff,
                 avg_num_neighbors, dtype=torch.float64):
        self.p = {k: v.detach().to("cpu", dtype).clone().requires_grad_(v.dtype.is_floating_point and "tp.weight" not in k)
                  for k, v in state_dict.items()}
        self.c, self.lmax, self.nl, self.corr = channels, lmax, num_interactions, correlation
        self.z = sorted(int(z) for z in atomic_numbers)
        self.cutoff, self.avg, self.dtype = float(cutoff), float(avg_num_neighbors), dtype

    def parameters(self):
        return {k: v for k, v in self.p.items() if v.requires_grad}

    def atomic_energies(self, pos, A, batch, src, dst, shifts, cell):
        c, p, dt = self.c, self.p, self.dtype
        order = torch.argsort(dst, stable=True)
        src, dst, shifts = src[order], dst[order], shifts[order]
        vec = pos[dst] - pos[src] + torch.einsum("ni,nij->nj", shifts.to(dt), cell.to(dt)[batch[src]])
        r = vec.norm(dim=1)
        unit = vec / r.clamp(min=1e-8).unsqueeze(-1)
        mask = (r <= self.cutoff).to(dt).detach()
        sh = torch.cat(O.direction_harmonics(unit, self.lmax), -1)
        feats = radial_embedding(r, self.cutoff)
        species = torch.tensor([self.z.index(int(a)) for a in A.tolist()])
        h = p["node_embedding.weight"].t()[species]
        n = pos.shape[0]
        total = None
        for layer in range(self.nl):
            pre = f"interactions.{layer}."
            lin = 0 if layer == 0 else self.lmax
            target = self.lmax if layer < self.nl - 1 else 0
            sc_lmax = 0 if layer == 0 else target
            blocks = _split(h, c, lin)
            up = {l: torch.einsum("oc,ncm->nom", p[pre + f"linear_up.adapters.{l}.weight"], blocks[l]) for l in blocks}
            g = feats
            for k in (0, 2, 4, 6):
                g = g @ p[pre + f"fc.{k}.weight"].t()
                if k < 6:
                    g = torch.nn.functional.silu(g) * O.SILU_SCALE
            paths = O.natural_paths(lin, self.lmax, self.lmax)
            tp = O.TensorProduct(c, self.lmax, paths, dtype=dt)
            xe = {l: up[l][src] for l in up}
            she = {l: sh[:, l * l:(l + 1) ** 2] for l in range(self.lmax + 1)}
            edge = tp(xe, she, g.reshape(-1, len(paths), c), p[pre + "tp.weight"])
            msg = {}
            for l in range(self.lmax + 1):
                agg = (edge[l] * mask.view(-1, 1, 1)).new_zeros(n, edge[l].shape[1], 2 * l + 1).index_add(
                    0, dst, edge[l] * mask.view(-1, 1, 1))
                msg[l] = torch.einsum("oc,ncm->nom", p[pre + f"message_linear.weights.{l}"], agg) / self.avg
            message = _merge(msg, self.lmax)
            sc_in = _split(h, c, lin)
            sc = _merge({l: torch.einsum("noi,nim->nom", p[pre + f"self_connection.weights.{l}"][species], sc_in[l])
                         for l in range(sc_lmax + 1)}, sc_lmax)
            # product
            pp = f"products.{layer}."
            xm = torch.cat([_split(message, c, self.lmax)[l] for l in range(self.lmax + 1)], -1)   # [N,C,9]
            weights = {}
            for l in range(target + 1):
                base = pp + f"symmetric_contractions.symmetric_contractions.contractions.{l}."
                lower = [p[base + f"weights.{k}"] for k in range(self.corr - 1)]
                weights[l] = list(reversed(lower)) + [p[base + "weights_max"]]
            y = O.symmetric_contraction(xm, species, weights, target, self.corr)
            yb = _split(y, c, target)
            out = _merge({l: torch.einsum("io,nim->nom", p[pp + f"linear.{l}"], yb[l]) / math.sqrt(c)
                          for l in range(target + 1)}, target)
            out = torch.cat((out[:, :c] + sc[:, :c], out[:, c:] + sc[:, c:]), -1) if sc.shape[1] == out.shape[1] else \
                torch.cat((out[:, :c] + sc, out[:, c:]), -1)
            h = out
            if layer < self.nl - 1:
                e = h[:, :c] @ p[f"layer_energy_readouts.{layer}.readout.weight"].t()
            else:
                hid = torch.nn.functional.silu(h @ p["last_layer_energy_readout.linear_1.weight"].t()) * O.SILU_SCALE
                e = hid @ p["last_layer_energy_readout.linear_2.weight"].t()
            total = e if total is None else total + e
        return total.reshape(n)

    def energy_and_forces(self, pos, A, batch, src, dst, shifts, cell, create_graph=False):
        pos = pos.detach().to(self.dtype).requires_grad_(True)
        atomic = self.atomic_energies(pos, A, batch, src, dst, shifts, cell)
        energy = atomic.new_zeros(cell.shape[0]).index_add(0, batch, atomic)
        forces = -torch.autograd.grad(energy.sum(), pos, create_graph=create_graph)[0]
        return {"energy": energy, "forces": forces, "atomic_energy": atomic}
