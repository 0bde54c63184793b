"""MACE-ICTC short-range model (baseline route: C channels, lmax 2, bridge-U style product, Bessel radial
basis) assembled from the B200 operators.

Structure and parameter names follow the reference's ``PureCartesianICTDFix`` baseline route:
backbone construction mace_ictc/models/mace/backbone.py:381-531, forward :860-1246;
interaction block mace_ictc/models/mace/layers.py:716-925 (construction) and :1042-1368 (forward);
product block mace_ictc/models/mace/products.py:792-841; readouts mace_ictc/models/mace/heads.py:12-27 and
mace_ictc/models/pure_cartesian_ictd_layers.py:89-113; radial embedding mace_ictc/models/radial_basis.py:11-92.

Node features are flat mul_ir rows ``[N, C*(l+1)^2]`` (degree blocks [C, 2l+1]) between blocks, exactly as
in the reference; the tensor-product kernels work on ir_mul rows and the conversion happens around them.
The equivariant linear of the product block (an e3nn ``o3.Linear`` in the reference) is a per-degree
channel matrix with N(0,1) entries applied as ``x @ W / sqrt(C)``.
"""
from __future__ import annotations

import math
from typing import Dict, List

import torch
from torch import nn

from ictc_o3.basis.ictd_irreps import EdgeWeightedPathPreservingTensorProduct
from ictc_o3.operators import (PackedGraphMessage, _RowsTimesWeight, _tc_eligible, channel_linear, convert_layout,
                               direction_harmonics, strict_fp32)
from ictc_o3.symmetric_contraction import ICTDBridgeUSymmetricContractionSO3

SILU_SCALE = 1.6791767923989418


def split_irreps(x: torch.Tensor, channels: int, lmax: int) -> Dict[int, torch.Tensor]:
    out, off = {}, 0
    for l in range(lmax + 1):
        w = channels * (2 * l + 1)
        out[l] = x[..., off:off + w].reshape(*x.shape[:-1], channels, 2 * l + 1)
        off += w
    return out


def merge_irreps(blocks: Dict[int, torch.Tensor], channels: int, lmax: int) -> torch.Tensor:
    return torch.cat([blocks[l].reshape(*blocks[l].shape[:-2], channels * (2 * l + 1)) for l in range(lmax + 1)], -1)


class Normalize2MomSiLU(nn.Module):
    def forward(self, x):
        return torch.nn.functional.silu(x) * SILU_SCALE


def bessel_embedding(r: torch.Tensor, r_max: float, num_basis: int, p: int) -> torch.Tensor:
    """sqrt(2/rc) sin(n pi r / rc)/r times the polynomial envelope (radial_basis.py:11-92)."""
    w = math.pi / r_max * torch.linspace(1.0, float(num_basis), num_basis, dtype=r.dtype, device=r.device)
    emb = math.sqrt(2.0 / r_max) * torch.sin(r.unsqueeze(-1) * w) / r.clamp_min(1e-12).unsqueeze(-1)
    u = r / r_max
    pf = float(p)
    env = (1.0 - ((pf + 1.0) * (pf + 2.0) / 2.0) * torch.pow(u, p) + pf * (pf + 2.0) * torch.pow(u, p + 1)
           - (pf * (pf + 1.0) / 2.0) * torch.pow(u, p + 2)) * (r < r_max).to(r.dtype)
    return emb * env.unsqueeze(-1)


class EquivariantChannelLinearSO3(nn.Module):
    """Per-degree channel linear (ictc_o3/basis/ictd_irreps.py:207-227)."""

    def __init__(self, channels, lmax):
        super().__init__()
        self.channels, self.lmax = channels, lmax
        self.adapters = nn.ModuleDict({str(l): nn.Linear(channels, channels, bias=False) for l in range(lmax + 1)})
        with torch.no_grad():
            for a in self.adapters.values():
                nn.init.eye_(a.weight)

    def forward(self, x):
        blocks = split_irreps(x, self.channels, self.lmax)
        for l in range(self.lmax + 1):
            blocks[l] = channel_linear(blocks[l], self.adapters[str(l)].weight)
        return merge_irreps(blocks, self.channels, self.lmax)


class PathPreservingLinearSO3(nn.Module):
    """[N, count_l*C, m] -> [N, C, m] per degree (mace_ictc/models/mace/layers.py:317-355)."""

    def __init__(self, in_channels_by_l, out_channels, lmax):
        super().__init__()
        self.out_channels, self.lmax = out_channels, lmax
        self.weights = nn.ParameterDict()
        for l in range(lmax + 1):
            cin = int(in_channels_by_l.get(l, 0))
            w = torch.empty(out_channels, cin)
            if cin:
                nn.init.normal_(w, mean=0.0, std=1.0 / math.sqrt(cin))
            self.weights[str(l)] = nn.Parameter(w)

    def forward(self, blocks):
        return merge_irreps({l: channel_linear(blocks[l], self.weights[str(l)]) for l in range(self.lmax + 1)},
                            self.out_channels, self.lmax)


class ElementConditionedLinearSO3(nn.Module):
    """Species-indexed channel linear, identity initialised (layers.py:21-87; init common.py:128-142)."""

    def __init__(self, num_elements, channels, lmax):
        super().__init__()
        self.num_elements, self.channels, self.lmax = num_elements, channels, lmax
        eye = torch.eye(channels).unsqueeze(0).repeat(num_elements, 1, 1)
        self.weights = nn.ParameterDict({str(l): nn.Parameter(eye.clone()) for l in range(lmax + 1)})

    def forward_type_idx(self, x, idx):
        blocks = split_irreps(x, self.channels, self.lmax)
        out = {}
        for l in range(self.lmax + 1):
            # all species at once, then pick the node's own: avoids a per-node [C,C] weight gather
            w = self.weights[str(l)]
            full = channel_linear(blocks[l], w.reshape(-1, w.shape[-1])).reshape(
                blocks[l].shape[0], self.num_elements, self.channels, 2 * l + 1)
            pick = idx.view(-1, 1, 1, 1).expand(-1, 1, self.channels, 2 * l + 1)
            out[l] = full.gather(1, pick).squeeze(1)
        return merge_irreps(out, self.channels, self.lmax)


class InteractionBlock(nn.Module):
    """``ICTDResidualInteractionBlock`` of the baseline route (attention-free, frozen unit TP weights)."""

    def __init__(self, *, channels, lmax, input_lmax, sc_lmax, number_of_basis, num_elements, avg_num_neighbors,
                 radial_mlp_hidden=(64, 64, 64)):
        super().__init__()
        self.channels, self.lmax, self.input_lmax, self.target_lmax, self.sc_lmax = channels, lmax, input_lmax, lmax, sc_lmax
        self.avg_num_neighbors = float(avg_num_neighbors)
        self.linear_up = EquivariantChannelLinearSO3(channels, input_lmax)
        paths = [(l1, l2, l3) for l1 in range(input_lmax + 1) for l2 in range(lmax + 1) for l3 in range(lmax + 1)
                 if abs(l1 - l2) <= l3 <= l1 + l2 and (l1 + l2 + l3) % 2 == 0]
        self.tp = EdgeWeightedPathPreservingTensorProduct(channels, lmax, allowed_paths=paths,
                                                           internal_compute_dtype=torch.float32)
        with torch.no_grad():
            self.tp.weight.fill_(1.0)
        self.tp.weight.requires_grad_(False)
        sizes = (number_of_basis, *radial_mlp_hidden, self.tp.num_paths * channels)
        layers: List[nn.Module] = []
        for k, (a, b) in enumerate(zip(sizes, sizes[1:])):
            lin = nn.Linear(a, b, bias=False)
            nn.init.normal_(lin.weight, mean=0.0, std=1.0 / math.sqrt(a))
            layers.append(lin)
            if k < len(sizes) - 2:
                layers.append(Normalize2MomSiLU())
        self.fc = nn.Sequential(*layers)
        self.message_linear = PathPreservingLinearSO3(
            {l: channels * self.tp.path_counts_by_l.get(l, 0) for l in range(lmax + 1)}, channels, lmax)
        self.self_connection = ElementConditionedLinearSO3(num_elements, channels, sc_lmax)
        self._message = None

    def message_op(self):
        if self._message is None:
            self._message = PackedGraphMessage(self.tp, input_lmax=self.input_lmax, edge_lmax=self.lmax)
        return self._message

    def radial_gates(self, edge_feats):
        """The gate MLP; layers whose sides are multiples of 64 (the hidden layers and the wide last one) run on
        the tcgen05 channel-linear kernel, the narrow first layer on the library GEMM."""
        h = edge_feats
        for mod in self.fc:
            if isinstance(mod, nn.Linear) and _tc_eligible(h, mod.weight):
                h = _RowsTimesWeight.apply(h, mod.weight)
            else:
                h = mod(h)
        return h

    def forward(self, h, sh, edge_feats, edge_src, edge_dst, edge_mask, species, topology=None):
        c = self.channels
        n = h.shape[0]
        up = self.linear_up(h)
        gates = self.radial_gates(edge_feats)
        op = self.message_op()
        x_packed = convert_layout(up, c, op.edge._in_blocks(), True)
        if topology is not None:
            op._topology, op._topology_key = topology, (edge_src.data_ptr(), edge_src._version, edge_dst.data_ptr(),
                                                        edge_dst._version, edge_src.numel(), n)
        out = convert_layout(op(x_packed, sh, gates, edge_src, edge_dst, edge_mask), c, op.edge._out_blocks(), False)
        blocks, start = {}, 0
        for l, (slots, mm) in enumerate(op.edge._out_blocks()):
            blocks[l] = out[:, start:start + slots * c * mm].reshape(n, slots * c, mm)
            start += slots * c * mm
        message = self.message_linear(blocks) / max(self.avg_num_neighbors, 1e-8)
        sc_in = h if self.sc_lmax == self.input_lmax else split_irreps(h, c, self.input_lmax)[0].reshape(n, c)
        sc = self.self_connection.forward_type_idx(sc_in, species)
        return message, sc


class ProductBlock(nn.Module):
    """Symmetric contraction + per-degree linear + self connection (products.py:792-841)."""

    def __init__(self, *, num_elements, channels, lmax, target_lmax, correlation):
        super().__init__()
        self.channels, self.lmax, self.target_lmax = channels, lmax, target_lmax
        self.symmetric_contractions = ICTDBridgeUSymmetricContractionSO3(
            num_elements=num_elements, channels=channels, lmax=lmax, target_lmax=target_lmax, correlation=correlation)
        self.linear = nn.ParameterDict({str(l): nn.Parameter(torch.randn(channels, channels))
                                        for l in range(target_lmax + 1)})

    def forward(self, message, sc, species):
        c = self.channels
        y = self.symmetric_contractions(message, None, species)
        blocks = split_irreps(y, c, self.target_lmax)
        out = merge_irreps({l: channel_linear(blocks[l], self.linear[str(l)].t() / math.sqrt(c))
                            for l in range(self.target_lmax + 1)}, c, self.target_lmax)
        if sc is not None:
            if sc.shape[-1] == out.shape[-1]:
                out = out + sc
            elif sc.shape[-1] == c:
                out = torch.cat((out[:, :c] + sc, out[:, c:]), -1)
            else:
                raise ValueError("unsupported self-connection width")
        return out


class ScalarReadout(nn.Module):
    def __init__(self, channels):
        super().__init__()
        self.channels = channels
        self.readout = nn.Linear(channels, 1, bias=False)
        nn.init.normal_(self.readout.weight, mean=0.0, std=1.0 / math.sqrt(channels))

    def forward(self, x):
        return self.readout(x[:, :self.channels])


class MLPReadout(nn.Module):
    def __init__(self, channels, hidden=16):
        super().__init__()
        self.linear_1 = nn.Linear(channels, hidden, bias=False)
        self.linear_2 = nn.Linear(hidden, 1, bias=False)
        self.activation = Normalize2MomSiLU()
        nn.init.normal_(self.linear_1.weight, mean=0.0, std=1.0 / math.sqrt(channels))
        nn.init.normal_(self.linear_2.weight, mean=0.0, std=1.0 / math.sqrt(hidden))

    def forward(self, x):
        return self.linear_2(self.activation(self.linear_1(x)))


class MaceIctcModel(nn.Module):
    """forward(pos [N,3], A [N] atomic numbers, batch [N], edge_src, edge_dst [E], edge_shifts [E,3], cell [B,3,3])
    -> per-atom energies [N,1].  Edge (src=j, dst=i): edge_vec = pos[dst] - pos[src] + shifts @ cell."""

    def __init__(self, *, channels=64, lmax=2, num_interactions=2, correlation=3, atomic_numbers=(1, 6, 8),
                 cutoff=5.0, avg_num_neighbors=50.0, number_of_basis=8, polynomial_cutoff_p=5,
                 radial_mlp_hidden=(64, 64, 64), readout_hidden_channels=16):
        super().__init__()
        self.channels, self.lmax, self.num_interaction = channels, lmax, num_interactions
        self.max_radius, self.number_of_basis, self.polynomial_cutoff_p = float(cutoff), number_of_basis, polynomial_cutoff_p
        self.atomic_numbers = sorted(int(z) for z in atomic_numbers)
        self.num_elements = len(self.atomic_numbers)
        table = torch.full((max(self.atomic_numbers) + 1,), -1, dtype=torch.long)
        for i, z in enumerate(self.atomic_numbers):
            table[z] = i
        self.register_buffer("atomic_number_to_index", table, persistent=False)
        self.node_embedding = nn.Linear(self.num_elements, channels, bias=False)
        self.interactions, self.products = nn.ModuleList(), nn.ModuleList()
        for layer in range(num_interactions):
            target = lmax if layer < num_interactions - 1 else 0
            self.interactions.append(InteractionBlock(
                channels=channels, lmax=lmax, input_lmax=0 if layer == 0 else lmax,
                sc_lmax=0 if layer == 0 else target, number_of_basis=number_of_basis,
                num_elements=self.num_elements, avg_num_neighbors=avg_num_neighbors,
                radial_mlp_hidden=radial_mlp_hidden))
            self.products.append(ProductBlock(num_elements=self.num_elements, channels=channels, lmax=lmax,
                                              target_lmax=target, correlation=correlation))
        self.layer_energy_readouts = nn.ModuleList([ScalarReadout(channels) for _ in range(num_interactions - 1)])
        self.last_layer_energy_readout = MLPReadout(channels, readout_hidden_channels)
        self.preserve_edge_order = False
        self.assume_edges_within_radius = False
        self.skip_input_validation = False

    def species_index(self, atomic_numbers):
        idx = self.atomic_number_to_index[atomic_numbers.long()]
        if not self.skip_input_validation and bool(torch.any(idx < 0)):
            raise ValueError(f"Encountered atomic numbers outside {self.atomic_numbers}")
        return idx

    def forward(self, pos, A, batch, edge_src, edge_dst, edge_shifts, cell, *, local_atom_count=None,
                layer_state_callback=None, topology=None):
        strict_fp32()
        dtype = self.node_embedding.weight.dtype
        pos, cell = pos.to(dtype), cell.to(dtype)
        if not self.preserve_edge_order:
            order = torch.argsort(edge_dst, stable=True)
            edge_src, edge_dst, edge_shifts = edge_src[order], edge_dst[order], edge_shifts[order]
            topology = None
        shift_vecs = torch.einsum("ni,nij->nj", edge_shifts.to(dtype), cell[batch[edge_src]])
        edge_vec = pos[edge_dst] - pos[edge_src] + shift_vecs
        length = edge_vec.norm(dim=1)
        unit = edge_vec / length.clamp(min=1e-8).unsqueeze(-1)
        mask = None if self.assume_edges_within_radius else (length <= self.max_radius).to(dtype).detach()
        sh = torch.cat(direction_harmonics(unit.contiguous(), self.lmax), -1)
        edge_feats = bessel_embedding(length, self.max_radius, self.number_of_basis, self.polynomial_cutoff_p)
        species = self.species_index(A)
        h = self.node_embedding.weight.t().index_select(0, species)
        owned = pos.shape[0] if local_atom_count is None else int(local_atom_count)
        total = None
        for layer, (interaction, product) in enumerate(zip(self.interactions, self.products)):
            message, sc = interaction(h, sh, edge_feats, edge_src, edge_dst, mask, species, topology)
            # only owned rows feed the product (ghost rows have no in-edges here)
            h = product(message[:owned], sc[:owned], species[:owned])
            if layer_state_callback is not None:
                h = layer_state_callback(layer, h)
            if layer < self.num_interaction - 1:
                e = self.layer_energy_readouts[layer](h[:owned])
            else:
                e = self.last_layer_energy_readout(h[:owned])
            total = e if total is None else total + e
        out = total.sum(dim=-1, keepdim=True)
        if owned < pos.shape[0]:
            out = torch.cat((out, out.new_zeros(pos.shape[0] - owned, 1)))
        return out
