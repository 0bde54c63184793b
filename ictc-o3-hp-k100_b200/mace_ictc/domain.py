"""Spatial domain decomposition of a periodic orthorhombic box over the GPUs of one node, and the halo
exchange of node features between interaction layers.

Semantics follow the reference's multi-rank runtime (mace_ictc/interfaces/lammps_hp.py:51-111, 213-284 and
lammps_user_mfftorch/src/USER-MFFTORCH/pair_mff_torch.cpp:209-274): every rank owns the atoms inside its
brick, sees ghost copies (periodic images included, as separate rows with explicit shifted coordinates,
so edge shifts are zero) of every atom within one cutoff of the brick, builds edges only for owned
centres, receives the ghost rows of the layer-1 input features from their owners
(``all_to_all_single`` with variable splits, adjoint = reverse exchange + ``index_add`` at the owner) and
returns position gradients of ghost rows to the owners.

Differences by design: positions and velocities are replicated on every rank (a million atoms are
24 MB), so there is no atom migration and no position halo; ownership and ghost lists are recomputed
from the replicated coordinates each step, and ghost-force contributions are returned by one
``all_reduce`` of the [N,3] gradient instead of per-peer messages.  Everything here is device-agnostic
torch code plus ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple

import torch
import torch.distributed as dist


def brick_grid(world: int, box) -> Tuple[int, int, int]:
    """Regular brick grid with ``world`` bricks (powers of two): always halve the axis with the longest brick."""
    grid = [1, 1, 1]
    lengths = [float(b) for b in box]
    n = world
    while n > 1:
        if n % 2:
            raise ValueError("world size must be a power of two")
        axis = max(range(3), key=lambda a: lengths[a] / grid[a])
        grid[axis] *= 2
        n //= 2
    return tuple(grid)


@dataclass
class LocalDomain:
    owned: torch.Tensor          # [n_owned] global ids, ascending
    ghost_ids: torch.Tensor      # [n_ghost] global ids of the ghost rows
    ghost_shift: torch.Tensor    # [n_ghost, 3] lattice shift of each ghost image (float)
    lo: torch.Tensor             # brick bounds [3] (float64, host)
    hi: torch.Tensor
    owner_rank: torch.Tensor     # [N] owning rank of every atom
    owner_row: torch.Tensor      # [N] row of every atom inside its owner's owned list

    @property
    def num_owned(self):
        return int(self.owned.numel())

    def local_positions(self, pos, box):
        ghosts = pos.index_select(0, self.ghost_ids) + self.ghost_shift.to(pos.dtype) * box.to(pos.dtype)
        return torch.cat((pos.index_select(0, self.owned), ghosts), 0)

    def local_ids(self):
        return torch.cat((self.owned, self.ghost_ids))


def decompose(pos: torch.Tensor, box: torch.Tensor, grid, rank: int, cutoff: float) -> LocalDomain:
    """Owned atoms and ghost images of brick ``rank``.  ``pos`` [N,3] wrapped into [0, box), ``box`` [3].

    A pure function of (pos, box, grid, rank, cutoff): every rank can evaluate it for every brick and
    gets the same answer, which keeps the replicated-state scheme consistent.
    """
    dev = pos.device
    g = torch.tensor(grid, device=dev)
    width = box.to(torch.float64) / g.to(torch.float64)
    cell = torch.clamp((pos.to(torch.float64) / width.to(dev)).floor().long(), min=0)
    cell = torch.minimum(cell, g - 1)
    owner = (cell[:, 0] * grid[1] + cell[:, 1]) * grid[2] + cell[:, 2]
    mine = (rank // (grid[1] * grid[2]), (rank // grid[2]) % grid[1], rank % grid[2])
    lo = torch.tensor([mine[a] * float(width[a]) for a in range(3)], dtype=torch.float64)
    hi = torch.tensor([(mine[a] + 1) * float(width[a]) for a in range(3)], dtype=torch.float64)
    owned = torch.nonzero(owner == rank).flatten()
    # row of each atom inside its owner's (ascending) owned list
    order = torch.argsort(owner, stable=True)
    counts = torch.bincount(owner, minlength=grid[0] * grid[1] * grid[2])
    starts = torch.cumsum(counts, 0) - counts
    owner_row = torch.empty_like(owner)
    owner_row[order] = torch.arange(owner.numel(), device=dev) - starts[owner[order]]
    # per axis, which of the three images (shift -1, 0, +1) of an atom falls inside the halo-extended brick
    p64 = pos.to(torch.float64)
    lo_d, hi_d, box_d = lo.to(dev), hi.to(dev), box.to(torch.float64).to(dev)
    shifts3 = torch.tensor([-1.0, 0.0, 1.0], dtype=torch.float64, device=dev)
    q = p64.unsqueeze(-1) + shifts3 * box_d.view(1, 3, 1)                       # [N, axis, image]
    inside = (q >= (lo_d - cutoff).view(1, 3, 1)) & (q < (hi_d + cutoff).view(1, 3, 1))
    # only atoms with at least one image inside the extended brick on EVERY axis can contribute: expand the 27
    # image combinations for those candidates alone (the replicated position table grows with the number of
    # ranks, the candidates do not)
    cand = torch.nonzero(inside.any(dim=2).all(dim=1)).flatten()
    inside_c = inside.index_select(0, cand)
    codes = torch.arange(27, device=dev)
    sx, sy, sz = codes // 9, (codes // 3) % 3, codes % 3                        # image index per axis
    valid = inside_c[:, 0, :][:, sx] & inside_c[:, 1, :][:, sy] & inside_c[:, 2, :][:, sz]   # [M, 27]
    valid[:, 13] &= owner.index_select(0, cand) != rank                         # zero shift: ghosts only
    pairs = torch.nonzero(valid.t())                                            # sorted by (image code, atom id)
    code, ghost_ids = pairs[:, 0], cand.index_select(0, pairs[:, 1]).contiguous()
    ghost_shift = torch.stack((code // 9 - 1, (code // 3) % 3 - 1, code % 3 - 1), 1).to(torch.float32)
    return LocalDomain(owned, ghost_ids, ghost_shift, lo, hi, owner, owner_row)


class ExchangePlan:
    """Who sends which owned rows to whom (reference: ``_Plan``, lammps_hp.py:51-78).

    Ghost rows are grouped by owner rank (stable, so the ghost order inside a group is kept); each rank
    tells every owner how many rows it wants and which owner-local rows those are.
    """

    def __init__(self, domain: LocalDomain, rank: int, world: int, group=None):
        self.rank, self.world, self.group = rank, world, group
        dev = domain.ghost_ids.device
        g_owner = domain.owner_rank.index_select(0, domain.ghost_ids)
        g_row = domain.owner_row.index_select(0, domain.ghost_ids)
        self.recv_perm = torch.argsort(g_owner, stable=True)          # ghost rows in receive order
        self.recv_counts = torch.bincount(g_owner, minlength=world)
        want_rows = g_row.index_select(0, self.recv_perm).contiguous()
        send_counts = torch.empty_like(self.recv_counts)
        if world > 1:
            dist.all_to_all_single(send_counts, self.recv_counts, group=group)
        else:
            send_counts.copy_(self.recv_counts)
        self.recv_split = [int(v) for v in self.recv_counts.tolist()]
        self.send_split = [int(v) for v in send_counts.tolist()]
        self.send_rows = torch.empty(sum(self.send_split), dtype=torch.long, device=dev)
        if world > 1:
            dist.all_to_all_single(self.send_rows, want_rows, self.send_split, self.recv_split, group=group)
        else:
            self.send_rows.copy_(want_rows)
        n_owned = domain.num_owned
        if self.send_rows.numel() and (int(self.send_rows.min()) < 0 or int(self.send_rows.max()) >= n_owned):
            raise RuntimeError("halo request names a row outside the owner's atoms")
        self.num_owned, self.num_ghost = n_owned, int(domain.ghost_ids.numel())

    def forward(self, owned_rows: torch.Tensor) -> torch.Tensor:
        """[n_owned, W] -> ghost rows [n_ghost, W] in the domain's ghost order."""
        send = owned_rows.index_select(0, self.send_rows).contiguous()
        recv = owned_rows.new_empty(sum(self.recv_split), owned_rows.shape[1])
        if self.world > 1:
            dist.all_to_all_single(recv, send, self.recv_split, self.send_split, group=self.group)
        else:
            recv.copy_(send)
        out = torch.empty_like(recv)
        out.index_copy_(0, self.recv_perm, recv)
        return out

    def forward_async(self, owned_rows: torch.Tensor):
        """Starts ``forward`` and returns a callable that waits for it and gives the ghost rows; kernels launched in
        between run while the rows travel (NCCL works on its own stream)."""
        if self.world == 1:
            out = self.forward(owned_rows)
            return lambda: out
        send = owned_rows.index_select(0, self.send_rows).contiguous()
        recv = owned_rows.new_empty(sum(self.recv_split), owned_rows.shape[1])
        work = dist.all_to_all_single(recv, send, self.recv_split, self.send_split, group=self.group, async_op=True)

        def finish():
            work.wait()
            out = torch.empty_like(recv)
            out.index_copy_(0, self.recv_perm, recv)
            return out
        return finish

    def adjoint_async(self, ghost_grad: torch.Tensor):
        """Starts ``adjoint`` and returns a callable that waits for it and gives the owners' cotangent rows."""
        if self.world == 1:
            out = self.adjoint(ghost_grad)
            return lambda: out
        send = ghost_grad.index_select(0, self.recv_perm).contiguous()
        recv = ghost_grad.new_empty(sum(self.send_split), ghost_grad.shape[1])
        work = dist.all_to_all_single(recv, send, self.send_split, self.recv_split, group=self.group, async_op=True)

        def finish():
            work.wait()
            out = ghost_grad.new_zeros(self.num_owned, ghost_grad.shape[1])
            out.index_add_(0, self.send_rows, recv)
            return out
        return finish

    def adjoint(self, ghost_grad: torch.Tensor) -> torch.Tensor:
        """Cotangent of the ghost rows -> cotangent of the owners' rows (repeated images accumulate)."""
        send = ghost_grad.index_select(0, self.recv_perm).contiguous()
        recv = ghost_grad.new_empty(sum(self.send_split), ghost_grad.shape[1])
        if self.world > 1:
            dist.all_to_all_single(recv, send, self.send_split, self.recv_split, group=self.group)
        else:
            recv.copy_(send)
        out = ghost_grad.new_zeros(self.num_owned, ghost_grad.shape[1])
        out.index_add_(0, self.send_rows, recv)
        return out


class _Exchange(torch.autograd.Function):
    """Differentiable halo exchange (reference: ``_Exchange``, lammps_hp.py:80-111); its adjoint is the
    reverse exchange, and the adjoint of that is the forward exchange again (force-loss training)."""

    @staticmethod
    def forward(ctx, owned_rows, plan):
        ctx.plan = plan
        return plan.forward(owned_rows)

    @staticmethod
    def backward(ctx, grad):
        return _ExchangeAdjoint.apply(grad.contiguous(), ctx.plan), None


class _ExchangeAdjoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ghost_grad, plan):
        ctx.plan = plan
        return plan.adjoint(ghost_grad)

    @staticmethod
    def backward(ctx, grad):
        return _Exchange.apply(grad.contiguous(), ctx.plan), None


def exchange(owned_rows: torch.Tensor, plan: ExchangePlan) -> torch.Tensor:
    return _Exchange.apply(owned_rows, plan)
