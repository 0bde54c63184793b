"""Spatial domain decomposition of a periodic orthorhombic box over the GPUs of one node: who owns which
atoms, which atoms each brick sees as ghosts, and the halo exchanges (positions, node features between the
interaction layers, gradients back to the owners).

Semantics follow the reference's multi-rank runtime (mace_ictc/interfaces/lammps_hp.py:51-111, 213-284 and
lammps_user_mfftorch/src/USER-MFFTORCH/pair_mff_torch.cpp:209-274): every rank holds its own atoms plus ghost
copies (periodic images included, as separate rows with explicit shifted coordinates, so edge shifts are zero)
of every atom within the halo width of its brick, builds edges only for owned centres, receives the ghost rows
of the layer-1 input features from their owners (``all_to_all_single``; adjoint = reverse exchange +
``index_add`` at the owner) and returns the position gradients of ghost rows to the owners the same way.

State is distributed: a rank never sees the coordinates of atoms outside its halo.  The exchange plan has a
FIXED capacity per pair of ranks, so that a refresh of the ghost lists (new senders, new images) rewrites index
tensors in place and every collective keeps its sizes: a step recorded as a CUDA graph, NCCL calls included,
stays valid across refreshes.  Unused rows of a capacity are padding: the position halo places them 10^6 A away
(no atom sees them), their feature rows are never read by an edge and their gradients are zero.

Everything here is device-agnostic torch code plus ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests).
"""
from __future__ import annotations

from typing import List, Tuple

import torch
import torch.distributed as dist

PAD_SHIFT = 1.0e6          # offset (A) of padding ghost rows: far outside every cutoff sphere


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


def brick_index(rank: int, grid) -> Tuple[int, int, int]:
    return rank // (grid[1] * grid[2]), (rank // grid[2]) % grid[1], rank % grid[2]


def brick_bounds(rank: int, grid, box) -> Tuple[List[float], List[float]]:
    """Lower and upper corner of brick ``rank``."""
    idx = brick_index(rank, grid)
    width = [float(box[a]) / grid[a] for a in range(3)]
    return [idx[a] * width[a] for a in range(3)], [(idx[a] + 1) * width[a] for a in range(3)]


def owner_of(pos: torch.Tensor, box, grid) -> torch.Tensor:
    """Rank of the brick that contains each position (positions wrapped into [0, box))."""
    g = torch.tensor(grid, device=pos.device)
    width = torch.tensor([float(box[a]) / grid[a] for a in range(3)], dtype=torch.float64, device=pos.device)
    cell = torch.clamp((pos.to(torch.float64) / width).floor().long(), min=0)
    cell = torch.minimum(cell, g - 1)
    return (cell[:, 0] * grid[1] + cell[:, 1]) * grid[2] + cell[:, 2]


def morton_order(pos: torch.Tensor, cell: float = 2.5) -> torch.Tensor:
    """Permutation that sorts positions along a Z-order (Morton) curve of cubic cells of edge ``cell``: rows that
    are close in the array are close in space, so the rows a kernel gathers for neighbouring centres (sender
    features, receiver cotangents) stay in L2 between uses.  Stable: equal codes keep their order."""
    q = torch.clamp(((pos - pos.amin(dim=0)) / cell).floor().long(), 0, 1023)
    code = torch.zeros(pos.shape[0], dtype=torch.long, device=pos.device)
    for bit in range(10):
        for axis in range(3):
            code |= ((q[:, axis] >> bit) & 1) << (3 * bit + axis)
    return torch.argsort(code, stable=True)


def outside_distance(pos: torch.Tensor, lo, hi) -> torch.Tensor:
    """Largest distance by which a position lies outside the brick [lo, hi) along any axis (0 inside)."""
    lo_t = torch.tensor(lo, dtype=pos.dtype, device=pos.device)
    hi_t = torch.tensor(hi, dtype=pos.dtype, device=pos.device)
    return torch.clamp(torch.maximum(lo_t - pos, pos - hi_t), min=0).amax(dim=1)


def same_on_all_ranks(flag: bool, group=None) -> bool:
    """True when ``flag`` is true on ANY rank; every rank gets the same answer, so ranks can raise together
    instead of one rank leaving the others inside a collective."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return bool(flag)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return bool(int(t.item()))


class HaloPlan:
    """Which owned rows go to which rank as ghosts (reference: ``_Plan``, lammps_hp.py:51-78), with fixed
    per-destination capacities.

    ``refresh(pos_own)`` selects, for every destination brick b and every periodic image s in {-1,0,1}^3, the
    owned atoms whose image lies within ``halo`` of brick b (a rank's own atoms with zero shift excepted) and
    writes them into the index tensors in place.  Ghost rows at the receiver are grouped by source rank at
    fixed offsets, ordered (image, sender row) inside a group, padding at the end of each group.
    """

    def __init__(self, rank: int, world: int, grid, box, halo: float, num_owned: int, device, margin: float = 1.10,
                 group=None):
        self.rank, self.world, self.grid, self.group = rank, world, tuple(grid), group
        self.box = [float(b) for b in box]
        self.halo, self.num_owned, self.device, self.margin = float(halo), int(num_owned), device, float(margin)
        self.send_cap: List[int] | None = None      # rows sent to each rank (capacity)
        self.recv_cap: List[int] | None = None      # rows received from each rank (capacity)
        self.send_rows = self.send_shift = None
        self.send_count = [0] * world               # rows in use of every send capacity
        self.recv_count = [0] * world

    # ------------------------------------------------------------------ ghost selection
    def _select(self, pos_own: torch.Tensor):
        """(destination rank, image code, owned row) of every ghost entry, sorted in that order."""
        dev, n = pos_own.device, pos_own.shape[0]
        p = pos_own.to(torch.float64)
        shifts = torch.tensor([-1.0, 0.0, 1.0], dtype=torch.float64, device=dev)
        masks = []
        for a in range(3):
            width = self.box[a] / self.grid[a]
            k = torch.arange(self.grid[a], dtype=torch.float64, device=dev)
            lo = (k * width - self.halo).view(-1, 1, 1)
            hi = ((k + 1) * width + self.halo).view(-1, 1, 1)
            q = p[:, a].view(1, 1, n) + (shifts * self.box[a]).view(1, 3, 1)
            masks.append((q >= lo) & (q < hi))                                    # [grid_a, 3, n]
        gx, gy, gz = self.grid
        full = (masks[0].view(gx, 1, 1, 3, 1, 1, n) & masks[1].view(1, gy, 1, 1, 3, 1, n)
                & masks[2].view(1, 1, gz, 1, 1, 3, n)).reshape(self.world, 27, n)
        full[self.rank, 13] = False            # a rank's own atoms with zero shift are not ghosts
        hits = torch.nonzero(full.reshape(self.world * 27, n))
        combo, rows = hits[:, 0], hits[:, 1]
        return combo // 27, combo % 27, rows

    def refresh(self, pos_own: torch.Tensor) -> bool:
        """Rebuild the send lists from the owners' current coordinates.  Returns False (on every rank) when some
        capacity is too small: the caller then calls ``allocate`` again and re-records whatever depends on the
        sizes.  Collective: every rank must call it."""
        dest, code, rows = self._select(pos_own)
        counts = torch.bincount(dest, minlength=self.world)
        count_list = [int(v) for v in counts.tolist()]
        if self.send_cap is None:
            self.allocate(count_list)
        fits = all(c <= cap for c, cap in zip(count_list, self.send_cap))
        if same_on_all_ranks(not fits, self.group):
            self.send_cap = None               # sizes must be renegotiated
            return False
        dev = pos_own.device
        starts = torch.cumsum(counts, 0) - counts
        offsets = torch.tensor([sum(self.send_cap[:b]) for b in range(self.world)], dtype=torch.long, device=dev)
        slot = offsets[dest] + (torch.arange(dest.numel(), device=dev) - starts[dest])
        self.send_rows.zero_()
        self.send_shift.fill_(PAD_SHIFT)
        self.send_rows[slot] = rows
        image = torch.stack((code // 9 - 1, (code // 3) % 3 - 1, code % 3 - 1), 1).to(torch.float32)
        self.send_shift[slot] = image * torch.tensor(self.box, dtype=torch.float32, device=dev)
        self.send_count = count_list
        got = torch.empty_like(counts)
        self._all_to_all(got, counts, [1] * self.world, [1] * self.world)
        self.recv_count = [int(v) for v in got.tolist()]
        return True

    def allocate(self, counts: List[int]):
        """Fix the capacities from the current counts (collective)."""
        dev = self.device
        self.send_cap = [int(c * self.margin) + 64 for c in counts]
        caps = torch.tensor(self.send_cap, dtype=torch.long, device=dev)
        got = torch.empty_like(caps)
        self._all_to_all(got, caps, [1] * self.world, [1] * self.world)
        self.recv_cap = [int(v) for v in got.tolist()]
        self.send_rows = torch.zeros(sum(self.send_cap), dtype=torch.long, device=dev)
        self.send_shift = torch.full((sum(self.send_cap), 3), PAD_SHIFT, dtype=torch.float32, device=dev)

    @property
    def num_ghost(self) -> int:
        """Ghost rows at this rank (capacity, padding included)."""
        return sum(self.recv_cap)

    def ghost_mask(self) -> torch.Tensor:
        """True for ghost rows that hold an atom, False for padding."""
        mask = torch.zeros(self.num_ghost, dtype=torch.bool, device=self.device)
        off = 0
        for cap, cnt in zip(self.recv_cap, self.recv_count):
            mask[off:off + cnt] = True
            off += cap
        return mask

    # ------------------------------------------------------------------ exchanges
    def _all_to_all(self, recv, send, recv_split, send_split, async_op=False):
        if self.world > 1:
            return dist.all_to_all_single(recv, send, recv_split, send_split, group=self.group, async_op=async_op)
        recv.copy_(send)
        return None

    def positions(self, pos_own: torch.Tensor) -> torch.Tensor:
        """Coordinates of the ghost rows [num_ghost, 3]: owner coordinates plus image shift (padding far away)."""
        send = pos_own.index_select(0, self.send_rows) + self.send_shift
        recv = pos_own.new_empty(self.num_ghost, 3)
        self._all_to_all(recv, send, self.recv_cap, self.send_cap)
        return recv

    def integers(self, values_own: torch.Tensor) -> torch.Tensor:
        """Per-atom integers (species, global ids) of the ghost rows; padding rows carry the sender's row 0."""
        send = values_own.index_select(0, self.send_rows).contiguous()
        recv = values_own.new_empty(self.num_ghost)
        self._all_to_all(recv, send, self.recv_cap, self.send_cap)
        return recv

    def forward(self, owned_rows: torch.Tensor) -> torch.Tensor:
        """[n_owned, W] -> ghost rows [num_ghost, W]."""
        return self.forward_async(owned_rows)()

    def forward_async(self, owned_rows: torch.Tensor):
        """Starts the exchange and returns a callable that waits for it and gives the ghost rows; kernels launched
        in between run while the rows travel (the collective works on its own stream)."""
        send = owned_rows.index_select(0, self.send_rows).contiguous()
        recv = owned_rows.new_empty(self.num_ghost, owned_rows.shape[1])
        work = self._all_to_all(recv, send, self.recv_cap, self.send_cap, async_op=self.world > 1)

        def finish():
            if work is not None:
                work.wait()
            return recv
        return finish

    def adjoint(self, ghost_grad: torch.Tensor) -> torch.Tensor:
        """Cotangent of the ghost rows -> cotangent of the owners' rows (repeated images accumulate)."""
        return self.adjoint_async(ghost_grad)()

    def adjoint_async(self, ghost_grad: torch.Tensor):
        send = ghost_grad.contiguous()
        recv = ghost_grad.new_empty(sum(self.send_cap), ghost_grad.shape[1])
        work = self._all_to_all(recv, send, self.send_cap, self.recv_cap, async_op=self.world > 1)

        def finish():
            if work is not None:
                work.wait()
            out = ghost_grad.new_zeros(self.num_owned, ghost_grad.shape[1])
            out.index_add_(0, self.send_rows, recv)
            return out
        return finish


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


def exchange(owned_rows: torch.Tensor, plan: HaloPlan) -> torch.Tensor:
    return _Exchange.apply(owned_rows, plan)


def migrate(dest: torch.Tensor, payload: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """Send row i of ``payload`` [n, W] to rank ``dest[i]`` and return the rows this rank receives (its own
    stay-at-home rows included), ordered by source rank.  Used when ownership is re-derived from the
    coordinates (atom migration; reference semantics: LAMMPS' exchange at re-neighbouring, which the pair
    style sees as a changed ``nlocal``, pair_mff_torch.cpp:222-242)."""
    order = torch.argsort(dest, stable=True)
    counts = torch.bincount(dest, minlength=world)
    send = payload.index_select(0, order).contiguous()
    if world == 1:
        return send
    got = torch.empty_like(counts)
    dist.all_to_all_single(got, counts, group=group)
    send_split, recv_split = [int(v) for v in counts.tolist()], [int(v) for v in got.tolist()]
    recv = payload.new_empty(sum(recv_split), payload.shape[1])
    dist.all_to_all_single(recv, send, recv_split, send_split, group=group)
    return recv


class PeerWatch:
    """Host-side liveness check between steps: every rank calls ``check()`` at the same points of the run (the
    driver does so before each block of steps); if a rank has left or hangs, the others get a ``RuntimeError``
    naming it after ``timeout`` seconds, BEFORE they launch collectives that would wait for it on the GPU.
    Runs over a gloo group of its own (``monitored_barrier`` is a gloo feature), so it works beside NCCL."""

    def __init__(self, timeout: float = 30.0):
        import datetime
        self.timeout = datetime.timedelta(seconds=float(timeout))
        self.group = dist.new_group(backend="gloo", timeout=self.timeout)

    def check(self):
        try:
            dist.monitored_barrier(group=self.group, timeout=self.timeout, wait_all_ranks=True)
        except RuntimeError as err:
            raise RuntimeError(f"a rank of the decomposed run is gone or not responding: {err}") from err
