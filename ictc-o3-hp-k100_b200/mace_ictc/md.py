"""Molecular-dynamics step on the B200 kernels: neighbour build, energy and forces, velocity Verlet, and
spatial domain decomposition over the GPUs of one node with distributed state.

The reference runs MD through LAMMPS (``examples/in.hco``: metal units, NVE, ``neighbor 0.5 bin``) with its
pair style building the edge list from LAMMPS' full neighbour list
(lammps_user_mfftorch/src/USER-MFFTORCH/pair_mff_torch_kokkos.cpp:661-871) and calling the model for
``E_local = sum over owned atoms`` and ``F = -dE/dpos`` (mff_torch_engine.cpp:1739-1859); every MPI rank holds
its own atoms and ghosts and ghost forces go back to the owners per peer (pair_mff_torch.cpp:222-274).
LAMMPS is not part of this build; this module is the stand-alone driver with the same step semantics.
Units: A, fs, eV, amu (1 eV/(A amu) = 9.64853321e-3 A/fs^2).

One rank: positions of all atoms, wrapped into the box; the step can be recorded as one CUDA graph.
Several ranks (``distributed=True``, one process per GPU): every rank keeps only the atoms of its brick
(positions, velocities, species, global ids) plus ghosts within ``cutoff + skin`` of the brick.  Per step:
position halo, edge list of the owned centres (rebuilt every step from the current coordinates, so the list is
exactly the ``r <= cutoff`` list), two feature halos inside the model, gradient halo back to the owners.
Ownership and the ghost LISTS change only at a refresh every few steps (re-neighbouring: atoms migrate to the
brick that contains them, ghosts are selected again); in between they stay valid while no atom has moved more
than skin/2 since the refresh, which a device-side flag watches.  All per-atom arrays, buffers and collectives
have FIXED capacities (unused rows are inert padding), a refresh rewrites them in place, and so the step, NCCL
calls included, is recorded once as a CUDA graph that survives the refreshes.
"""
from __future__ import annotations

import ctypes as C
import math

import numpy as np
import torch

from ictc_o3 import _lib
from ictc_o3.ops.topology import Topology
from . import domain as D

KB_EV = 8.617333262e-5
ACCEL = 9.64853321e-3
MASSES = {1: 1.008, 6: 12.011, 8: 15.999}


def _bucket(rows):
    """Allocation size for a per-edge array: see ``ForceEngine.bucket`` (sizes that repeat from step to step)."""
    rows = int(rows)
    if rows <= 4096:
        return 4096
    g = 1 << (rows.bit_length() - 5)
    return (rows + g - 1) // g * g


def _arr(values, ctype):
    return (ctype * 3)(*[values[i] for i in range(3)])


def neighbor_list(pos, num_centres, lo, hi, box, periodic, cutoff, return_keys=False):
    """Edges (src=j, dst=i) of the first ``num_centres`` rows, sorted by (dst, src, shift).

    pos [N,3] fp32 CUDA; lo/hi: bounds of the cell grid; box: periodic lengths; periodic: 3 flags.
    Returns src, dst (int64 [E]), shifts (float32 [E,3], lattice units), rowptr (int64 [centres+1]).
    """
    lib, dev = _lib.load(), pos.device
    n = pos.shape[0]
    lo_c, hi_c = _arr([float(x) for x in lo], C.c_double), _arr([float(x) for x in hi], C.c_double)
    box_c, per_c = _arr([float(x) for x in box], C.c_double), _arr([int(x) for x in periodic], C.c_int)
    nbytes = int(lib.ictc_neighbor_scratch_bytes(n, lo_c, hi_c, float(cutoff)))
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    rowptr = torch.empty(num_centres + 1, dtype=torch.int64, device=dev)
    scan = torch.empty(int(lib.ictc_scan_scratch_bytes(num_centres + 1)), dtype=torch.uint8, device=dev)
    pos = pos.contiguous()
    with _lib.on_device(dev):
        st = _lib.stream(dev)
        _lib.check(lib.ictc_neighbor_count(pos.data_ptr(), n, num_centres, lo_c, hi_c, box_c, per_c, float(cutoff),
                                           rowptr.data_ptr(), scratch.data_ptr(), st), "ictc_neighbor_count")
        _lib.check(lib.ictc_inclusive_scan_i64(rowptr.data_ptr(), num_centres + 1, scan.data_ptr(), st),
                   "ictc_inclusive_scan_i64")
        e = int(rowptr[-1].item())
        eb = _bucket(e)
        src = torch.empty(eb, dtype=torch.int64, device=dev)[:e]
        dst = torch.empty(eb, dtype=torch.int64, device=dev)[:e]
        shifts = torch.empty(eb, 3, dtype=torch.float32, device=dev)[:e]
        keys = torch.empty(eb, dtype=torch.int64, device=dev)[:e]
        _lib.check(lib.ictc_neighbor_fill(pos.data_ptr(), n, num_centres, lo_c, hi_c, box_c, per_c, float(cutoff),
                                          rowptr.data_ptr(), e, _lib.ptr(src), _lib.ptr(dst), _lib.ptr(shifts),
                                          _lib.ptr(keys), scratch.data_ptr(), st), "ictc_neighbor_fill")
    if return_keys:
        return src, dst, shifts, rowptr, keys
    return src, dst, shifts, rowptr


def edge_pairs(rowptr, dst, keys, num_centres):
    """Radial pairing of a neighbour list (edge and reverse edge share their length): returns
    (gate_row [E], rep_edge [U], other_edge [U]); see ``ictc_neighbor_pairs``."""
    lib, dev = _lib.load(), dst.device
    e = int(dst.numel())
    eb = _bucket(e)
    rev = torch.empty(eb, dtype=torch.int64, device=dev)
    scan = torch.empty(eb, dtype=torch.int64, device=dev)
    gate_row = torch.empty(eb, dtype=torch.int64, device=dev)[:e]
    rep = torch.empty(eb, dtype=torch.int64, device=dev)
    other = torch.empty(eb, dtype=torch.int64, device=dev)
    num = torch.zeros(1, dtype=torch.int64, device=dev)
    scratch = torch.empty(int(lib.ictc_scan_scratch_bytes(eb)), dtype=torch.uint8, device=dev)
    with _lib.on_device(dev):
        _lib.check(lib.ictc_neighbor_pairs(rowptr.data_ptr(), _lib.ptr(dst), _lib.ptr(keys), num_centres, e, e,
                                           rowptr.data_ptr() + 8 * num_centres, _lib.ptr(rev), _lib.ptr(scan),
                                           _lib.ptr(gate_row), _lib.ptr(rep), _lib.ptr(other), num.data_ptr(),
                                           scratch.data_ptr(), _lib.stream(dev)), "ictc_neighbor_pairs")
    u = int(num.item())
    return gate_row, rep[:u], other[:u]


class StaticNeighborList:
    """Neighbour list into fixed-capacity buffers, with no host read-back: the tail of the edge arrays
    is padded with inert edges (sender = the extra row ``num_atoms`` of the position buffer, which the
    sender CSR ignores; receiver 0) and an overflow flag stays on the device.  All buffers are allocated
    once, so the sequence can be recorded in a CUDA graph.

    ``num_centres`` (default: all atoms) rows get edges; ``lo`` / ``hi`` bound the cell grid (default: the
    periodic box); ``periodic`` = three flags (a domain-decomposed rank passes zeros: its ghost rows already
    carry the image shifts); ``pair_fraction`` sizes the pair table relative to the edge capacity (0.5 when
    every edge has its reverse in the list, more when senders can be ghosts)."""

    def __init__(self, num_atoms, box, cutoff, capacity, device, *, num_centres=None, lo=None, hi=None,
                 periodic=(1, 1, 1), pair_fraction=0.5):
        self.n, self.cap, self.cutoff, self.dev = int(num_atoms), int(capacity), float(cutoff), device
        self.centres = self.n if num_centres is None else int(num_centres)
        lib = _lib.load()
        self.lo = _arr([0.0, 0.0, 0.0] if lo is None else [float(v) for v in lo], C.c_double)
        self.hi = _arr([float(b) for b in box] if hi is None else [float(v) for v in hi], C.c_double)
        self.box, self.per = _arr([float(b) for b in box], C.c_double), _arr([int(v) for v in periodic], C.c_int)
        n1 = self.n + 1                                   # the position buffer carries one extra (dummy) row
        self.scratch = torch.empty(int(lib.ictc_neighbor_scratch_bytes(n1, self.lo, self.hi, self.cutoff)),
                                   dtype=torch.uint8, device=device)
        self.scan = torch.empty(int(lib.ictc_scan_scratch_bytes(self.centres + 1)), dtype=torch.uint8, device=device)
        self.rowptr = torch.zeros(self.centres + 1, dtype=torch.int64, device=device)
        self.src = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.dst = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.shifts = torch.zeros(self.cap, 3, dtype=torch.float32, device=device)
        self.keys = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=device)
        self.ucap = int(self.cap * pair_fraction) + 1024
        self.rev = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.pscan = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.gate_row = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.rep = torch.zeros(self.ucap, dtype=torch.int64, device=device)
        self.other = torch.zeros(self.ucap, dtype=torch.int64, device=device)
        self.num_unique = torch.zeros(1, dtype=torch.int64, device=device)
        self.pscratch = torch.empty(int(lib.ictc_scan_scratch_bytes(self.cap)), dtype=torch.uint8, device=device)

    def build(self, pos_ext):
        """pos_ext [n+1, 3]: the atoms followed by the dummy row (far away from every atom)."""
        lib, st = _lib.load(), _lib.stream(self.dev)
        n, n1 = self.centres, self.n + 1
        _lib.check(lib.ictc_neighbor_count(pos_ext.data_ptr(), n1, n, self.lo, self.hi, self.box, self.per,
                                           self.cutoff, self.rowptr.data_ptr(), self.scratch.data_ptr(), st),
                   "ictc_neighbor_count")
        _lib.check(lib.ictc_inclusive_scan_i64(self.rowptr.data_ptr(), n + 1, self.scan.data_ptr(), st), "scan")
        _lib.check(lib.ictc_neighbor_clamp(self.rowptr.data_ptr(), n, self.cap - 1, self.overflow.data_ptr(), st),
                   "ictc_neighbor_clamp")       # cap - 1: the last slot always stays an inert edge
        _lib.check(lib.ictc_neighbor_fill(pos_ext.data_ptr(), n1, n, self.lo, self.hi, self.box, self.per, self.cutoff,
                                          self.rowptr.data_ptr(), self.cap, self.src.data_ptr(), self.dst.data_ptr(),
                                          self.shifts.data_ptr(), self.keys.data_ptr(), self.scratch.data_ptr(), st),
                   "ictc_neighbor_fill")
        _lib.check(lib.ictc_neighbor_pad(self.rowptr.data_ptr() + 8 * n, self.cap, self.n, 0, self.src.data_ptr(),
                                         self.dst.data_ptr(), self.shifts.data_ptr(), None, st),
                   "ictc_neighbor_pad")
        _lib.check(lib.ictc_neighbor_pairs(self.rowptr.data_ptr(), self.dst.data_ptr(), self.keys.data_ptr(), n,
                                           self.cap, self.ucap, self.rowptr.data_ptr() + 8 * n, self.rev.data_ptr(),
                                           self.pscan.data_ptr(), self.gate_row.data_ptr(), self.rep.data_ptr(),
                                           self.other.data_ptr(), self.num_unique.data_ptr(),
                                           self.pscratch.data_ptr(), st), "ictc_neighbor_pairs")

    def pairs(self):
        return self.gate_row, self.rep, self.other, self.num_unique


def maxwell_boltzmann(masses: np.ndarray, temperature: float, seed: int) -> np.ndarray:
    """Gaussian velocities (A/fs) at ``temperature`` with zero total momentum, rescaled to the exact
    target (LAMMPS ``velocity all create T seed mom yes rot no dist gaussian``)."""
    rng = np.random.default_rng(seed)
    sigma = np.sqrt(KB_EV * temperature * ACCEL / masses)[:, None]
    v = rng.normal(size=(masses.shape[0], 3)) * sigma
    v -= (v * masses[:, None]).sum(0) / masses.sum()
    ke = 0.5 * (masses[:, None] * v * v).sum() / ACCEL
    dof = 3 * masses.shape[0] - 3
    v *= math.sqrt(0.5 * dof * KB_EV * temperature / ke)
    return v.astype(np.float32)


class MolecularDynamics:
    """NVE velocity-Verlet driver around a model created by ``mace_ictc.hp.create_model``.

    ``positions`` [N,3], ``atomic_numbers`` [N] and ``velocities`` describe the WHOLE system on every rank; with
    ``distributed=True`` (``torch.distributed`` initialised, one rank per GPU) each rank keeps the atoms of its
    brick and forgets the rest.  ``pos``, ``vel``, ``forces`` hold this rank's atoms only, in an internal order
    (``sort_atoms``: along a space-filling curve, for cache locality of the gathers); ``gid`` gives their indices
    in the arrays passed here and ``gather`` reassembles an array in that original order.  Positions outside the box are
    wrapped into it; an atomic number the model does not know raises ``ValueError``.
    ``skin``: extra halo width of the decomposed run (see the module text).  ``chunk_rows``: owner rows per
    chunk of the force engine's streamed gate evaluation (None: whole tables) and ``stream_gates`` whether the
    gates themselves are streamed or only their gradient (``ForceEngine.stream_gates``).  ``use_engine``: None picks the
    tape-free force engine for the 64-channel two-interaction model and autograd through the same kernels
    otherwise.  ``watch_peers``: check before every block of steps that all ranks are still there.
    ``capture_collectives``: whether ``enable_graph`` of a decomposed run records the step, collectives included, as
    one CUDA graph.  On four ranks the replay of such a graph never completed with the collective library's defaults
    (every rank waiting in the host read after the replays; the same step run eagerly before it was fine; no GPU
    fault) and completes with in-switch reduction and capture-time buffer registration switched off
    (NCCL_NVLS_ENABLE=0, NCCL_GRAPH_REGISTER=0, set before the process group is created).  None = record with two
    ranks, with three or four ranks when the environment shows both settings (the rank counts the recording was run
    on), otherwise launch the step eagerly — same kernels, same fixed buffers, no host read-back inside a block of
    steps.  True records at any rank count.
    """

    def __init__(self, model, positions, atomic_numbers, box, *, dt=1.0, temperature=300.0, seed=0,
                 velocities=None, distributed=False, use_engine=None, share_gates=True, skin=2.0, chunk_rows=None,
                 stream_gates=None, watch_peers=False, sort_atoms=True, capture_collectives=None):
        self.model = model
        dev = next(model.parameters()).device
        self.device = dev
        self.box = torch.as_tensor(np.asarray(box, dtype=np.float64))
        self.box_f = self.box.to(dev, torch.float32)
        self.cutoff = float(model.max_radius)
        z_all = np.asarray(atomic_numbers).astype(np.int64)
        pos_all = np.asarray(positions, dtype=np.float32)
        if pos_all.ndim != 2 or pos_all.shape[1] != 3 or z_all.shape != (pos_all.shape[0],):
            raise ValueError("positions must be [N, 3] and atomic_numbers [N]")
        if not np.isfinite(pos_all).all():
            raise ValueError("positions must be finite")
        model.skip_input_validation = False
        species_all = model.species_index(torch.as_tensor(z_all).to(dev))        # raises ValueError on an unknown Z
        unknown = [int(a) for a in np.unique(z_all) if int(a) not in MASSES]
        if unknown:
            raise ValueError(f"no mass tabulated for atomic numbers {unknown}")
        masses_all = np.array([MASSES[int(a)] for a in z_all], dtype=np.float64)
        if velocities is None:
            velocities = maxwell_boltzmann(masses_all, temperature, seed)
        vel_all = np.asarray(velocities, dtype=np.float32)
        box32 = np.asarray(box, dtype=np.float32)
        pos_all = pos_all - np.floor(pos_all / box32) * box32                    # wrap into [0, box)
        pos_all = np.where(pos_all >= box32, pos_all - box32, pos_all).astype(np.float32)
        self.num_atoms_total = int(pos_all.shape[0])
        self.dt = float(dt)
        self.skin = float(skin)
        self.distributed = bool(distributed)
        if self.distributed:
            import torch.distributed as dist
            self.rank, self.world = dist.get_rank(), dist.get_world_size()
            self.grid = D.brick_grid(self.world, self.box.tolist())
        else:
            self.rank, self.world, self.grid = 0, 1, (1, 1, 1)
        model.preserve_edge_order = True
        model.skip_input_validation = True
        pos_t = torch.as_tensor(pos_all).to(dev)
        if self.world > 1:
            owner = D.owner_of(pos_t, self.box.tolist(), self.grid)
            counts = torch.bincount(owner, minlength=self.world)
            if int(counts.min()) == 0:      # the same decision on every rank: all ranks hold the whole system here
                raise RuntimeError("a brick owns no atoms; use fewer ranks for this box")
            mine = torch.nonzero(owner == self.rank).flatten()
        else:
            mine = torch.arange(self.num_atoms_total, device=dev)
        self.sort_atoms = bool(sort_atoms)
        if self.sort_atoms:          # rows along a space-filling curve: gathered neighbour rows stay in L2
            mine = mine.index_select(0, D.morton_order(pos_t.index_select(0, mine)))
        self.gid = mine
        self.num_owned = int(mine.numel())       # rows of pos / vel / forces that hold atoms (the rest is padding)
        self.pos = pos_t.index_select(0, mine).contiguous()
        self.vel = torch.as_tensor(vel_all).to(dev).index_select(0, mine).contiguous()
        self.z = torch.as_tensor(z_all).to(dev).index_select(0, mine)
        self.species = species_all.index_select(0, mine)
        self.masses = torch.as_tensor(masses_all, dtype=torch.float32).to(dev).index_select(0, mine)
        self.inv_mass = (1.0 / self.masses).contiguous()
        if use_engine is None:       # the tape-free engine exists for the 64-channel model; other widths differentiate
            use_engine = model.channels == 64 and len(model.interactions) == 2      # through the same kernels by autograd
        if use_engine:
            from .engine import ForceEngine
            self.engine = ForceEngine(model, chunk_rows=chunk_rows, stream_gates=stream_gates)
        else:
            self.engine = None
        self.forces = None
        self.energy = None
        self.num_edges = 0
        self.num_gate_rows = 0       # rows of the gate table of the last force call (edge pairs, or edges)
        self.graph = None
        self._static = None
        self._dist = None            # buffers of the decomposed step
        self.share_gates = bool(share_gates)     # evaluate the radial MLP once per (edge, reverse edge) pair
        self.graph_rebuilds = 0
        self.refreshes = 0           # ghost-list refreshes of the decomposed run
        self.redecompositions = 0
        self.block = 8               # steps between refreshes; set at every refresh from the atoms' speeds
        self._period_stale = False
        self._stale_block = 8
        self.refresh_seconds = 0.0   # host time spent in refreshes (they synchronise)
        self.events = []             # (what, steps, host seconds) of the decomposed run's blocks and refreshes
        if capture_collectives is None:
            import os
            capture_collectives = self.world <= 2 or (self.world <= 4 and os.environ.get("NCCL_NVLS_ENABLE") == "0"
                                                      and os.environ.get("NCCL_GRAPH_REGISTER") == "0")
        self.capture_collectives = bool(capture_collectives)
        self.zero_box = torch.zeros(3, dtype=torch.float32, device=dev)
        self._watch = D.PeerWatch() if (watch_peers and self.world > 1) else None

    # ------------------------------------------------------------------ forces
    def compute_forces(self):
        if self.world == 1:
            return self._forces_single()
        if self._dist is None:
            self._setup_distributed()
        self._forces_distributed()
        return self.forces

    def _forces_single(self):
        n = self.pos.shape[0]
        box = self.box.tolist()
        src, dst, shifts, rowptr, keys = neighbor_list(self.pos, n, [0, 0, 0], box, box, (1, 1, 1), self.cutoff, True)
        self.num_edges = int(src.numel())
        if self.engine is not None:
            pairs = edge_pairs(rowptr, dst, keys, n) if self.share_gates else None
            self.num_gate_rows = int(pairs[1].numel()) if pairs is not None else self.num_edges
            energy, grad, _ = self.engine.energy_and_gradient(self.pos, self.species, src, dst, shifts, box, n, rowptr,
                                                              pairs=pairs)
            if self._static is not None:            # keep the buffers the recorded graph reads and writes
                self._static["energy"].copy_(energy.reshape(1))
                self.forces.copy_(grad).neg_()
            else:
                self.energy = energy
                self.forces = (-grad).contiguous()
            return self.forces
        topo = Topology(src, dst, n, dst_sorted=True)
        topo._by_dst = (rowptr, None)
        pos = self.pos.detach().requires_grad_(True)
        batch = torch.zeros(n, dtype=torch.long, device=self.device)
        cell = torch.diag(self.box_f).unsqueeze(0)
        with torch.enable_grad():
            atomic = self.model(pos, self.z, batch, src, dst, shifts, cell, topology=topo)
            energy = atomic.sum()
            (grad,) = torch.autograd.grad(energy, pos)
        self.energy = energy.detach()
        self.forces = (-grad).contiguous()
        return self.forces

    # ------------------------------------------------------------------ decomposed run: set-up and refresh
    def _pad_rows(self, count, own_cap):
        """Coordinates of the padding rows [count, own_cap): a far line with 16 A spacing on the NEGATIVE side
        (padding ghost rows sit at +10^6 A, the sender of inert edges at -10^6 A), so that padding rows are
        neighbours neither of atoms, nor of padding ghosts, nor of each other."""
        k = torch.arange(own_cap - count, dtype=torch.float32, device=self.device)
        pad = torch.full((own_cap - count, 3), -3.0 * D.PAD_SHIFT, dtype=torch.float32, device=self.device)
        pad[:, 0] -= 16.0 * k
        return pad

    def _store_owned(self, pos, vel, forces, gid, z):
        """Write this rank's atoms (sorted along the Morton curve when ``sort_atoms``) into the fixed-capacity
        arrays in place; rows beyond the count become inert padding (far away, no velocity, infinite mass)."""
        d, dev = self._dist, self.device
        n, cap = int(pos.shape[0]), d["own_cap"]
        if self.sort_atoms:
            order = D.morton_order(pos)
            pos, vel, forces, gid, z = (t.index_select(0, order) for t in (pos, vel, forces, gid, z))
        self.pos[:n].copy_(pos)
        self.pos[n:].copy_(self._pad_rows(n, cap))
        self.vel[:n].copy_(vel)
        self.vel[n:].zero_()
        self.forces[:n].copy_(forces)
        self.forces[n:].zero_()
        self.gid[:n].copy_(gid)
        self.gid[n:].fill_(-1)
        self.z[:n].copy_(z)
        self.z[n:].fill_(int(self.model.atomic_numbers[0]))
        self.species.copy_(self.model.atomic_number_to_index[self.z])
        mass = torch.tensor([MASSES[int(a)] for a in self.model.atomic_numbers], dtype=torch.float32, device=dev)
        self.masses.copy_(mass[self.species])
        self.inv_mass.copy_(1.0 / self.masses)
        self.inv_mass[n:].zero_()
        d["own_mask"][:n].fill_(1.0)
        d["own_mask"][n:].zero_()
        d["n_own"] = n
        self.num_owned = n

    def _setup_distributed(self, edge_margin=1.15, own_margin=1.01):
        """Fixed-capacity arrays of this rank's atoms, halo plan, local buffers and neighbour-list buffers
        (collective).  On entry ``pos``, ``vel``, ``gid``, ``z`` (and ``forces``, if any) hold exactly the rank's
        atoms; afterwards they have ``own_cap`` rows, the first ``num_owned`` of them atoms."""
        if self.engine is None:
            raise RuntimeError("the decomposed run uses the force engine (use_engine=True)")
        dev = self.device
        n_own = int(self.num_owned)
        peak = torch.tensor([float(n_own)], device=dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(peak, op=dist.ReduceOp.MAX)
        own_cap = int(float(peak.item()) * own_margin) + 256           # the same on every rank
        cur = (self.pos[:n_own].clone(), self.vel[:n_own].clone(),
               torch.zeros(n_own, 3, device=dev) if self.forces is None else self.forces[:n_own].clone(),
               self.gid[:n_own].clone(), self.z[:n_own].clone())
        self.pos = torch.zeros(own_cap, 3, dtype=torch.float32, device=dev)
        self.vel = torch.zeros(own_cap, 3, dtype=torch.float32, device=dev)
        self.forces = torch.zeros(own_cap, 3, dtype=torch.float32, device=dev)
        self.gid = torch.zeros(own_cap, dtype=torch.long, device=dev)
        self.z = torch.zeros(own_cap, dtype=torch.long, device=dev)
        self.species = torch.zeros(own_cap, dtype=torch.long, device=dev)
        self.masses = torch.ones(own_cap, dtype=torch.float32, device=dev)
        self.inv_mass = torch.zeros(own_cap, dtype=torch.float32, device=dev)
        self._dist = {"own_cap": own_cap, "own_mask": torch.zeros(own_cap, dtype=torch.float32, device=dev)}
        self._store_owned(*cur)
        halo = self.cutoff + self.skin
        lo, hi = D.brick_bounds(self.rank, self.grid, self.box.tolist())
        plan = D.HaloPlan(self.rank, self.world, self.grid, self.box.tolist(), halo, own_cap, dev)
        while not plan.refresh(self.pos):
            pass
        n_local = own_cap + plan.num_ghost
        # cell grid: the halo plus the room atoms may move before the next refresh
        ext = halo + self.skin
        grid_lo, grid_hi = [v - ext for v in lo], [v + ext for v in hi]
        pos_ext = torch.zeros(n_local + 1, 3, dtype=torch.float32, device=dev)
        pos_ext[n_local] = -1.0e6
        species_ext = torch.zeros(n_local + 1, dtype=torch.long, device=dev)
        species_ext[:own_cap] = self.species
        species_ext[own_cap:n_local] = plan.integers(self.species)
        pos_ext[:own_cap] = self.pos
        pos_ext[own_cap:n_local] = plan.positions(self.pos)
        # edge capacity from one eager build
        src, _d, _s, rowptr = neighbor_list(pos_ext[:n_local], own_cap, grid_lo, grid_hi, self.box.tolist(), (0, 0, 0),
                                            self.cutoff)
        edges = torch.tensor([float(src.numel())], device=dev)
        if self.world > 1:
            dist.all_reduce(edges, op=dist.ReduceOp.MAX)
        cap = int(float(edges.item()) * edge_margin) + 4096
        nl = StaticNeighborList(n_local, self.box.tolist(), self.cutoff, cap, dev, num_centres=own_cap, lo=grid_lo,
                                hi=grid_hi, periodic=(0, 0, 0), pair_fraction=0.7)
        self._dist.update({"plan": plan, "nl": nl, "pos_ext": pos_ext, "species_ext": species_ext,
                           "n_local": n_local, "cap": cap, "edge_margin": edge_margin,
                           "pos_ref": self.pos.clone(), "stale": torch.zeros(1, dtype=torch.int32, device=dev),
                           "energy": torch.zeros(1, dtype=torch.float32, device=dev),
                           "limit2": torch.full((1,), (0.5 * self.skin) ** 2, dtype=torch.float32, device=dev),
                           "since_refresh": 0})
        self.energy = self._dist["energy"][0]
        self.graph = None

    def refresh(self):
        """Re-neighbouring of the decomposed run (collective): coordinates are wrapped into the box, every atom moves
        to the rank whose brick contains it (reference semantics: LAMMPS' exchange at re-neighbouring, seen by the
        pair style as a changed ``nlocal``, pair_mff_torch.cpp:222-242), the rows are sorted again and the ghost
        lists are rebuilt.  Everything is rewritten IN PLACE in fixed-capacity arrays, so a recorded step stays
        valid.  Returns False when a capacity no longer fits: the caller sets the buffers up again."""
        d = self._dist
        n = d["n_own"]
        box32 = self.box_f
        pos = self.pos[:n]
        pos = pos - torch.floor(pos / box32) * box32
        pos = torch.where(pos >= box32, pos - box32, pos)
        dest = D.owner_of(pos, self.box.tolist(), self.grid)
        payload = torch.cat((pos.double(), self.vel[:n].double(), self.forces[:n].double(),
                             self.gid[:n].double().unsqueeze(1), self.z[:n].double().unsqueeze(1)), 1)
        got = D.migrate(dest, payload, self.world)
        count = int(got.shape[0])
        if D.same_on_all_ranks(count == 0):
            raise RuntimeError("a brick owns no atoms; use fewer ranks for this box")
        got = got.index_select(0, torch.argsort(got[:, 9].long()))       # ascending global id: a reproducible order
        fresh = (got[:, 0:3].float(), got[:, 3:6].float(), got[:, 6:9].float(), got[:, 9].long(), got[:, 10].long())
        if D.same_on_all_ranks(count > d["own_cap"]):
            self.pos, self.vel, self.forces, self.gid, self.z = (t.contiguous() for t in fresh)
            self.num_owned = count
            return False
        self._store_owned(*fresh)
        if not d["plan"].refresh(self.pos):
            return False
        d["species_ext"][:d["own_cap"]] = self.species
        d["species_ext"][d["own_cap"]:d["n_local"]] = d["plan"].integers(self.species)
        d["pos_ref"].copy_(self.pos)
        d["stale"].zero_()
        self.refreshes += 1
        return True

    def _steps_within_budget(self):
        """How many steps the fastest atom (of any rank) needs to use up 70 % of the displacement budget skin/2 at
        its present speed: the length of the next period between refreshes (collective)."""
        n = self.num_owned
        vmax = self.vel[:n].square().sum(1).max().sqrt().reshape(1)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(vmax, op=dist.ReduceOp.MAX)
        speed = max(float(vmax.item()), 1e-12)
        return int(max(1, min(64, 0.7 * 0.5 * self.skin / (speed * self.dt))))

    def redecompose(self):
        """Refresh, and set all buffers up again (a recorded graph is dropped) when a capacity did not fit."""
        if not self.refresh():
            edge_margin = self._dist["edge_margin"]
            forces = self.forces[:self.num_owned].clone() if self.forces.shape[0] >= self.num_owned else None
            self.graph, self._dist = None, None
            self._setup_distributed(edge_margin=edge_margin)
            if forces is not None:
                self.forces[:self.num_owned].copy_(forces)
            self.redecompositions += 1
            return False
        return True

    # ------------------------------------------------------------------ decomposed run: one step
    def _forces_distributed(self):
        """Forces of the owned atoms from their current coordinates, on fixed buffers only: no host read-back, no
        data-dependent host control flow (the sequence is what a recorded graph replays)."""
        d = self._dist
        plan, nl, n_own, n_local = d["plan"], d["nl"], d["own_cap"], d["n_local"]
        pos_ext = d["pos_ext"]
        pos_ext[:n_own].copy_(self.pos)
        pos_ext[n_own:n_local].copy_(plan.positions(self.pos))
        # has any owned atom used up its displacement budget?  (sticky flag, read by ``run`` between blocks)
        moved2 = (self.pos - d["pos_ref"]).square().sum(1).max()
        d["stale"].logical_or_(moved2 > d["limit2"])
        with _lib.on_device(self.device):
            nl.build(pos_ext)
        energy, grad, _ = self.engine.energy_and_gradient(pos_ext, d["species_ext"], nl.src, nl.dst, None,
                                                          self.box.tolist(), n_own, nl.rowptr, plan=plan,
                                                          n_rows=n_local, row_mask=d["own_mask"],
                                                          pairs=nl.pairs() if self.share_gates else None)
        back = plan.adjoint(grad[n_own:n_local])          # ghost rows' gradients return to their owners
        torch.add(grad[:n_own], back, out=self.forces)
        self.forces.neg_()
        e = energy.reshape(1).clone()
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(e)
        d["energy"].copy_(e)

    def _step_distributed(self):
        self._kick(True)
        self._forces_distributed()
        self._kick(False)

    def _flags(self):
        """(edge or chunk or pair capacity exceeded, displacement budget used up), agreed between the ranks."""
        d = self._dist
        nl = d["nl"]
        over = (nl.overflow.to(torch.int64) + self.engine.overflow.to(torch.int64)
                + (nl.num_unique > nl.ucap).to(torch.int64)).clamp(max=1)
        both = torch.cat((over, d["stale"].to(torch.int64)))
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(both, op=dist.ReduceOp.MAX)
        v = both.tolist()
        return bool(v[0]), bool(v[1])

    def _reset_flags(self):
        d = self._dist
        d["nl"].overflow.zero_()
        self.engine.overflow.zero_()
        d["stale"].zero_()

    # ------------------------------------------------------------------ CUDA-graph replay
    def _step_static(self):
        """One full single-GPU step on fixed buffers only (no host read-back, no data-dependent host control flow)."""
        st = self._static
        n = self.pos.shape[0]
        self._kick(True)
        st["pos_ext"][:n].copy_(self.pos)
        st["nl"].build(st["pos_ext"])
        nl = st["nl"]
        energy, grad, _ = self.engine.energy_and_gradient(st["pos_ext"], st["species_ext"], nl.src, nl.dst, nl.shifts,
                                                          self.box.tolist(), n, nl.rowptr, n_rows=n,
                                                          pairs=nl.pairs() if self.share_gates else None)
        st["energy"].copy_(energy.reshape(1))
        self.forces.copy_(grad).neg_()
        self._kick(False)

    def run(self, steps, check_every=25, margin=1.10, on_step=None):
        """Advance ``steps`` MD steps.

        One rank with a recorded graph: the capacity flags are read every ``check_every`` steps; when the
        neighbour list (or a gate chunk) outgrew its buffers the block of steps is repeated from a snapshot with
        a larger capacity.  Several ranks: steps run in blocks that start with a ghost-list refresh; after a
        block the ranks agree on the flags, and a block that used up its displacement budget is repeated from
        the snapshot with half the length.  ``on_step`` is called on the host after every step was launched."""
        if self.world > 1:
            return self._run_distributed(steps, on_step)
        if self.graph is None:
            for _ in range(steps):
                self.step()
                if on_step is not None:
                    on_step()
            return
        done = 0
        while done < steps:
            block = min(check_every, steps - done)
            snap = (self.pos.clone(), self.vel.clone())
            for _ in range(block):
                self.graph.replay()
                if on_step is not None:
                    on_step()
            self.check_kernels()
            if self.check_overflow():
                self.pos.copy_(snap[0])
                self.vel.copy_(snap[1])
                self.graph, self._static = None, None
                if bool(int(self.engine.overflow.item())):
                    self.engine.chunk_margin += 0.15
                self.engine.overflow.zero_()
                self.compute_forces()
                self.enable_graph(margin=margin)
                self.graph_rebuilds += 1
                continue
            done += block

    def _run_distributed(self, steps, on_step):
        if self._dist is None:
            self.compute_forces()
        done = 0
        while done < steps:
            if self._watch is not None:
                self._watch.check()          # a missing rank is noticed here, on the host, before the next collectives
            d = self._dist
            if d["since_refresh"] >= self.block:
                import time
                t0 = time.perf_counter()
                recorded = self.graph is not None
                if not self.redecompose() and recorded:
                    self.enable_graph()
                torch.cuda.synchronize(self.device)
                self.refresh_seconds += time.perf_counter() - t0
                self.events.append(("refresh", 0, time.perf_counter() - t0))
                d = self._dist
                d["since_refresh"] = 0
                ahead = self._steps_within_budget()
                # after a period that ran out of budget, at most half its length; otherwise what the speeds allow
                self.block = min(ahead, max(1, self._stale_block // 2)) if self._period_stale else ahead
                self._period_stale = False
            block = min(self.block - d["since_refresh"], steps - done)
            snap = (self.pos.clone(), self.vel.clone(), self.forces.clone())
            import time
            t_block = time.perf_counter()
            for _ in range(block):
                if self.graph is not None:
                    self.graph.replay()
                else:
                    self._step_distributed()
                if on_step is not None:
                    on_step()
            over, stale = self._flags()
            self.check_kernels()
            self.events.append(("repeat" if (over or stale) else "block", block, time.perf_counter() - t_block))
            if over or stale:
                self.pos.copy_(snap[0])
                self.vel.copy_(snap[1])
                self.forces.copy_(snap[2])
                self._reset_flags()
                if over:                    # larger capacities: new buffers, new recording
                    recorded = self.graph is not None
                    margin = d["edge_margin"] + 0.15
                    self.engine.chunk_margin += 0.15
                    since, n = d["since_refresh"], d["n_own"]
                    self.graph, self._dist = None, None
                    self.pos, self.vel, self.gid, self.z = (t[:n].contiguous() for t in (self.pos, self.vel, self.gid, self.z))
                    self.forces = snap[2][:n].contiguous()
                    self._setup_distributed(edge_margin=margin)
                    self._dist["since_refresh"] = since
                    if recorded:
                        self.enable_graph()
                    self.graph_rebuilds += 1
                if stale:
                    if block == 1 and d["since_refresh"] == 0:
                        raise RuntimeError("an atom uses up the skin within one step: use a larger skin or a smaller dt")
                    self._stale_block = max(1, min(self.block, d["since_refresh"] + block))
                    self.block = 0                                # the repeated block starts with a refresh
                    self._period_stale = True
                continue
            done += block
            d["since_refresh"] += block

    def enable_graph(self, margin=1.10, warmup=2, spare=1024):
        """Record the whole MD step (integration, neighbour build, forces, halo exchanges) as one CUDA graph.

        One rank: edge buffers get a fixed capacity of ``margin`` times the current edge count plus ``spare``; the
        device-side overflow flag is checked by ``check_overflow``.  Several ranks: the decomposed step already
        runs on fixed buffers; the recording includes its collectives (collective call)."""
        if self.engine is None:
            raise RuntimeError("graph replay covers the engine path")
        dev = self.device
        torch.cuda.empty_cache()        # the eager steps' cached blocks go back before the recording gets its own pool
        if self.world > 1:
            if self._dist is None:
                self.compute_forces()
            if not self.capture_collectives:        # the step stays an eager launch sequence on the fixed buffers
                return self._dist["cap"]
            keep = (self.pos.clone(), self.vel.clone(), self.forces.clone(), self._dist["energy"].clone())
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                for _ in range(warmup):
                    self._step_distributed()
            torch.cuda.current_stream(dev).wait_stream(side)
            torch.cuda.synchronize(dev)
            # thread-local capture mode: the collective library's watchdog thread keeps polling its events
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                self._step_distributed()
            self.graph = graph
            self.pos.copy_(keep[0])
            self.vel.copy_(keep[1])
            self.forces.copy_(keep[2])
            self._dist["energy"].copy_(keep[3])
            self._reset_flags()
            return self._dist["cap"]
        if self.forces is None:
            self.compute_forces()
        n = self.pos.shape[0]
        cap = int(self.num_edges * margin) + int(spare)
        pos_ext = torch.zeros(n + 1, 3, dtype=torch.float32, device=dev)
        pos_ext[n] = -1.0e6          # the dummy row sits far outside every cutoff sphere
        species_ext = torch.cat((self.species, self.species.new_zeros(1)))
        self._static = {"nl": StaticNeighborList(n, self.box.tolist(), self.cutoff, cap, dev), "pos_ext": pos_ext,
                        "species_ext": species_ext, "energy": torch.zeros(1, device=dev), "cap": cap}
        self.forces = self.forces.clone()
        keep = (self.pos.clone(), self.vel.clone(), self.forces.clone(), self.energy.detach().clone().reshape(1))
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                self._step_static()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step_static()
        # the warm-up steps advanced the state: put it back so that recording is invisible to the caller
        self.pos.copy_(keep[0])
        self.vel.copy_(keep[1])
        self.forces.copy_(keep[2])
        self._static["energy"].copy_(keep[3])
        self._static["nl"].overflow.zero_()
        self.engine.overflow.zero_()
        self.energy = self._static["energy"][0]
        return cap

    def check_overflow(self):
        """True when a replayed step needed more edges than a recorded capacity (results invalid)."""
        if self._static is None:
            return False
        nl = self._static["nl"]
        return (bool(int(nl.overflow.item())) or int(nl.num_unique.item()) > nl.ucap
                or bool(int(self.engine.overflow.item())))

    def check_kernels(self):
        """Raise when a kernel with bounded waits gave up (its results are then invalid)."""
        status = _lib.kernel_status()
        if status != 0:
            raise RuntimeError(f"a kernel gave up a bounded wait (status {status}); the step's results are invalid")

    def close(self):
        """Release the recorded graph.  A decomposed run MUST call this before the process group is destroyed: a
        live CUDA graph that holds captured collectives keeps the communicator busy and its tear-down waits
        forever."""
        if self.graph is not None:
            torch.cuda.synchronize(self.device)
            self.graph = None
            import gc
            gc.collect()
            torch.cuda.synchronize(self.device)

    # ------------------------------------------------------------------ integration
    def _kick(self, drift):
        lib = _lib.load()
        # a decomposed run keeps coordinates unwrapped between re-decompositions (ghost images are owner + shift)
        box = self.box_f if self.world == 1 else self.zero_box
        with _lib.on_device(self.device):
            _lib.check(lib.ictc_md_kick(self.pos.shape[0], self.dt, self.forces.data_ptr(), self.inv_mass.data_ptr(),
                                        self.vel.data_ptr(), self.pos.data_ptr(), box.data_ptr(), int(drift),
                                        _lib.stream(self.device)), "ictc_md_kick")

    def step(self):
        """One velocity-Verlet step; the edge list is rebuilt from the current coordinates every step."""
        if self.world > 1:
            return self._run_distributed(1, None)
        if self.graph is not None:
            self.graph.replay()
            return
        if self.forces is None:
            self.compute_forces()
        self._kick(True)
        self.compute_forces()
        self._kick(False)

    # ------------------------------------------------------------------ observables
    def gather(self, owned_rows: torch.Tensor) -> torch.Tensor:
        """Rows of this rank's atoms (``pos``, ``vel``, ``forces`` are stored in an internal, spatially sorted order)
        -> the array of the whole system in the order of the constructor's arguments (row = ``gid``), on every
        rank."""
        n = self.num_owned
        full = owned_rows.new_zeros(self.num_atoms_total, *owned_rows.shape[1:])
        full.index_copy_(0, self.gid[:n], owned_rows[:n])
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(full)
        return full

    def kinetic_energy(self):
        ke = 0.5 * (self.masses.double().unsqueeze(1) * self.vel.double() ** 2).sum().reshape(1) / ACCEL
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(ke)
        return float(ke)

    def temperature(self):
        return 2.0 * self.kinetic_energy() / ((3 * self.num_atoms_total - 3) * KB_EV)
