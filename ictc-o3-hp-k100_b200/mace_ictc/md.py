"""Molecular-dynamics step on the B200 kernels: neighbour build, energy and forces, velocity Verlet,
optional spatial domain decomposition over the GPUs of one node.

The reference runs MD through LAMMPS (``examples/in.hco``: metal units, NVE, neighbour rebuild with
0.5 A skin) with its pair style building the edge list from LAMMPS' full neighbour list
(lammps_user_mfftorch/src/USER-MFFTORCH/pair_mff_torch_kokkos.cpp:661-871) and calling the model for
``E_local = sum over owned atoms`` and ``F = -dE/dpos`` (mff_torch_engine.cpp:1739-1859).  LAMMPS is not
part of this build; this module is the stand-alone driver with the same step semantics.
Units: A, fs, eV, amu (1 eV/(A amu) = 9.64853321e-3 A/fs^2).
"""
from __future__ import annotations

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


def neighbor_list(pos, num_centres, lo, hi, box, periodic, cutoff, return_keys=False):
    """Edges (src=j, dst=i) of the first ``num_centres`` rows, sorted by (dst, src, shift).

    pos [N,3] fp32 CUDA; lo/hi: bounds of the cell grid; box: periodic lengths; periodic: 3 flags.
    Returns src, dst (int64 [E]), shifts (float32 [E,3], lattice units), rowptr (int64 [centres+1]).
    """
    import ctypes as C
    lib, dev = _lib.load(), pos.device
    n = pos.shape[0]
    arr = lambda v, t: (t * 3)(*[v[i] for i in range(3)])
    lo_c, hi_c, box_c = arr([float(x) for x in lo], C.c_double), arr([float(x) for x in hi], C.c_double), \
        arr([float(x) for x in box], C.c_double)
    per_c = arr([int(x) for x in periodic], C.c_int)
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
    once, so the sequence can be recorded in a CUDA graph."""

    def __init__(self, num_atoms, box, cutoff, capacity, device):
        import ctypes as C
        self.n, self.cap, self.cutoff, self.dev = int(num_atoms), int(capacity), float(cutoff), device
        lib = _lib.load()
        arr = lambda v, t: (t * 3)(*[v[i] for i in range(3)])
        self.lo, self.hi = arr([0.0, 0.0, 0.0], C.c_double), arr([float(b) for b in box], C.c_double)
        self.box, self.per = arr([float(b) for b in box], C.c_double), arr([1, 1, 1], C.c_int)
        n1 = self.n + 1                                   # the position buffer carries one extra (dummy) row
        self.scratch = torch.empty(int(lib.ictc_neighbor_scratch_bytes(n1, self.lo, self.hi, self.cutoff)),
                                   dtype=torch.uint8, device=device)
        self.scan = torch.empty(int(lib.ictc_scan_scratch_bytes(self.n + 1)), dtype=torch.uint8, device=device)
        self.rowptr = torch.zeros(self.n + 1, dtype=torch.int64, device=device)
        self.src = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.dst = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.shifts = torch.zeros(self.cap, 3, dtype=torch.float32, device=device)
        self.keys = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.overflow = torch.zeros(1, dtype=torch.int32, device=device)
        # radial pairing: on one GPU every edge has its reverse in the list, so there are E/2 pairs
        self.ucap = self.cap // 2 + 1024
        self.rev = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.pscan = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.gate_row = torch.zeros(self.cap, dtype=torch.int64, device=device)
        self.rep = torch.zeros(self.ucap, dtype=torch.int64, device=device)
        self.other = torch.zeros(self.ucap, dtype=torch.int64, device=device)
        self.num_unique = torch.zeros(1, dtype=torch.int64, device=device)
        self.pscratch = torch.empty(int(lib.ictc_scan_scratch_bytes(self.cap)), dtype=torch.uint8, device=device)

    def build(self, pos_ext):
        """pos_ext [n+1, 3]: the real atoms followed by the dummy row (far away from every atom)."""
        lib, st = _lib.load(), _lib.stream(self.dev)
        n, n1 = self.n, self.n + 1
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
        _lib.check(lib.ictc_neighbor_pad(self.rowptr.data_ptr() + 8 * n, self.cap, n, 0, self.src.data_ptr(),
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

    With ``torch.distributed`` initialised (one rank per GPU) atoms are split over a brick grid: each
    rank evaluates energies of its own atoms, node features of ghost atoms cross ranks inside the model
    (``domain.exchange``) and the position gradients are summed over ranks.
    """

    def __init__(self, model, positions, atomic_numbers, box, *, dt=1.0, temperature=300.0, seed=0,
                 velocities=None, distributed=False, use_engine=True, share_gates=True):
        self.model = model
        dev = next(model.parameters()).device
        self.device = dev
        self.box = torch.as_tensor(np.asarray(box, dtype=np.float64))
        self.box_f = self.box.to(dev, torch.float32)
        self.pos = torch.as_tensor(np.asarray(positions, dtype=np.float32)).to(dev).contiguous()
        self.z = torch.as_tensor(np.asarray(atomic_numbers)).long().to(dev)
        masses = np.array([MASSES[int(a)] for a in np.asarray(atomic_numbers)], dtype=np.float64)
        self.masses = torch.as_tensor(masses, dtype=torch.float32).to(dev)
        self.inv_mass = (1.0 / self.masses).contiguous()
        if velocities is None:
            velocities = maxwell_boltzmann(masses, temperature, seed)
        self.vel = torch.as_tensor(np.asarray(velocities, dtype=np.float32)).to(dev).contiguous()
        self.dt = float(dt)
        self.cutoff = float(model.max_radius)
        self.distributed = bool(distributed)
        if self.distributed:
            import torch.distributed as dist
            self.rank, self.world = dist.get_rank(), dist.get_world_size()
            self.grid = D.brick_grid(self.world, self.box.tolist())
        else:
            self.rank, self.world, self.grid = 0, 1, (1, 1, 1)
        model.preserve_edge_order = True
        model.skip_input_validation = True
        self.species = model.species_index(self.z)
        if use_engine:
            from .engine import ForceEngine
            self.engine = ForceEngine(model)
        else:
            self.engine = None
        self.forces = None
        self.energy = None
        self.num_edges = 0
        self.num_gate_rows = 0       # rows of the gate table of the last force call (edge pairs, or edges)
        self.launches = 0
        self.graph = None
        self._static = None
        self.share_gates = bool(share_gates)     # evaluate the radial MLP once per (edge, reverse edge) pair

    # ------------------------------------------------------------------ forces
    def compute_forces(self):
        if self.world == 1:
            return self._forces_single()
        return self._forces_decomposed()

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

    def _forces_decomposed(self):
        import torch.distributed as dist
        dom = D.decompose(self.pos, self.box.to(self.device), self.grid, self.rank, self.cutoff)
        plan = D.ExchangePlan(dom, self.rank, self.world)
        n_owned = dom.num_owned
        if n_owned == 0:
            raise RuntimeError("a rank owns no atoms; use fewer ranks for this box")
        local = dom.local_positions(self.pos, self.box.to(self.device)).contiguous()
        ids = dom.local_ids()
        lo = (dom.lo - self.cutoff).tolist()
        hi = (dom.hi + self.cutoff).tolist()
        src, dst, shifts, rowptr, keys = neighbor_list(local, n_owned, lo, hi, self.box.tolist(), (0, 0, 0),
                                                       self.cutoff, True)
        self.num_edges = int(src.numel())
        n_local = local.shape[0]
        if self.engine is not None:
            pairs = edge_pairs(rowptr, dst, keys, n_owned) if self.share_gates else None
            self.num_gate_rows = int(pairs[1].numel()) if pairs is not None else self.num_edges
            energy, grad, _ = self.engine.energy_and_gradient(local, self.species.index_select(0, ids), src, dst, None,
                                                              self.box.tolist(), n_owned, rowptr, plan, pairs=pairs)
            total = torch.zeros_like(self.pos)
            total.index_add_(0, ids, grad)
            e = energy.reshape(1).clone()
            dist.all_reduce(total)
            dist.all_reduce(e)
            self.energy = e[0]
            self.forces = (-total).contiguous()
            return self.forces
        topo = Topology(src, dst, n_local, dst_sorted=True)
        pad = rowptr.new_full((n_local - n_owned,), int(rowptr[-1].item()))
        topo._by_dst = (torch.cat((rowptr, pad)), None)
        pos = local.detach().requires_grad_(True)
        batch = torch.zeros(n_local, dtype=torch.long, device=self.device)
        cell = torch.diag(self.box_f).unsqueeze(0)

        def callback(layer, h_owned):
            if layer == len(self.model.interactions) - 1:
                return h_owned
            return torch.cat((h_owned, D.exchange(h_owned, plan)), 0)

        with torch.enable_grad():
            atomic = self.model(pos, self.z.index_select(0, ids), batch, src, dst, shifts, cell,
                                local_atom_count=n_owned, layer_state_callback=callback, topology=topo)
            energy = atomic[:n_owned].sum()
            (grad,) = torch.autograd.grad(energy, pos)
        total = torch.zeros_like(self.pos)
        total.index_add_(0, ids, grad)
        e = energy.detach().reshape(1).clone()
        dist.all_reduce(total)
        dist.all_reduce(e)
        self.energy = e[0]
        self.forces = (-total).contiguous()
        return self.forces

    # ------------------------------------------------------------------ CUDA-graph replay (single GPU)
    def _step_static(self):
        """One full step on fixed buffers only (no host read-back, no data-dependent host control flow)."""
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

    graph_rebuilds = 0

    def run(self, steps, check_every=25, margin=1.10, on_step=None):
        """Advance ``steps`` MD steps.  With a recorded graph the edge-capacity flag is read every
        ``check_every`` steps; if the neighbour list outgrew the recorded buffers the block of steps is
        repeated from a snapshot with a larger capacity (steps run after an overflow are invalid).
        ``on_step`` is called on the host after every step has been launched."""
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
            if self.check_overflow():
                self.pos.copy_(snap[0])
                self.vel.copy_(snap[1])
                self.graph, self._static = None, None
                self.compute_forces()
                self.enable_graph(margin=margin)
                self.graph_rebuilds += 1
                continue
            done += block

    def enable_graph(self, margin=1.10, warmup=2, spare=1024):
        """Record the whole MD step (integration, neighbour build, forces) as one CUDA graph.

        Edge buffers get a fixed capacity of ``margin`` times the current edge count plus ``spare``; the device-side
        overflow flag is checked by ``check_overflow``.  Single-GPU, engine path only."""
        if self.world != 1 or self.engine is None:
            raise RuntimeError("graph replay covers the single-GPU engine path")
        if self.forces is None:
            self.compute_forces()
        n, dev = self.pos.shape[0], self.device
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
        self.energy = self._static["energy"][0]
        return cap

    def check_overflow(self):
        """True when a replayed step needed more edges than the recorded capacity (results invalid)."""
        if self._static is None:
            return False
        nl = self._static["nl"]
        return bool(int(nl.overflow.item())) or int(nl.num_unique.item()) > nl.ucap

    # ------------------------------------------------------------------ integration
    def _kick(self, drift):
        lib = _lib.load()
        with _lib.on_device(self.device):
            _lib.check(lib.ictc_md_kick(self.pos.shape[0], self.dt, self.forces.data_ptr(), self.inv_mass.data_ptr(),
                                        self.vel.data_ptr(), self.pos.data_ptr(), self.box_f.data_ptr(), int(drift),
                                        _lib.stream(self.device)), "ictc_md_kick")

    def step(self):
        """One velocity-Verlet step; neighbours are rebuilt every step."""
        if self.graph is not None:
            self.graph.replay()
            return
        if self.forces is None:
            self.compute_forces()
        self._kick(True)
        self.compute_forces()
        self._kick(False)

    def kinetic_energy(self):
        return 0.5 * float((self.masses.double().unsqueeze(1) * self.vel.double() ** 2).sum()) / ACCEL

    def temperature(self):
        return 2.0 * self.kinetic_energy() / ((3 * self.pos.shape[0] - 3) * KB_EV)
