#!/usr/bin/env python
"""Benchmark of the ICTC hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload md|fused_message|sc|train]
                    [--scaling strong|weak]

Workload ``md`` (default; BASELINE configuration 5): NVE molecular dynamics of the C64 / lmax 2 /
2-interaction / correlation-3 random-init model on a jittered simple-cubic H/C/O lattice (spacing 2.15 A,
sigma 0.1 A, 1:2:1), cutoff 4.5 A, 1 fs velocity-Verlet steps from a 300 K Maxwell-Boltzmann start.  A "step" is
one full MD step: integration, position halo, neighbour rebuild, energy, forces, feature and gradient halos.
Metric: atom-steps per second over all GPUs.
  --scaling strong (default): ONE system of 1,048,576 atoms (128 x 128 x 64 sites) split over the N GPUs;
      on one GPU the gates are streamed in chunks of owner rows, so no per-edge table wider than 64 floats
      exists whole.
  --scaling weak: 131,072 atoms per GPU (64 x 64 x 32 sites per brick; 8 GPUs = the same 1,048,576-atom box).
With N > 1 (torchrun) the box is split into N bricks: distributed state, NCCL halo exchanges, the step recorded
as one CUDA graph.

At N = 1 the line also carries the other BASELINE configurations as extra keys, each measured in this run:
``tp_edges_per_s`` (configuration 2, fused tensor product + scatter, forward + adjoint, 65,536 atoms),
``sc_nodes_per_s`` (configuration 3, symmetric contraction forward + feature gradient, 262,144 nodes),
``train_atom_steps_per_s`` (configuration 4, force-loss training step, 32,768 atoms), ``parity`` (GPU against the
float64 CPU oracle on a small periodic sample) and ``cpu_baseline``.  At N > 1 it carries ``parity_multi_gpu``:
a small system evaluated decomposed over the N ranks against rank 0 alone.

Workloads ``fused_message``, ``sc`` and ``train`` print their own line for the single configuration.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "ictc-o3-hp-k100_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")

import numpy as np  # noqa: E402
import torch  # noqa: E402

CHANNELS, LMAX, NUM_ATOMS, DENSITY, CUTOFF = 64, 2, 65536, 0.1, 4.5
NX, NH, NP, NO = 9, 9, 11, 35
SC_NODES = 262144


def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        return float(json.load(open(path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback"


def algorithmic_bytes(n, e, c=CHANNELS):
    """Bytes that one launch must move when every operand crosses HBM exactly once."""
    fwd = 4 * (n * NX * c + e * NH + e * NP * c + n * NO * c) + 16 * e
    bwd = 4 * (n * NX * c + e * NH + e * NP * c + n * NO * c) + 16 * e + 4 * (n * NX * c + e * NH + e * NP * c)
    return fwd, bwd


def make_system(seed, num_atoms=NUM_ATOMS):
    from mace_ictc import synthetic as S
    pos, box = S.uniform_box(num_atoms, DENSITY, seed)
    src, dst, shifts = S.neighbor_list_host(pos, box, CUTOFF)
    return pos, box, src, dst, shifts


def make_inputs(seed, device, num_atoms=NUM_ATOMS, dtype=torch.float32):
    """Inputs of the fused message on ``device`` (torch ops only; untimed set-up)."""
    from mace_ictc import synthetic as S
    pos, box, src, dst, shifts = make_system(seed, num_atoms)
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(num_atoms, NX * CHANNELS, generator=gen).to(device=device, dtype=dtype)
    p = torch.as_tensor(pos, dtype=torch.float64)
    vec = p[dst] - p[src] + torch.as_tensor(shifts * box, dtype=torch.float64)
    r = vec.norm(dim=-1)
    unit = (vec / r.unsqueeze(-1)).to(device=device, dtype=dtype)
    r = r.to(device=device, dtype=dtype)
    weights = S.random_radial_mlp([8, 64, 64, 64, NP * CHANNELS], seed + 1, device)
    weights = [w.to(dtype) for w in weights]
    gates = torch.cat([S.radial_gates(S.bessel_basis(rr, CUTOFF), weights) for rr in r.split(262144)], 0)
    v = torch.randn(num_atoms, NO * CHANNELS, generator=gen).to(device=device, dtype=dtype)
    return {"x": x, "unit": unit, "gates": gates.contiguous(), "v": v,
            "src": torch.as_tensor(src, device=device), "dst": torch.as_tensor(dst, device=device)}


# ------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """SM clock and throttle reasons of one GPU, read through NVML inside the benchmark's own process (a light
    thread, at most one reading per ``period`` seconds).  A separate sampling process or an nvidia-smi loop slows an
    eager multi-GPU step by tens of per cent on these hosts; two in-process queries per reading do not."""

    def __init__(self, gpu_index, period=0.25):
        self.rows, self.period, self.last, self.active = [], period, 0.0, False
        self.nvml = self.handle = None
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        gpu = int(visible.split(",")[gpu_index]) if visible and visible.replace(",", "").isdigit() else gpu_index
        try:
            import pynvml as N
            N.nvmlInit()
            self.nvml, self.handle = N, N.nvmlDeviceGetHandleByIndex(gpu)
            self.max = float(N.nvmlDeviceGetMaxClockInfo(self.handle, N.NVML_CLOCK_SM))
            self.masks = {"hw_slowdown": N.nvmlClocksThrottleReasonHwSlowdown,
                          "hw_thermal_slowdown": N.nvmlClocksThrottleReasonHwThermalSlowdown,
                          "sw_thermal_slowdown": N.nvmlClocksThrottleReasonSwThermalSlowdown,
                          "sw_power_cap": N.nvmlClocksThrottleReasonSwPowerCap}
        except Exception:       # noqa: BLE001 - no NVML on this box: the bench line says so
            self.nvml = None

    def start(self):
        """Sample from a daemon thread of this process every ``period`` seconds until ``stop`` (a recorded step is
        queued in milliseconds, so the host thread would otherwise see the GPU only before and after the region)."""
        import threading
        self.active, self.last = True, 0.0

        def loop():
            while self.active:
                self.tick()
                time.sleep(self.period)
        self.thread = threading.Thread(target=loop, daemon=True)
        self.thread.start()

    def tick(self):
        """One reading (rate limited); also called between steps of the timed region."""
        if not self.active or self.nvml is None:
            return
        now = time.perf_counter()
        if now - self.last < 0.8 * self.period:
            return
        self.last = now
        try:
            sm = self.nvml.nvmlDeviceGetClockInfo(self.handle, self.nvml.NVML_CLOCK_SM)
            r = self.nvml.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
            self.rows.append((float(sm), [k for k, b in self.masks.items() if r & b]))
        except Exception:       # noqa: BLE001
            pass

    def stop(self):
        self.active = False
        if self.nvml is None or not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["sampler unavailable"]}
        reasons = sorted({x for _, rs in self.rows for x in rs})
        return {"sm_mhz": float(np.median([sm for sm, _ in self.rows])), "sm_max_mhz": self.max, "reasons": reasons,
                "samples": len(self.rows)}


def wait_and_sample(event, sampler):
    """The launches are queued; the host polls for completion and reads the clocks meanwhile."""
    while not event.query():
        sampler.tick()
        time.sleep(0.02)


# ------------------------------------------------------------------------------------ CPU arms (oracle port)
def cpu_fused_message_step_factory(seed, sample_atoms):
    """The oracle's restatement of the reference torch path (fp32, all host threads) on a bounded
    sample: the first ``sample_atoms`` receivers of the workload and all their in-edges."""
    from oracle import ictc_oracle as O
    inp = make_inputs(seed, "cpu")
    rowend = int(torch.searchsorted(inp["dst"], torch.tensor(sample_atoms)))
    src, dst = inp["src"][:rowend], inp["dst"][:rowend]
    paths = O.natural_paths(LMAX, LMAX, LMAX)
    tp = O.TensorProduct(CHANNELS, LMAX, paths, dtype=torch.float32)
    w = torch.ones(NP, CHANNELS)
    x = inp["x"].clone().requires_grad_(True)
    unit = inp["unit"][:rowend].clone().requires_grad_(True)
    g = inp["gates"][:rowend].reshape(rowend, NP, CHANNELS).clone().requires_grad_(True)
    v = inp["v"]

    def step():
        sh = torch.cat(O.direction_harmonics(unit, LMAX), -1)
        out = O.graph_message(tp, x, sh, g, w, src, dst, None, LMAX, LMAX)
        torch.autograd.grad(out, [x, unit, g], v)
        return rowend

    return step, rowend


def run_cpu_fused_message(seed, steps, warmup, sample_atoms):
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    step, edges = cpu_fused_message_step_factory(seed, sample_atoms)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return {"value": edges / dt, "unit": "edges/s", "cores": threads, "kind": "port",
            "sample": f"first {sample_atoms} receivers of the workload with all their in-edges ({edges} edges), "
                      f"fp32 torch CPU, forward + adjoint, {steps} timed steps",
            "ms_per_step": dt * 1e3}


MD_BRICK = (64, 64, 32)          # lattice sites per GPU of the weak series
MD_STRONG = (128, 128, 64)       # lattice sites of the strong series: 1,048,576 atoms
MD_SPACING, MD_SIGMA, MD_CUTOFF, MD_DT, MD_T = 2.15, 0.1, 4.5, 1.0, 300.0


def md_lattice_dims(world):
    dims = list(MD_BRICK)
    n = world
    while n > 1:                      # double the currently shortest box edge, so bricks stay 64x64x32
        axis = min(range(3), key=lambda a: dims[a])
        dims[axis] *= 2
        n //= 2
    return tuple(dims)


def md_oracle(side, dtype):
    """(oracle model, inputs) of a side^3-atom periodic sample of the benchmark lattice and model."""
    from mace_ictc import synthetic as S
    from mace_ictc.model import MaceIctcModel
    from oracle.model_oracle import ModelOracle
    torch.manual_seed(0)
    pos, box, species = S.jittered_lattice(side, side, side, MD_SPACING, MD_SIGMA, 0)
    z = np.array([1, 6, 8])[species]
    weights = MaceIctcModel(channels=CHANNELS, cutoff=MD_CUTOFF, avg_num_neighbors=32.0).state_dict()
    oracle = ModelOracle(weights, channels=CHANNELS, lmax=2, num_interactions=2, correlation=3,
                         atomic_numbers=(1, 6, 8), cutoff=MD_CUTOFF, avg_num_neighbors=32.0, dtype=dtype)
    return oracle, weights, pos, box, z


def run_cpu_md(steps, warmup, side):
    """The oracle model (fp32, all host threads): neighbour list, energy and forces of a side^3-atom periodic
    sample of the same lattice, per step."""
    from mace_ictc import synthetic as S
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    oracle, _w, pos, box, z = md_oracle(side, torch.float32)
    p, zt = torch.as_tensor(pos), torch.as_tensor(z)
    batch = torch.zeros(p.shape[0], dtype=torch.long)
    cell = torch.as_tensor(np.diag(box)).float().unsqueeze(0)

    def step():
        src, dst, shifts = S.neighbor_list_host(pos, box, MD_CUTOFF)
        oracle.energy_and_forces(p, zt, batch, torch.as_tensor(src), torch.as_tensor(dst), torch.as_tensor(shifts), cell)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    atoms = p.shape[0]
    return {"value": atoms / dt, "unit": "atom-steps/s", "cores": threads, "kind": "port",
            "sample": f"{atoms}-atom periodic sample ({side}^3 sites) of the same lattice and model, fp32 torch CPU, "
                      f"neighbour list + energy + forces per step, {steps} timed steps",
            "ms_per_step": dt * 1e3, "sample_atoms": atoms}


def parity_against_oracle(dev, side=10):
    """GPU (float32, force engine) against the float64 CPU oracle on a side^3-atom periodic sample of the benchmark
    lattice with identical weights: relative error of forces (max |d| / max |ref|) and of the energy."""
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model
    from mace_ictc.md import MolecularDynamics
    oracle, weights, pos, box, z = md_oracle(side, torch.float64)
    src, dst, shifts = S.neighbor_list_host(pos, box, MD_CUTOFF)
    n = pos.shape[0]
    ref = oracle.energy_and_forces(torch.as_tensor(pos), torch.as_tensor(z), torch.zeros(n, dtype=torch.long),
                                   torch.as_tensor(src), torch.as_tensor(dst), torch.as_tensor(shifts),
                                   torch.as_tensor(np.diag(box)).unsqueeze(0))
    model = create_model(channels=CHANNELS, lmax=2, num_interactions=2, correlation=3, cutoff=MD_CUTOFF,
                         atomic_numbers=(1, 6, 8), avg_num_neighbors=32.0, device=dev)
    model.load_state_dict(weights)
    md = MolecularDynamics(model, pos, z, box, dt=MD_DT, seed=1)
    f = md.gather(md.compute_forces()).double().cpu()
    rf = ref["forces"].detach()
    return {"forces_rel": float((f - rf).abs().max() / rf.abs().max()),
            "energy_rel": abs(float(md.energy) - float(ref["energy"])) / abs(float(ref["energy"])),
            "atoms": n, "edges": md.num_edges, "oracle": "float64 CPU restatement pinned on the reference's own model",
            "tolerance": 1e-5}


def parity_multi_gpu(model, dev, rank, world):
    """A small fixed system evaluated decomposed over the ranks and on rank 0 alone: max force error / max force,
    relative energy error (every rank computes the single-GPU value itself, so no rank idles in a collective)."""
    from mace_ictc import synthetic as S
    from mace_ictc.md import MolecularDynamics
    pos, box, species = S.jittered_lattice(24, 20, 16, MD_SPACING, MD_SIGMA, 17)
    z = np.array([1, 6, 8])[species]
    single = MolecularDynamics(model, pos, z, box, dt=MD_DT, seed=2)
    f_ref = single.gather(single.compute_forces())
    e_ref = float(single.energy)
    multi = MolecularDynamics(model, pos, z, box, dt=MD_DT, seed=2, distributed=True)
    f = multi.gather(multi.compute_forces())
    out = {"forces_rel": float((f - f_ref).abs().max() / f_ref.abs().max()),
           "energy_rel": abs(float(multi.energy) - e_ref) / abs(e_ref), "atoms": int(pos.shape[0]),
           "ranks": world, "tolerance": 2e-5}
    multi.close()
    del single, multi
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------ fused message (configuration 2)
def measure_fused_message(dev, atoms, steps, warmup, seed, sampler=None, e2e=True):
    from ictc_o3 import PackedGraphMessage, direction_harmonics
    from ictc_o3.ops import tensor_product as tpmod
    inp = make_inputs(seed, dev, atoms)
    n, e = atoms, int(inp["src"].numel())
    op = PackedGraphMessage.create(channels=CHANNELS, input_lmax=LMAX, edge_lmax=LMAX, output_lmax=LMAX, device=dev)
    sh = torch.cat(direction_harmonics(inp["unit"], LMAX), -1).contiguous()
    x = inp["x"].requires_grad_(True)
    shg = sh.requires_grad_(True)
    g = inp["gates"].requires_grad_(True)
    src, dst, v = inp["src"], inp["dst"], inp["v"]

    def step():
        out = op(x, shg, g, src, dst)
        return torch.autograd.grad(out, [x, shg, g], v)

    for _ in range(max(3, warmup)):
        step()
    tpmod.PROFILE = []
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
        if sampler is not None:
            sampler.tick()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    profile, tpmod.PROFILE = tpmod.PROFILE, None
    kern = {}
    for name, a, b in profile:
        kern.setdefault(name, []).append(a.elapsed_time(b))
    kern_ms = {k: float(np.mean(vv)) for k, vv in kern.items()}
    res = {"ms": ms, "edges": e, "launches": len(profile), "kernels_ms": kern_ms, "e2e": None}
    if e2e:
        import psutil
        host = {k: t.detach() for k, t in (("x", x), ("sh", sh), ("g", g), ("v", v), ("src", src), ("dst", dst))}
        need = sum(t.numel() * t.element_size() for t in host.values()) * 2.2
        if psutil.virtual_memory().available > need * 1.5:
            pin = {k: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for k, t in host.items()}
            outs = None

            def e2e_step():
                nonlocal outs
                d = {k: t.to(dev, non_blocking=True) for k, t in pin.items()}
                xs, ss, gs = (d[k].requires_grad_(True) for k in ("x", "sh", "g"))
                out = op(xs, ss, gs, d["src"], d["dst"])
                grads = torch.autograd.grad(out, [xs, ss, gs], d["v"])
                got = (out.detach(),) + grads
                if outs is None:
                    outs = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in got]
                for o, t in zip(outs, got):
                    o.copy_(t, non_blocking=True)

            e2e_steps = max(1, min(steps, 5))
            for _ in range(2):
                e2e_step()
            torch.cuda.synchronize()
            s2, t2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s2.record()
            for _ in range(e2e_steps):
                e2e_step()
            t2.record()
            torch.cuda.synchronize()
            res["e2e"] = [s2.elapsed_time(t2) / e2e_steps, sum(t.numel() * t.element_size() for t in pin.values()),
                          sum(t.numel() * t.element_size() for t in outs), e2e_steps]
            del pin, outs
    peak, peak_src = hbm_peak()
    fwd_b, bwd_b = algorithmic_bytes(n, e)
    dom = max(kern_ms, key=kern_ms.get) if kern_ms else None
    dom_bytes = {"graph_forward": fwd_b, "graph_adjoint": bwd_b}.get(dom, 0)
    achieved = dom_bytes / (kern_ms[dom] * 1e-3) / 1e9 if dom else None
    res["roofline"] = {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
                       "frac": achieved / peak if achieved else None, "peak_source": peak_src,
                       "algorithmic_bytes_per_launch": dom_bytes, "traffic": None}
    return res


# ------------------------------------------------------------------------------------ symmetric contraction (configuration 3)
def measure_sc(dev, nodes, steps, warmup, sampler=None):
    """Symmetric contraction, correlation 3, C64, lmax 2, 4 species: forward plus gradient with respect to the
    features.  FP32-pipe bound: reports multiply-adds per second beside the HBM fraction."""
    from ictc_o3 import create_symmetric_contraction
    from ictc_o3 import tables
    torch.manual_seed(3)
    sc = create_symmetric_contraction(num_elements=4, lmax=2, target_lmax=2, channels=CHANNELS, device=dev)
    x = torch.randn(nodes, 9 * CHANNELS, device=dev).requires_grad_(True)
    species = torch.randint(0, 4, (nodes,), device=dev)
    cot = torch.randn(nodes, 9 * CHANNELS, device=dev)

    def step():
        y = sc(x, None, species)
        return torch.autograd.grad(y, x, cot)

    for _ in range(max(3, warmup)):
        step()
    torch.cuda.synchronize()
    marks = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    fwd_ms = bwd_ms = 0.0
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
        if sampler is not None:
            sampler.tick()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    with torch.no_grad():                              # the forward kernel alone, for its roofline
        marks[0].record()
        for _ in range(steps):
            sc(x, None, species)
        marks[1].record()
    torch.cuda.synchronize()
    fwd_ms = marks[0].elapsed_time(marks[1]) / steps
    bwd_ms = ms - fwd_ms
    # non-zero couplings of the U tensors: one multiply-add each per (node, channel) in the forward polynomial
    nnz = sum(int(np.count_nonzero(tables.sc_u_tensor(l, nu))) for l in range(3) for nu in (1, 2, 3))
    peak, peak_src = hbm_peak()
    bytes_fwd = 8 * nodes * 9 * CHANNELS + 8 * nodes
    return {"ms": ms, "nodes": nodes, "forward_ms": fwd_ms, "adjoint_ms": bwd_ms,
            "roofline": {"bound": "fp32 pipe", "kernel": "sc_node_kernel (forward)", "u_nonzeros": nnz,
                         "coupling_fma_per_s": nnz * nodes * CHANNELS / (fwd_ms * 1e-3),
                         "hbm": {"achieved": bytes_fwd / (fwd_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                                 "frac": bytes_fwd / (fwd_ms * 1e-3) / 1e9 / peak, "peak_source": peak_src,
                                 "algorithmic_bytes_per_launch": bytes_fwd}}}


# ------------------------------------------------------------------------------------ training step (configuration 4)
def measure_train(dev, side, steps, warmup, seed, sampler=None):
    """Energy-and-force training step: forces with create_graph, force loss whose gradient needs the mixed second
    derivatives, AdamW; side^3-atom jittered lattice, neighbour list built once (the reference's protocol)."""
    from ictc_o3 import _lib
    from mace_ictc import synthetic as S
    from mace_ictc.hp import configure_model, create_model, energy_and_forces
    from mace_ictc.md import neighbor_list
    n_atoms = side ** 3
    pos, box, species = S.jittered_lattice(side, side, side, MD_SPACING, MD_SIGMA, seed)
    z = np.array([1, 6, 8])[species]
    torch.manual_seed(0)
    model = create_model(channels=CHANNELS, lmax=2, num_interactions=2, correlation=3, cutoff=MD_CUTOFF,
                         atomic_numbers=(1, 6, 8), avg_num_neighbors=32.0, device=dev)
    configure_model(model, policy="generated")
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
    p = torch.as_tensor(pos, dtype=torch.float32, device=dev)
    src, dst, shifts, _ = neighbor_list(p, n_atoms, [0, 0, 0], list(box), list(box), (1, 1, 1), MD_CUTOFF)
    zt = torch.as_tensor(z, device=dev)
    batch = torch.zeros(n_atoms, dtype=torch.long, device=dev)
    cell = torch.as_tensor(np.diag(box), dtype=torch.float32, device=dev).unsqueeze(0)
    target = torch.randn(n_atoms, 3, device=dev) * 0.05
    host_pos = torch.empty(n_atoms, 3, pin_memory=True).copy_(p)
    host_target = torch.empty(n_atoms, 3, pin_memory=True).copy_(target)
    host_loss = torch.empty(1, pin_memory=True)

    def step(from_host=False):
        if from_host:
            p.copy_(host_pos, non_blocking=True)
            target.copy_(host_target, non_blocking=True)
        opt.zero_grad(set_to_none=True)
        res = energy_and_forces(model, p, zt, batch, src, dst, shifts, cell, training=True)
        loss = (res["energy"] / n_atoms).square().mean() + (res["forces"] - target).square().mean()
        loss.backward()
        opt.step()
        if from_host:
            host_loss.copy_(loss.detach().reshape(1), non_blocking=True)
            torch.cuda.synchronize()

    for _ in range(max(3, warmup)):
        step()
    calls0 = _lib.CALLS
    step()
    torch.cuda.synchronize()
    calls_per_step = _lib.CALLS - calls0
    torch.cuda.reset_peak_memory_stats()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        step()
        if sampler is not None:
            sampler.tick()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    e2e_steps = max(3, min(steps, 10))
    start.record()
    for _ in range(e2e_steps):
        step(True)
    stop.record()
    torch.cuda.synchronize()
    return {"ms": ms, "atoms": n_atoms, "edges": int(src.numel()), "calls_per_step": calls_per_step,
            "e2e_ms": start.elapsed_time(stop) / e2e_steps, "e2e_steps": e2e_steps,
            "peak_memory_gib": torch.cuda.max_memory_allocated() / 2 ** 30}


# ------------------------------------------------------------------------------------ MD workload
def main_md(args, rank, world, local):
    global MD_BRICK
    if args.md_brick:
        MD_BRICK = tuple(int(v) for v in args.md_brick.lower().split("x"))
    if args.scaling == "strong":
        dims = tuple(int(v) for v in args.strong_lattice.lower().split("x")) if args.strong_lattice else MD_STRONG
    else:
        dims = md_lattice_dims(world)
    atoms_total = dims[0] * dims[1] * dims[2]
    per_gpu = atoms_total // world
    chunk_rows = args.chunk_rows if args.chunk_rows >= 0 else (65536 if per_gpu > 300000 else 0)
    workload = {"workload": f"md: NVE velocity-Verlet, C{CHANNELS}/lmax2/2 interactions/corr3 random-init, jittered "
                            f"H/C/O lattice {dims[0]}x{dims[1]}x{dims[2]} = {atoms_total} atoms "
                            f"({per_gpu} per GPU), cutoff {MD_CUTOFF} A, dt {MD_DT} fs, "
                            f"{MD_T} K, edge list rebuilt every step",
                "l2": "per-edge tensors (GBs per layer) are far larger than L2", "atoms_per_gpu": per_gpu,
                "series": args.scaling}
    if args.impl == "reference":
        if rank != 0:
            return
        steps, warmup = max(1, min(args.steps, 3)), 1
        res = run_cpu_md(steps, warmup, args.cpu_md_side)
        line = {"impl": "reference", "metric": "MD atom-steps/s", "value": res["value"], "unit": "atom-steps/s",
                "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": dict(workload, cpu_sample_atoms=res["sample_atoms"]),
                "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": res["value"], "unit": "atom-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        if world > 2 and args.capture_collectives != "no":
            # recorded collectives on more than two ranks need the collective library without in-switch reduction and
            # without buffer registration at capture time (the replay never completed with the defaults); plain ring /
            # peer-copy kernels are all the small exchanges of this step need
            os.environ["NCCL_NVLS_ENABLE"] = "0"
            os.environ["NCCL_GRAPH_REGISTER"] = "0"
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from ictc_o3 import _lib
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model
    from mace_ictc.md import MolecularDynamics
    torch.manual_seed(0)
    model = create_model(channels=CHANNELS, lmax=2, num_interactions=2, correlation=3, cutoff=MD_CUTOFF,
                         atomic_numbers=(1, 6, 8), avg_num_neighbors=32.0, device=dev)
    if world > 1:
        for p in model.parameters():
            dist.broadcast(p.data, 0)
    par_multi = parity_multi_gpu(model, dev, rank, world) if (world > 1 and not args.no_parity) else None
    pos, box, species = S.jittered_lattice(*dims, MD_SPACING, MD_SIGMA, 0)
    z = np.array([1, 6, 8])[species]
    md = MolecularDynamics(model, pos, z, box, dt=MD_DT, temperature=MD_T, seed=1, distributed=world > 1,
                           skin=args.skin, chunk_rows=chunk_rows or None, sort_atoms=not args.no_sort,
                           stream_gates={"auto": None, "yes": True, "no": False}[args.stream_gates],
                           capture_collectives={"auto": None, "yes": True, "no": False}[args.capture_collectives])
    del pos, species
    warm = max(3, args.warmup)
    md.compute_forces()
    md.run(warm)
    # per-kernel CUDA-event timings and the launch count come from eager steps (events cannot be read
    # inside a replayed graph); the timed region below replays the recorded step
    md.engine.profile = []
    calls0 = _lib.CALLS
    probe_steps = 2
    md.run(probe_steps)
    torch.cuda.synchronize()
    calls_per_step = (_lib.CALLS - calls0) // probe_steps
    profile, md.engine.profile = md.engine.profile, None
    kern = {}
    for name, a, b in profile:
        kern.setdefault(name, []).append(a.elapsed_time(b))
    kern_ms = {k: float(np.sum(v)) / probe_steps for k, v in kern.items()}          # per step (chunks summed)
    kern_launches = {k: len(v) // probe_steps for k, v in kern.items()}
    del profile, kern
    graph_cap = None
    if not args.no_graph:
        graph_cap = md.enable_graph()
        md.run(2)
    if world > 1:
        md.redecompose()          # one refresh before the timed region: the first one pays one-time set-up costs
        md._dist["since_refresh"] = 0
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    rebuilds0 = md.graph_rebuilds
    md.events.clear()
    start.record()
    md.run(args.steps, on_step=sampler.tick)
    stop.record()
    wait_and_sample(stop, sampler)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = start.elapsed_time(stop) / args.steps
    run_events = [(k, n, round(t * 1e3, 2)) for k, n, t in md.events]
    calls = calls_per_step * args.steps
    peak_mem = torch.cuda.max_memory_reserved() / 2 ** 30       # whole run so far: set-up, eager steps, recorded step
    if md.world == 1:
        nl = md._static["nl"] if md._static is not None else None
        edges = int(nl.rowptr[-1].item()) if nl is not None else md.num_edges
        gate_rows = int(nl.num_unique.item()) if nl is not None else md.num_gate_rows
    else:
        nl = md._dist["nl"]
        edges, gate_rows = int(nl.rowptr[-1].item()), int(nl.num_unique.item())

    # end to end: the caller owns the coordinates on the host: they go in every step, the step runs, and forces,
    # energy and the new coordinates come back
    e2e = None
    if not args.no_e2e:
        n = md.pos.shape[0]
        host_pos = torch.empty(n, 3, pin_memory=True).copy_(md.pos)
        host_f = torch.empty(n, 3, pin_memory=True)
        host_e = torch.empty(1, pin_memory=True)

        def e2e_step():
            nonlocal host_pos, host_f
            if host_pos.shape[0] != md.pos.shape[0]:       # the decomposed run re-sized its per-atom arrays
                host_pos = torch.empty(md.pos.shape[0], 3, pin_memory=True).copy_(md.pos)
                host_f = torch.empty(md.pos.shape[0], 3, pin_memory=True)
            md.pos.copy_(host_pos, non_blocking=True)
            md.run(1)
            if host_pos.shape[0] != md.pos.shape[0]:
                return
            host_f.copy_(md.forces, non_blocking=True)
            host_e.copy_(md.energy.reshape(1), non_blocking=True)
            host_pos.copy_(md.pos, non_blocking=True)

        e2e_steps = max(1, min(args.steps, 10))
        for _ in range(2):
            e2e_step()
        barrier()
        s2, t2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        for _ in range(e2e_steps):
            e2e_step()
        t2.record()
        barrier()
        e2e = [s2.elapsed_time(t2) / e2e_steps, n * 12, n * 12 + 4 + n * 12, e2e_steps]
    streamed = bool(chunk_rows) and md.engine._streaming(gate_rows)
    status = _lib.kernel_status()
    if world > 1:
        t = torch.tensor([ms, e2e[0] if e2e else 0.0, float(edges), peak_mem], device=dev, dtype=torch.float64)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t)
        ms, peak_mem = float(tmax[0]), float(tmax[3])
        if e2e:
            e2e[0] = float(tmax[1])
        total_edges = float(t[2])
    else:
        total_edges = float(edges)
    if rank == 0:
        peak, peak_src = hbm_peak()
        n_local = md.pos.shape[0] if world == 1 else md._dist["n_local"]
        # layer-1 adjoint, every operand once: reads x, sh, the gates (one row per edge PAIR when the pair table is
        # kept whole, one per edge when streamed in chunks), cotangent rows, indices (edge id, neighbour, gate
        # row); writes dx, dsh and the per-edge gate gradient
        g_rows = edges if streamed else gate_rows
        bwd_b = (4 * (n_local * NX * CHANNELS + edges * NH + g_rows * NP * CHANNELS + per_gpu * NO * CHANNELS)
                 + 24 * edges + 4 * (n_local * NX * CHANNELS + edges * NH + edges * NP * CHANNELS))
        adj_ms = kern_ms.get("graph_adjoint_l1")
        achieved = bwd_b / (adj_ms * 1e-3) / 1e9 if adj_ms else None
        line = {"metric": "MD atom-steps/s", "value": atoms_total / (ms * 1e-3), "unit": "atom-steps/s",
                "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True,
                "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": dict(workload, edges_total=total_edges, edges_per_atom=total_edges / atoms_total,
                               step_replayed_as_cuda_graph=md.graph is not None, edge_capacity=graph_cap,
                               atoms_sorted_along_morton_curve=not args.no_sort, gate_chunk_rows=chunk_rows or None, gates_streamed=streamed, skin=args.skin if world > 1 else None,
                               timed_region_events_ms=run_events, ghost_refreshes=md.refreshes, refresh_seconds_total=md.refresh_seconds, refresh_period_steps=md.block, redecompositions=md.redecompositions,
                               graph_rebuilds_in_timed_region=md.graph_rebuilds - rebuilds0,
                               kernels_ms_from=f"{probe_steps} eager steps before the timed region (per step, "
                                               "chunk launches summed)"),
                "gpu_launches": calls, "kernel_status": status, "clocks": clocks, "peak_memory_gib": peak_mem,
                "kernels_ms": kern_ms, "kernel_launches_per_step": kern_launches,
                "roofline": {"bound": "hbm", "kernel": "tp_adjoint_tma_kernel (layer-1 graph adjoint: dx, dsh, dg)",
                             "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak if achieved else None, "peak_source": peak_src,
                             "algorithmic_bytes_per_launch": bwd_b / max(1, kern_launches.get("graph_adjoint_l1", 1)),
                             "launches_per_step": kern_launches.get("graph_adjoint_l1", 1),
                             "traffic": TRAFFIC_PER_EDGE * edges / max(1, kern_launches.get("graph_adjoint_l1", 1)),
                             "traffic_source": TRAFFIC_SOURCE},
                "e2e": ({"value": atoms_total / (e2e[0] * 1e-3), "unit": "atom-steps/s", "h2d_bytes_per_step": e2e[1],
                         "d2h_bytes_per_step": e2e[2], "ms_per_step": e2e[0], "steps": e2e[3]} if e2e else None)}
        if par_multi is not None:
            line["parity_multi_gpu"] = par_multi
    md.close()
    del md
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_extras:
        line["parity"] = parity_against_oracle(dev)
        torch.cuda.empty_cache()
        fm = measure_fused_message(dev, NUM_ATOMS, 5, 3, 1000, e2e=False)
        line["tp_edges_per_s"] = {"value": fm["edges"] / (fm["ms"] * 1e-3), "unit": "edges/s", "ms_per_step": fm["ms"],
                                  "edges": fm["edges"], "atoms": NUM_ATOMS, "step": "forward + adjoint(dx,dsh,dg)",
                                  "kernels_ms": fm["kernels_ms"], "roofline": fm["roofline"]}
        del fm
        torch.cuda.empty_cache()
        sc = measure_sc(dev, SC_NODES, 10, 3)
        line["sc_nodes_per_s"] = {"value": sc["nodes"] / (sc["ms"] * 1e-3), "unit": "nodes/s", "ms_per_step": sc["ms"],
                                  "nodes": sc["nodes"], "step": "forward + feature gradient",
                                  "forward_ms": sc["forward_ms"], "adjoint_ms": sc["adjoint_ms"],
                                  "roofline": sc["roofline"]}
        torch.cuda.empty_cache()
        tr = measure_train(dev, 32, 5, 3, 0)
        line["train_atom_steps_per_s"] = {"value": tr["atoms"] / (tr["ms"] * 1e-3), "unit": "atom-steps/s",
                                          "ms_per_step": tr["ms"], "atoms": tr["atoms"],
                                          "peak_memory_gib": tr["peak_memory_gib"],
                                          "step": "E+F with create_graph, force loss, backward, AdamW"}
        torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        res = run_cpu_md(2, 1, args.cpu_md_side)
        line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes per edge of one layer-1 adjoint launch, measured by ncu (dram__bytes_read.sum + dram__bytes_write.sum)
# on the 32,768-atom case; traffic grows in proportion to the edge count at fixed density
TRAFFIC_PER_EDGE = 6235.0
TRAFFIC_SOURCE = "ncu on 32768 atoms, scaled by edges"


# ------------------------------------------------------------------------------------ single-configuration lines
def setup_single(local, world):
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    return dev


def reduce_max(values, dev, world):
    t = torch.tensor(values, device=dev, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(v) for v in t]


def main_train(args, rank, world, local):
    """BASELINE configuration 4 on every GPU (independent replicas: no collective)."""
    side = args.train_side
    workload = {"workload": f"train: energy+force loss step (mixed second derivatives, AdamW), C{CHANNELS}/lmax2/2 "
                            f"interactions/corr3 random-init, jittered H/C/O lattice {side}^3 = {side ** 3} atoms per GPU, "
                            f"cutoff {MD_CUTOFF} A, neighbour list built once (as in the reference's protocol)",
                "l2": "edge tensors (gates 3 GB per layer) are larger than L2", "atoms_per_gpu": side ** 3}
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the CPU port times the MD step only; use --workload md"}))
        return
    dev = setup_single(local, world)
    from ictc_o3 import _lib
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    tr = measure_train(dev, side, args.steps, args.warmup, rank, sampler)
    clocks = sampler.stop() if rank == 0 else None
    ms, e2e_ms = reduce_max([tr["ms"], tr["e2e_ms"]], dev, world)
    status = _lib.kernel_status()
    if rank == 0:
        total = tr["atoms"] * world
        print(json.dumps({
            "metric": "training atom-steps/s", "value": total / (ms * 1e-3), "unit": "atom-steps/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(workload, edges_per_gpu=tr["edges"], parallelism="independent replicas"),
            "gpu_launches": tr["calls_per_step"] * args.steps, "kernel_status": status, "clocks": clocks,
            "peak_memory_gib": tr["peak_memory_gib"],
            "e2e": {"value": total / (e2e_ms * 1e-3), "unit": "atom-steps/s", "h2d_bytes_per_step": 24 * tr["atoms"],
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms, "steps": tr["e2e_steps"]}}))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def main_sc(args, rank, world, local):
    """BASELINE configuration 3 on every GPU (independent replicas)."""
    workload = {"workload": f"sc: symmetric contraction corr 3, C{CHANNELS}, lmax 2, 4 species, {args.nodes} nodes per GPU, "
                            "forward + feature gradient", "l2": "features in + out are 1.2 GB, larger than L2"}
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the CPU port times the MD step only; use --workload md"}))
        return
    dev = setup_single(local, world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sc = measure_sc(dev, args.nodes, args.steps, args.warmup, sampler)
    clocks = sampler.stop() if rank == 0 else None
    (ms,) = reduce_max([sc["ms"]], dev, world)
    if rank == 0:
        print(json.dumps({"metric": "SC nodes/s", "value": sc["nodes"] * world / (ms * 1e-3), "unit": "nodes/s",
                          "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                          "data": "synthetic", "config": workload, "gpu_launches": 2 * args.steps, "clocks": clocks,
                          "forward_ms": sc["forward_ms"], "adjoint_ms": sc["adjoint_ms"], "roofline": sc["roofline"],
                          "e2e": None}))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def main_fused_message(args, rank, world, local):
    workload = {"workload": f"fused_message: TP+scatter forward+adjoint, fp32, C{CHANNELS}, lmax {LMAX}, "
                            f"{args.atoms} atoms/GPU uniform density {DENSITY}, cutoff {CUTOFF}",
                "l2": "inputs larger than L2 (gates alone are 7 GB)", "atoms_per_gpu": args.atoms}
    if args.impl == "reference":
        if rank != 0:
            return
        steps, warmup = max(1, min(args.steps, 3)), max(1, min(args.warmup, 1))
        res = run_cpu_fused_message(0, steps, warmup, args.cpu_sample_atoms)
        print(json.dumps({"impl": "reference", "metric": "TP edges/s", "value": res["value"], "unit": "edges/s",
                          "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": res["ms_per_step"],
                          "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                          "data": "synthetic", "config": workload,
                          "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
                          "e2e": {"value": res["value"], "unit": "edges/s", "h2d_bytes_per_step": 0,
                                  "d2h_bytes_per_step": 0}, "gpu_launches": 0}))
        return
    dev = setup_single(local, world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    fm = measure_fused_message(dev, args.atoms, args.steps, args.warmup, 1000 + rank, sampler, e2e=not args.no_e2e)
    clocks = sampler.stop() if rank == 0 else None
    ms, e2e_ms = reduce_max([fm["ms"], fm["e2e"][0] if fm["e2e"] else 0.0], dev, world)
    tot = torch.tensor([fm["edges"]], device=dev, dtype=torch.float64)
    if world > 1:
        import torch.distributed as dist
        dist.all_reduce(tot)
    total_edges = float(tot[0])
    if rank == 0:
        line = {"metric": "TP edges/s", "value": total_edges / (ms * 1e-3), "unit": "edges/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": dict(workload, edges_per_gpu=fm["edges"], step="forward + adjoint(dx,dsh,dg)"),
                "gpu_launches": fm["launches"], "clocks": clocks, "kernels_ms": fm["kernels_ms"],
                "roofline": fm["roofline"],
                "e2e": ({"value": total_edges / (e2e_ms * 1e-3), "unit": "edges/s", "h2d_bytes_per_step": fm["e2e"][1],
                         "d2h_bytes_per_step": fm["e2e"][2], "ms_per_step": e2e_ms, "steps": fm["e2e"][3]}
                        if fm["e2e"] else None)}
        if world == 1 and not args.no_cpu_baseline:
            res = run_cpu_fused_message(1000, 2, 1, args.cpu_sample_atoms)
            line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="md", choices=["md", "fused_message", "sc", "train"])
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"],
                    help="md workload: strong = one 1,048,576-atom system split over the GPUs (default), "
                         "weak = 131,072 atoms per GPU")
    ap.add_argument("--strong-lattice", default=None, help="lattice sites of the strong-scaling system (default 128x128x64)")
    ap.add_argument("--md-brick", default=None, help="weak series: lattice sites per GPU as XxYxZ (small profiling cases)")
    ap.add_argument("--chunk-rows", type=int, default=-1,
                    help="owner rows per chunk of the streamed gate evaluation (0: whole tables; default: 65536 above "
                         "300,000 atoms per GPU)")
    ap.add_argument("--stream-gates", default="auto", choices=["auto", "yes", "no"],
                    help="with chunks: stream the gates too (yes), keep the pair table and stream only the gate "
                         "gradient (no), or decide by the table's size (auto)")
    ap.add_argument("--skin", type=float, default=2.0, help="extra halo width of the decomposed run (A)")
    ap.add_argument("--train-side", type=int, default=32, help="train workload: lattice sites per edge (atoms = side^3)")
    ap.add_argument("--cpu-md-side", type=int, default=24, help="CPU arm: sites per edge of the periodic sample")
    ap.add_argument("--no-sort", action="store_true", help="keep the atoms in lattice order (no space-filling-curve sort)")
    ap.add_argument("--no-graph", action="store_true", help="do not record the MD step as a CUDA graph")
    ap.add_argument("--capture-collectives", default="auto", choices=["auto", "yes", "no"],
                    help="decomposed run: record the step with its collectives as one CUDA graph (auto: yes; beyond two ranks "
                         "the benchmark then switches NVLS and graph buffer registration off before NCCL starts)")
    ap.add_argument("--atoms", type=int, default=NUM_ATOMS)
    ap.add_argument("--nodes", type=int, default=SC_NODES)
    ap.add_argument("--cpu-sample-atoms", type=int, default=2048)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="md at N=1: skip the configuration 2/3/4 and parity keys")
    ap.add_argument("--no-parity", action="store_true", help="md at N>1: skip the decomposed-vs-single parity check")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return {"md": main_md, "train": main_train, "sc": main_sc, "fused_message": main_fused_message}[args.workload](
        args, rank, world, local)


if __name__ == "__main__":
    main()
