#!/usr/bin/env python
"""Benchmark of the ICTC hot path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload fused_message]

Workload ``md`` (default; BASELINE configuration 5, weak-scaling series): NVE molecular dynamics of the
C64 / lmax 2 / 2-interaction / correlation-3 random-init model on a jittered simple-cubic H/C/O lattice
(spacing 2.15 A, sigma 0.1 A, 1:2:1), 131,072 atoms per GPU (64x64x32 sites per brick; 8 GPUs = the
1,048,576-atom box), cutoff 4.5 A, 1 fs velocity-Verlet steps from a 300 K Maxwell-Boltzmann start.  A
"step" is one full MD step: neighbour rebuild, energy, forces (autograd through the kernels), halo
exchange when N > 1, integration.  Metric: atom-steps per second over all GPUs.

Workload ``fused_message`` (BASELINE configuration 2): fused edge tensor product + receiver
scatter-sum, forward and first adjoint (dx, dsh, dg), fp32, C=64, lmax 2, 65,536 atoms at uniform
random positions in a periodic cube of density 0.1 / A^3, cutoff 4.5 A (about 38 neighbours per
atom, ~2.5 M directed edges sorted by receiver), node features ~ N(0,1), gates from a random-init
radial MLP 8 -> 64 -> 64 -> 64 -> 704 over an 8-function Bessel basis.  A "step" is one forward plus
one adjoint over the whole edge list; the metric is directed edges processed per second.

One JSON line is printed by rank 0.  With N > 1 (torchrun) the MD box is split into N bricks (spatial
domain decomposition, NCCL halo exchange); the fused_message workload gives every rank its own
independent system (no data-path collective).  Both are weak scaling.
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

import numpy as np  # noqa: E402
import torch  # noqa: E402

CHANNELS, LMAX, NUM_ATOMS, DENSITY, CUTOFF = 64, 2, 65536, 0.1, 4.5
NX, NH, NP, NO = 9, 9, 11, 35


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
    """SM clock and throttle reasons of one GPU, read through NVML from the benchmark's own thread between
    steps (``tick``; at most one reading per ``period`` seconds).  A separate sampling process or an nvidia-smi
    loop slows an eager multi-GPU step by tens of per cent on these hosts; two in-process queries do not."""

    _BITS = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

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
        self.active, self.last = True, 0.0

    def tick(self):
        """Called between steps of the timed region."""
        if not self.active or self.nvml is None:
            return
        now = time.perf_counter()
        if now - self.last < self.period:
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


# ------------------------------------------------------------------------------------ CPU arm
def cpu_reference_step_factory(seed, sample_atoms):
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


def run_cpu(seed, steps, warmup, sample_atoms):
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    step, edges = cpu_reference_step_factory(seed, sample_atoms)
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



# ------------------------------------------------------------------------------------ MD workload
MD_BRICK = (64, 64, 32)          # lattice sites per GPU
MD_SPACING, MD_SIGMA, MD_CUTOFF, MD_DT, MD_T = 2.15, 0.1, 4.5, 1.0, 300.0


def md_lattice_dims(world):
    from mace_ictc.domain import brick_grid
    dims = list(MD_BRICK)
    n = world
    while n > 1:                      # double the currently shortest box edge, so bricks stay 64x64x32
        axis = min(range(3), key=lambda a: dims[a])
        dims[axis] *= 2
        n //= 2
    return tuple(dims)


def md_cpu_step_factory(side):
    """The oracle model (fp32, all host threads): energy and forces of a side^3-atom periodic sample of
    the same lattice, neighbour list included."""
    from mace_ictc import synthetic as S
    from mace_ictc.model import MaceIctcModel
    from oracle.model_oracle import ModelOracle
    torch.manual_seed(0)
    pos, box, species = S.jittered_lattice(side, side, side, MD_SPACING, MD_SIGMA, 0)
    z = torch.as_tensor(np.array([1, 6, 8])[species])
    weights = MaceIctcModel(channels=CHANNELS, cutoff=MD_CUTOFF, avg_num_neighbors=32.0).state_dict()
    oracle = ModelOracle(weights, channels=CHANNELS, lmax=2, num_interactions=2, correlation=3,
                         atomic_numbers=(1, 6, 8), cutoff=MD_CUTOFF, avg_num_neighbors=32.0, dtype=torch.float32)
    p = torch.as_tensor(pos)
    batch = torch.zeros(p.shape[0], dtype=torch.long)
    cell = torch.as_tensor(np.diag(box)).float().unsqueeze(0)

    def step():
        src, dst, shifts = S.neighbor_list_host(pos, box, MD_CUTOFF)
        oracle.energy_and_forces(p, z, batch, torch.as_tensor(src), torch.as_tensor(dst), torch.as_tensor(shifts), cell)
        return p.shape[0]

    return step, p.shape[0]


def run_cpu_md(steps, warmup, side):
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    step, atoms = md_cpu_step_factory(side)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / steps
    return {"value": atoms / dt, "unit": "atom-steps/s", "cores": threads, "kind": "port",
            "sample": f"{atoms}-atom periodic sample ({side}^3 sites) of the same lattice and model, fp32 torch CPU, "
                      f"neighbour list + energy + forces per step, {steps} timed steps",
            "ms_per_step": dt * 1e3}


def main_md(args, rank, world, local):
    global MD_BRICK
    if args.md_brick:
        MD_BRICK = tuple(int(v) for v in args.md_brick.lower().split("x"))
    if args.scaling == "strong":          # one fixed system (default: the reference's 262,144-atom strong series)
        dims = tuple(int(v) for v in args.strong_lattice.lower().split("x"))
    else:
        dims = md_lattice_dims(world)
    atoms_total = dims[0] * dims[1] * dims[2]
    workload = {"workload": f"md: NVE velocity-Verlet, C{CHANNELS}/lmax2/2 interactions/corr3 random-init, jittered "
                            f"H/C/O lattice {dims[0]}x{dims[1]}x{dims[2]} = {atoms_total} atoms "
                            f"({atoms_total // world} per GPU), cutoff {MD_CUTOFF} A, dt {MD_DT} fs, "
                            f"{MD_T} K, neighbours rebuilt every step",
                "l2": "edge tensors (gates 12 GB per layer) are larger than L2", "atoms_per_gpu": atoms_total // world}
    if args.impl == "reference":
        if rank != 0:
            return
        steps, warmup = max(1, min(args.steps, 3)), 1
        res = run_cpu_md(steps, warmup, args.cpu_md_side)
        line = {"impl": "reference", "metric": "MD atom-steps/s", "value": res["value"], "unit": "atom-steps/s",
                "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "f32",
                "data": "synthetic",
                "config": workload, "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
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
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from ictc_o3 import _lib
    from ictc_o3.ops import tensor_product as tpmod
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model
    from mace_ictc.md import MolecularDynamics
    torch.manual_seed(0)
    pos, box, species = S.jittered_lattice(*dims, MD_SPACING, MD_SIGMA, 0)
    z = np.array([1, 6, 8])[species]
    model = create_model(channels=CHANNELS, lmax=2, num_interactions=2, correlation=3, cutoff=MD_CUTOFF,
                         atomic_numbers=(1, 6, 8), avg_num_neighbors=32.0, device=dev)
    if world > 1:
        for p in model.parameters():
            dist.broadcast(p.data, 0)
    md = MolecularDynamics(model, pos, z, box, dt=MD_DT, temperature=MD_T, seed=1, distributed=world > 1)
    warm = max(3, args.warmup)
    for _ in range(warm):
        md.step()
    # per-kernel CUDA-event timings and the launch count come from eager steps (events cannot be read
    # inside a replayed graph); the timed region below replays the recorded step when N = 1
    md.engine.profile = []
    calls0 = _lib.CALLS
    probe_steps = 3
    for _ in range(probe_steps):
        md.step()
    torch.cuda.synchronize()
    calls_per_step = (_lib.CALLS - calls0) // probe_steps
    profile, md.engine.profile = md.engine.profile, None
    kern = {}
    for name, a, b in profile:
        kern.setdefault(name, []).append(a.elapsed_time(b))
    kern_ms = {k: float(np.mean(v)) for k, v in kern.items()}
    edges = md.num_edges
    gate_rows = md.num_gate_rows
    graph_cap = None
    if world == 1 and not args.no_graph:
        graph_cap = md.enable_graph()
        for _ in range(2):
            md.step()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for attempt in range(3):
        start.record()
        if md.graph is not None:
            # the replays are queued at once; the host then polls for completion and reads the clocks meanwhile
            for _ in range(args.steps):
                md.step()
            stop.record()
            while not stop.query():
                sampler.tick()
                time.sleep(0.02)
            if not md.check_overflow():
                break
            md.graph, md._static = None, None          # the edge list outgrew the recorded buffers: record again
            md.compute_forces()
            graph_cap = md.enable_graph(margin=1.10 + 0.1 * (attempt + 1))
        else:
            md.run(args.steps, on_step=sampler.tick)
            stop.record()
            break
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = start.elapsed_time(stop) / args.steps
    calls = calls_per_step * args.steps
    edges = md.num_edges

    # end to end: positions arrive from the host every step, forces and energy go back to the host
    e2e = None
    if not args.no_e2e:
        n = md.pos.shape[0]
        host_pos = torch.empty(n, 3, pin_memory=True).copy_(md.pos)
        host_f = torch.empty(n, 3, pin_memory=True)
        host_e = torch.empty(1, pin_memory=True)

        def e2e_step():
            # the caller owns the coordinates on the host: they go in, the step runs (integration, neighbour
            # build, energy, forces), and forces, energy and the new coordinates come back
            md.pos.copy_(host_pos, non_blocking=True)
            md.step()
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
    status = _lib.kernel_status()
    if world > 1:
        t = torch.tensor([ms, e2e[0] if e2e else 0.0, float(edges)], device=dev, dtype=torch.float64)
        tmax = t.clone()
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(t)
        ms = float(tmax[0])
        if e2e:
            e2e[0] = float(tmax[1])
        total_edges = float(t[2])
    else:
        total_edges = float(edges)
    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(peaks_path):
            peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_src = 6650.0, "fallback"
        n_local = atoms_total // world
        # layer-1 adjoint, every operand once: reads x, sh, one gate row per edge PAIR, cotangent rows, indices
        # (edge id, neighbour, gate row); writes dx, dsh and dg per edge
        bwd_b = (4 * (n_local * NX * CHANNELS + edges * NH + gate_rows * NP * CHANNELS + n_local * NO * CHANNELS)
                 + 24 * edges + 4 * (n_local * NX * CHANNELS + edges * NH + edges * NP * CHANNELS))
        adj_ms = kern_ms.get("graph_adjoint_l1")
        achieved = bwd_b / (adj_ms * 1e-3) / 1e9 if adj_ms else None
        line = {"metric": "MD atom-steps/s", "value": atoms_total / (ms * 1e-3), "unit": "atom-steps/s",
                "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True,
                "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": dict(workload, edges_total=total_edges, edges_per_atom=total_edges / atoms_total,
                               step_replayed_as_cuda_graph=graph_cap is not None, edge_capacity=graph_cap,
                               kernels_ms_from="3 eager steps before the timed region"),
                "gpu_launches": calls, "kernel_status": status, "clocks": clocks,
                "kernels_ms": kern_ms,
                "roofline": {"bound": "hbm", "kernel": "tp_adjoint_tma_kernel (layer-1 graph adjoint: dx, dsh, dg)",
                             "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak if achieved else None, "peak_source": peak_src,
                             "algorithmic_bytes_per_launch": bwd_b,
                             # DRAM bytes per launch: 5,995 B per edge measured by ncu on the 32,768-atom case
                             # (dram__bytes_read.sum + dram__bytes_write.sum), scaled by this launch's edge count
                             "traffic": 5995.0 * edges, "traffic_source": "ncu on 32768 atoms, scaled by edges"},
                "e2e": ({"value": atoms_total / (e2e[0] * 1e-3), "unit": "atom-steps/s", "h2d_bytes_per_step": e2e[1],
                         "d2h_bytes_per_step": e2e[2], "ms_per_step": e2e[0], "steps": e2e[3]} if e2e else None)}
        if world == 1 and not args.no_cpu_baseline:
            res = run_cpu_md(2, 1, args.cpu_md_side)
            line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------ training step
def main_train(args, rank, world, local):
    """BASELINE configuration 4: energy-and-force training step (forces with create_graph, force loss whose
    gradient needs the mixed second derivatives, AdamW) of the C64 model on a 32^3-site jittered lattice per GPU
    (independent replicas: no collective)."""
    side = args.train_side
    n_atoms = side ** 3
    workload = {"workload": f"train: energy+force loss step (mixed second derivatives, AdamW), C{CHANNELS}/lmax2/2 "
                            f"interactions/corr3 random-init, jittered H/C/O lattice {side}^3 = {n_atoms} atoms per GPU, "
                            f"cutoff {MD_CUTOFF} A, neighbour list built once (as in the reference's protocol)",
                "l2": "edge tensors (gates 3 GB per layer) are larger than L2", "atoms_per_gpu": n_atoms}
    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the CPU port times the MD step only; use --workload md"}))
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    from ictc_o3 import _lib
    from mace_ictc import synthetic as S
    from mace_ictc.hp import configure_model, create_model, energy_and_forces
    from mace_ictc.md import neighbor_list
    pos, box, species = S.jittered_lattice(side, side, side, MD_SPACING, MD_SIGMA, rank)
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

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    calls0 = _lib.CALLS
    step()
    torch.cuda.synchronize()
    calls_per_step = _lib.CALLS - calls0
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
        sampler.tick()
    stop.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = start.elapsed_time(stop) / args.steps
    e2e_steps = max(3, min(args.steps, 10))
    barrier()
    start.record()
    for _ in range(e2e_steps):
        step(True)
    stop.record()
    barrier()
    e2e_ms = start.elapsed_time(stop) / e2e_steps
    t = torch.tensor([ms, e2e_ms], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])
    status = _lib.kernel_status()
    if rank == 0:
        total = n_atoms * world
        print(json.dumps({
            "metric": "training atom-steps/s", "value": total / (ms * 1e-3), "unit": "atom-steps/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(workload, edges_per_gpu=int(src.numel()), parallelism="independent replicas"),
            "gpu_launches": calls_per_step * args.steps, "kernel_status": status, "clocks": clocks,
            "peak_memory_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
            "e2e": {"value": total / (e2e_ms * 1e-3), "unit": "atom-steps/s", "h2d_bytes_per_step": 24 * n_atoms,
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms, "steps": e2e_steps}}))
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------ GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="md", choices=["md", "fused_message", "train"])
    ap.add_argument("--train-side", type=int, default=32, help="train workload: lattice sites per edge (atoms = side^3)")
    ap.add_argument("--cpu-md-side", type=int, default=12)
    ap.add_argument("--no-graph", action="store_true", help="do not record the single-GPU MD step as a CUDA graph")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="md workload: weak = 131,072 atoms per GPU (default), strong = one fixed system")
    ap.add_argument("--strong-lattice", default="64x64x64", help="lattice sites of the strong-scaling system")
    ap.add_argument("--md-brick", default=None, help="lattice sites per GPU as XxYxZ (profiling of small cases)")
    ap.add_argument("--atoms", type=int, default=NUM_ATOMS)
    ap.add_argument("--cpu-sample-atoms", type=int, default=2048)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.workload == "md":
        return main_md(args, rank, world, local)
    if args.workload == "train":
        return main_train(args, rank, world, local)
    workload = {"workload": f"fused_message: TP+scatter forward+adjoint, fp32, C{CHANNELS}, lmax {LMAX}, "
                            f"{args.atoms} atoms/GPU uniform density {DENSITY}, cutoff {CUTOFF}",
                "l2": "inputs larger than L2 (gates alone are 7 GB)", "atoms_per_gpu": args.atoms}

    if args.impl == "reference":
        if rank != 0:
            return
        steps, warmup = max(1, min(args.steps, 3)), max(1, min(args.warmup, 1))
        res = run_cpu(0, steps, warmup, args.cpu_sample_atoms)
        line = {"impl": "reference", "metric": "TP edges/s", "value": res["value"], "unit": "edges/s",
                "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": workload,
                "cpu_baseline": {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": res["value"], "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    from ictc_o3 import PackedGraphMessage, direction_harmonics
    from ictc_o3.ops import tensor_product as tpmod

    inp = make_inputs(1000 + rank, dev, args.atoms)
    n, e = args.atoms, int(inp["src"].numel())
    op = PackedGraphMessage.create(channels=CHANNELS, input_lmax=LMAX, edge_lmax=LMAX, output_lmax=LMAX, device=dev)
    sh = torch.cat(direction_harmonics(inp["unit"], LMAX), -1).contiguous()
    x = inp["x"].requires_grad_(True)
    shg = sh.requires_grad_(True)
    g = inp["gates"].requires_grad_(True)
    src, dst, v = inp["src"], inp["dst"], inp["v"]

    def step():
        out = op(x, shg, g, src, dst)
        return torch.autograd.grad(out, [x, shg, g], v)

    for _ in range(max(3, args.warmup)):
        step()
    sampler = ClockSampler(local)
    tpmod.PROFILE = []
    barrier()
    if rank == 0:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        step()
        sampler.tick()
    stop.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = start.elapsed_time(stop) / args.steps
    profile, tpmod.PROFILE = tpmod.PROFILE, None
    launches = len(profile)
    kern = {}
    for name, a, b in profile:
        kern.setdefault(name, []).append(a.elapsed_time(b))
    kern_ms = {k: float(np.mean(vv)) for k, vv in kern.items()}

    # end to end: host (pinned) buffers in, host buffers out, copies inside the timed region
    e2e = None
    if not args.no_e2e:
        import psutil
        host = {k: t.detach() for k, t in (("x", x), ("sh", sh), ("g", g), ("v", v), ("src", src), ("dst", dst))}
        need = sum(t.numel() * t.element_size() for t in host.values()) * 2.2
        if psutil.virtual_memory().available > need * 1.5 * max(1, world):
            pin = {k: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for k, t in host.items()}
            outs = None

            def e2e_step():
                nonlocal outs
                d = {k: t.to(dev, non_blocking=True) for k, t in pin.items()}
                xs, ss, gs = (d[k].requires_grad_(True) for k in ("x", "sh", "g"))
                out = op(xs, ss, gs, d["src"], d["dst"])
                grads = torch.autograd.grad(out, [xs, ss, gs], d["v"])
                res = (out.detach(),) + grads
                if outs is None:
                    outs = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True) for t in res]
                for o, t in zip(outs, res):
                    o.copy_(t, non_blocking=True)

            e2e_steps = max(1, min(args.steps, 5))
            for _ in range(2):
                e2e_step()
            barrier()
            s2, t2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s2.record()
            for _ in range(e2e_steps):
                e2e_step()
            t2.record()
            barrier()
            e2e_ms = s2.elapsed_time(t2) / e2e_steps
            h2d = sum(t.numel() * t.element_size() for t in pin.values())
            d2h = sum(t.numel() * t.element_size() for t in outs)
            e2e = [e2e_ms, h2d, d2h, e2e_steps]
            del pin, outs

    if world > 1:
        t = torch.tensor([ms, e2e[0] if e2e else 0.0], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        if e2e:
            e2e[0] = float(t[1])
        tot = torch.tensor([e], device=dev, dtype=torch.float64)
        dist.all_reduce(tot)
        total_edges = float(tot[0])
    else:
        total_edges = float(e)

    if rank == 0:
        peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
        if os.path.exists(peaks_path):
            peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        else:
            peak, peak_src = 6650.0, "fallback"
        fwd_b, bwd_b = algorithmic_bytes(n, e)
        dom = max(kern_ms, key=kern_ms.get) if kern_ms else None
        dom_bytes = {"graph_forward": fwd_b, "graph_adjoint": bwd_b}.get(dom, 0)
        achieved = dom_bytes / (kern_ms[dom] * 1e-3) / 1e9 if dom else None
        line = {"metric": "TP edges/s", "value": total_edges / (ms * 1e-3), "unit": "edges/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": dict(workload, edges_per_gpu=e, step="forward + adjoint(dx,dsh,dg)"),
                "gpu_launches": launches, "clocks": clocks,
                "kernels_ms": kern_ms,
                "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak if achieved else None, "peak_source": peak_src,
                             "algorithmic_bytes_per_launch": dom_bytes, "traffic": None},
                "e2e": ({"value": total_edges / (e2e[0] * 1e-3), "unit": "edges/s", "h2d_bytes_per_step": e2e[1],
                         "d2h_bytes_per_step": e2e[2], "ms_per_step": e2e[0], "steps": e2e[3]} if e2e else None)}
        if world == 1 and not args.no_cpu_baseline:
            res = run_cpu(1000, 2, 1, args.cpu_sample_atoms)
            line["cpu_baseline"] = {k: res[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
