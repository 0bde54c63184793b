"""Neighbour list (bit-exact), MD integrator and the MD force path on one GPU."""
import numpy as np
import pytest
import torch

from oracle import ictc_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _status():
    yield
    from ictc_o3 import _lib
    assert _lib.kernel_status() == 0


@pytest.mark.parametrize("n,box,periodic,centres,seed", [
    (300, (14.0, 15.0, 16.0), (1, 1, 1), 300, 0),      # 3 cells per axis
    (120, (9.5, 10.0, 4.6), (1, 1, 1), 120, 1),        # 2 and 1 cells per axis: same cell, several images
    (200, (12.0, 13.0, 11.0), (0, 0, 0), 150, 2),      # open boundaries, centres = first 150 rows
    (180, (10.0, 20.0, 10.0), (1, 0, 1), 180, 3),      # mixed
    (1, (10.0, 10.0, 10.0), (1, 1, 1), 1, 4), (5, (10.0, 10.0, 10.0), (1, 1, 1), 0, 5)])
def test_neighbor_list_bit_exact(n, box, periodic, centres, seed):
    from mace_ictc.md import neighbor_list
    rng = np.random.default_rng(seed)
    pos = (rng.random((n, 3)) * np.array(box)).astype(np.float32)
    cutoff = 4.5
    rs, rd, rsh = O.neighbor_list_bruteforce(pos, centres, box, periodic, cutoff)
    src, dst, shifts, rowptr = neighbor_list(torch.as_tensor(pos).cuda(), centres, [0, 0, 0], box, box, periodic, cutoff)
    assert src.numel() == rs.shape[0]
    assert torch.equal(src.cpu(), torch.as_tensor(rs))
    assert torch.equal(dst.cpu(), torch.as_tensor(rd))
    assert torch.equal(shifts.cpu().long(), torch.as_tensor(rsh))
    assert torch.equal(rowptr.cpu(), torch.as_tensor(np.concatenate([[0], np.cumsum(np.bincount(rd, minlength=centres))])))


def test_neighbor_list_matches_host_builder_on_config_sized_system():
    """32,768-atom jittered lattice (BASELINE configuration 4): same edges as the host k-d tree builder."""
    from mace_ictc import synthetic as S
    from mace_ictc.md import neighbor_list
    pos, box, _species = S.jittered_lattice(32, 32, 32, 2.15, 0.1, 0)
    hs, hd, hsh = S.neighbor_list_host(pos, box, 4.5)
    src, dst, shifts, _ = neighbor_list(torch.as_tensor(pos).cuda(), pos.shape[0], [0, 0, 0], box, box, (1, 1, 1), 4.5)
    assert torch.equal(src.cpu(), torch.as_tensor(hs)) and torch.equal(dst.cpu(), torch.as_tensor(hd))
    assert torch.equal(shifts.cpu().long(), torch.as_tensor(hsh))
    assert 30.0 < src.numel() / pos.shape[0] < 36.0


def test_md_forces_match_public_api_and_energy_is_conserved():
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model, energy_and_forces
    from mace_ictc.md import MolecularDynamics
    torch.manual_seed(1)
    pos, box, species = S.jittered_lattice(8, 8, 8, 2.15, 0.1, 3)
    z = np.array([1, 6, 8])[species]
    model = create_model(channels=32, lmax=2, cutoff=4.5, avg_num_neighbors=32.0)
    md = MolecularDynamics(model, pos, z, box, dt=0.5, temperature=300.0, seed=7)
    f = md.gather(md.compute_forces())
    hs, hd, hsh = S.neighbor_list_host(pos, box, 4.5)
    n = pos.shape[0]
    dev = "cuda"
    model.preserve_edge_order = False
    ref = energy_and_forces(model, torch.as_tensor(pos).to(dev), torch.as_tensor(z).to(dev),
                            torch.zeros(n, dtype=torch.long, device=dev), torch.as_tensor(hs).to(dev),
                            torch.as_tensor(hd).to(dev), torch.as_tensor(hsh).to(dev),
                            torch.as_tensor(np.diag(box)).float().unsqueeze(0).to(dev))
    model.preserve_edge_order = True
    assert float((f - ref["forces"]).abs().max()) < 1e-5 * float(ref["forces"].abs().max())
    assert abs(float(md.energy) - float(ref["energy"])) < 1e-5 * abs(float(ref["energy"]))
    assert abs(md.temperature() - 300.0) < 1e-3
    e0 = float(md.energy) + md.kinetic_energy()
    for _ in range(20):
        md.step()
    e1 = float(md.energy) + md.kinetic_energy()
    ke = md.kinetic_energy()
    assert abs(e1 - e0) < 2e-3 * ke, (e0, e1, ke)      # NVE: total energy drift far below the kinetic energy
    assert float(md.pos.min()) >= 0.0 and bool((md.pos < md.box_f).all())


def test_force_engine_matches_autograd_path():
    """The explicit forward/reverse sweep gives the forces and energy of autograd through the model."""
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model
    from mace_ictc.md import MolecularDynamics
    torch.manual_seed(5)
    pos, box, species = S.jittered_lattice(9, 8, 7, 2.15, 0.1, 8)
    z = np.array([1, 6, 8])[species]
    model = create_model(channels=64, lmax=2, cutoff=4.5, avg_num_neighbors=32.0)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "linear_up" in name or "self_connection" in name:
                p.add_(0.05 * torch.randn_like(p))
    auto = MolecularDynamics(model, pos, z, box, seed=2, use_engine=False)
    fast = MolecularDynamics(model, pos, z, box, seed=2, use_engine=True)
    fa, ff = auto.compute_forces(), fast.compute_forces()
    scale = float(fa.abs().max())
    assert float((fa - ff).abs().max()) < 1e-5 * scale, float((fa - ff).abs().max()) / scale
    assert abs(float(auto.energy) - float(fast.energy)) < 1e-5 * abs(float(auto.energy))
    # bitwise repeatable: the engine has no float atomics
    f2 = fast.compute_forces()
    assert torch.equal(ff, f2)


def test_chunked_gate_streaming_is_bitwise_equal_to_whole_tables():
    """Streaming the gates in chunks of owner rows (no [E, P*C] tensor exists whole; the reverse sweep recomputes
    each chunk's gates) gives bit-identical energy and forces, eagerly and in a recorded step; a chunk buffer
    that is too small raises the device flag and nothing is written out of bounds."""
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model
    from mace_ictc.md import MolecularDynamics
    torch.manual_seed(6)
    pos, box, species = S.jittered_lattice(10, 9, 8, 2.15, 0.1, 21)
    z = np.array([1, 6, 8])[species]
    model = create_model(channels=64, lmax=2, cutoff=4.5, avg_num_neighbors=32.0)
    whole = MolecularDynamics(model, pos, z, box, seed=2)
    f0 = whole.compute_forces().clone()
    unshared = MolecularDynamics(model, pos, z, box, seed=2, share_gates=False).compute_forces().clone()
    for rows in (97, 256):
        for share in (True, False):
            for stream in (True, False):      # gates and gate gradients per chunk / gate gradients only
                part = MolecularDynamics(model, pos, z, box, seed=2, chunk_rows=rows, share_gates=share,
                                         stream_gates=stream)
                assert torch.equal(part.compute_forces(), f0 if share else unshared), (rows, share, stream)
                assert int(part.engine.overflow.item()) == 0
    a = MolecularDynamics(model, pos, z, box, dt=1.0, seed=4)
    b = MolecularDynamics(model, pos, z, box, dt=1.0, seed=4, chunk_rows=128, stream_gates=True)
    a.compute_forces()
    b.compute_forces()
    assert float(a.energy) == float(b.energy)
    a.enable_graph()
    b.enable_graph()
    a.run(4)
    b.run(4)
    assert torch.equal(a.pos, b.pos) and torch.equal(a.forces, b.forces) and not b.check_overflow()
    tight = MolecularDynamics(model, pos, z, box, seed=2, chunk_rows=97, stream_gates=True)
    tight.engine.chunk_margin = 0.5
    tight.engine.bucket = lambda rows: int(rows)          # exact sizes: the buffer really is too small
    tight.compute_forces()
    assert int(tight.engine.overflow.item()) == 1


def test_positions_are_wrapped_and_unknown_species_raise():
    """Coordinates outside the box are wrapped on entry (same forces as the wrapped system); an atomic number the
    model has no embedding for raises ValueError on the host."""
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model
    from mace_ictc.md import MolecularDynamics
    torch.manual_seed(8)
    pos, box, species = S.jittered_lattice(8, 8, 8, 2.15, 0.1, 13)
    z = np.array([1, 6, 8])[species]
    model = create_model(channels=64, lmax=2, cutoff=4.5, avg_num_neighbors=32.0)
    inside = MolecularDynamics(model, pos, z, box, seed=1)
    rng = np.random.default_rng(3)
    images = rng.integers(-2, 3, size=pos.shape).astype(np.float64)
    outside = MolecularDynamics(model, np.asarray(pos, dtype=np.float64) + images * box, z, box, seed=1)
    assert float(outside.pos.min()) >= 0.0 and bool((outside.pos < outside.box_f).all())
    f_in, f_out = inside.gather(inside.compute_forces()), outside.gather(outside.compute_forces())
    assert outside.num_edges == inside.num_edges
    assert float((f_in - f_out).abs().max()) < 1e-4 * float(f_in.abs().max())
    bad = z.copy()
    bad[5] = 7
    with pytest.raises(ValueError):
        MolecularDynamics(model, pos, bad, box, seed=1)


def test_graph_replay_matches_eager_steps():
    """The recorded MD step (fixed-capacity edge buffers, no host read-back) follows the eager trajectory."""
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model
    from mace_ictc.md import MolecularDynamics
    torch.manual_seed(2)
    pos, box, species = S.jittered_lattice(10, 9, 8, 2.15, 0.1, 6)
    z = np.array([1, 6, 8])[species]
    model = create_model(channels=64, lmax=2, cutoff=4.5, avg_num_neighbors=32.0)
    eager = MolecularDynamics(model, pos, z, box, dt=1.0, seed=4)
    fast = MolecularDynamics(model, pos, z, box, dt=1.0, seed=4)
    eager.compute_forces()
    fast.compute_forces()
    p0, v0 = fast.pos.clone(), fast.vel.clone()
    cap = fast.enable_graph()
    assert cap > fast.num_edges
    assert torch.equal(fast.pos, p0) and torch.equal(fast.vel, v0)     # recording leaves the state alone
    for _ in range(5):
        eager.step()
        fast.step()
    assert not fast.check_overflow()
    assert float((fast.pos - eager.pos).abs().max()) < 2e-5
    assert float((fast.forces - eager.forces).abs().max()) < 2e-5 * float(eager.forces.abs().max())
    assert abs(float(fast.energy) - float(eager.energy)) < 1e-5 * abs(float(eager.energy))


def test_edge_capacity_overflow_is_flagged_and_stays_in_bounds():
    """A neighbour list that does not fit the fixed buffers is truncated inside them and raises the sticky
    device flag; every index the consumers read stays in range."""
    from mace_ictc import synthetic as S
    from mace_ictc.md import StaticNeighborList, neighbor_list
    pos, box, _ = S.jittered_lattice(8, 8, 8, 2.15, 0.1, 3)
    dev = torch.device("cuda:0")
    p = torch.as_tensor(pos, dtype=torch.float32, device=dev)
    n = p.shape[0]
    full = neighbor_list(p, n, [0, 0, 0], list(box), list(box), [1, 1, 1], 4.5)[0].shape[0]
    cap = full // 2
    nl = StaticNeighborList(n, list(box), 4.5, cap, dev)
    ext = torch.cat((p, torch.full((1, 3), -1.0e6, device=dev)))
    nl.build(ext)
    if hasattr(nl, "pairs"):
        nl.pairs()
    torch.cuda.synchronize()
    assert int(nl.overflow.item()) == 1
    rp = nl.rowptr.cpu()
    assert int(rp[-1]) == cap - 1 and bool((rp[1:] >= rp[:-1]).all())
    assert int(nl.src.min()) >= 0 and int(nl.src.max()) <= n
    assert int(nl.dst.min()) >= 0 and int(nl.dst.max()) < n
    assert int(nl.gate_row.min()) >= 0 and int(nl.gate_row.max()) < nl.ucap
    assert int(nl.rep.min()) >= 0 and int(nl.rep.max()) < cap and int(nl.other.max()) < cap
    # a list that fits leaves the flag alone (it is sticky) and a fresh one reports no overflow
    ok = StaticNeighborList(n, list(box), 4.5, full + 8, dev)
    ok.build(ext)
    torch.cuda.synchronize()
    assert int(ok.overflow.item()) == 0 and int(ok.rowptr[-1]) == full


def test_run_recovers_from_edge_capacity_overflow():
    """``run`` notices that the recorded capacity was exceeded, re-records with a larger one and repeats the
    block, so the trajectory equals the eager one."""
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model
    from mace_ictc.md import MolecularDynamics
    torch.manual_seed(2)
    # spacing 2.02: the (2,1,0) shell sits 0.017 A outside the cutoff, so thermal motion adds edges quickly
    pos, box, species = S.jittered_lattice(8, 8, 8, 2.02, 0.02, 6)
    z = np.array([1, 6, 8])[species]
    model = create_model(channels=64, lmax=2, cutoff=4.5, avg_num_neighbors=32.0)
    eager = MolecularDynamics(model, pos, z, box, dt=1.0, temperature=600.0, seed=4)
    fast = MolecularDynamics(model, pos, z, box, dt=1.0, temperature=600.0, seed=4)
    eager.compute_forces()
    fast.compute_forces()
    e0 = fast.num_edges
    fast.enable_graph(margin=1.0, spare=16)
    eager.run(12)
    fast.run(12, check_every=4, margin=1.5)
    assert eager.num_edges > e0 + 16, "the test system must outgrow the first capacity"
    assert fast.graph_rebuilds >= 1 and not fast.check_overflow()
    assert float((fast.pos - eager.pos).abs().max()) < 5e-5
    assert float((fast.forces - eager.forces).abs().max()) < 5e-5 * float(eager.forces.abs().max())


def test_radial_pairs_are_exact_and_do_not_change_forces():
    """Every edge and its reverse share one gate row, their lengths are bitwise equal, and evaluating the
    radial MLP per pair gives the same forces as evaluating it per directed edge."""
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model
    from mace_ictc.md import MolecularDynamics, edge_pairs, neighbor_list
    pos, box, species = S.jittered_lattice(9, 7, 8, 2.15, 0.1, 12)
    z = np.array([1, 6, 8])[species]
    p = torch.as_tensor(pos).cuda()
    n = p.shape[0]
    src, dst, shifts, rowptr, keys = neighbor_list(p, n, [0, 0, 0], box, box, (1, 1, 1), 4.5, True)
    gate_row, rep, other = edge_pairs(rowptr, dst, keys, n)
    e = src.numel()
    assert rep.numel() * 2 == e and bool((other >= 0).all())          # single GPU: all edges are paired
    assert torch.equal(gate_row[rep], torch.arange(rep.numel(), device="cuda"))
    assert torch.equal(gate_row[other], torch.arange(rep.numel(), device="cuda"))
    assert torch.equal(src[other], dst[rep]) and torch.equal(dst[other], src[rep])
    assert torch.equal(shifts[other], -shifts[rep])
    vec = p[dst] - p[src] + shifts * torch.as_tensor(box, dtype=torch.float32, device="cuda")
    length = vec.norm(dim=1)
    assert torch.equal(length[rep], length[other])
    # centres restricted to a prefix: edges whose sender is not a centre stay single
    half = n // 2
    s2, d2, sh2, rp2, k2 = neighbor_list(p, half, [0, 0, 0], box, box, (1, 1, 1), 4.5, True)
    g2, r2, o2 = edge_pairs(rp2, d2, k2, half)
    single = o2 < 0
    assert bool((s2[r2[single]] >= half).all()) and bool((s2[r2[~single]] < half).all())
    assert int(g2.max()) + 1 == r2.numel()
    torch.manual_seed(3)
    model = create_model(channels=64, lmax=2, cutoff=4.5, avg_num_neighbors=32.0)
    a = MolecularDynamics(model, pos, z, box, seed=1, share_gates=True)
    b = MolecularDynamics(model, pos, z, box, seed=1, share_gates=False)
    fa, fb = a.compute_forces(), b.compute_forces()
    assert float((fa - fb).abs().max()) < 5e-6 * float(fb.abs().max())
    assert abs(float(a.energy) - float(b.energy)) < 1e-6 * abs(float(b.energy))


@pytest.mark.parametrize("p", [5, 6])
def test_edge_geometry_kernel_matches_the_reference_radial_embedding(p):
    """The fused geometry kernel's radial basis and its length derivative against vectors computed by the
    reference's own `mace_radial_embedding` (tests/golden/radial_bessel8_rmax4p5.npz)."""
    import os
    from ictc_o3 import _lib
    lib = _lib.load()
    g = np.load(os.path.join(os.path.dirname(__file__), "golden", "radial_bessel8_rmax4p5.npz"))
    keep = g["r"] < 4.5
    r = torch.tensor(g["r"][keep], dtype=torch.float64)
    e = r.numel()
    torch.manual_seed(0)
    unit = torch.nn.functional.normalize(torch.randn(e, 3, dtype=torch.float64), dim=-1)
    pos = torch.zeros(2 * e, 3, dtype=torch.float64)
    pos[0::2] = torch.rand(e, 3, dtype=torch.float64) * 3.0 + 5.0
    pos[1::2] = pos[0::2] + unit * r[:, None]
    dev = "cuda"
    posd = pos.float().to(dev)
    src = torch.arange(1, 2 * e, 2, device=dev)          # one edge per pair of points, length r
    dst = torch.arange(0, 2 * e, 2, device=dev)
    sh = torch.empty(e, 9, device=dev)
    rb = torch.empty(e, 8, device=dev)
    un = torch.empty(e, 3, device=dev)
    ln = torch.empty(e, device=dev)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.ictc_edge_geometry_forward(posd.data_ptr(), src.data_ptr(), dst.data_ptr(), None, None, 4.5, 8, p, e,
                                              sh.data_ptr(), rb.data_ptr(), un.data_ptr(), ln.data_ptr(), st), "geom")
    # the fp32 positions give a slightly different length: compare at the length the kernel saw
    want = torch.tensor(g[f"emb_p{p}"][keep])
    slope = torch.tensor(g[f"grad_p{p}"][keep])
    assert float((ln.double().cpu() - r).abs().max()) < 5e-6
    err = float((rb.double().cpu() - want).abs().max() / want.abs().max())
    assert err < 1e-5, err
    w = torch.tensor(g["w"], dtype=torch.float32, device=dev)
    drb = w.unsqueeze(0).expand(e, -1).contiguous()
    dsh = torch.zeros(e, 9, device=dev)
    dvec = torch.empty(e, 3, device=dev)
    _lib.check(lib.ictc_edge_geometry_backward(un.data_ptr(), ln.data_ptr(), 4.5, 8, p, e, dsh.data_ptr(), drb.data_ptr(),
                                               dvec.data_ptr(), st), "geom bwd")
    dr = (dvec * un).sum(-1).double().cpu()
    assert float((dr - slope).abs().max() / slope.abs().max()) < 1e-5


def test_full_size_step_properties():
    """Size-independent checks at the benchmark size (131,072 atoms, 4.2 M edges): total force vanishes, energy
    and forces are invariant under a rigid translation through the periodic box, results are bitwise
    repeatable, and the neighbour list is symmetric (every edge has its reverse: E = 2 x pairs)."""
    from mace_ictc import synthetic as S
    from mace_ictc.hp import create_model
    from mace_ictc.md import MolecularDynamics
    torch.manual_seed(0)
    pos, box, species = S.jittered_lattice(64, 64, 32, 2.15, 0.1, 0)
    z = np.array([1, 6, 8])[species]
    model = create_model(channels=64, lmax=2, cutoff=4.5, avg_num_neighbors=32.0)
    md = MolecularDynamics(model, pos, z, box, dt=1.0, seed=1)
    f1 = md.compute_forces().clone()
    e1 = float(md.energy)
    assert md.num_edges == 2 * md.num_gate_rows
    fmax = float(f1.abs().max())
    assert float(f1.sum(0).abs().max()) < 2e-3 * fmax
    assert torch.equal(md.compute_forces(), f1)
    shift = np.array([0.37, -1.21, 2.05])
    moved = np.mod(np.asarray(pos, dtype=np.float64) + shift, box)
    md2 = MolecularDynamics(model, moved, z, box, dt=1.0, seed=1)
    f2 = md2.gather(md2.compute_forces())
    f1 = md.gather(f1)
    # the translated fp32 coordinates round differently (1e-5 A at 100 A): forces agree to that rounding
    assert float((f2 - f1).abs().max()) < 1e-4 * fmax
    assert abs(float(md2.energy) - e1) < 2e-6 * abs(e1)
    from ictc_o3 import _lib
    assert _lib.kernel_status() == 0
