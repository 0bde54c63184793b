"""GPU parity against vectors produced by the reference's own model classes (tests/golden/make_golden_model.py):
the symmetric-contraction kernels, the channel linears and the whole C64 model (autograd route and force
engine), float32 kernels against float64 reference values at 1e-5 relative."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-5
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _rel(a, b):
    a, b = torch.as_tensor(a).detach().double().cpu(), torch.as_tensor(b).detach().double().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.fixture(autouse=True)
def _status():
    yield
    from ictc_o3 import _lib
    assert _lib.kernel_status() == 0


@pytest.mark.parametrize("target", [0, 2])
def test_symmetric_contraction_kernels_match_reference_recursion(target):
    from ictc_o3 import create_symmetric_contraction
    g = np.load(os.path.join(GOLD, "sc_pureu_c8.npz"))
    tag = f"t{target}/"
    sc = create_symmetric_contraction(num_elements=3, lmax=2, target_lmax=target, channels=8)
    named = {}
    with torch.no_grad():
        for l, con in enumerate(sc.symmetric_contractions.contractions):
            con.weights_max.copy_(torch.tensor(g[tag + f"w/contractions.{l}.weights_max"]))
            named[f"contractions.{l}.weights_max"] = con.weights_max
            for k, w in enumerate(con.weights):
                w.copy_(torch.tensor(g[tag + f"w/contractions.{l}.weights.{k}"]))
                named[f"contractions.{l}.weights.{k}"] = w
    x = torch.tensor(g[tag + "x"]).float().cuda().requires_grad_(True)
    y = sc(x, None, torch.tensor(g[tag + "species"]).cuda())
    assert _rel(y, g[tag + "y"]) < TOL
    names = sorted(named)
    grads = torch.autograd.grad((y * torch.tensor(g[tag + "cot"]).float().cuda()).sum(), [x] + [named[k] for k in names])
    assert _rel(grads[0], g[tag + "dx"]) < TOL
    for k, got in zip(names, grads[1:]):
        assert _rel(got, g[tag + "dw/" + k]) < TOL, k


def test_channel_linears_match_reference_modules():
    from mace_ictc.model import ElementConditionedLinearSO3, EquivariantChannelLinearSO3, PathPreservingLinearSO3
    g = np.load(os.path.join(GOLD, "linears_c8.npz"))
    c = 8
    up = EquivariantChannelLinearSO3(c, 2).cuda()
    up.load_state_dict({k[len("up/w/"):]: torch.tensor(g[k]).float() for k in g.files if k.startswith("up/w/")})
    assert _rel(up(torch.tensor(g["up/x"]).float().cuda()), g["up/y"]) < TOL
    counts = {0: 3, 1: 4, 2: 4}
    ppl = PathPreservingLinearSO3({l: c * counts[l] for l in counts}, c, 2).cuda()
    ppl.load_state_dict({k[len("message/w/"):]: torch.tensor(g[k]).float() for k in g.files
                         if k.startswith("message/w/")})
    blocks = {l: torch.tensor(g[f"message/x{l}"]).float().cuda() for l in counts}
    assert _rel(ppl(blocks), g["message/y"]) < TOL
    ecl = ElementConditionedLinearSO3(3, c, 2).cuda()
    ecl.load_state_dict({k[len("element/w/"):]: torch.tensor(g[k]).float() for k in g.files
                         if k.startswith("element/w/")})
    got = ecl.forward_type_idx(torch.tensor(g["element/x"]).float().cuda(), torch.tensor(g["element/idx"]).cuda())
    assert _rel(got, g["element/y"]) < TOL


def _golden_model(g):
    from mace_ictc.checkpoint import load_reference_state_dict
    from mace_ictc.hp import create_model
    model = create_model(channels=int(g["channels"]), lmax=2, num_interactions=2, correlation=3,
                         cutoff=float(g["cutoff"]), atomic_numbers=(1, 6, 8),
                         avg_num_neighbors=float(g["avg_num_neighbors"]))
    load_reference_state_dict(model, {k[len("state/"):]: torch.tensor(g[k]) for k in g.files if k.startswith("state/")})
    return model


def test_model_matches_reference_model_c64():
    """The reference's own model (float64 CPU, 'ictd-pure-u' backend) on 125 atoms: energy, atomic energies and
    forces through the autograd route, and the force-loss gradient of seven parameters of different blocks
    (mixed second derivatives)."""
    from mace_ictc.checkpoint import from_reference_state_dict
    from mace_ictc.hp import energy_and_forces
    g = np.load(os.path.join(GOLD, "model_pureu_c64_n125.npz"))
    model = _golden_model(g)
    n, dev = g["pos"].shape[0], "cuda"
    args = (torch.tensor(g["pos"]).float().to(dev), torch.tensor(g["z"]).to(dev), torch.zeros(n, dtype=torch.long, device=dev),
            torch.tensor(g["src"]).to(dev), torch.tensor(g["dst"]).to(dev), torch.tensor(g["shifts"]).float().to(dev),
            torch.tensor(np.diag(g["box"])).float().unsqueeze(0).to(dev))
    got = energy_and_forces(model, *args)
    assert _rel(got["energy"], g["energy"]) < TOL
    assert _rel(got["atomic_energy"], g["atomic_energy"]) < TOL
    assert _rel(got["forces"], g["forces"]) < TOL
    res = energy_and_forces(model, *args, training=True)
    loss = (res["energy"] / n).square().mean() + res["forces"].square().mean()
    assert _rel(loss, g["loss"]) < TOL
    ref = from_reference_state_dict({k[len("grad/"):]: torch.tensor(g[k]) for k in g.files if k.startswith("grad/")}, 64)
    params = dict(model.named_parameters())
    keys = sorted(ref)
    assert len(keys) >= 7
    grads = torch.autograd.grad(loss, [params[k] for k in keys])
    for k, got_g in zip(keys, grads):
        assert _rel(got_g, ref[k]) < 3 * TOL, k


def test_force_engine_matches_reference_model_c64():
    """Same golden system through the tape-free force engine (the MD path: neighbour list built on the device,
    tcgen05 gate MLP and channel linears, paired gates)."""
    from mace_ictc.md import MolecularDynamics
    g = np.load(os.path.join(GOLD, "model_pureu_c64_n125.npz"))
    model = _golden_model(g)
    md = MolecularDynamics(model, g["pos"], g["z"], g["box"], dt=1.0, seed=1)
    forces = md.gather(md.compute_forces())
    assert md.num_edges == g["src"].shape[0]
    assert _rel(forces, g["forces"]) < TOL
    assert abs(float(md.energy) - float(g["energy"][0])) < TOL * abs(float(g["energy"][0]))
