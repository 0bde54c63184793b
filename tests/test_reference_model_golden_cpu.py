"""Pins the CPU oracle of the symmetric contraction, the channel linears and the whole model on vectors that
the reference's own classes produced (tests/golden/make_golden_model.py), and checks the checkpoint key
translation on the reference's state dict.  No GPU needed."""
import os

import numpy as np
import pytest
import torch

from oracle import ictc_oracle as O
from oracle.model_oracle import ModelOracle

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _rel(a, b):
    a, b = torch.as_tensor(a).detach().double(), torch.as_tensor(b).detach().double()
    assert a.shape == b.shape, (a.shape, b.shape)
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-300))


def _blocks(flat, c):
    n = flat.shape[0]
    return {l: flat[:, c * l * l:c * (l + 1) ** 2].reshape(n, c, 2 * l + 1) for l in range(3)}


@pytest.mark.parametrize("target", [0, 2])
def test_symmetric_contraction_oracle_matches_reference_recursion(target):
    g = np.load(os.path.join(GOLD, "sc_pureu_c8.npz"))
    tag, c = f"t{target}/", 8
    x = torch.tensor(g[tag + "x"], requires_grad=True)
    species = torch.tensor(g[tag + "species"])
    weights, names = {}, {}
    for l in range(target + 1):
        base = tag + f"w/contractions.{l}."
        lower = [torch.tensor(g[base + f"weights.{k}"], requires_grad=True) for k in range(2)]
        top = torch.tensor(g[base + "weights_max"], requires_grad=True)
        weights[l] = list(reversed(lower)) + [top]
        names[l] = [f"contractions.{l}.weights.1", f"contractions.{l}.weights.0", f"contractions.{l}.weights_max"]
    xm = torch.cat([_blocks(x, c)[l] for l in range(3)], -1)                    # [N, C, 9]
    y = O.symmetric_contraction(xm, species, weights, target, 3)
    assert _rel(y, g[tag + "y"]) < 1e-12
    flat_w = [w for l in sorted(weights) for w in weights[l]]
    grads = torch.autograd.grad((y * torch.tensor(g[tag + "cot"])).sum(), [x] + flat_w)
    assert _rel(grads[0], g[tag + "dx"]) < 1e-12
    flat_names = [nm for l in sorted(names) for nm in names[l]]
    for nm, got in zip(flat_names, grads[1:]):
        assert _rel(got, g[tag + "dw/" + nm]) < 1e-12, nm


def test_channel_linears_match_reference_modules():
    g = np.load(os.path.join(GOLD, "linears_c8.npz"))
    c = 8
    x = _blocks(torch.tensor(g["up/x"]), c)
    up = torch.cat([O.channel_linear(x[l], torch.tensor(g[f"up/w/adapters.{l}.weight"])).reshape(x[l].shape[0], -1)
                    for l in range(3)], -1)
    assert _rel(up, g["up/y"]) < 1e-13
    msg = torch.cat([O.channel_linear(torch.tensor(g[f"message/x{l}"]), torch.tensor(g[f"message/w/weights.{l}"]))
                     .reshape(-1, c * (2 * l + 1)) for l in range(3)], -1)
    assert _rel(msg, g["message/y"]) < 1e-13
    idx = torch.tensor(g["element/idx"])
    xe = _blocks(torch.tensor(g["element/x"]), c)
    el = torch.cat([torch.einsum("noi,nim->nom", torch.tensor(g[f"element/w/weights.{l}"])[idx], xe[l])
                    .reshape(idx.numel(), -1) for l in range(3)], -1)
    assert _rel(el, g["element/y"]) < 1e-13


def _reference_state(g):
    return {k[len("state/"):]: torch.tensor(g[k]) for k in g.files if k.startswith("state/")}


def test_model_oracle_matches_reference_model():
    """Energy, atomic energies, forces and the force-loss gradient of every parameter (mixed second derivatives)
    of the reference's own model (float64, 'ictd-pure-u' product backend), 64 atoms, C = 8."""
    from mace_ictc.checkpoint import from_reference_state_dict
    g = np.load(os.path.join(GOLD, "model_pureu_c8_n64.npz"))
    c = int(g["channels"])
    state = from_reference_state_dict(_reference_state(g), c)
    oracle = ModelOracle(state, channels=c, lmax=2, num_interactions=2, correlation=3, atomic_numbers=(1, 6, 8),
                         cutoff=float(g["cutoff"]), avg_num_neighbors=float(g["avg_num_neighbors"]))
    n = g["pos"].shape[0]
    res = oracle.energy_and_forces(torch.tensor(g["pos"]), torch.tensor(g["z"]), torch.zeros(n, dtype=torch.long),
                                   torch.tensor(g["src"]), torch.tensor(g["dst"]), torch.tensor(g["shifts"]),
                                   torch.tensor(np.diag(g["box"])).unsqueeze(0), create_graph=True)
    assert _rel(res["energy"], g["energy"]) < 1e-11
    assert _rel(res["atomic_energy"], g["atomic_energy"]) < 1e-11
    assert _rel(res["forces"], g["forces"]) < 1e-10
    loss = (res["energy"] / n).square().mean() + res["forces"].square().mean()
    assert _rel(loss, g["loss"]) < 1e-10
    params = oracle.parameters()
    ref_grads = from_reference_state_dict({k[len("grad/"):]: torch.tensor(g[k]) for k in g.files
                                           if k.startswith("grad/")}, c)
    assert len(ref_grads) >= 30
    keys = [k for k in ref_grads if k in params]
    assert len(keys) == len(ref_grads)
    grads = torch.autograd.grad(loss, [params[k] for k in keys])
    for k, got in zip(keys, grads):
        assert _rel(got, ref_grads[k]) < 1e-8, k


def test_checkpoint_key_translation_round_trip(tmp_path):
    from mace_ictc import checkpoint as CK
    g = np.load(os.path.join(GOLD, "model_pureu_c8_n64.npz"))
    ref = _reference_state(g)
    ours = CK.from_reference_state_dict(ref, 8)
    assert "products.0.linear.2" in ours and ours["products.0.linear.2"].shape == (8, 8)
    assert "products.0.symmetric_contractions.symmetric_contractions.contractions.1.weights_max" in ours
    back = CK.to_reference_state_dict(ours)
    assert set(back) == set(ref)
    for k in ref:
        assert torch.equal(back[k], ref[k]), k
    with pytest.raises(ValueError, match="bridge-u"):
        CK.from_reference_state_dict({"products.0.symmetric_contractions.symmetric_contractions.contractions.0."
                                      "weights_max": torch.zeros(1)}, 8)
    # a checkpoint file in the reference trainer's layout loads into this build's model class
    from mace_ictc.model import MaceIctcModel
    model = MaceIctcModel(channels=8, cutoff=4.5, avg_num_neighbors=32.0)
    path = os.path.join(tmp_path, "ref.pth")
    torch.save({"e3trans_state_dict": ref, "max_radius": 4.5, "dtype": "float64", "default_state_source": "raw",
                "epoch": 3}, path)
    meta = CK.load_checkpoint(model, path)
    assert meta["epoch"] == 3
    assert torch.equal(model.interactions[1].fc[6].weight, ref["interactions.1.fc.6.weight"])
    out = os.path.join(tmp_path, "ours.pth")
    CK.save_checkpoint(model, out, epoch=4, atomic_energies={1: -13.6, 6: -1029.0})
    saved = torch.load(out, weights_only=False)
    assert set(saved["e3trans_state_dict"]) == set(ref)
    other = MaceIctcModel(channels=8, cutoff=4.5, avg_num_neighbors=32.0)
    assert CK.load_checkpoint(other, out)["epoch"] == 4
    for a, b in zip(model.parameters(), other.parameters()):
        assert torch.equal(a, b)
    with pytest.raises(ValueError, match="cutoff"):
        CK.load_checkpoint(MaceIctcModel(channels=8, cutoff=5.0), out)
