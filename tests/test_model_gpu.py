"""GPU parity of the whole model (energy, forces, force-loss parameter gradients) against the fp64 CPU
oracle model with identical weights, on small periodic systems."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-5


def _rel(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    assert a.shape == b.shape
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.fixture(autouse=True)
def _status():
    yield
    from ictc_o3 import _lib
    assert _lib.kernel_status() == 0


def _system(n_side, seed, cutoff):
    from mace_ictc import synthetic as S
    pos, box, species = S.jittered_lattice(n_side, n_side, n_side, 2.15, 0.1, seed)
    src, dst, shifts = S.neighbor_list_host(pos, box, cutoff)
    z = np.array([1, 6, 8])[species]
    return (torch.as_tensor(pos), torch.as_tensor(z), torch.as_tensor(src), torch.as_tensor(dst),
            torch.as_tensor(shifts), torch.as_tensor(np.diag(box)).unsqueeze(0))


@pytest.mark.parametrize("channels,n_side", [(64, 5), (32, 5)])
def test_energy_forces_and_training_gradients(channels, n_side):
    from mace_ictc.hp import configure_model, create_model, energy_and_forces
    from oracle.model_oracle import ModelOracle
    torch.manual_seed(3)
    cutoff = 4.5
    pos, z, src, dst, shifts, cell = _system(n_side, 5, cutoff)
    n = pos.shape[0]
    model = create_model(channels=channels, lmax=2, num_interactions=2, correlation=3, cutoff=cutoff,
                         atomic_numbers=(1, 6, 8), avg_num_neighbors=32.0)
    info = configure_model(model, policy="generated")
    assert info["selected"] == "generated"
    # perturb the identity-initialised maps so every parameter matters
    with torch.no_grad():
        for name, p in model.named_parameters():
            if "linear_up" in name or "self_connection" in name:
                p.add_(0.05 * torch.randn_like(p))
    oracle = ModelOracle(model.state_dict(), channels=channels, lmax=2, num_interactions=2, correlation=3,
                         atomic_numbers=(1, 6, 8), cutoff=cutoff, avg_num_neighbors=32.0)
    batch = torch.zeros(n, dtype=torch.long)
    ref = oracle.energy_and_forces(pos, z, batch, src, dst, shifts, cell, create_graph=True)
    dev = "cuda"
    args = (pos.to(dev), z.to(dev), batch.to(dev), src.to(dev), dst.to(dev), shifts.to(dev), cell.float().to(dev))
    got = energy_and_forces(model, *args)
    assert _rel(got["energy"], ref["energy"]) < TOL
    assert _rel(got["atomic_energy"], ref["atomic_energy"]) < TOL
    assert _rel(got["forces"], ref["forces"]) < TOL
    assert float(got["forces"].sum(0).abs().max()) < 1e-3 * float(got["forces"].abs().max())
    # training step: loss = E^2 + mean F^2, gradient w.r.t. every trainable parameter (mixed second derivatives)
    res = energy_and_forces(model, *args, training=True)
    loss = res["energy"].square().mean() + res["forces"].square().mean()
    names = [k for k, p in model.named_parameters() if p.requires_grad]
    grads = torch.autograd.grad(loss, [dict(model.named_parameters())[k] for k in names])
    rloss = ref["energy"].square().mean() + ref["forces"].square().mean()
    rparams = oracle.parameters()
    rgrads = torch.autograd.grad(rloss, [rparams[k] for k in names])
    assert abs(float(loss.detach()) - float(rloss.detach())) < TOL * abs(float(rloss))
    scale = max(float(g.abs().max()) for g in rgrads)
    for k, g, r in zip(names, grads, rgrads):
        err = float((g.double().cpu() - r).abs().max())
        assert err < 2 * TOL * max(float(r.abs().max()), 1e-3 * scale), (k, err, float(r.abs().max()))


def test_unsorted_edges_and_owned_mask():
    from mace_ictc.hp import create_model, energy_and_forces
    torch.manual_seed(0)
    pos, z, src, dst, shifts, cell = _system(4, 9, 4.5)
    n = pos.shape[0]
    model = create_model(channels=32, lmax=2, cutoff=4.5, avg_num_neighbors=32.0)
    batch = torch.zeros(n, dtype=torch.long)
    dev = "cuda"
    base = energy_and_forces(model, pos.to(dev), z.to(dev), batch.to(dev), src.to(dev), dst.to(dev), shifts.to(dev),
                             cell.float().to(dev))
    perm = torch.randperm(src.numel())
    shuf = energy_and_forces(model, pos.to(dev), z.to(dev), batch.to(dev), src[perm].to(dev), dst[perm].to(dev),
                             shifts[perm].to(dev), cell.float().to(dev))
    assert _rel(shuf["forces"], base["forces"]) < TOL and _rel(shuf["energy"], base["energy"]) < TOL
    mask = (torch.arange(n) % 2 == 0).float().to(dev)
    half = energy_and_forces(model, pos.to(dev), z.to(dev), batch.to(dev), src.to(dev), dst.to(dev), shifts.to(dev),
                             cell.float().to(dev), owned_mask=mask)
    assert _rel(half["energy"], (base["atomic_energy"] * mask).sum().reshape(1)) < TOL
    with pytest.raises(ValueError):
        create_model(channels=32, lmax=3)
    with pytest.raises(ValueError):
        energy_and_forces(model, pos.to(dev)[:, :2], z.to(dev), batch.to(dev), src.to(dev), dst.to(dev),
                          shifts.to(dev), cell.float().to(dev))
