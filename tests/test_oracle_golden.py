"""The CPU oracle against the golden vectors produced by the reference's own torch code."""
import os

import numpy as np
import pytest
import torch

from oracle import ictc_oracle as O

F64 = torch.float64


def _load(golden_dir, name):
    with np.load(os.path.join(golden_dir, name + ".npz")) as d:
        return {k: np.array(d[k]) for k in d.files}


def _t(a):
    return torch.as_tensor(np.asarray(a, dtype=np.float64))


def _close(a, b, tol=1e-11):
    a, b = np.asarray(a), np.asarray(b)
    scale = max(1.0, float(np.abs(b).max()))
    assert a.shape == b.shape
    assert float(np.abs(a - b).max()) <= tol * scale


@pytest.mark.parametrize("name", ["tp_c8_l222_e37", "tp_c8_l022_e19", "tp_c5_l111_e13_w", "tp_cfg1_c32_l222_e257"])
def test_edge_tp_first_and_second(golden_dir, name):
    g = _load(golden_dir, name)
    c, lin, ledge, lout, keep = (int(g[k]) for k in ("channels", "lin", "ledge", "lout", "rows_kept"))
    paths = [tuple(int(v) for v in p) for p in g["paths"]]
    assert paths == O.natural_paths(lin, ledge, lout)
    tp = O.TensorProduct(c, max(lin, ledge, lout), paths)
    blocks = {l: _t(g[f"x{l}"]).requires_grad_(True) for l in range(lin + 1)}
    vec = _t(g["vec"]).requires_grad_(True)
    gates = _t(g["gates"]).requires_grad_(True)
    n = torch.nn.functional.normalize(vec, dim=-1)
    sh = O.direction_harmonics(n, ledge)
    _close(torch.cat(sh, -1).detach().numpy()[::keep], g["sh"])
    out = tp(blocks, {l: sh[l] for l in range(ledge + 1)}, gates.reshape(-1, len(paths), c), _t(g["weight"]))
    for l, v in out.items():
        _close(v.detach().numpy()[::keep], g[f"out{l}"])
    loss = sum(v.square().sum() for v in out.values()) / sum(v.numel() for v in out.values())
    assert abs(float(loss.detach()) - float(g["loss"])) < 1e-12
    inputs = [blocks[l] for l in range(lin + 1)] + [vec, gates]
    first = torch.autograd.grad(loss, inputs, create_graph=True)
    for l in range(lin + 1):
        _close(first[l].detach().numpy()[::keep], g[f"dx{l}"])
    _close(first[-2].detach().numpy()[::keep], g["dvec"])
    _close(first[-1].detach().numpy()[::keep], g["dgates"])
    loss2 = sum((v * v).sum() for v in first)
    second = torch.autograd.grad(loss2, inputs)
    for l in range(lin + 1):
        _close(second[l].numpy()[::keep], g[f"ddx{l}"])
    _close(second[-2].numpy()[::keep], g["ddvec"])
    _close(second[-1].numpy()[::keep], g["ddgates"])


@pytest.mark.parametrize("name", ["message_c8_l2_n23_e120", "message_c8_l0_n17_e90"])
def test_graph_message(golden_dir, name):
    g = _load(golden_dir, name)
    c, lin = int(g["channels"]), int(g["lin"])
    paths = [tuple(int(v) for v in p) for p in g["paths"]]
    tp = O.TensorProduct(c, 2, paths)
    x = _t(g["x"]).requires_grad_(True)
    vec = _t(g["vec"]).requires_grad_(True)
    gate = _t(g["g"]).requires_grad_(True)
    src, dst = torch.as_tensor(g["src"]), torch.as_tensor(g["dst"])
    sh = torch.cat(O.direction_harmonics(torch.nn.functional.normalize(vec, dim=-1), 2), -1)
    _close(sh.detach().numpy(), g["sh"])
    out = O.graph_message(tp, x, sh, gate, _t(g["weight"]), src, dst, _t(g["mask"]), lin, 2, layout="ir_mul")
    _close(out.detach().numpy(), g["out"])
    first = torch.autograd.grad((out * _t(g["cot"])).sum(), [x, vec, gate], create_graph=True)
    for v, key in zip(first, ("dx", "dvec", "dg")):
        _close(v.detach().numpy(), g[key])
    second = torch.autograd.grad(sum((v * v).sum() for v in first), [x, vec, gate])
    for v, key in zip(second, ("ddx", "ddvec", "ddg")):
        _close(v.numpy(), g[key], tol=1e-10)


def test_direction_harmonics(golden_dir):
    g = _load(golden_dir, "harmonics_l2_e41")
    n = _t(g["n"]).requires_grad_(True)
    y = torch.cat(O.direction_harmonics(n, 2), -1)
    _close(y.detach().numpy(), g["y"])
    dn = torch.autograd.grad((y * _t(g["cot"])).sum(), n)[0]
    _close(dn.numpy(), g["dn"])
    # component normalisation: |Y_l|^2 = 2l+1 on the unit sphere; l=1 is sqrt(3)*(z,y,x)
    yv = y.detach()
    assert torch.allclose((yv[:, 1:4] ** 2).sum(-1), torch.full((41,), 3.0, dtype=F64))
    assert torch.allclose((yv[:, 4:9] ** 2).sum(-1), torch.full((41,), 5.0, dtype=F64))
    assert torch.allclose(yv[:, 1:4], n.detach()[:, [2, 1, 0]] * 3 ** 0.5)


def test_layout_round_trips():
    torch.manual_seed(0)
    blocks = {l: torch.randn(7, 4, 2 * l + 1, dtype=F64) for l in range(3)}
    flat = O.features_to_ir_mul(blocks)
    back = O.features_from_ir_mul(flat, 4, 2)
    for l in blocks:
        assert torch.equal(back[l], blocks[l])
    flat2 = O.features_to_mul_ir(blocks)
    back2 = O.features_from_mul_ir(flat2, 4, 2)
    for l in blocks:
        assert torch.equal(back2[l], blocks[l])
    counts = {0: 3, 1: 4, 2: 4}
    outs = {l: torch.randn(7, counts[l] * 4, 2 * l + 1, dtype=F64) for l in range(3)}
    f = O.output_to_ir_mul(outs, 4)
    rb = O.output_from_ir_mul(f, 4, counts)
    for l in outs:
        assert torch.equal(rb[l], outs[l])


def test_symmetric_contraction_equivariant_scalar_output():
    """The scalar (lout=0) contraction of a rotated input equals that of the original input.

    Rotation acts on the l=1 block (stored z,y,x) as a proper rotation and on the l=2 block through
    the harmonics; instead of building the l=2 rotation matrix we compare node features built from
    harmonics of rotated directions, which transform covariantly by construction.
    """
    torch.manual_seed(3)
    c, s = 3, 2
    dirs = torch.nn.functional.normalize(torch.randn(5, 6, 3, dtype=F64), dim=-1)
    amp = torch.randn(5, 6, c, dtype=F64)
    q, _ = torch.linalg.qr(torch.randn(3, 3, dtype=F64))
    if torch.det(q) < 0:
        q[:, 0] = -q[:, 0]

    def feats(d):
        y = torch.cat(O.direction_harmonics(d, 2), -1)          # [5,6,9]
        return torch.einsum("nkc,nkh->nch", amp, y)             # [5,c,9]

    species = torch.tensor([0, 1, 1, 0, 1])
    t = O.tables()
    weights = {0: [torch.randn(s, t[f"u_0_{nu}"].shape[-1], c, dtype=F64) for nu in (1, 2, 3)]}
    a = O.symmetric_contraction(feats(dirs), species, weights, 0)
    b = O.symmetric_contraction(feats(dirs @ q.T), species, weights, 0)
    assert a.shape == (5, c)
    assert torch.allclose(a, b, atol=1e-10, rtol=1e-10)


@pytest.mark.parametrize("p", [5, 6])
def test_radial_embedding_matches_the_reference_function(golden_dir, p):
    """Bessel basis x polynomial cutoff of the model oracle against vectors computed by the reference's own
    `mace_radial_embedding` (tests/golden/make_golden_radial.py), values and derivative."""
    from oracle.model_oracle import radial_embedding
    g = np.load(os.path.join(golden_dir, "radial_bessel8_rmax4p5.npz"))
    r = torch.tensor(g["r"], dtype=torch.float64, requires_grad=True)
    emb = radial_embedding(r, float(g["r_max"]), 8, p)
    assert torch.allclose(emb, torch.tensor(g[f"emb_p{p}"]), rtol=1e-12, atol=1e-13)
    (grad,) = torch.autograd.grad((emb * torch.tensor(g["w"])).sum(), r)
    assert torch.allclose(grad, torch.tensor(g[f"grad_p{p}"]), rtol=1e-11, atol=1e-12)
    assert float(emb[-2:].abs().max()) == 0.0          # beyond the cutoff
