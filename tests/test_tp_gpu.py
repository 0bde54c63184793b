"""GPU parity of the tensor product, graph message and harmonics kernels against the CPU oracle.

Tolerance (stated by the task): fp32 kernel result within 1e-5 relative (max|d| / max|ref|) of the
fp64 oracle.  All calls go through the public operators, i.e. through the C ABI.
"""
import os

import numpy as np
import pytest
import torch

from oracle import ictc_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-5


@pytest.fixture(autouse=True)
def _kernel_status_is_clean():
    """No kernel may have given up on a bounded wait."""
    yield
    from ictc_o3 import _lib
    assert _lib.kernel_status() == 0


def _rel(a, b, floor=None):
    """max|a-b| / max|b|; ``floor`` (a tensor of the same problem) bounds the denominator from below
    for references that vanish by symmetry."""
    a = a.detach().double().cpu()
    b = b.detach().double().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    scale = b.abs().max()
    if floor is not None:
        scale = torch.maximum(scale, floor.detach().double().abs().max().cpu())
    return float((a - b).abs().max() / scale.clamp_min(1e-30))


def _load(golden_dir, name):
    with np.load(os.path.join(golden_dir, name + ".npz")) as d:
        return {k: np.array(d[k]) for k in d.files}


def _dev(a, grad=False):
    t = torch.as_tensor(np.asarray(a), dtype=torch.float32).cuda()
    return t.requires_grad_(True) if grad else t


@pytest.mark.parametrize("name", ["tp_c8_l222_e37", "tp_c8_l022_e19", "tp_c5_l111_e13_w", "tp_cfg1_c32_l222_e257"])
@pytest.mark.parametrize("layout", ["ir_mul", "mul_ir"])
def test_edge_tp_against_reference_golden(golden_dir, name, layout):
    """Forward, first gradients and force-loss-like mixed second gradients vs the reference's output."""
    from ictc_o3 import EdgeTensorProduct, direction_harmonics
    g = _load(golden_dir, name)
    c, lin, ledge, lout, keep = (int(g[k]) for k in ("channels", "lin", "ledge", "lout", "rows_kept"))
    tp = EdgeTensorProduct.create(input_lmax=lin, edge_lmax=ledge, output_lmax=lout, channels=c, layout=layout)
    assert [list(p) for p in tp.paths] == g["paths"].tolist()
    with torch.no_grad():
        tp.tp.weight.copy_(_dev(g["weight"]))
    blocks = {l: _dev(g[f"x{l}"], True) for l in range(lin + 1)}
    vec, gates = _dev(g["vec"], True), _dev(g["gates"], True)
    sh = torch.cat(direction_harmonics(torch.nn.functional.normalize(vec, dim=-1), ledge), -1)
    assert _rel(sh[::keep], torch.as_tensor(g["sh"])) < TOL
    out = tp(tp.pack_input(blocks), sh, gates)
    assert out.shape == (vec.shape[0], tp.output_width)
    parts = tp.unpack_output(out)
    for l, v in parts.items():
        if f"out{l}" in g:
            assert _rel(v[::keep], torch.as_tensor(g[f"out{l}"])) < TOL
    loss = out.square().mean()
    assert abs(float(loss.detach()) - float(g["loss"])) < 1e-5 * abs(float(g["loss"]))
    inputs = [blocks[l] for l in range(lin + 1)] + [vec, gates]
    first = torch.autograd.grad(loss, inputs, create_graph=True)
    for l in range(lin + 1):
        assert _rel(first[l][::keep], torch.as_tensor(g[f"dx{l}"])) < TOL
    assert _rel(first[-2][::keep], torch.as_tensor(g["dvec"]), torch.as_tensor(g["dgates"])) < TOL
    assert _rel(first[-1][::keep], torch.as_tensor(g["dgates"])) < TOL
    loss2 = sum((v * v).sum() for v in first)
    second = torch.autograd.grad(loss2, inputs)
    for l in range(lin + 1):
        assert _rel(second[l][::keep], torch.as_tensor(g[f"ddx{l}"])) < 2 * TOL
    assert _rel(second[-2][::keep], torch.as_tensor(g["ddvec"]), torch.as_tensor(g["ddgates"])) < 2 * TOL
    assert _rel(second[-1][::keep], torch.as_tensor(g["ddgates"])) < 2 * TOL


@pytest.mark.parametrize("name", ["message_c8_l2_n23_e120", "message_c8_l0_n17_e90"])
def test_graph_message_against_reference_golden(golden_dir, name):
    """Unsorted, repeated receivers + fixed mask + non-unit base coefficients."""
    from ictc_o3 import PackedGraphMessage, direction_harmonics
    from ictc_o3.basis.ictd_irreps import EdgeWeightedPathPreservingTensorProduct
    g = _load(golden_dir, name)
    c, lin = int(g["channels"]), int(g["lin"])
    paths = [tuple(int(v) for v in p) for p in g["paths"]]
    mod = EdgeWeightedPathPreservingTensorProduct(c, 2, allowed_paths=paths).cuda()
    with torch.no_grad():
        mod.weight.copy_(_dev(g["weight"]))
    mod.weight.requires_grad_(False)
    op = PackedGraphMessage(mod, input_lmax=lin, edge_lmax=2)
    x, vec, gate = _dev(g["x"], True), _dev(g["vec"], True), _dev(g["g"], True)
    src, dst = torch.as_tensor(g["src"]).cuda(), torch.as_tensor(g["dst"]).cuda()
    sh = torch.cat(direction_harmonics(torch.nn.functional.normalize(vec, dim=-1), 2), -1)
    out = op(x, sh, gate, src, dst, _dev(g["mask"]))
    assert _rel(out, torch.as_tensor(g["out"])) < TOL
    first = torch.autograd.grad((out * _dev(g["cot"])).sum(), [x, vec, gate], create_graph=True)
    for v, key in zip(first, ("dx", "dvec", "dg")):
        assert _rel(v, torch.as_tensor(g[key])) < TOL, key
    second = torch.autograd.grad(sum((v * v).sum() for v in first), [x, vec, gate])
    for v, key in zip(second, ("ddx", "ddvec", "ddg")):
        assert _rel(v, torch.as_tensor(g[key])) < 2 * TOL, key
    # bitwise reproducible: no atomics anywhere in the reduction
    out2 = op(x, sh, gate, src, dst, _dev(g["mask"]))
    assert torch.equal(out, out2)


def _random_graph(n, e, seed, sorted_dst):
    gen = torch.Generator().manual_seed(seed)
    src = torch.randint(0, n, (e,), generator=gen)
    dst = torch.randint(0, n, (e,), generator=gen)
    if sorted_dst:
        dst, perm = torch.sort(dst, stable=True)
        src = src[perm]
    return src, dst


@pytest.mark.parametrize("channels,lin,n,e,sorted_dst", [
    (64, 2, 300, 9000, True), (64, 0, 300, 9000, True), (32, 2, 50, 700, False), (40, 2, 64, 900, True),
    (96, 2, 40, 500, False), (64, 2, 10, 0, True), (64, 2, 33, 5, False)])
def test_graph_message_against_oracle(channels, lin, n, e, sorted_dst):
    """Sizes the oracle finishes in seconds: C64 paths of both interaction layers, ragged channel
    counts (40, 96), empty edge list, receivers without edges."""
    from ictc_o3 import PackedGraphMessage
    torch.manual_seed(n + e + channels)
    op = PackedGraphMessage.create(channels=channels, input_lmax=lin, edge_lmax=2, output_lmax=2)
    paths = [tuple(p) for p in op.edge.paths]
    tp = O.TensorProduct(channels, 2, paths)
    src, dst = _random_graph(n, e, 5, sorted_dst)
    x = torch.randn(n, channels * (lin + 1) ** 2, dtype=torch.float64)
    vec = torch.nn.functional.normalize(torch.randn(e, 3, dtype=torch.float64), dim=-1)
    gate = torch.randn(e, len(paths) * channels, dtype=torch.float64)
    cot = torch.randn(n, op.output_width, dtype=torch.float64)
    xr, shr, gr = (t.clone().requires_grad_(True) for t in (x, torch.cat(O.direction_harmonics(vec, 2), -1), gate))
    xd, shd, gd = (t.detach().float().cuda().requires_grad_(True) for t in (xr, shr, gr))
    out = op(xd, shd, gd, src.cuda(), dst.cuda())
    if e == 0:
        assert out.shape == (n, op.output_width) and float(out.detach().abs().max()) == 0.0
        return
    ref = O.graph_message(tp, xr, shr, gr.reshape(e, len(paths), channels), torch.ones(len(paths), channels, dtype=torch.float64),
                          src, dst, None, lin, 2)
    assert _rel(out, ref) < TOL
    rgrads = torch.autograd.grad((ref * cot).sum(), [xr, shr, gr])
    dgrads = torch.autograd.grad((out * cot.float().cuda()).sum(), [xd, shd, gd])
    for a, b in zip(dgrads, rgrads):
        assert _rel(a, b) < TOL


def test_graph_message_is_linear_and_matches_edge_rows_at_full_size():
    """BASELINE-sized property checks (no oracle): C64, 65,536 nodes, ~38 edges per node.

    (1) trilinearity: F(a*x1 + x2) = a*F(x1) + F(x2); (2) scatter consistency: the node rows equal the
    segment sums of the edge-owned product; (3) adjoint consistency <v, F(x)> = <A_x(v), x>.
    """
    from ictc_o3 import EdgeTensorProduct, PackedGraphMessage
    torch.manual_seed(0)
    n, deg, c = 65536, 38, 64
    e = n * deg
    op = PackedGraphMessage.create(channels=c, input_lmax=2, edge_lmax=2, output_lmax=2)
    dst = torch.arange(n, device="cuda").repeat_interleave(deg)
    src = torch.randint(0, n, (e,), device="cuda")
    x1 = torch.randn(n, 9 * c, device="cuda")
    x2 = torch.randn(n, 9 * c, device="cuda")
    sh = torch.randn(e, 9, device="cuda")
    g = torch.randn(e, 11 * c, device="cuda")
    f1, f2 = op(x1, sh, g, src, dst), op(x2, sh, g, src, dst)
    f12 = op(0.5 * x1 + x2, sh, g, src, dst)
    scale = float(f12.abs().max())
    assert float((f12 - (0.5 * f1 + f2)).abs().max()) < 2e-5 * scale
    # scatter consistency on a slice of receivers (edge rows of the first 4096 nodes)
    m = 4096
    edge = EdgeTensorProduct(op.tp, input_lmax=2, edge_lmax=2)
    rows = edge(x1[src[:m * deg]], sh[:m * deg], g[:m * deg]).reshape(m, deg, -1).sum(1)
    assert float((rows - f1[:m]).abs().max()) < 2e-5 * float(f1[:m].abs().max())
    # adjoint identity
    xg = x1.clone().requires_grad_(True)
    v = torch.randn_like(f1)
    out = op(xg, sh, g, src, dst)
    (dx,) = torch.autograd.grad((out * v).sum(), xg)
    lhs = float((out.detach().double() * v.double()).sum())
    rhs = float((dx.double() * x1.double()).sum())
    assert abs(lhs - rhs) < 1e-5 * abs(lhs)


def test_harmonics_first_and_second(golden_dir):
    from ictc_o3 import direction_harmonics
    g = _load(golden_dir, "harmonics_l2_e41")
    n = _dev(g["n"], True)
    y = torch.cat(direction_harmonics(n, 2), -1)
    assert _rel(y, torch.as_tensor(g["y"])) < TOL
    (dn,) = torch.autograd.grad((y * _dev(g["cot"])).sum(), n, create_graph=True)
    assert _rel(dn, torch.as_tensor(g["dn"])) < TOL
    # second order against the oracle's autograd
    nr = torch.as_tensor(g["n"]).requires_grad_(True)
    cr = torch.as_tensor(g["cot"]).requires_grad_(True)
    yr = torch.cat(O.direction_harmonics(nr, 2), -1)
    (dr,) = torch.autograd.grad((yr * cr).sum(), nr, create_graph=True)
    ref2 = torch.autograd.grad(dr.square().sum(), [nr, cr])
    cot = _dev(g["cot"], True)
    y2 = torch.cat(direction_harmonics(n, 2), -1)
    (d2,) = torch.autograd.grad((y2 * cot).sum(), n, create_graph=True)
    got2 = torch.autograd.grad(d2.square().sum(), [n, cot])
    for a, b in zip(got2, ref2):
        assert _rel(a, b) < TOL
    for lmax in (0, 1):
        yl = torch.cat(direction_harmonics(n.detach(), lmax), -1)
        assert _rel(yl, torch.as_tensor(g["y"])[:, :(lmax + 1) ** 2]) < TOL


def test_csr_build_matches_stable_sort():
    from ictc_o3.ops.topology import build_csr
    gen = torch.Generator().manual_seed(1)
    for n, e in ((1, 1), (7, 100), (5000, 200000), (70000, 10), (3, 0)):
        keys = torch.randint(0, n, (e,), generator=gen)
        rowptr, order = build_csr(keys.cuda(), n)
        counts = torch.bincount(keys, minlength=n)
        assert torch.equal(rowptr.cpu(), torch.cat([torch.zeros(1, dtype=torch.int64), counts.cumsum(0)]))
        expect = torch.sort(keys, stable=True)[1]
        if order is None:
            assert torch.equal(expect, torch.arange(e))
        else:
            assert torch.equal(order.cpu(), expect)
    keys = torch.sort(torch.randint(0, 100, (5000,), generator=gen))[0]
    rowptr, order = build_csr(keys.cuda(), 100)
    assert order is None
    with pytest.raises(ValueError):
        build_csr(torch.tensor([0, 5, 1]).cuda(), 3)


def test_public_api_validation():
    from ictc_o3 import EdgeTensorProduct
    with pytest.raises(ValueError):
        EdgeTensorProduct.create(input_lmax=2, edge_lmax=2, channels=0)
    with pytest.raises(ValueError):
        EdgeTensorProduct.create(input_lmax=2, edge_lmax=2, channels=8, device="cpu")
    with pytest.raises(ValueError):
        EdgeTensorProduct.create(input_lmax=2, edge_lmax=2, channels=8, layout="bad")
    tp = EdgeTensorProduct.create(input_lmax=2, edge_lmax=2, channels=8)
    assert tp.gate_width == 88 and tp.output_width == 280 and len(tp.paths) == 11
    x = torch.randn(4, 72, device="cuda")
    with pytest.raises(ValueError):
        tp(x, torch.randn(4, 8, device="cuda"), torch.randn(4, 88, device="cuda"))
    with pytest.raises(ValueError):
        tp(x.double(), torch.randn(4, 9, device="cuda"), torch.randn(4, 88, device="cuda"))
    out = tp(x[:0], torch.randn(0, 9, device="cuda"), torch.randn(0, 88, device="cuda"))
    assert out.shape == (0, 280)


def test_bounded_wait_gives_up_and_reports_without_a_fault():
    """A wait that nothing satisfies runs out after its (short) limit, the kernel returns normally, the status word
    carries the code, resetting it works and the context keeps computing; an MD driver turns a non-zero status into
    an exception instead of silently using the step's results."""
    from ictc_o3 import _lib
    lib = _lib.load()
    assert _lib.kernel_status() == 0
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.ictc_selftest_bounded_wait(200000, 77, st), "selftest")          # ~0.1 ms of polling
    assert _lib.kernel_status(reset=False) == 77
    from mace_ictc.md import MolecularDynamics
    with pytest.raises(RuntimeError, match="gave up a bounded wait"):
        MolecularDynamics.check_kernels(None)
    assert _lib.kernel_status() == 0                                                  # the check above reset it
    x = torch.arange(8, device="cuda").float()
    assert float((x * 2).sum()) == 56.0                                               # the context is alive
    assert lib.ictc_selftest_bounded_wait(0, 77, st) == -2 and lib.ictc_selftest_bounded_wait(1000, 0, st) == -2


def test_graph_message_layouts_and_channel_linear_on_the_tensor_cores():
    """GraphMessage converts its dictionaries with the one-launch layout kernel for 'fused_pack' / 'canonical' and with
    reshapes for 'packed': same values and gradients; channel_linear with a 64-wide side runs on the tcgen05 kernel:
    values and both gradients against float64."""
    from ictc_o3 import EdgeTensorProduct, GraphMessage, channel_linear, direction_harmonics
    torch.manual_seed(4)
    n, e, c = 37, 210, 64
    seed = EdgeTensorProduct.create(input_lmax=2, edge_lmax=2, channels=c)
    feats = {l: torch.randn(n, c, 2 * l + 1, device="cuda", requires_grad=True) for l in range(3)}
    unit = torch.nn.functional.normalize(torch.randn(e, 3, device="cuda"), dim=-1)
    harm = {l: y.unsqueeze(1) for l, y in enumerate(direction_harmonics(unit, 2))}
    gates = torch.randn(e, seed.gate_width, device="cuda", requires_grad=True)
    src, dst = torch.randint(0, n, (e,), device="cuda"), torch.randint(0, n, (e,), device="cuda")
    outs = {}
    for layout in ("packed", "fused_pack", "canonical"):
        op = GraphMessage(seed.tp, input_lmax=2, edge_lmax=2, layout=layout)
        out = op(feats, harm, gates, src, dst)
        grads = torch.autograd.grad(sum((o * o).sum() for o in out.values()), list(feats.values()) + [gates])
        outs[layout] = ([out[l] for l in range(3)], grads)
    for layout in ("fused_pack", "canonical"):
        for a, b in zip(outs[layout][0] + list(outs[layout][1]), outs["packed"][0] + list(outs["packed"][1])):
            assert a.shape == b.shape and float((a - b).abs().max()) <= 1e-6 * float(b.abs().max())
    for cin, cout, m in ((64, 64, 5), (64, 192, 3), (256, 64, 1)):
        x = torch.randn(23, cin, m, device="cuda", requires_grad=True)
        w = (torch.randn(cout, cin, device="cuda") / cin ** 0.5).requires_grad_(True)
        y = channel_linear(x, w)
        cot = torch.randn_like(y)
        gx, gw = torch.autograd.grad((y * cot).sum(), [x, w])
        xr, wr = x.detach().double().cpu().requires_grad_(True), w.detach().double().cpu().requires_grad_(True)
        yr = torch.einsum("oi,nim->nom", wr, xr)
        rx, rw = torch.autograd.grad((yr * cot.double().cpu()).sum(), [xr, wr])
        for got, want in ((y, yr), (gx, rx), (gw, rw)):
            assert float((got.double().cpu() - want).abs().max() / want.abs().max()) < 5e-6
