"""GPU parity of the symmetric contraction (forward, first adjoints, mixed second derivatives) against
the CPU oracle's restatement of the reference recursion with the reference's U tensors."""
import pytest
import torch

from oracle import ictc_oracle as O

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


def _oracle_weights(module):
    return {l: [w.detach().double().cpu().requires_grad_(True) for w in c.by_order()]
            for l, c in enumerate(module.symmetric_contractions.contractions)}


@pytest.mark.parametrize("target_lmax,channels,nodes,species", [(2, 64, 257, 4), (0, 64, 300, 3), (2, 8, 5, 1),
                                                                (0, 40, 130, 2)])
def test_sc_forward_first_and_second(target_lmax, channels, nodes, species):
    from ictc_o3 import create_symmetric_contraction
    torch.manual_seed(7 + nodes)
    sc = create_symmetric_contraction(num_elements=species, lmax=2, target_lmax=target_lmax, channels=channels)
    x = torch.randn(nodes, channels, 9, dtype=torch.float64) * 0.7
    idx = torch.randint(0, species, (nodes,))
    cot = torch.randn(nodes, channels * (target_lmax + 1) ** 2, dtype=torch.float64)
    # oracle (fp64, mul_ir rows: degree block [C, 2l+1])
    xr = x.clone().requires_grad_(True)
    wr = _oracle_weights(sc)
    ref = O.symmetric_contraction(xr, idx, wr, target_lmax)
    flat_w = [w for l in sorted(wr) for w in wr[l]]
    rg = torch.autograd.grad((ref * cot).sum(), [xr] + flat_w, create_graph=True)
    # device
    def to_flat(t):   # [N,C,9] -> mul_ir rows
        return torch.cat([t[:, :, l * l:(l + 1) ** 2].reshape(nodes, -1) for l in range(3)], -1)
    xd = to_flat(x).float().cuda().requires_grad_(True)
    out = sc(xd, None, idx.cuda())
    assert _rel(out, ref) < TOL
    params = [w for c in sc.symmetric_contractions.contractions for w in c.by_order()]
    dg = torch.autograd.grad((out * cot.float().cuda()).sum(), [xd] + params, create_graph=True)
    assert _rel(dg[0], to_flat(rg[0])) < TOL
    for a, b in zip(dg[1:], rg[1:]):
        assert _rel(a, b) < TOL
    # force-loss-like scalar of the feature gradient -> mixed second derivatives wrt features and weights
    r2 = torch.autograd.grad(rg[0].square().sum() + sum((g * g).sum() for g in rg[1:]), [xr] + flat_w)
    d2 = torch.autograd.grad(dg[0].square().sum() + sum((g * g).sum() for g in dg[1:]), [xd] + params)
    assert _rel(d2[0], to_flat(r2[0])) < 2 * TOL
    for a, b in zip(d2[1:], r2[1:]):
        assert _rel(a, b) < 2 * TOL


def test_sc_full_size_properties():
    """BASELINE configuration 3 (262,144 nodes, C64, 4 species): homogeneity per order and bitwise
    repeatability (no float atomics in the weight-gradient reduction)."""
    from ictc_o3 import create_symmetric_contraction
    torch.manual_seed(0)
    n, c = 262144, 64
    sc = create_symmetric_contraction(num_elements=4, lmax=2, target_lmax=2, channels=c)
    x = torch.randn(n, 9 * c, device="cuda").requires_grad_(True)
    idx = torch.randint(0, 4, (n,), device="cuda")
    y1 = sc(x, None, idx)
    # y(t x) = t y_1 + t^2 y_2 + t^3 y_3 : check the cubic through three scalings
    with torch.no_grad():
        ys = {t: sc(t * x, None, idx) for t in (2.0, -1.0)}
        # y(2x) + y(-x)... eliminate orders: y(2x) - 8*y(x) = -6 y1' - 4 y2' where primes are order parts
        a = ys[2.0] - 8 * y1          # = -6*o1 - 4*o2
        b = ys[-1.0] + y1             # = 2*o2
        o2 = b / 2
        o1 = (a + 4 * o2) / -6
        o3 = y1 - o1 - o2
        t = 0.5
        pred = t * o1 + t * t * o2 + t ** 3 * o3
        got = sc(t * x, None, idx)
        assert float((got - pred).abs().max()) < 2e-4 * float(got.abs().max())
    params = list(sc.parameters())
    g1 = torch.autograd.grad(y1.square().mean(), [x] + params, retain_graph=True)
    g2 = torch.autograd.grad(y1.square().mean(), [x] + params)
    for a, b in zip(g1, g2):
        assert torch.equal(a, b)
