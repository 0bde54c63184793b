"""Tensor-core radial MLP (error-compensated TF32) against an fp64 evaluation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("edges,nb,nout", [(1000, 8, 704), (257, 8, 192), (128, 5, 64), (1, 8, 704), (70000, 8, 704)])
def test_radial_mlp_forward_backward(edges, nb, nout):
    from ictc_o3 import _lib
    lib = _lib.load()
    torch.manual_seed(edges)
    scale = 1.6791767923989418
    rb = (torch.randn(edges, nb) * 0.7).cuda()
    ws = [torch.randn(64, nb) / nb ** 0.5, torch.randn(64, 64) / 8, torch.randn(64, 64) / 8, torch.randn(nout, 64) / 8]
    ws = [w.cuda().contiguous() for w in ws]
    wt = [w.t().contiguous() for w in ws]
    def split(w):
        out = torch.empty(*w.shape, 2, device="cuda")
        _lib.check(lib.ictc_split_tf32(w.numel(), w.data_ptr(), out.data_ptr(), None), "split")
        return out
    w3s, w3ts = split(ws[3]), split(wt[3])
    assert float((w3s.sum(-1) - ws[3]).abs().max()) < 1e-6 * float(ws[3].abs().max())   # big + small ~ w to 2^-21
    gates = torch.empty(edges, nout, device="cuda")
    zs = [torch.empty(edges, 64, device="cuda") for _ in range(3)]
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.ictc_radial_mlp_forward(edges, nb, nout, rb.data_ptr(), *[w.data_ptr() for w in ws[:3]],
                                           w3s.data_ptr(), gates.data_ptr(), *[z.data_ptr() for z in zs], st), "fwd")
    x = rb.double().cpu().requires_grad_(True)
    h = x
    ref_z = []
    for k, w in enumerate(ws):
        h = h @ w.double().cpu().t()
        if k < 3:
            ref_z.append(h)
            h = torch.nn.functional.silu(h) * scale
    err = float((gates.double().cpu() - h.detach()).abs().max() / h.detach().abs().max())
    print('fwd err', err)
    assert err < 4e-6, err
    for z, r in zip(zs, ref_z):
        assert float((z.double().cpu() - r).abs().max() / r.abs().max()) < 2e-6
    dg = torch.randn(edges, nout)
    (ref_d,) = torch.autograd.grad((h * dg.double()).sum(), x)
    drb = torch.empty(edges, nb, device="cuda")
    dgd = dg.cuda()
    _lib.check(lib.ictc_radial_mlp_backward(edges, nb, nout, dgd.data_ptr(), *[w.data_ptr() for w in wt[:3]],
                                            w3ts.data_ptr(), *[z.data_ptr() for z in zs], drb.data_ptr(), st), "bwd")
    err = float((drb.double().cpu() - ref_d).abs().max() / ref_d.abs().max())
    print('bwd err', err)
    assert err < 1e-5, err
    assert lib.ictc_radial_mlp_forward(10, 9, 704, *([None] * 10), None) == -1
    assert lib.ictc_radial_mlp_forward(10, 8, 100, *([None] * 10), None) == -1
