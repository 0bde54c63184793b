"""Last layer of the gate MLP on the tcgen05 tensor cores (three-term TF32 split) against fp64."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SCALE = 1.6791767923989418


def _status(lib):
    import ctypes
    s = ctypes.c_int(0)
    assert lib.ictc_kernel_status(ctypes.byref(s), 1) == 0
    return s.value


def _pack(lib, w, transpose):
    from ictc_o3 import _lib
    out = torch.empty(2 * w.numel(), device="cuda")
    _lib.check(lib.ictc_gate_pack_weights(w.shape[0], w.data_ptr(), transpose, out.data_ptr(), None), "pack")
    return out


@pytest.mark.parametrize("rows,nout,act", [(128, 64, 0), (1000, 192, 1), (1, 704, 1), (70001, 704, 1), (148 * 128 * 3 + 5, 192, 0)])
def test_gate_gemm_forward(rows, nout, act):
    from ictc_o3 import _lib
    lib = _lib.load()
    torch.manual_seed(rows + nout)
    z3 = torch.randn(rows, 64).cuda()
    w3 = (torch.randn(nout, 64) / 8).cuda().contiguous()
    gates = torch.full((rows, nout), float("nan"), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.ictc_gate_gemm_forward(rows, nout, z3.data_ptr(), _pack(lib, w3, 0).data_ptr(), gates.data_ptr(),
                                          act, None, st), "fwd")
    assert _status(lib) == 0
    sample = torch.arange(0, rows, max(1, rows // 4000))
    h = z3[sample].double().cpu()
    if act:
        h = torch.nn.functional.silu(h) * SCALE
    ref = h @ w3.double().cpu().t()
    got = gates[sample].double().cpu()
    assert torch.isfinite(gates).all()
    err = float((got - ref).abs().max() / ref.abs().max())
    assert err < 2e-6, err


@pytest.mark.parametrize("rows,nout,paired", [(128, 64, False), (1000, 192, True), (1, 704, False), (70001, 704, True)])
def test_gate_gemm_backward(rows, nout, paired):
    from ictc_o3 import _lib
    lib = _lib.load()
    torch.manual_seed(rows + nout + 1)
    src_rows = 2 * rows + 3 if paired else rows
    dg = torch.randn(src_rows, nout).cuda()
    w3 = (torch.randn(nout, 64) / 8).cuda().contiguous()
    da3 = torch.full((rows, 64), float("nan"), device="cuda")
    if paired:
        pa = torch.randint(0, src_rows, (rows,)).cuda()
        pb = torch.randint(-1, src_rows, (rows,)).cuda()
        pa_p, pb_p = pa.data_ptr(), pb.data_ptr()
    else:
        pa_p = pb_p = None
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.ictc_gate_gemm_backward(rows, nout, dg.data_ptr(), pa_p, pb_p, _pack(lib, w3, 1).data_ptr(),
                                           da3.data_ptr(), None, st), "bwd")
    assert _status(lib) == 0
    sample = torch.arange(0, rows, max(1, rows // 4000))
    if paired:
        a, b = pa.cpu()[sample], pb.cpu()[sample]
        d = dg.cpu().double()
        summed = d[a] + torch.where((b >= 0)[:, None], d[b.clamp(min=0)], torch.zeros(1, dtype=torch.float64))
    else:
        summed = dg[sample].double().cpu()
    ref = summed @ w3.double().cpu()
    got = da3[sample].double().cpu()
    assert torch.isfinite(da3).all()
    err = float((got - ref).abs().max() / ref.abs().max())
    # K = num_out products per output, accumulated by the tensor cores without rounding to nearest
    assert err < 1e-5, err


def test_row_windows_match_the_whole_products_bit_for_bit():
    """Streamed gate evaluation: the forward over a window of an index list and the backward with scattered output
    rows give exactly the rows of the whole-table products; the window bounds are device scalars and an under-sized
    buffer truncates instead of overrunning."""
    from ictc_o3 import _lib
    lib = _lib.load()
    torch.manual_seed(12)
    pairs, edges, nout = 900, 1700, 704
    z3 = torch.randn(pairs, 64).cuda()
    w3 = (torch.randn(nout, 64) / 8).cuda().contiguous()
    packed, packed_t = _pack(lib, w3, 0), _pack(lib, w3, 1)
    st = torch.cuda.current_stream().cuda_stream
    table = torch.empty(pairs, nout, device="cuda")
    _lib.check(lib.ictc_gate_gemm_forward(pairs, nout, z3.data_ptr(), packed.data_ptr(), table.data_ptr(), 1, None, st),
               "fwd")
    index = torch.randint(0, pairs, (edges,)).cuda()
    bounds = torch.tensor([0, 130, 131, 800, 1700], dtype=torch.int64, device="cuda")      # a CSR-like offset array
    cap = 700
    for k in range(4):
        lo, hi = int(bounds[k]), int(bounds[k + 1])
        buf = torch.full((cap, nout), float("nan"), device="cuda")
        _lib.check(lib.ictc_gate_gemm_forward_rows(cap, nout, z3.data_ptr(), index.data_ptr(), bounds.data_ptr() + 8 * k,
                                                   bounds.data_ptr() + 8 * (k + 1), packed.data_ptr(), buf.data_ptr(), 1,
                                                   st), "fwd rows")
        used = min(hi - lo, cap)
        assert torch.equal(buf[:used], table[index[lo:lo + used]])
        assert bool(torch.isnan(buf[used:]).all())
    # identity index (no pairing): row = list entry
    buf = torch.empty(cap, nout, device="cuda")
    _lib.check(lib.ictc_gate_gemm_forward_rows(cap, nout, z3.data_ptr(), None, bounds.data_ptr() + 8, bounds.data_ptr() + 24,
                                               packed.data_ptr(), buf.data_ptr(), 1, st), "fwd rows id")
    assert torch.equal(buf[:669], table[130:799])
    # backward: chunk rows in, rows scattered through an index out
    dg = torch.randn(edges, nout).cuda()
    whole = torch.empty(edges, 64, device="cuda")
    _lib.check(lib.ictc_gate_gemm_backward(edges, nout, dg.data_ptr(), None, None, packed_t.data_ptr(), whole.data_ptr(),
                                           None, st), "bwd")
    order = torch.randperm(edges).cuda()
    out = torch.full((edges, 64), float("nan"), device="cuda")
    for k in range(4):
        lo, hi = int(bounds[k]), int(bounds[k + 1])
        if hi - lo > cap:
            continue
        chunk = dg[lo:hi].contiguous()
        _lib.check(lib.ictc_gate_gemm_backward_rows(cap, nout, chunk.data_ptr(), bounds.data_ptr() + 8 * k,
                                                    bounds.data_ptr() + 8 * (k + 1), order.data_ptr(),
                                                    packed_t.data_ptr(), out.data_ptr(), st), "bwd rows")
        assert torch.equal(out[order[lo:hi]], whole[lo:hi])
    assert _status(lib) == 0


def test_chain_backward_adds_the_two_edges_of_a_pair_on_load():
    from ictc_o3 import _lib
    lib = _lib.load()
    torch.manual_seed(13)
    pairs, edges, nb = 500, 900, 8
    ws = [w.cuda().contiguous() for w in (torch.randn(64, nb) / nb ** 0.5, torch.randn(64, 64) / 8, torch.randn(64, 64) / 8)]
    packed = [_pack(lib, ws[1], 0), _pack(lib, ws[2], 0), _pack(lib, ws[1], 1), _pack(lib, ws[2], 1)]
    st = torch.cuda.current_stream().cuda_stream
    rb = (torch.randn(pairs, nb) * 0.7).cuda()
    zs = [torch.empty(pairs, 64, device="cuda") for _ in range(3)]
    _lib.check(lib.ictc_mlp_chain_forward(pairs, nb, rb.data_ptr(), None, ws[0].data_ptr(), packed[0].data_ptr(),
                                          packed[1].data_ptr(), *[z.data_ptr() for z in zs], None, st), "fwd")
    per_edge = torch.randn(edges, 64).cuda()
    pa = torch.randint(0, edges, (pairs,)).cuda()
    pb = torch.randint(-1, edges, (pairs,)).cuda()
    summed = per_edge[pa] + torch.where((pb >= 0).unsqueeze(1), per_edge[pb.clamp(min=0)], torch.zeros((), device="cuda"))
    want = torch.empty(pairs, nb, device="cuda")
    _lib.check(lib.ictc_mlp_chain_backward(pairs, nb, summed.data_ptr(), ws[0].data_ptr(), packed[2].data_ptr(),
                                           packed[3].data_ptr(), *[z.data_ptr() for z in zs], want.data_ptr(), None, 0,
                                           None, st), "bwd")
    got = torch.empty(pairs, nb, device="cuda")
    _lib.check(lib.ictc_mlp_chain_backward_paired(pairs, nb, per_edge.data_ptr(), pa.data_ptr(), pb.data_ptr(),
                                                  ws[0].data_ptr(), packed[2].data_ptr(), packed[3].data_ptr(),
                                                  *[z.data_ptr() for z in zs], got.data_ptr(), None, 0, None, st),
               "bwd paired")
    assert _status(lib) == 0
    assert torch.equal(got, want)
    assert lib.ictc_gate_gemm_forward(10, 100, *([None] * 3), 1, None, None) == -1


@pytest.mark.parametrize("nodes,mm,cnt", [(777, 3, 4), (1000, 5, 4), (300, 1, 3), (513, 3, 1)])
def test_channel_linear_reads_and_writes_slot_major_blocks_in_place(nodes, mm, cnt):
    """Message linear (K = cnt * 64 -> 64) and its adjoint (64 -> cnt * 64) on a [node][slot][m][C] block that sits
    inside a wider row, against fp64 einsum."""
    from ictc_o3 import _lib
    lib = _lib.load()
    torch.manual_seed(nodes + mm)
    c, ld_wide, ld_narrow, off_wide, off_narrow = 64, 35 * 64, 9 * 64, 2 * 64, 64
    wide = torch.randn(nodes, ld_wide).cuda()
    w = (torch.randn(cnt * c, c) / 8).cuda()                  # [K = (slot, channel), N]
    st = torch.cuda.current_stream().cuda_stream
    # K-loop direction
    narrow = torch.zeros(nodes, ld_narrow, device="cuda")
    _lib.check(lib.ictc_channel_linear_tc(nodes * mm, cnt, 1, wide.data_ptr() + 4 * off_wide, mm, ld_wide,
                                          _pack(lib, w.contiguous(), 1).data_ptr(), narrow.data_ptr() + 4 * off_narrow,
                                          mm, ld_narrow, st), "lin")
    block = wide[:, off_wide:off_wide + cnt * mm * c].view(nodes, cnt, mm, c).double().cpu()
    ref = torch.einsum("nsic,scd->nid", block, w.view(cnt, c, c).double().cpu())
    got = narrow[:, off_narrow:off_narrow + mm * c].view(nodes, mm, c).double().cpu()
    assert float((got - ref).abs().max() / ref.abs().max()) < 5e-6
    assert float(narrow[:, :off_narrow].abs().max()) == 0 and float(narrow[:, off_narrow + mm * c:].abs().max()) == 0
    # N-wide direction (adjoint): narrow block -> wide block
    src = torch.randn(nodes, ld_narrow).cuda()
    dst = torch.zeros(nodes, ld_wide, device="cuda")
    wt = w.t().contiguous()                                   # [N = 64 in, cnt*64 out] used as x @ wt
    _lib.check(lib.ictc_channel_linear_tc(nodes * mm, 1, cnt, src.data_ptr() + 4 * off_narrow, mm, ld_narrow,
                                          _pack(lib, w.contiguous(), 0).data_ptr(), dst.data_ptr() + 4 * off_wide,
                                          mm, ld_wide, st), "lin adjoint")
    assert _status(lib) == 0
    x = src[:, off_narrow:off_narrow + mm * c].view(nodes, mm, c).double().cpu()
    ref = torch.einsum("nid,scd->nsic", x, w.view(cnt, c, c).double().cpu())
    got = dst[:, off_wide:off_wide + cnt * mm * c].view(nodes, cnt, mm, c).double().cpu()
    assert float((got - ref).abs().max() / ref.abs().max()) < 5e-6
    assert float(dst[:, :off_wide].abs().max()) == 0
    assert lib.ictc_channel_linear_tc(10, 2, 2, *([None] * 1), 1, 64, None, None, 1, 64, None) == -1


@pytest.mark.parametrize("edges,nb", [(1000, 8), (129, 5), (1, 8), (148 * 128 * 2 + 77, 8), (70001, 8)])
def test_mlp_chain_hidden_layers(edges, nb):
    """TMEM chain kernels of the hidden layers against fp64 (values and input gradient)."""
    from ictc_o3 import _lib
    lib = _lib.load()
    torch.manual_seed(edges + nb)
    rb = (torch.randn(edges, nb) * 0.7).cuda()
    ws = [torch.randn(64, nb) / nb ** 0.5, torch.randn(64, 64) / 8, torch.randn(64, 64) / 8]
    ws = [w.cuda().contiguous() for w in ws]
    st = torch.cuda.current_stream().cuda_stream
    zs = [torch.full((edges, 64), float("nan"), device="cuda") for _ in range(3)]
    packed = [_pack(lib, ws[1], 0), _pack(lib, ws[2], 0), _pack(lib, ws[1], 1), _pack(lib, ws[2], 1)]
    _lib.check(lib.ictc_mlp_chain_forward(edges, nb, rb.data_ptr(), None, ws[0].data_ptr(), packed[0].data_ptr(),
                                          packed[1].data_ptr(), *[z.data_ptr() for z in zs], None, st), "chain fwd")
    assert _status(lib) == 0
    x = rb.double().cpu().requires_grad_(True)
    h, ref = x, []
    for w in ws:
        z = h @ w.double().cpu().t()
        ref.append(z)
        h = torch.nn.functional.silu(z) * SCALE
    errs = [float((z.double().cpu() - r.detach()).abs().max() / r.detach().abs().max()) for z, r in zip(zs, ref)]
    assert all(torch.isfinite(z).all() for z in zs)
    assert max(errs) < 4e-6, errs
    da3 = torch.randn(edges, 64)
    (ref_d,) = torch.autograd.grad((h * da3.double()).sum(), x)
    drb = torch.full((edges, nb), float("nan"), device="cuda")
    da3d = da3.cuda()
    _lib.check(lib.ictc_mlp_chain_backward(edges, nb, da3d.data_ptr(), ws[0].data_ptr(), packed[2].data_ptr(),
                                           packed[3].data_ptr(), *[z.data_ptr() for z in zs], drb.data_ptr(),
                                           None, 0, None, st), "chain bwd")
    assert _status(lib) == 0
    assert torch.isfinite(drb).all()
    err = float((drb.double().cpu() - ref_d).abs().max() / ref_d.abs().max())
    assert err < 5e-6, err


def test_mlp_chain_row_indices_gather_and_scatter():
    """Row indices: the forward reads rb[rows[r]], the backward writes or adds to drb[rows[r]]."""
    from ictc_o3 import _lib
    lib = _lib.load()
    torch.manual_seed(3)
    total, edges, nb = 900, 400, 8
    rb = (torch.randn(total, nb) * 0.7).cuda()
    rows = torch.randperm(total)[:edges].cuda()
    ws = [w.cuda().contiguous() for w in (torch.randn(64, nb) / nb ** 0.5, torch.randn(64, 64) / 8, torch.randn(64, 64) / 8)]
    packed = [_pack(lib, ws[1], 0), _pack(lib, ws[2], 0), _pack(lib, ws[1], 1), _pack(lib, ws[2], 1)]
    st = torch.cuda.current_stream().cuda_stream
    za = [torch.empty(edges, 64, device="cuda") for _ in range(3)]
    zb = [torch.empty(edges, 64, device="cuda") for _ in range(3)]
    sub = rb[rows].contiguous()
    _lib.check(lib.ictc_mlp_chain_forward(edges, nb, sub.data_ptr(), None, ws[0].data_ptr(), packed[0].data_ptr(),
                                          packed[1].data_ptr(), *[z.data_ptr() for z in za], None, st), "fwd")
    _lib.check(lib.ictc_mlp_chain_forward(edges, nb, rb.data_ptr(), rows.data_ptr(), ws[0].data_ptr(),
                                          packed[0].data_ptr(), packed[1].data_ptr(), *[z.data_ptr() for z in zb], None, st),
               "fwd rows")
    for x, y in zip(za, zb):
        assert torch.equal(x, y)
    da3 = torch.randn(edges, 64, device="cuda")
    dense = torch.empty(edges, nb, device="cuda")
    _lib.check(lib.ictc_mlp_chain_backward(edges, nb, da3.data_ptr(), ws[0].data_ptr(), packed[2].data_ptr(),
                                           packed[3].data_ptr(), *[z.data_ptr() for z in za], dense.data_ptr(), None, 0,
                                           None, st), "bwd")
    out = torch.ones(total, nb, device="cuda")
    _lib.check(lib.ictc_mlp_chain_backward(edges, nb, da3.data_ptr(), ws[0].data_ptr(), packed[2].data_ptr(),
                                           packed[3].data_ptr(), *[z.data_ptr() for z in za], out.data_ptr(),
                                           rows.data_ptr(), 1, None, st), "bwd rows")
    assert _status(lib) == 0
    expect = torch.ones(total, nb, device="cuda")
    expect[rows] += dense
    assert torch.equal(out, expect)


def test_row_limit_on_the_device_bounds_the_work():
    """A device-side row count smaller than the host row count leaves the tail of the outputs untouched."""
    from ictc_o3 import _lib
    lib = _lib.load()
    torch.manual_seed(9)
    rows, live, nout = 1000, 333, 192
    z3 = torch.randn(rows, 64).cuda()
    w3 = (torch.randn(nout, 64) / 8).cuda().contiguous()
    limit = torch.tensor([live], dtype=torch.int64, device="cuda")
    gates = torch.full((rows, nout), float("nan"), device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    packed = _pack(lib, w3, 0)
    _lib.check(lib.ictc_gate_gemm_forward(rows, nout, z3.data_ptr(), packed.data_ptr(), gates.data_ptr(), 0,
                                          limit.data_ptr(), st), "fwd")
    ref = z3[:live].double().cpu() @ w3.double().cpu().t()
    assert float((gates[:live].double().cpu() - ref).abs().max() / ref.abs().max()) < 2e-6
    assert bool(torch.isnan(gates[live:]).all())
    da3 = torch.full((rows, 64), float("nan"), device="cuda")
    dg = torch.randn(rows, nout).cuda()
    packed_t = _pack(lib, w3, 1)
    _lib.check(lib.ictc_gate_gemm_backward(rows, nout, dg.data_ptr(), None, None, packed_t.data_ptr(), da3.data_ptr(),
                                           limit.data_ptr(), st), "bwd")
    ref = dg[:live].double().cpu() @ w3.double().cpu()
    assert float((da3[:live].double().cpu() - ref).abs().max() / ref.abs().max()) < 1e-5
    assert bool(torch.isnan(da3[live:]).all())
    assert _status(lib) == 0


@pytest.mark.parametrize("rows,nout,pad", [(1, 64, 0), (7, 192, 0), (1000, 704, 0), (70001, 704, 0), (9, 768, 0),
                                           (148 * 8 * 5 + 3, 64, 32), (0, 192, 0)])
def test_weight_gradient_on_the_tensor_cores(rows, nout, pad):
    """dW = grad^T @ rows contracted over the rows (tcgen05, both operands transposed into shared memory): against
    float64, with strided operands, bitwise repeatable."""
    from ictc_o3 import _lib
    lib = _lib.load()
    torch.manual_seed(rows + nout)
    grad_full = torch.randn(max(rows, 1), nout + pad).cuda()
    rows_full = torch.randn(max(rows, 1), 64 + pad).cuda()
    need = lib.ictc_weight_grad_workspace(rows, nout)
    assert need > 0
    work = torch.empty(need // 4, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    outs = []
    for _ in range(2):
        dw = torch.full((nout, 64 + pad), float("nan"), device="cuda")
        _lib.check(lib.ictc_weight_grad_tc(rows, nout, grad_full.data_ptr(), nout + pad, rows_full.data_ptr(), 64 + pad,
                                           dw.data_ptr(), 64 + pad, work.data_ptr(), st), "weight_grad")
        outs.append(dw[:, :64].clone())
        assert bool(torch.isnan(dw[:, 64:]).all())
    assert _status(lib) == 0
    assert torch.equal(outs[0], outs[1])
    ref = grad_full[:rows, :nout].double().cpu().t() @ rows_full[:rows, :64].double().cpu()
    scale = float(ref.abs().max()) if rows else 1.0
    assert float((outs[0].double().cpu() - ref).abs().max()) <= 1e-5 * max(scale, 1e-30)      # fp32 accumulation
    assert lib.ictc_weight_grad_workspace(10, 100) < 0 and lib.ictc_weight_grad_workspace(10, 832) < 0


def test_gate_mlp_weight_gradients_through_autograd():
    """The autograd route of the gate MLP: layers with 64-multiple sides run forward, input gradient and weight gradient
    on the tcgen05 kernels; all of them against float64, force-loss style (a gradient of a gradient)."""
    from ictc_o3.operators import _RowsTimesWeight
    torch.manual_seed(11)
    rows = torch.randn(3001, 64, device="cuda", requires_grad=True)
    w1 = (torch.randn(64, 64, device="cuda") / 8).requires_grad_(True)
    w2 = (torch.randn(1472, 64, device="cuda") / 8).requires_grad_(True)      # wider than one 768-column block

    def run(r, a, b, op):
        h = torch.nn.functional.silu(op(r, a))
        g = op(h, b)
        first, = torch.autograd.grad((g * g).sum(), r, create_graph=True)
        return torch.autograd.grad((first * first).sum() + g.sum(), [r, a, b])

    got = run(rows, w1, w2, _RowsTimesWeight.apply)
    ref = run(*(t.detach().double().cpu().requires_grad_(True) for t in (rows, w1, w2)), lambda r, w: r @ w.t())
    for a, b in zip(got, ref):
        assert float((a.double().cpu() - b).abs().max() / b.abs().max()) < 5e-5     # second order, fp32 sums 1,472 wide
