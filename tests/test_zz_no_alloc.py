"""The allocation-free CSR builder (ictc_csr_build_static) against the ordinary entry point.

Some hosts of this library cannot allocate device memory at the point where they rebuild the edge
topology: an MD loop in which a cudaMalloc would stall the whole device every few steps, or a plugin
host that gives away all device memory at start-up.  For them the library carries its own fixed
scratch array; this test drives that entry point through the C ABI exactly as such a host would
(ctypes, raw pointers, no helper of the package in between) and checks that it returns what
ictc_csr_build returns with caller-owned scratch — twice in a row, the second time on a smaller and
differently ordered input, so anything the first call left behind in the shared array would show.
It is collected last on purpose.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _build(lib, fn_static, keys, n):
    dev = keys.device
    e = keys.numel()
    stream = torch.cuda.current_stream(dev).cuda_stream
    out = {}
    for name in ("ref", "static"):
        rowptr = torch.full((n + 1,), -7, dtype=torch.int64, device=dev)
        order = torch.full((max(e, 1),), -7, dtype=torch.int64, device=dev)
        flag = torch.full((1,), -7, dtype=torch.int32, device=dev)
        if name == "ref":
            scratch = torch.empty(int(lib.ictc_csr_scratch_bytes(n, e)), dtype=torch.uint8, device=dev)
            rc = lib.ictc_csr_build(keys.data_ptr(), n, e, rowptr.data_ptr(), order.data_ptr(), flag.data_ptr(),
                                    scratch.data_ptr(), stream)
        else:
            rc = fn_static(keys.data_ptr(), n, e, rowptr.data_ptr(), order.data_ptr(), flag.data_ptr(), stream)
        assert rc == 0, lib.ictc_last_error().decode()
        torch.cuda.synchronize()
        out[name] = (rowptr.cpu(), order[:e].cpu(), int(flag.item()))
    return out


def test_static_scratch_csr_matches_allocating_entry_point_twice():
    from ictc_o3 import _lib
    lib = _lib.load()
    fn_static = lib.ictc_csr_build_static
    max_n, max_e = C.c_int64(), C.c_int64()
    assert lib.ictc_csr_static_limits(C.byref(max_n), C.byref(max_e)) == 0
    assert max_n.value == 65536 and max_e.value == 1048576
    gen = torch.Generator().manual_seed(123)
    cases = [(40000, 700000, False), (900, 30000, False), (5000, 100000, True)]
    for n, e, presorted in cases:                      # consecutive calls share the built-in scratch
        keys = torch.randint(0, n, (e,), generator=gen)
        if presorted:
            keys = torch.sort(keys)[0]
        res = _build(lib, fn_static, keys.cuda(), n)
        ref, got = res["ref"], res["static"]
        assert torch.equal(got[0], ref[0])             # integer work: bit-exact
        assert torch.equal(got[1], ref[1])
        assert got[2] == ref[2] == (1 if presorted else 0)
        expect = torch.sort(keys, stable=True)[1]
        assert torch.equal(got[1], expect)
    # sizes beyond the built-in scratch are refused with a clear message and touch nothing
    dev = torch.device("cuda")
    rowptr = torch.zeros(8, dtype=torch.int64, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    keys = torch.zeros(8, dtype=torch.int64, device=dev)
    rc = fn_static(keys.data_ptr(), max_n.value + 1, 8, rowptr.data_ptr(), keys.data_ptr(), flag.data_ptr(), None)
    assert rc == -4 and "exceed the built-in scratch" in lib.ictc_last_error().decode()
    rc = fn_static(keys.data_ptr(), 7, max_e.value + 1, rowptr.data_ptr(), keys.data_ptr(), flag.data_ptr(), None)
    assert rc == -4
    assert _lib.kernel_status() == 0
