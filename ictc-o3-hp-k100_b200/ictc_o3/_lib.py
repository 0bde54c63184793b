"""ctypes binding of ``libictc_b200.so`` (C ABI declared in ``include/ictc_b200.h``).

The library is the only compute path: if it is missing the import fails loudly, there is no CPU or
PyTorch fallback.  Signatures contain plain pointers and sizes only; tensors are passed as
``data_ptr()`` and the launch goes to torch's current CUDA stream of the tensor's device.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libictc_b200.so")

_P, _I, _L = C.c_void_p, C.c_int, C.c_int64

# name -> (restype, argtypes); mirrors include/ictc_b200.h one to one
SIGNATURES = {
    "ictc_last_error": (C.c_char_p, []),
    "ictc_version": (C.c_char_p, []),
    "ictc_kernel_status": (_I, [C.POINTER(C.c_int), _I]),
    "ictc_selftest_bounded_wait": (_I, [_L, _I, _P]),
    "ictc_tp_spec": (_I, [_I, _I, _I]),
    "ictc_tp_spec_info": (_I, [_I] + [C.POINTER(C.c_int)] * 5),
    "ictc_tp_edge_forward": (_I, [_I, _I, _L, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_tp_edge_adjoint": (_I, [_I, _I, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_tp_graph_forward": (_I, [_I, _I, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_tp_graph_adjoint": (_I, [_I, _I, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_tp_graph_forward_shared": (_I, [_I, _I, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_tp_graph_adjoint_shared": (_I, [_I, _I, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_tp_graph_forward_chunk": (_I, [_I, _I, _L, _P, _P, _P, _P, _P, _P, _L, _P, _P, _P, _P, _P, _P]),
    "ictc_tp_graph_adjoint_chunk": (_I, [_I, _I, _L, _P, _P, _P, _P, _P, _I, _P, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                         _L, _P]),
    "ictc_gate_gemm_forward_rows": (_I, [_L, _I, _P, _P, _P, _P, _P, _P, _I, _P]),
    "ictc_gate_gemm_backward_rows": (_I, [_L, _I, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_mlp_chain_backward_paired": (_I, [_L, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P]),
    "ictc_gate_pack_weights": (_I, [_I, _P, _I, _P, _P]),
    "ictc_gate_gemm_forward": (_I, [_L, _I, _P, _P, _P, _I, _P, _P]),
    "ictc_gate_gemm_backward": (_I, [_L, _I, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_mlp_chain_forward": (_I, [_L, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_mlp_chain_backward": (_I, [_L, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _P, _P]),
    "ictc_channel_linear_tc": (_I, [_L, _I, _I, _P, _I, _L, _P, _P, _I, _L, _P]),
    "ictc_weight_grad_workspace": (_L, [_L, _I]),
    "ictc_weight_grad_tc": (_I, [_L, _I, _P, _L, _P, _L, _P, _L, _P, _P]),
    "ictc_csr_scratch_bytes": (_L, [_L, _L]),
    "ictc_csr_build": (_I, [_P, _L, _L, _P, _P, _P, _P, _P]),
    "ictc_csr_build_static": (_I, [_P, _L, _L, _P, _P, _P, _P]),
    "ictc_csr_static_limits": (_I, [C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "ictc_scan_scratch_bytes": (_L, [_L]),
    "ictc_inclusive_scan_i64": (_I, [_P, _L, _P, _P]),
    "ictc_neighbor_scratch_bytes": (_L, [_L, C.POINTER(C.c_double), C.POINTER(C.c_double), C.c_double]),
    "ictc_neighbor_count": (_I, [_P, _L, _L, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double),
                                 C.POINTER(C.c_int), C.c_double, _P, _P, _P]),
    "ictc_neighbor_fill": (_I, [_P, _L, _L, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double),
                                C.POINTER(C.c_int), C.c_double, _P, _L, _P, _P, _P, _P, _P, _P]),
    "ictc_neighbor_clamp": (_I, [_P, _L, _L, _P, _P]),
    "ictc_neighbor_pad": (_I, [_P, _L, _L, _L, _P, _P, _P, _P, _P]),
    "ictc_neighbor_pairs": (_I, [_P, _P, _P, _L, _L, _L, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_md_kick": (_I, [_L, C.c_float, _P, _P, _P, _P, _P, _I, _P]),
    "ictc_edge_geometry_forward": (_I, [_P, _P, _P, _P, C.POINTER(C.c_float), C.c_float, _I, _I, _L, _P, _P, _P, _P, _P]),
    "ictc_edge_geometry_backward": (_I, [_P, _P, C.c_float, _I, _I, _L, _P, _P, _P, _P]),
    "ictc_position_gradient": (_I, [_L, _L, _P, _P, _P, _P, _P, _P]),
    "ictc_silu_forward": (_I, [_L, C.c_float, _P, _P, _P]),
    "ictc_silu_backward": (_I, [_L, C.c_float, _P, _P, _P, _P]),
    "ictc_layout_copy": (_I, [_L, _I, _I, C.POINTER(C.c_int), C.POINTER(C.c_int), _P, _P, _I, _P]),
    "ictc_harmonics_forward": (_I, [_I, _L, _P, _P, _P]),
    "ictc_harmonics_vjp": (_I, [_I, _L, _P, _P, _P, _P]),
    "ictc_harmonics_second": (_I, [_I, _L, _P, _P, _P, _P, _P, _P]),
    "ictc_sc_num_weights": (_I, [_I, _I]),
    "ictc_sc_scratch_bytes": (_L, [_I, _I, _I, _L, _I]),
    "ictc_sc_forward": (_I, [_I, _I, _I, _L, _I, _I, _P, _P, _P, _P, _P]),
    "ictc_sc_adjoint": (_I, [_I, _I, _I, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P]),
    "ictc_sc_second": (_I, [_I, _I, _I, _L, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P]),
}

_lib = None


def load():
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(
                f"{LIB_PATH} is missing: build it with `python ictc-o3-hp-k100_b200/csrc/build.py` "
                "(nvcc, sm_100a). There is no fallback path.")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def last_error() -> str:
    return load().ictc_last_error().decode()


# number of successful C-ABI calls that launch kernels (each call launches one or more kernels)
CALLS = 0


def check(rc: int, what: str):
    global CALLS
    CALLS += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}: {last_error()}")


def kernel_status(reset: bool = True) -> int:
    """Synchronise the current device and return its kernel status word (0 = ok)."""
    value = C.c_int(0)
    check(load().ictc_kernel_status(C.byref(value), int(reset)), "ictc_kernel_status")
    return value.value


def ptr(t):
    """Device pointer of a tensor, or NULL for None / empty tensors."""
    if t is None or t.numel() == 0:
        return None
    return t.data_ptr()


def stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


class on_device:
    """Make ``device`` current for the launch when it is not already."""

    def __init__(self, device):
        self.index = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.index:
            self.prev = cur
            torch.cuda.set_device(self.index)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)


def tp_spec(input_lmax: int, edge_lmax: int, output_lmax: int) -> int:
    spec = load().ictc_tp_spec(input_lmax, edge_lmax, output_lmax)
    if spec < 0:
        raise ValueError(f"unsupported tensor-product degrees: {last_error()}")
    return spec


def tp_spec_info(spec: int):
    vals = [C.c_int() for _ in range(5)]
    check(load().ictc_tp_spec_info(spec, *[C.byref(v) for v in vals]), "ictc_tp_spec_info")
    return tuple(v.value for v in vals)
