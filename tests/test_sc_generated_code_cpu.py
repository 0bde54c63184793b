"""The GENERATED symmetric-contraction source the CUDA kernels compile (csrc/generated/sc_code.cuh), built for the host
in double precision (tests/host/sc_host.cpp, g++) and pinned on the vectors of the reference's own recursion
(tests/golden/sc_pureu_c8.npz from mace_ictc/models/mace/products.py:845-949): values, feature gradient and weight
gradient for target lmax 0 and 2.  This checks the kernel arithmetic itself without a GPU."""
import ctypes
import os
import shutil
import subprocess

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "..", "ictc-o3-hp-k100_b200", "csrc")


@pytest.fixture(scope="module")
def host_lib(tmp_path_factory):
    gxx = shutil.which("g++")
    if gxx is None:
        pytest.skip("g++ not available")
    out = str(tmp_path_factory.mktemp("sc_host") / "sc_host.so")
    subprocess.run([gxx, "-O1", "-shared", "-fPIC", "-I", CSRC, os.path.join(HERE, "host", "sc_host.cpp"), "-o", out],
                   check=True)
    lib = ctypes.CDLL(out)
    lib.sc_host_num_weights.restype = ctypes.c_int
    lib.sc_host.restype = None
    return lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _run(lib, lt, mode, x, species, bank, gy=None):
    n, c = x.shape[0], x.shape[1] // 9
    ny = (lt + 1) ** 2
    y = np.zeros((n, ny * c)) if mode == 0 else None
    gx = np.zeros((n, 9 * c)) if mode == 1 else None
    gw = np.zeros_like(bank) if mode == 2 else None
    lib.sc_host(ctypes.c_int(lt), ctypes.c_int(mode), ctypes.c_int64(n), ctypes.c_int(c), _ptr(x), _ptr(species),
                _ptr(bank), _ptr(gy), _ptr(y), _ptr(gx), _ptr(gw))
    return (y, gx, gw)[mode]


@pytest.mark.parametrize("target", [0, 2])
def test_generated_sc_code_matches_reference_recursion(host_lib, target):
    g = np.load(os.path.join(HERE, "golden", "sc_pureu_c8.npz"))
    tag = f"t{target}/"
    x = np.ascontiguousarray(g[tag + "x"])
    species = np.ascontiguousarray(g[tag + "species"])
    # kernel order of the weight bank: per output degree the orders nu = 1, 2, 3 (reference module: weights.1, weights.0,
    # weights_max), concatenated along the weight axis -> [S, NW, C]
    names = [f"contractions.{l}.{part}" for l in range(target + 1) for part in ("weights.1", "weights.0", "weights_max")]
    bank = np.ascontiguousarray(np.concatenate([g[tag + "w/" + k] for k in names], axis=1))
    assert bank.shape[1] == host_lib.sc_host_num_weights(target)
    cot = np.ascontiguousarray(g[tag + "cot"])
    y = _run(host_lib, target, 0, x, species, bank)
    assert np.abs(y - g[tag + "y"]).max() <= 2e-7 * np.abs(g[tag + "y"]).max()          # couplings are float32 literals
    dx = _run(host_lib, target, 1, x, species, bank, cot)
    assert np.abs(dx - g[tag + "dx"]).max() <= 2e-7 * np.abs(g[tag + "dx"]).max()
    gw = _run(host_lib, target, 2, x, species, bank, cot)
    start = 0
    for k in names:
        ref = g[tag + "dw/" + k]
        got = gw[:, start:start + ref.shape[1]]
        start += ref.shape[1]
        assert np.abs(got - ref).max() <= 2e-7 * max(np.abs(ref).max(), 1e-30), k
