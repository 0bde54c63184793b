"""Regenerate ``ictc_tables_lmax{L}.npz`` from the reference's frozen Cartesian-harmonic basis.

The ICTC harmonic basis for l >= 2 is a set of SHA-pinned binary assets of the reference
(``ictc_o3/basis/_ictd_basis/v1``), so every coupling constant used by the kernels has to be
*derived from those assets by the reference's own code*; nothing here re-derives a basis.
This script is the only file of the package that imports the reference.  It is run by a
maintainer on a machine that has the reference checkout, never at import or test time:

    python make_tables.py --reference <path to the reference checkout> [--lmax 2]

Arrays written (all float64 unless noted):
  cg_{l1}{l2}{l3}      raw ``build_cg_tensor(l1,l2,l3)`` [2l1+1,2l2+1,2l3+1], natural parity only
                       (reference: ictc_o3/basis/ictd_irreps.py:1264-1303)
  cgfull_{l1}_{l2}_{l3} raw ``build_full_cg_tensor_so3`` incl. odd-parity couplings
                       (ictd_irreps.py:1345-1414), l1 <= 2*lmax, l2 <= lmax
  u_{lout}_{nu}        ``ictd_u_matrix_so3(lmax, lout, nu, "component")`` (ictd_irreps.py:1535-1557)
  harm_exps_{l}        int64 [n_mono,3] monomial exponents in reference row order
                       (ictc_o3/basis/ictd_fast.py:41-48)
  harm_coef_{l}        [n_mono, 2l+1]: multinomial * projector * component scale, so that
                       Y_l[h] = sum_r x^a y^b z^c * harm_coef[r,h]  (ictd_irreps.py:1153-1208)
"""
import argparse
import os
import sys

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--lmax", type=int, default=2)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    os.environ.setdefault("FSCETP_ICTD_CACHE_DIR", "/tmp/ictd_cache")
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    import torch
    import ictc_o3.basis.ictd_irreps as B

    L = args.lmax
    out = {"lmax": np.int64(L)}
    for l1 in range(L + 1):
        for l2 in range(L + 1):
            for l3 in range(abs(l1 - l2), min(l1 + l2, L) + 1):
                if (l1 + l2 + l3) % 2:
                    continue
                out[f"cg_{l1}{l2}{l3}"] = B.build_cg_tensor(l1, l2, l3).double().numpy()
    for l1 in range(2 * L + 1):
        for l2 in range(L + 1):
            for l3 in range(abs(l1 - l2), min(l1 + l2, 2 * L) + 1):
                out[f"cgfull_{l1}_{l2}_{l3}"] = B.build_full_cg_tensor_so3(l1, l2, l3).double().numpy()
    for lout in range(L + 1):
        for nu in (1, 2, 3):
            out[f"u_{lout}_{nu}"] = B.ictd_u_matrix_so3(
                lmax=L, output_l=lout, correlation=nu, irrep_normalization="component",
                dtype=torch.float64).numpy()
    for l in range(1, L + 1):
        exps, coefs = B._dir_monomial_exps_coefs(l)
        proj = B._dir_proj_cpu_f64(l).double()
        scale = float(B._direction_component_scale_cpu_f64(l))
        assert [tuple(int(v) for v in row) for row in exps] == [tuple(t) for t in B._counts_list(l)]
        out[f"harm_exps_{l}"] = exps.long().numpy()
        out[f"harm_coef_{l}"] = (coefs.double()[:, None] * proj * scale).numpy()
    path = args.out or os.path.join(os.path.dirname(os.path.abspath(__file__)), f"ictc_tables_lmax{L}.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
