"""Golden vectors of the radial embedding, computed by the REFERENCE's own function on CPU.

    python tests/golden/make_golden_radial.py --reference <path to the reference checkout>

``mace_ictc/models/radial_basis.py`` is loaded as a single file: its package ``__init__`` imports e3nn, which is
not installed where this runs, and the file itself needs e3nn only for a basis type that is not used here, so a
placeholder module stands in for ``e3nn.math``.  Everything that is evaluated (``mace_radial_embedding`` with
the Bessel basis and ``mace_polynomial_cutoff``) is the reference's code, in float64.
"""
import argparse
import importlib.util
import os
import sys
import types

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    import torch
    e3nn, e3nn_math = types.ModuleType("e3nn"), types.ModuleType("e3nn.math")

    def unavailable(*a, **k):
        raise RuntimeError("e3nn is not installed")
    e3nn_math.soft_one_hot_linspace = unavailable
    e3nn.math = e3nn_math
    sys.modules.setdefault("e3nn", e3nn)
    sys.modules.setdefault("e3nn.math", e3nn_math)
    path = os.path.join(args.reference, "mace_ictc", "models", "radial_basis.py")
    spec = importlib.util.spec_from_file_location("reference_radial_basis", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    rng = np.random.default_rng(11)
    r = np.concatenate((np.linspace(0.35, 4.49, 40), rng.uniform(0.5, 4.5, 20), [4.5, 4.6, 5.0]))
    w = rng.normal(size=(8,))
    out = {"r": r, "w": w, "r_max": np.array(4.5)}
    for p in (5, 6):
        rt = torch.tensor(r, dtype=torch.float64, requires_grad=True)
        emb = mod.mace_radial_embedding(rt, r_max=4.5, number_of_basis=8, function_type="bessel",
                                        polynomial_cutoff_p=p, sqrt_num_basis_norm=False)
        (grad,) = torch.autograd.grad((emb * torch.tensor(w)).sum(), rt)
        out[f"emb_p{p}"] = emb.detach().numpy()
        out[f"grad_p{p}"] = grad.numpy()
    here = os.path.dirname(os.path.abspath(__file__))
    np.savez(os.path.join(here, "radial_bessel8_rmax4p5.npz"), **out)
    print("wrote radial_bessel8_rmax4p5.npz", out["emb_p5"].shape)


if __name__ == "__main__":
    main()
