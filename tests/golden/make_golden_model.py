"""Golden vectors of the symmetric contraction, the channel linears and the whole model, computed by the
REFERENCE's own classes on CPU in float64.

    python tests/golden/make_golden_model.py --reference <path to the reference checkout>

What runs is the reference's code: ``build_baseline_model`` (mace_ictc/models/factory.py) with the arguments of
its ``create_model`` factory (mace_ictc/hp/runtime.py:6-79) except ``product_backend="ictd-pure-u"``, its
``energy_and_forces`` (hp/runtime.py:82-111), ``ICTDPureUSymmetricContractionSO3`` / ``_ICTDPureUContraction``
(mace_ictc/models/mace/products.py:845-1035), ``EquivariantChannelLinearSO3`` (ictc_o3/basis/ictd_irreps.py:185-227),
``PathPreservingLinearSO3`` and ``ElementConditionedLinearSO3`` (mace_ictc/models/mace/layers.py:21-87, 317-355).

Two third-party packages of the reference are not installed where this runs, so stand-ins are registered
before the reference is imported:
  * ``opt_einsum_fx.optimize_einsums_full`` returns the traced einsum module unchanged (it only reorders
    contractions; the arithmetic is the einsum the reference wrote);
  * ``e3nn.o3``: ``Irreps`` (parsing of "64x0e+64x1o+64x2e" and iteration) and ``Linear`` restated from e3nn's
    published definition for equal input and output irreps: one N(0,1) matrix per degree,
    y[n,o,m] = sum_i x[n,i,m] W[i,o] / sqrt(C_in), no bias.  Everything else of e3nn is a placeholder that is
    never evaluated on this route.
The default product backend of the reference factory ("ictd-bridge-u") takes its U tensors from e3nn's Wigner
symbols and cannot run here; "ictd-pure-u" is the same model class with the U tensors of the reference's own
``ictd_u_matrix_so3``, which is the contraction this build implements.

All stored weights are rounded to float32 values first, so a float32 model can load them exactly.
"""
import argparse
import importlib.abc
import importlib.machinery
import importlib.util
import math
import os
import re
import sys
import types

import numpy as np


class _Placeholder:
    def __init__(self, *a, **k):
        pass

    def __call__(self, *a, **k):
        return _Placeholder()

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return _Placeholder()

    def __iter__(self):
        return iter(())


class _StubModule(types.ModuleType):
    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        full = self.__name__ + "." + name
        return sys.modules[full] if full in sys.modules else _Placeholder


_ABSENT = {"e3nn", "opt_einsum_fx", "ase", "matscipy", "mpi4py", "mace", "cuequivariance", "cuequivariance_torch",
           "openequivariance", "lammps"}


class _StubFinder(importlib.abc.MetaPathFinder, importlib.abc.Loader):
    def find_spec(self, name, path, target=None):
        if name.split(".")[0] in _ABSENT:
            return importlib.machinery.ModuleSpec(name, self, is_package=True)
        return None

    def create_module(self, spec):
        mod = _StubModule(spec.name)
        mod.__path__ = []
        return mod

    def exec_module(self, module):
        pass


def install_stand_ins():
    import torch
    sys.meta_path.insert(0, _StubFinder())
    import e3nn
    import e3nn.o3 as o3
    import opt_einsum_fx
    opt_einsum_fx.optimize_einsums_full = lambda model, example_inputs=None, **k: model
    e3nn.get_optimization_defaults = lambda: {}
    e3nn.set_optimization_defaults = lambda **k: None

    class Irrep:
        def __init__(self, l, p):
            self.l, self.p, self.dim = int(l), int(p), 2 * int(l) + 1

    class Irreps:
        def __init__(self, spec):
            if isinstance(spec, Irreps):
                self.items = list(spec.items)
                return
            self.items = []
            for part in str(spec).split("+"):
                part = part.strip()
                if part:
                    m = re.fullmatch(r"(?:(\d+)x)?(\d+)([eo])", part)
                    self.items.append((int(m.group(1) or 1), Irrep(int(m.group(2)), 1 if m.group(3) == "e" else -1)))

        def __iter__(self):
            return iter(self.items)

        def __len__(self):
            return len(self.items)

        @property
        def dim(self):
            return sum(mul * ir.dim for mul, ir in self.items)

        def __repr__(self):
            return "+".join(f"{m}x{ir.l}{'e' if ir.p == 1 else 'o'}" for m, ir in self.items)

    class Linear(torch.nn.Module):
        def __init__(self, irreps_in, irreps_out, **kwargs):
            super().__init__()
            a, b = Irreps(irreps_in), Irreps(irreps_out)
            if repr(a) != repr(b):
                raise NotImplementedError("stand-in Linear: equal input and output irreps only")
            self.muls, self.dims = [m for m, _ in a], [ir.dim for _, ir in a]
            self.weight = torch.nn.Parameter(torch.randn(sum(m * m for m in self.muls)))

        def forward(self, x):
            outs, off, woff = [], 0, 0
            for mul, d in zip(self.muls, self.dims):
                block = x[:, off:off + mul * d].reshape(-1, mul, d)
                w = self.weight[woff:woff + mul * mul].reshape(mul, mul)
                outs.append((torch.einsum("nim,io->nom", block, w) / math.sqrt(mul)).reshape(-1, mul * d))
                off, woff = off + mul * d, woff + mul * mul
            return torch.cat(outs, -1)

    o3.Irrep, o3.Irreps, o3.Linear = Irrep, Irreps, Linear


def round_to_fp32(module):
    import torch
    with torch.no_grad():
        for p in module.parameters():
            p.copy_(p.float().double())


def lattice(side, seed, spacing=2.15, sigma=0.1, cutoff=4.5):
    """Jittered simple-cubic H/C/O sample with a brute-force periodic neighbour list (r^2 <= cutoff^2)."""
    rng = np.random.default_rng(seed)
    grid = np.stack(np.meshgrid(*[np.arange(side)] * 3, indexing="ij"), -1).reshape(-1, 3) * spacing
    box = np.array([side * spacing] * 3)
    pos = (grid + rng.normal(scale=sigma, size=grid.shape)) % box
    pos = pos.astype(np.float32).astype(np.float64)
    src, dst, shifts = [], [], []
    for image in np.stack(np.meshgrid(*[np.arange(-1, 2)] * 3, indexing="ij"), -1).reshape(-1, 3):
        vec = pos[:, None, :] - pos[None, :, :] + (image * box)[None, None, :]      # [dst i, src j]
        r2 = (vec * vec).sum(-1)
        i, j = np.nonzero((r2 <= cutoff ** 2) & (r2 > 1e-12))
        src += list(j)
        dst += list(i)
        shifts += [image] * len(i)
    order = np.lexsort((np.array(src), np.array(dst)))
    z = np.array([1, 6, 6, 8])[rng.integers(0, 4, len(pos))]
    return pos, box, z, np.array(src)[order], np.array(dst)[order], np.array(shifts, dtype=np.float64)[order]


def model_case(torch, reference, channels, side, seed, grad_keys):
    from mace_ictc.models.factory import build_baseline_model
    from mace_ictc.utils.config import ModelConfig
    spec = importlib.util.spec_from_file_location("reference_hp_runtime",
                                                  os.path.join(reference, "mace_ictc", "hp", "runtime.py"))
    runtime = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(runtime)
    dt = torch.float64
    torch.manual_seed(seed)
    config = ModelConfig(dtype=dt, internal_compute_dtype=dt, channel_in=channels,
                         irreps_output_conv_channels=channels, lmax=2, max_radius=4.5, max_radius_main=4.5,
                         function_type="bessel")
    model = build_baseline_model(
        config, avg_num_neighbors=32.0, num_interaction=2, route="baseline", product_backend="ictd-pure-u",
        correlation=3, use_reduced_cg=False, freeze_conv_tp_weight=True, radial_sqrt_num_basis=False, edge_lmax=2,
        attn_heads=0, atomic_numbers=[1, 6, 8], ictd_save_tp_mode="fully-connected", invariant_channels=32,
        device=torch.device("cpu"), dtype=dt)
    round_to_fp32(model)
    pos, box, z, src, dst, shifts = lattice(side, seed)
    n = len(pos)
    t = lambda a, d=dt: torch.as_tensor(a, dtype=d)
    args = (t(pos), t(z, torch.long), torch.zeros(n, dtype=torch.long), t(src, torch.long), t(dst, torch.long),
            t(shifts), t(np.diag(box)).unsqueeze(0))
    res = runtime.energy_and_forces(model, *args, training=True)
    loss = (res["energy"] / n).square().mean() + res["forces"].square().mean()
    params = dict(model.named_parameters())
    keys = [k for k in params if params[k].requires_grad] if grad_keys is None else grad_keys
    grads = torch.autograd.grad(loss, [params[k] for k in keys], allow_unused=True)
    out = {"pos": pos, "box": box, "z": z, "src": src, "dst": dst, "shifts": shifts,
           "energy": res["energy"].detach().numpy(), "forces": res["forces"].detach().numpy(),
           "atomic_energy": res["atomic_energy"].detach().numpy(), "loss": loss.detach().numpy(),
           "channels": np.array(channels), "avg_num_neighbors": np.array(32.0), "cutoff": np.array(4.5)}
    for k, v in model.state_dict().items():
        if "U_matrix" not in k:
            out["state/" + k] = v.detach().numpy().astype(np.float32)
    for k, g in zip(keys, grads):
        if g is not None:
            out["grad/" + k] = g.numpy()
    return out


def contraction_cases(torch):
    from mace_ictc.models.mace.products import ICTDPureUSymmetricContractionSO3
    out = {}
    torch.set_default_dtype(torch.float64)
    try:
        for target in (0, 2):
            torch.manual_seed(40 + target)
            n, c, s = 23, 8, 3
            mod = ICTDPureUSymmetricContractionSO3(num_elements=s, channels=c, lmax=2, target_lmax=target,
                                                    correlation=3)
            round_to_fp32(mod)
            x = (torch.randn(n, 9 * c) * 0.7).float().double().requires_grad_(True)
            species = torch.randint(0, s, (n,))
            attrs = torch.nn.functional.one_hot(species, s).double()
            y = mod(x, attrs)
            cot = torch.randn_like(y)
            params = list(mod.parameters())
            grads = torch.autograd.grad((y * cot).sum(), [x] + params)
            tag = f"t{target}/"
            out.update({tag + "x": x.detach().numpy(), tag + "species": species.numpy(), tag + "y": y.detach().numpy(),
                        tag + "cot": cot.numpy(), tag + "dx": grads[0].numpy()})
            for (name, p), g in zip(mod.named_parameters(), grads[1:]):
                out[tag + "w/" + name] = p.detach().numpy()
                out[tag + "dw/" + name] = g.numpy()
    finally:
        torch.set_default_dtype(torch.float32)
    return out


def linear_cases(torch):
    from ictc_o3.basis.ictd_irreps import EquivariantChannelLinearSO3
    from mace_ictc.models.mace.layers import ElementConditionedLinearSO3, PathPreservingLinearSO3
    torch.manual_seed(77)
    n, c, s = 19, 8, 3
    out = {}
    x = torch.randn(n, 9 * c, dtype=torch.float64)
    up = EquivariantChannelLinearSO3(c, 2).double()
    with torch.no_grad():
        for p in up.parameters():
            p.copy_(torch.randn_like(p))
    out["up/x"], out["up/y"] = x.numpy(), up(x).detach().numpy()
    for k, v in up.state_dict().items():
        out["up/w/" + k] = v.numpy()
    counts = {0: 3, 1: 4, 2: 4}
    ppl = PathPreservingLinearSO3({l: c * counts[l] for l in counts}, c, 2).double()
    blocks = {l: torch.randn(n, c * counts[l], 2 * l + 1, dtype=torch.float64) for l in counts}
    out["message/y"] = ppl(blocks).detach().numpy()
    for l in counts:
        out[f"message/x{l}"] = blocks[l].numpy()
    for k, v in ppl.state_dict().items():
        out["message/w/" + k] = v.detach().numpy()
    ecl = ElementConditionedLinearSO3(s, c, 2).double()
    with torch.no_grad():
        for p in ecl.parameters():
            p.copy_(torch.randn_like(p))
    idx = torch.randint(0, s, (n,))
    out["element/x"], out["element/idx"] = x.numpy(), idx.numpy()
    out["element/y"] = ecl.forward_type_idx(x, idx).detach().numpy()
    for k, v in ecl.state_dict().items():
        out["element/w/" + k] = v.detach().numpy()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--cache", default="/tmp/ictd_cache", help="writable folder for the reference's basis cache")
    args = ap.parse_args()
    sys.dont_write_bytecode = True
    os.makedirs(args.cache, exist_ok=True)
    os.environ.setdefault("FSCETP_ICTD_CACHE_DIR", args.cache)
    import torch
    install_stand_ins()
    sys.path.insert(0, args.reference)
    here = os.path.dirname(os.path.abspath(__file__))
    small = model_case(torch, args.reference, channels=8, side=4, seed=3, grad_keys=None)
    np.savez_compressed(os.path.join(here, "model_pureu_c8_n64.npz"), **small)
    big_keys = ["interactions.1.linear_up.adapters.1.weight", "interactions.0.fc.2.weight",
                "interactions.1.message_linear.weights.2", "products.0.linear.weight",
                "products.0.symmetric_contractions.contractions.1.weights_max",
                "last_layer_energy_readout.linear_1.weight", "node_embedding.weight"]
    big = model_case(torch, args.reference, channels=64, side=5, seed=5, grad_keys=big_keys)
    np.savez_compressed(os.path.join(here, "model_pureu_c64_n125.npz"), **big)
    np.savez_compressed(os.path.join(here, "sc_pureu_c8.npz"), **contraction_cases(torch))
    np.savez_compressed(os.path.join(here, "linears_c8.npz"), **linear_cases(torch))
    print("energy c8", small["energy"], "c64", big["energy"], "max force", np.abs(big["forces"]).max())


if __name__ == "__main__":
    main()
