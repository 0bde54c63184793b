"""Generate the golden vectors under tests/golden/ by running the REFERENCE's own torch code on CPU.

Run by a maintainer where the reference checkout is available (it cannot run on the GPU box):

    python tests/golden/make_golden.py --reference <path to the reference checkout>

Everything is computed in float64 with the reference's modules:
  * ``EdgeWeightedPathPreservingTensorProduct`` + ``direction_harmonics_all``
    (ictc_o3/basis/ictd_irreps.py:2681-2971, 1153-1208) for the edge tensor product, its first
    gradients and a force-loss-like mixed second derivative;
  * ``ictc_o3.ops.rematerialized_message._native`` (gather + TP + gate + mask + index_add, ir_mul
    "native_packed" buffers) for the graph message;
  * ``ictd_u_matrix_so3`` is already frozen in the constants file, so the symmetric contraction has no
    separate golden here.
Inputs are stored next to the outputs so that no RNG stream has to be reproduced.
"""
import argparse
import os
import sys

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    args = ap.parse_args()
    os.environ.setdefault("FSCETP_ICTD_CACHE_DIR", "/tmp/ictd_cache")
    sys.dont_write_bytecode = True
    sys.path.insert(0, args.reference)
    import torch
    from ictc_o3.basis.ictd_irreps import EdgeWeightedPathPreservingTensorProduct, direction_harmonics_all
    from ictc_o3.ops.fused_message import _plan
    from ictc_o3.ops.bond_projection import projection_plan
    from ictc_o3.ops.rematerialized_message import _native

    here = os.path.dirname(os.path.abspath(__file__))
    f64 = torch.float64

    def make_tp(channels, lin, ledge, lout):
        paths = [(i, j, k) for i in range(lin + 1) for j in range(ledge + 1) for k in range(lout + 1)
                 if abs(i - j) <= k <= i + j and (i + j + k) % 2 == 0]
        tp = EdgeWeightedPathPreservingTensorProduct(
            channels=channels, lmax=max(lin, ledge, lout), allowed_paths=paths, path_policy="full",
            internal_compute_dtype=f64).to(f64)
        with torch.no_grad():
            tp.weight.fill_(1.0)
        tp.weight.requires_grad_(False)
        return tp, paths

    def tp_case(name, channels, lin, ledge, lout, edges, seed, rows_kept=None, unit_weight=True, f32_inputs=False):
        torch.manual_seed(seed)
        tp, paths = make_tp(channels, lin, ledge, lout)
        if not unit_weight:
            with torch.no_grad():
                tp.weight.copy_(torch.randn(len(paths), channels, dtype=f64))
        # f32_inputs: draw fp32 values (exactly representable), evaluate in fp64, store as fp32
        draw = torch.float32 if f32_inputs else f64
        store = (lambda a: a.astype(np.float32)) if f32_inputs else (lambda a: a)
        blocks = {l: torch.randn(edges, channels, 2 * l + 1, dtype=draw).to(f64).requires_grad_(True)
                  for l in range(lin + 1)}
        vec = torch.randn(edges, 3, dtype=draw).to(f64).requires_grad_(True)
        gates = torch.randn(edges, len(paths) * channels, dtype=draw).to(f64).requires_grad_(True)
        n = torch.nn.functional.normalize(vec, dim=-1)
        sh = direction_harmonics_all(n, ledge)
        out = tp(blocks, {l: sh[l].unsqueeze(-2) for l in range(ledge + 1)}, gates)
        loss = sum(v.square().sum() for v in out.values()) / sum(v.numel() for v in out.values())
        inputs = [blocks[l] for l in range(lin + 1)] + [vec, gates]
        first = torch.autograd.grad(loss, inputs, create_graph=True)
        # force-loss-like scalar of the first gradients -> mixed second derivatives
        loss2 = sum((g * g).sum() for g in first)
        second = torch.autograd.grad(loss2, inputs)
        keep = slice(None) if rows_kept is None else slice(0, None, rows_kept)
        data = {"channels": channels, "lin": lin, "ledge": ledge, "lout": lout, "rows_kept": rows_kept or 1,
                "paths": np.array(paths), "weight": tp.weight.detach().numpy(),
                "vec": store(vec.detach().numpy()), "gates": store(gates.detach().numpy()),
                "sh": torch.cat(sh, -1).detach().numpy()[keep], "loss": float(loss.detach()), "loss2": float(loss2.detach())}
        for l in range(lin + 1):
            data[f"x{l}"] = store(blocks[l].detach().numpy())
            data[f"dx{l}"] = first[l].detach().numpy()[keep]
            data[f"ddx{l}"] = second[l].detach().numpy()[keep]
        for l, v in out.items():
            data[f"out{l}"] = v.detach().numpy()[keep]
        data["dvec"], data["dgates"] = first[-2].detach().numpy()[keep], first[-1].detach().numpy()[keep]
        data["ddvec"], data["ddgates"] = second[-2].detach().numpy()[keep], second[-1].detach().numpy()[keep]
        np.savez_compressed(os.path.join(here, name + ".npz"), **data)
        print(name, "loss", float(loss), "loss2", float(loss2))

    tp_case("tp_c8_l222_e37", 8, 2, 2, 2, 37, 11)
    tp_case("tp_c8_l022_e19", 8, 0, 2, 2, 19, 12)
    tp_case("tp_c5_l111_e13_w", 5, 1, 1, 1, 13, 13, unit_weight=False)
    # BASELINE config 1 (C32, lmax 2, 257 edges): inputs in full, outputs for every 8th edge
    tp_case("tp_cfg1_c32_l222_e257", 32, 2, 2, 2, 257, 0, rows_kept=8, f32_inputs=True)

    def message_case(name, channels, lin, nodes, edges, seed):
        torch.manual_seed(seed)
        tp, paths = make_tp(channels, lin, 2, 2)
        with torch.no_grad():
            tp.weight.copy_(1.0 + 0.1 * torch.randn(len(paths), channels, dtype=f64))
        plan = dict(_plan(tp, list(range(lin + 1)), torch.device("cpu"), True))
        plan["native_packed"] = True
        proj = projection_plan(tp, tp._get_bond_projectors(torch.device("cpu"), f64), torch.device("cpu"), f64)
        x = torch.randn(nodes, plan["xdim"], dtype=f64, requires_grad=True)
        vec = torch.randn(edges, 3, dtype=f64, requires_grad=True)
        g = torch.randn(edges, len(paths), channels, dtype=f64, requires_grad=True)
        src = torch.randint(0, nodes, (edges,))
        dst = torch.randint(0, nodes, (edges,))
        mask = (torch.rand(edges, dtype=f64) > 0.2).to(f64)
        sh = torch.cat(direction_harmonics_all(torch.nn.functional.normalize(vec, dim=-1), 2), -1)
        out = _native(x, sh, tp.weight, g, src, dst, mask, plan, proj)
        cot = torch.randn_like(out)
        first = torch.autograd.grad((out * cot).sum(), [x, vec, g], create_graph=True)
        loss2 = sum((v * v).sum() for v in first)
        second = torch.autograd.grad(loss2, [x, vec, g])
        np.savez_compressed(os.path.join(here, name + ".npz"), channels=channels, lin=lin, nodes=nodes,
                            paths=np.array(paths), weight=tp.weight.detach().numpy(), x=x.detach().numpy(),
                            vec=vec.detach().numpy(), sh=sh.detach().numpy(), g=g.detach().numpy(),
                            src=src.numpy(), dst=dst.numpy(), mask=mask.numpy(), out=out.detach().numpy(),
                            cot=cot.numpy(), dx=first[0].detach().numpy(), dvec=first[1].detach().numpy(),
                            dg=first[2].detach().numpy(), ddx=second[0].numpy(), ddvec=second[1].numpy(),
                            ddg=second[2].numpy())
        print(name, "odim", out.shape[1], "loss2", float(loss2))

    message_case("message_c8_l2_n23_e120", 8, 2, 23, 120, 21)
    message_case("message_c8_l0_n17_e90", 8, 0, 17, 90, 22)

    # direction harmonics, value and vector-Jacobian product
    torch.manual_seed(31)
    n = torch.nn.functional.normalize(torch.randn(41, 3, dtype=f64), dim=-1).requires_grad_(True)
    y = torch.cat(direction_harmonics_all(n, 2), -1)
    cot = torch.randn_like(y)
    dn = torch.autograd.grad((y * cot).sum(), n)[0]
    np.savez_compressed(os.path.join(here, "harmonics_l2_e41.npz"), n=n.detach().numpy(), y=y.detach().numpy(),
                        cot=cot.numpy(), dn=dn.numpy())
    print("harmonics ok")


if __name__ == "__main__":
    main()
