"""Reading and writing the reference's checkpoints and export side-car files.

The reference trainer saves a dictionary with the model's ``state_dict()`` under ``e3trans_state_dict`` (plus
``e3trans_ema_state_dict`` / ``e3trans_swa_state_dict`` and ``default_state_source`` naming the one to use),
``max_radius``, ``dtype``, ``tensor_product_mode``, ``atomic_energy_keys`` / ``atomic_energy_values`` and its
optimiser state (mace_ictc/training/train_loop.py:1917-1938).  Its LAMMPS export writes a ``<name>.json`` side-car
with ``elements``, ``atomic_numbers``, ``max_radius``, ``avg_num_neighbors``, ``message_passing_depth`` and
optional ``e0_keys`` / ``e0_values`` next to a copy of that checkpoint (mace_ictc/interfaces/lammps_hp.py:387-404).

Parameter names of this build's ``MaceIctcModel`` follow the reference's baseline route, with two differences
that the functions below translate:
  * the product block's equivariant linear is an e3nn ``o3.Linear`` there, whose single flat ``weight`` holds
    one [C_in, C_out] matrix per degree back to back; here it is one parameter per degree
    (``products.K.linear.L``);
  * the contraction weights of the ``ictd-pure-u`` backend sit under
    ``products.K.symmetric_contractions.contractions.L.*`` there and one module level deeper here.
Buffers that hold constant tables (``U_matrix_*``) are dropped: the kernels carry their own copies.

A checkpoint of the reference's default ``ictd-bridge-u`` backend keeps its contraction weights in the gauge of
e3nn's Wigner symbols; those weights have no image in the pure-U gauge (the reference says the same about the
opposite direction, mace_ictc/models/mace/products.py:961-970), so such a checkpoint is refused.
"""
from __future__ import annotations

import json
import os
import re
from typing import Dict

import torch

_PURE_U = re.compile(r"^(products\.\d+\.symmetric_contractions)\.(contractions\.\d+\..+)$")
_OURS_U = re.compile(r"^(products\.\d+\.symmetric_contractions)\.symmetric_contractions\.(contractions\.\d+\..+)$")
_FLAT_LINEAR = re.compile(r"^(products\.\d+\.linear)\.weight$")
_DEGREE_LINEAR = re.compile(r"^(products\.\d+\.linear)\.(\d+)$")


def from_reference_state_dict(state: Dict[str, torch.Tensor], channels: int) -> Dict[str, torch.Tensor]:
    """Reference parameter names -> this build's names (see the module text).  Unknown keys pass through, so
    ``load_state_dict(strict=True)`` still reports anything that does not fit."""
    out = {}
    for key, value in state.items():
        if ".U_matrix_" in key:
            continue
        if ".symmetric_contractions.symmetric_contractions." in key and "U_matrix" not in key:
            raise ValueError(
                "this state dict comes from the 'ictd-bridge-u' product backend: its contraction weights live in "
                "the gauge of e3nn's Wigner symbols and cannot be carried into the pure-U contraction of this build")
        m = _PURE_U.match(key)
        if m:
            out[f"{m.group(1)}.symmetric_contractions.{m.group(2)}"] = value
            continue
        m = _FLAT_LINEAR.match(key)
        if m:
            cc = channels * channels
            if value.ndim != 1 or value.numel() % cc:
                raise ValueError(f"{key}: expected a flat vector of per-degree [{channels}, {channels}] blocks")
            for l in range(value.numel() // cc):
                out[f"{m.group(1)}.{l}"] = value[l * cc:(l + 1) * cc].reshape(channels, channels)
            continue
        out[key] = value
    return out


def to_reference_state_dict(state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """This build's parameter names -> the reference's (``ictd-pure-u`` backend); inverse of the above apart
    from the constant tables, which the reference rebuilds on construction (load there with strict=False)."""
    out, linear = {}, {}
    for key, value in state.items():
        m = _OURS_U.match(key)
        if m:
            out[f"{m.group(1)}.{m.group(2)}"] = value
            continue
        m = _DEGREE_LINEAR.match(key)
        if m:
            linear.setdefault(m.group(1), {})[int(m.group(2))] = value
            continue
        out[key] = value
    for prefix, blocks in linear.items():
        out[prefix + ".weight"] = torch.cat([blocks[l].reshape(-1) for l in sorted(blocks)])
    return out


def load_reference_state_dict(model, state: Dict[str, torch.Tensor], strict: bool = True):
    """Copy a reference state dict into ``model`` (a ``MaceIctcModel``), casting to the model's dtype."""
    p = next(model.parameters())
    mapped = {k: v.to(device=p.device, dtype=p.dtype) if v.is_floating_point() else v.to(p.device)
              for k, v in from_reference_state_dict(state, model.channels).items()}
    return model.load_state_dict(mapped, strict=strict)


def load_checkpoint(model, path: str, source: str | None = None, strict: bool = True) -> dict:
    """Load a checkpoint written by the reference trainer (or by ``save_checkpoint``) into ``model``.

    ``source`` picks 'raw', 'ema' or 'swa'; None follows the file's ``default_state_source``.  The cutoff stored
    in the file must equal the model's.  Returns the checkpoint's metadata (everything but the state dicts and
    the optimiser state)."""
    ckpt = torch.load(path, map_location="cpu", weights_only=False)
    if "e3trans_state_dict" not in ckpt:
        raise ValueError(f"{path}: no 'e3trans_state_dict' entry, not a checkpoint of this model family")
    source = source or ckpt.get("default_state_source", "raw")
    key = {"raw": "e3trans_state_dict", "ema": "e3trans_ema_state_dict", "swa": "e3trans_swa_state_dict"}.get(source)
    if key is None:
        raise ValueError(f"source: {source!r} is not one of 'raw', 'ema', 'swa'")
    if key not in ckpt:
        raise ValueError(f"{path}: holds no {source!r} state")
    if "max_radius" in ckpt and abs(float(ckpt["max_radius"]) - float(model.max_radius)) > 1e-9:
        raise ValueError(f"{path}: cutoff {ckpt['max_radius']} differs from the model's {model.max_radius}")
    load_reference_state_dict(model, ckpt[key], strict=strict)
    skip = {"e3trans_state_dict", "e3trans_ema_state_dict", "e3trans_swa_state_dict", "optimizer_state_dict"}
    return {k: v for k, v in ckpt.items() if k not in skip}


def save_checkpoint(model, path: str, *, epoch: int = 0, global_step: int = 0, optimizer=None,
                    atomic_energies: Dict[int, float] | None = None) -> None:
    """Write ``model`` in the reference trainer's checkpoint layout, with the reference's parameter names."""
    atomic_energies = atomic_energies or {}
    keys = sorted(atomic_energies)
    ckpt = {
        "epoch": int(epoch), "global_step": int(global_step),
        "e3trans_state_dict": {k: v.detach().cpu() for k, v in to_reference_state_dict(model.state_dict()).items()},
        "optimizer_state_dict": optimizer.state_dict() if optimizer is not None else {},
        "dtype": "float32", "max_radius": float(model.max_radius), "tensor_product_mode": "pure-cartesian-ictd",
        "atomic_energy_keys": torch.tensor(keys, dtype=torch.long),
        "atomic_energy_values": torch.tensor([atomic_energies[k] for k in keys], dtype=torch.float64),
        "default_state_source": "raw", "product_backend": "ictd-pure-u",
        "channels": int(model.channels), "lmax": int(model.lmax), "num_interaction": int(model.num_interaction),
        "atomic_numbers": list(model.atomic_numbers),
    }
    os.makedirs(os.path.dirname(os.path.abspath(path)) or ".", exist_ok=True)
    torch.save(ckpt, path)


def model_from_export(json_path: str, *, channels: int = 64, correlation: int = 3, device="cuda"):
    """Build a model from the ``<name>.json`` side-car of the reference's LAMMPS export and load the checkpoint
    copy it names (``checkpoint`` entry, relative to the side-car).  Returns (model, metadata)."""
    from .hp.runtime import create_model
    with open(json_path) as f:
        meta = json.load(f)
    if meta.get("backend") != "ictc-hp":
        raise ValueError(f"{json_path}: backend {meta.get('backend')!r} is not 'ictc-hp'")
    model = create_model(channels=channels, lmax=2, num_interactions=int(meta["message_passing_depth"]),
                         correlation=correlation, atomic_numbers=tuple(meta["atomic_numbers"]),
                         cutoff=float(meta["max_radius"]), avg_num_neighbors=float(meta.get("avg_num_neighbors", 50.0)),
                         device=device)
    load_checkpoint(model, os.path.join(os.path.dirname(os.path.abspath(json_path)), meta["checkpoint"]))
    return model, meta
