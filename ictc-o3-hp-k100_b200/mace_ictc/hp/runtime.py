"""create_model / configure_model / energy_and_forces (reference: mace_ictc/hp/runtime.py:6-297)."""
from __future__ import annotations

import torch

from ..model import MaceIctcModel


from ictc_o3.operators import _need_degree, _need_positive


def create_model(*, channels=64, lmax=3, edge_lmax=None, num_interactions=2, correlation=3, use_reduced_cg=False,
                 atomic_numbers=(1, 6, 8), cutoff=5.0, avg_num_neighbors=50.0, device="cuda", dtype=torch.float32,
                 electrostatics=None):
    """A freshly initialised short-range model (reference factory: mace_ictc/hp/runtime.py:6-79): tensor-product
    base coefficients fixed to one, radial MLP / channel linears / contraction weights trainable.

    Compiled coverage of this build: lmax = edge_lmax = 2, float32, CUDA, no electrostatics head.  Arguments
    outside the reference's own domain raise the reference's exception types; arguments the reference accepts
    but this build has no kernels for raise ValueError naming the limit.
    """
    _need_positive(num_interactions, "num_interactions")
    _need_positive(channels, "channels")
    _need_positive(correlation, "correlation")
    if correlation > 3:
        raise ValueError(f"correlation: orders 1 to 3 are provided, got {correlation}")
    if not isinstance(use_reduced_cg, bool):
        raise TypeError(f"use_reduced_cg: expected True or False, got {type(use_reduced_cg).__name__}")
    if use_reduced_cg:
        raise ValueError("use_reduced_cg: this factory builds the full Clebsch-Gordan basis only")
    _need_degree(lmax, "lmax")
    if edge_lmax is None:
        edge_lmax = lmax
    _need_degree(edge_lmax, "edge_lmax")
    if edge_lmax < lmax:
        raise ValueError(f"edge_lmax ({edge_lmax}) may not be smaller than lmax ({lmax})")
    if electrostatics is not None:
        raise ValueError("electrostatics: the long-range head is not part of this build (short-range model only)")
    if (lmax, edge_lmax) != (2, 2):
        raise ValueError("lmax / edge_lmax: kernels are compiled for degree 2 only")
    if dtype != torch.float32:
        raise ValueError("dtype: the kernels compute in float32")
    if torch.device(device).type != "cuda":
        raise ValueError(f"device: a CUDA device is required, got {device!r}")
    model = MaceIctcModel(channels=channels, lmax=lmax, num_interactions=num_interactions, correlation=correlation,
                          atomic_numbers=atomic_numbers, cutoff=cutoff, avg_num_neighbors=avg_num_neighbors)
    return model.to(device=device, dtype=dtype)


def energy_and_forces(model, positions, atomic_numbers, batch, edge_src, edge_dst, edge_shifts, cell, *,
                      training=False, owned_mask=None):
    """Energies per graph [B], forces [N, 3] = -dE/dpositions and per-atom energies [N] of a graph whose edges
    the caller has built (reference: mace_ictc/hp/runtime.py:82-111).

    ``edge_shifts`` are lattice coordinates, ``cell`` is [B, 3, 3].  ``owned_mask`` [N] (constant) selects the
    atoms whose energies count; the derivative is still taken with respect to every row of ``positions``,
    ghost rows included.  With ``training=True`` the force computation stays on the tape, so a loss on the
    forces can be differentiated (mixed second derivatives); otherwise everything returned is detached.
    """
    if torch.is_inference_mode_enabled():
        raise ValueError("forces need the autograd tape: call under torch.no_grad(), not torch.inference_mode()")
    count = positions.shape[0] if positions.ndim == 2 else -1
    if count < 0 or positions.shape[1] != 3:
        raise ValueError(f"positions: expected [N, 3], got {tuple(positions.shape)}")
    if cell.ndim != 3 or tuple(cell.shape[1:]) != (3, 3):
        raise ValueError(f"cell: expected [B, 3, 3], got {tuple(cell.shape)}")
    for name, value in (("atomic_numbers", atomic_numbers), ("batch", batch)):
        if tuple(value.shape) != (count,):
            raise ValueError(f"{name}: expected shape [{count}], got {tuple(value.shape)}")
    if owned_mask is not None:
        if tuple(owned_mask.shape) != (count,) or owned_mask.requires_grad:
            raise ValueError(f"owned_mask: expected a constant tensor of shape [{count}]")
    with torch.enable_grad():
        coords = positions if positions.requires_grad else positions.detach().requires_grad_(True)
        per_atom = model(coords, atomic_numbers, batch, edge_src, edge_dst, edge_shifts, cell)
        if isinstance(per_atom, tuple):
            per_atom = per_atom[0]
        per_atom = per_atom.reshape(count)
        counted = per_atom if owned_mask is None else per_atom * owned_mask.to(per_atom.dtype)
        energy = torch.zeros(cell.shape[0], dtype=counted.dtype, device=counted.device).index_add_(0, batch, counted)
        # the zero-weighted coordinate sum keeps `coords` in the graph when there is no edge at all
        total = energy.sum() + 0.0 * coords.sum()
        (gradient,) = torch.autograd.grad(total, coords, create_graph=training, retain_graph=training)
    forces = -gradient
    if training:
        return {"energy": energy, "forces": forces, "atomic_energy": per_atom}
    return {"energy": energy.detach(), "forces": forces.detach(), "atomic_energy": per_atom.detach()}


_LEGACY_KEYS = {"policy", "training", "capture", "layout", "message_schedule", "edge_chunk_size", "gate_schedule",
                "training_gate_schedule", "training_message_linear_layout", "species_schedule", "fuse_activation",
                "inference_message_layout", "radial_checkpoint", "assume_edges_within_radius",
                "preserve_edge_order", "skip_input_validation"}


def configure_model(model, *, policy="auto", training=False, **options):
    """Bind a runtime plan to the model (hp/runtime.py:136-297).

    The reference selects among K100 kernel schedules here; this build has one kernel path, so the
    call validates its arguments, applies the options that change semantics (``preserve_edge_order``,
    ``assume_edges_within_radius``, ``skip_input_validation``) and reports the same info-dict keys.
    """
    if not isinstance(model, MaceIctcModel):
        raise TypeError("Expected a model created by mace_ictc.hp.create_model")
    if policy not in ("auto", "generated", "reference"):
        raise ValueError("policy must be auto, generated or reference")
    if not isinstance(training, bool):
        raise TypeError("training must be a boolean")
    unknown = set(options) - _LEGACY_KEYS
    if unknown:
        raise ValueError(f"Unknown runtime options: {sorted(unknown)}")
    for key in ("preserve_edge_order", "assume_edges_within_radius", "skip_input_validation"):
        if key in options:
            if not isinstance(options[key], bool):
                raise TypeError(f"{key} must be a boolean")
            setattr(model, key, options[key])
    parameter = next(model.parameters())
    supported = parameter.is_cuda and parameter.dtype == torch.float32
    if policy == "generated" and not supported:
        raise ValueError("generated plan requires a CUDA FP32 model")
    return {"selected": "generated" if supported and policy != "reference" else "reference",
            "reasons": [] if supported else ["model is not CUDA FP32"],
            "counts": {"interactions": len(model.interactions), "products": len(model.products)},
            "layout": options.get("layout", "packed"),
            "training_gate_schedule": "materialized", "training_message_linear_layout": "node_component",
            "training": training}


def check_model(model, *, training=False, capture=False):
    """Read-only coverage check (hp/runtime.py:119-133)."""
    reasons = []
    if not isinstance(model, MaceIctcModel):
        reasons.append("not a model created by create_model")
    else:
        p = next(model.parameters())
        if not p.is_cuda or p.dtype != torch.float32:
            reasons.append("model is not CUDA FP32")
    if capture:
        reasons.append("whole-model capture is not provided")
    return {"supported": not reasons, "reasons": reasons}
