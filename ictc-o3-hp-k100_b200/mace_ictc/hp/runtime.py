"""create_model / configure_model / energy_and_forces (reference: mace_ictc/hp/runtime.py:6-297)."""
from __future__ import annotations

import torch

from ..model import MaceIctcModel


def _degree(value, name):
    if not isinstance(value, int) or isinstance(value, bool) or value < 0:
        raise ValueError(f"{name} must be a nonnegative integer")


def _positive_integer(value, name):
    if not isinstance(value, int) or isinstance(value, bool) or value < 1:
        raise ValueError(f"{name} must be a positive integer")


def create_model(*, channels=64, lmax=3, edge_lmax=None, num_interactions=2, correlation=3, use_reduced_cg=False,
                 atomic_numbers=(1, 6, 8), cutoff=5.0, avg_num_neighbors=50.0, device="cuda", dtype=torch.float32,
                 electrostatics=None):
    """Create a parameterised Cartesian model with freshly initialised weights (hp/runtime.py:6-79).

    TP base coefficients are fixed to one; radial, linear and contraction weights are trainable.
    Compiled coverage: lmax = edge_lmax = 2, fp32, short-range only (``electrostatics`` must be None).
    """
    if not isinstance(num_interactions, int) or isinstance(num_interactions, bool) or num_interactions < 1:
        raise ValueError("num_interactions must be a positive integer")
    _positive_integer(channels, "channels")
    _positive_integer(correlation, "correlation")
    if correlation not in (1, 2, 3):
        raise ValueError("HP correlation currently supports 1, 2, 3; cor4/5 experiments are separate")
    if not isinstance(use_reduced_cg, bool):
        raise TypeError("use_reduced_cg must be a boolean")
    if use_reduced_cg:
        raise ValueError("The independent HP factory uses native full CG; cuEq reduced-basis generation is not enabled")
    _degree(lmax, "lmax")
    edge_lmax = lmax if edge_lmax is None else edge_lmax
    _degree(edge_lmax, "edge_lmax")
    if edge_lmax < lmax:
        raise ValueError("edge_lmax must be at least lmax")
    if electrostatics is not None:
        raise ValueError("the long-range electrostatics head is outside this build (short-range model only)")
    if lmax != 2 or edge_lmax != 2:
        raise ValueError("kernels are compiled for lmax = edge_lmax = 2")
    if dtype != torch.float32:
        raise ValueError("the kernels compute in fp32")
    if torch.device(device).type != "cuda":
        raise ValueError("the model requires a CUDA device")
    model = MaceIctcModel(channels=channels, lmax=lmax, num_interactions=num_interactions, correlation=correlation,
                          atomic_numbers=atomic_numbers, cutoff=cutoff, avg_num_neighbors=avg_num_neighbors)
    return model.to(device=device, dtype=dtype)


def energy_and_forces(model, positions, atomic_numbers, batch, edge_src, edge_dst, edge_shifts, cell, *,
                      training=False, owned_mask=None):
    """Energy [B], forces [N,3] = -dE/dpos, atomic_energy [N] of a prebuilt graph (hp/runtime.py:82-111).

    ``training=True`` keeps the graph of the force computation (mixed second derivatives for a force
    loss); otherwise results are detached.  Shifts are lattice coordinates, cell is [B,3,3].
    """
    if torch.is_inference_mode_enabled():
        raise ValueError("Full forces require autograd; use no_grad instead of inference_mode")
    if positions.ndim != 2 or positions.shape[1] != 3 or cell.ndim != 3 or cell.shape[1:] != (3, 3):
        raise ValueError("Expected positions [N,3] and cell [B,3,3]")
    n = positions.shape[0]
    if atomic_numbers.shape != (n,) or batch.shape != (n,):
        raise ValueError("Atomic numbers and graph batch must have shape [N]")
    if owned_mask is not None and (owned_mask.shape != (n,) or owned_mask.requires_grad):
        raise ValueError("owned_mask must be a fixed [N] tensor")
    with torch.enable_grad():
        pos = positions if positions.requires_grad else positions.detach().requires_grad_(True)
        output = model(pos, atomic_numbers, batch, edge_src, edge_dst, edge_shifts, cell)
        atomic = (output[0] if isinstance(output, tuple) else output).reshape(n)
        selected = atomic if owned_mask is None else atomic * owned_mask.to(atomic)
        energy = selected.new_zeros(cell.shape[0]).index_add(0, batch, selected)
        force = -torch.autograd.grad(energy.sum() + pos.sum() * 0.0, pos, create_graph=training,
                                     retain_graph=training)[0]
        result = {"energy": energy, "forces": force, "atomic_energy": atomic}
        return result if training else {key: value.detach() for key, value in result.items()}


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
