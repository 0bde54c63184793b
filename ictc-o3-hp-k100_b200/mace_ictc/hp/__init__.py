"""Whole-network entry points, same names as the reference's ``mace_ictc.hp``."""
from .runtime import check_model, configure_model, create_model, energy_and_forces  # noqa: F401

__all__ = ["create_model", "configure_model", "energy_and_forces", "check_model"]
