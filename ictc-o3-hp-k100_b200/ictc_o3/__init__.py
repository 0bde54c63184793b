"""ICTC O(3) operators on B200 — drop-in for the ``ictc_o3`` package of the reference."""
from .operators import (EdgeTensorProduct, GraphMessage, PackedGraphMessage, channel_linear,  # noqa: F401
                        configure_symmetric_contraction, create_symmetric_contraction, direction_harmonics,
                        normalized_silu)

__all__ = [
    "EdgeTensorProduct", "GraphMessage", "PackedGraphMessage", "direction_harmonics",
    "create_symmetric_contraction", "configure_symmetric_contraction", "channel_linear", "normalized_silu",
]
