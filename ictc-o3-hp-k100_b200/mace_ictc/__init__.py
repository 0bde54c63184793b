"""MACE-ICTC model-level API on B200 (drop-in names of the reference's ``mace_ictc`` package)."""
