"""Comparison baseline built from library calls only: NCCL all-to-all(v) + cuBLAS GEMMs."""
