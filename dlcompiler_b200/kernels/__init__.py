"""Operator wrappers; module names follow python/dlBLAS/dlblas/kernels/ of the reference."""
