"""Operators: the fused all-reduce family, standalone hot ops, GEMMs and attention."""
from . import activation, gemm, norm, quant, reference, rope  # noqa: F401
