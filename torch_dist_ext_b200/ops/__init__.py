"""Operators: the fused all-reduce family, standalone hot ops, GEMMs and attention."""
from . import activation, attention, gemm, norm, quant, reference, rope, sampling  # noqa: F401
from . import fused_gemm  # noqa: F401,E402
