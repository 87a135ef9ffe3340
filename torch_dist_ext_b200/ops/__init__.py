"""Operators: the fused all-reduce family, standalone hot ops, GEMMs and attention."""
from . import reference  # noqa: F401
