"""Benchmarks: fused all-reduce sweeps, baselines (NCCL + separate kernels, the reference build) and models."""
