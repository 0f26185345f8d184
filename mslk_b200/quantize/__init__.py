"""Quantizers of the low-precision GEMM path (CUDA-backed; same module layout as the reference)."""
