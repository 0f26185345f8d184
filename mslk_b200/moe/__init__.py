"""Mirror of the reference's ``mslk.moe`` symbols that sit beside the FP8 GEMM path (activation only)."""

from .activation import silu_mul, silu_mul_quant  # noqa: F401
