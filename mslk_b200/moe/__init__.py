"""Mirror of the reference's ``mslk.moe`` symbols that sit beside the FP8 GEMM path: the SwiGLU
activation (``activation``) and the token gather / scatter steps (``gather_scatter``)."""

from .activation import silu_mul, silu_mul_quant  # noqa: F401
from .gather_scatter import (  # noqa: F401
    gather_scale_dense_tokens,
    gather_scale_quant_dense_tokens,
    scatter_add_dense_tokens,
    scatter_add_padded_tokens,
)
