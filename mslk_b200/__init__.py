"""mslk_b200 -- B200 (sm_100a) kernels for MSLK's low-precision GEMM path.

Per-row FP8 quantization, the rowwise-scaled FP8 GEMM (dense and grouped/stacked)
and the NVFP4 quantizer + GEMM, as hand-written CUDA behind a C ABI
(``include/mslk_b200.h``).  ``mslk_b200.ops`` holds tensor-level wrappers;
``mslk_b200.compat`` installs the reference's module paths and ``torch.ops.mslk``
operator names on top of them.  There is no CPU or eager fallback: importing
``mslk_b200.ops`` without the built library raises.
"""

__version__ = "0.1.0"
