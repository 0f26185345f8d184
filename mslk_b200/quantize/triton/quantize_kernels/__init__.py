"""Mirror of ``mslk/quantize/triton/quantize_kernels``: the MXFP4 quantizers on this library's CUDA kernels."""
