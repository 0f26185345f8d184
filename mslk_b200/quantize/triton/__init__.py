"""Module path kept from the reference (``mslk.quantize.triton``); the kernels here are CUDA, not Triton."""
