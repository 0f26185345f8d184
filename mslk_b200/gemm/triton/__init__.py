"""Mirror of the reference's ``mslk.gemm.triton`` entry points that this library serves."""
