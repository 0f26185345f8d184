"""Mirror of ``mslk/quantize/triton/quantize_kernels``: the MXFP4 quantizers on this library's CUDA kernels."""
from typing import Optional

import torch


def _resolve_seed(seed: Optional[int], stochastic: bool, device: torch.device) -> int:
    """Seed of the stochastic rounding mode as the reference resolves it
    (``mslk/quantize/triton/quantize_kernels/__init__.py:20-44``): 0 when the mode is not stochastic, the caller's seed
    masked to 63 bits, else the CUDA generator's initial seed (so ``torch.manual_seed`` is respected), 0 on CPU."""
    if not stochastic:
        return 0
    if seed is None:
        if device.type != "cuda":
            return 0
        seed = torch.cuda.default_generators[device.index].initial_seed()
    return int(seed) & ((1 << 63) - 1)
