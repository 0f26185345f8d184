"""Shared helpers for the test-suite: golden-fixture loading and raw <-> torch views."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_golden(name):
    path = os.path.join(GOLDEN, name)
    if not os.path.exists(path):
        return None
    return np.load(path)


def bf16(arr) -> torch.Tensor:
    return torch.from_numpy(arr.view(np.int16).copy()).view(torch.bfloat16)


def fp8(arr) -> torch.Tensor:
    return torch.from_numpy(arr.copy()).view(torch.float8_e4m3fn)


def u8(t: torch.Tensor) -> torch.Tensor:
    return t.contiguous().view(torch.uint8)


def randn_bf16(shape, seed, scale=1.0, device="cpu"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g, dtype=torch.float32) * scale).to(torch.bfloat16).to(device)
