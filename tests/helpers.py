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


def bf16_ulp_distance(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """|a - b| counted in bf16 steps: the bit patterns are mapped to a monotone integer line."""
    def key(t):
        i = t.contiguous().view(torch.int16).to(torch.int32)
        return torch.where(i < 0, -(i & 0x7FFF), i)
    return (key(a.to(torch.bfloat16)) - key(b.to(torch.bfloat16))).abs()


def assert_sharp_bf16(y: torch.Tensor, y_ref: torch.Tensor, tag: str, within_1ulp: float = 0.999, max_ulp: int = 2,
                      floor_abs: float = None):
    """The sharp GEMM check beside the reference's rtol/atol bound.  Both sides accumulate exact products in
    fp32 and round once to bf16, so they may differ only where the fp32 sums (different summation order)
    straddle a bf16 rounding boundary: at least `within_1ulp` of the elements must be within one bf16 step of
    `y_ref` and none further than `max_ulp` steps.  Elements that are tiny through cancellation
    (|y_ref| < rms/128) are held to the absolute step of that magnitude (rms * 2^-15) instead, since the
    summation-order error does not shrink with the result; `floor_abs` overrides that absolute step (sums of
    bf16-rounded partial products carry the rounding of the LARGER partials).  Returns the figures for the log."""
    y, y_ref = y.to(torch.bfloat16), y_ref.to(torch.bfloat16)
    d = bf16_ulp_distance(y, y_ref)
    rms = float(y_ref.float().pow(2).mean().sqrt())
    if floor_abs is None:
        floor_abs = rms * 2.0 ** -15
    tiny_ok = (y.float() - y_ref.float()).abs() <= floor_abs
    d_eff = torch.where(tiny_ok, torch.zeros_like(d), d)
    n = d.numel()
    frac1 = float((d_eff <= 1).sum()) / max(n, 1)
    worst = int(d_eff.max()) if n else 0
    report = {"case": tag, "elements": n, "max_ulp": worst, "frac_within_1ulp": frac1,
              "frac_equal": float((d == 0).sum()) / max(n, 1), "raw_max_ulp": int(d.max()) if n else 0}
    log = os.environ.get("MSLK_B200_PARITY_LOG")
    if log:
        import json
        with open(log, "a") as f:
            f.write(json.dumps(report) + "\n")
    print(report)
    assert frac1 >= within_1ulp, f"{tag}: only {frac1:.6f} of the elements are within 1 bf16 ulp ({report})"
    assert worst <= max_ulp, f"{tag}: an element is {worst} bf16 ulps from the fp32 formula ({report})"
    return report


def fp8_rowwise_formula_chunked(xq, wq, xs, ws, bias=None, rows_per_chunk=2048):
    """The reference tests' fp32 formula (dequantize, fp32 matmul, row x column scales, optional bias) over row
    chunks on the tensors' device, so that full benchmark sizes fit (test/gemm/triton/grouped_gemm_test.py:124-129)."""
    import oracle
    wf = None
    out = torch.empty((xq.shape[0], wq.shape[0]), dtype=torch.bfloat16, device=xq.device)
    for r in range(0, xq.shape[0], rows_per_chunk):
        out[r:r + rows_per_chunk] = oracle.gemm_f8_rowwise_torch(xq[r:r + rows_per_chunk], wq, xs[r:r + rows_per_chunk], ws, bias)
    del wf
    return out
