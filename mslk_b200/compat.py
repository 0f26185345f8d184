"""Drop-in aliasing: make ``import mslk.gemm`` / ``mslk.quantize.triton.*`` resolve to this package.

``install()`` registers this package's mirror modules under the reference's module names in
``sys.modules``, so code written against MSLK's FP8-rowwise / NVFP4 path
(``torch.ops.mslk.f8f8bf16_rowwise``, ``mslk.quantize.triton.fp8_quantize.quantize_fp8_row``,
``mslk.quantize.triton.fp4_quantize.triton_quantize_nvfp4``, ``mslk.quantize.triton.fp4_utils.*``, ``mslk.moe.activation.silu_mul_quant``)
runs unchanged on the B200 kernels.  It refuses to shadow a real ``mslk`` that is already imported.
"""

import importlib
import sys

_ALIASES = {
    "mslk": "mslk_b200",
    "mslk.gemm": "mslk_b200.gemm",
    "mslk.gemm.triton": "mslk_b200.gemm.triton",
    "mslk.gemm.triton.grouped_gemm": "mslk_b200.gemm.triton.grouped_gemm",
    "mslk.quantize": "mslk_b200.quantize",
    "mslk.quantize.triton": "mslk_b200.quantize.triton",
    "mslk.quantize.triton.fp8_quantize": "mslk_b200.quantize.triton.fp8_quantize",
    "mslk.quantize.triton.fp4_quantize": "mslk_b200.quantize.triton.fp4_quantize",
    "mslk.quantize.triton.fp4_utils": "mslk_b200.quantize.triton.fp4_utils",
    "mslk.quantize.triton.fp4_primitives": "mslk_b200.quantize.triton.fp4_primitives",
    "mslk.quantize.triton.quantize_kernels": "mslk_b200.quantize.triton.quantize_kernels",
    "mslk.quantize.triton.quantize_kernels.mx4": "mslk_b200.quantize.triton.quantize_kernels.mx4",
    "mslk.quantize.triton.quantize_kernels.mx4_stacked": "mslk_b200.quantize.triton.quantize_kernels.mx4_stacked",
    "mslk.moe": "mslk_b200.moe",
    "mslk.moe.activation": "mslk_b200.moe.activation",
    "mslk.moe.gather_scatter": "mslk_b200.moe.gather_scatter",
}


def install() -> None:
    existing = sys.modules.get("mslk")
    if existing is not None and getattr(existing, "__name__", "") != "mslk_b200":
        raise RuntimeError("a different 'mslk' package is already imported; refusing to shadow it")
    for alias, target in _ALIASES.items():
        sys.modules[alias] = importlib.import_module(target)
