"""Loads the operator library and registers the fake (meta) kernels.

Mirror of the reference's ``mslk/gemm/__init__.py:15-26``: after ``import mslk_b200.gemm``
(or ``import mslk.gemm`` once :func:`mslk_b200.compat.install` has run) the operators
``torch.ops.mslk.{f8f8bf16_rowwise, f8f8bf16_rowwise_out, f8f8bf16_rowwise_batched,
f8f8bf16_rowwise_grouped_stacked, f4f4bf16}`` exist, backed by the sm_100a kernels.  Importing fails loudly if the native
libraries have not been built.
"""

import os

import torch

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_OPS_LIB = os.path.join(_PKG, "_torch_ops.so")

if not os.path.exists(_OPS_LIB):
    raise ImportError(
        f"{_OPS_LIB} is missing: build it with `python -m mslk_b200.build`. "
        "The mslk:: operators have no Python or CPU fallback.")

# the C-ABI library must be loadable first (the operator library links against it by rpath)
from .. import _lib  # noqa: F401,E402

torch.ops.load_library(_OPS_LIB)

from . import _meta  # noqa: F401,E402

from . import _grouped_fp4  # noqa: F401,E402  mslk::f4f4bf16_grouped_stacked / mslk::f4f4bf16_grouped_mm
