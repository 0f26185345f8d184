"""Constants of the reference's ``mslk/quantize/triton/fp4_primitives`` package that callers pass to the quantizers."""
from enum import IntEnum


class RoundingMode(IntEnum):
    """How the shared exponent of an MX group is rounded (``mslk/quantize/triton/fp4_primitives/constants.py:42-60``).
    This library implements floor, even and ceil."""

    nearest = 0
    floor = 1
    even = 2
    stochastic = 3
    ceil = 4
