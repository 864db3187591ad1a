"""B200-native implementation of MPTorch's simulated-arithmetic hot path.

Mirrors the reference package layout (``mptorch`` -> ``mptorch_b200``): number formats at the top level,
the quantization API under ``mptorch_b200.quant``.
"""
from .number import *  # noqa: F401,F403

__version__ = "0.1.0"

__all__ = ["FixedPoint", "BlockFloatingPoint", "FloatingPoint", "Binary8", "SuperNormalFloat"]
