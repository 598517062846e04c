"""forge_b200: B200 (sm_100a) implementation of Forge's quantized-inference hot path.

The compute lives in libforge_b200.so (hand-written CUDA behind a C ABI, see
include/forge_b200.h); this package is the Python side of that boundary.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib"]
