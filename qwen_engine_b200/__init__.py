"""B200 (sm_100a) implementation of the W4A16 group-128 projection path of qwen-engine.

The product is the CUDA library `libw4a16_b200.so` behind the C ABI in
`include/w4a16_b200.h`; `ops` is a thin Python mirror of the reference's launch functions
over that ABI (torch supplies device memory and streams only).
"""
from . import _lib  # noqa: F401
from .ops import *  # noqa: F401,F403
