"""gem16_b200 -- B200 (sm_100a) operator library for gem16's quantized-weight contraction path.

The product is the C-ABI shared library `libgemb200.so` (declared in include/gemb200.h, sources
under gem16_b200/csrc).  This Python package only builds it, loads it through ctypes and offers
thin helpers that pass torch device pointers; there is no Python or CPU compute path.
"""
from .lib import GembError, Lib, load  # noqa: F401
