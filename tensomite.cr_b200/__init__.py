"""B200-native decode engine for tensomite's quantised token loop: Python access to the C ABI.

The product is `libtsm_b200.so` (CUDA for sm_100a + C++ host runtime, `csrc/`), whose
entry points are declared in `include/tsm_b200.h`.  This package only loads that library
through ctypes and mirrors the reference's host-side names on top of it; there is no
Python or CPU implementation of any operator here, and every call fails loudly when the
library or a CUDA device is missing.
"""
from . import build, gguf, groups  # noqa: F401
from .binding import *  # noqa: F401,F403
