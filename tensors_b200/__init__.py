"""B200-native dense-contraction path for tensorforge: ctypes binding of libtfb.so.

The shared library is the product; this package only loads it, declares the C-ABI of
``include/tfb.h`` and offers thin helpers that take raw device pointers. There is no
CPU or library fallback: importing :mod:`tensors_b200.capi` fails if libtfb.so is missing.
"""
from .capi import lib, TfbError, check, DTYPE_F32, DTYPE_F16, DTYPE_BF16  # noqa: F401
