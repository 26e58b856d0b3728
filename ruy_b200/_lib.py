"""Loader for the in-tree CUDA library (ruy_b200/libruy_b200.so).

There is no fallback of any kind: if the shared library is missing or cannot be
loaded, importing code gets an ImportError that says how to build it.
"""
import ctypes as C
import os

from . import _abi

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libruy_b200.so")
_lib = None


def lib():
    """Returns the loaded C-ABI library with prototypes declared."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} has not been built; run `python -m ruy_b200.build` "
            "(needs nvcc with sm_100a support). There is no CPU fallback.")
    handle = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    for name, (restype, argtypes) in _abi.PROTOTYPES.items():
        fn = getattr(handle, name)  # AttributeError here = header / library mismatch
        fn.restype = restype
        fn.argtypes = argtypes
    got = handle.ruyb200_abi_version()
    if got != _abi.ABI_VERSION:
        raise ImportError(f"{LIB_PATH}: ABI version {got}, expected {_abi.ABI_VERSION}")
    _lib = handle
    return _lib
