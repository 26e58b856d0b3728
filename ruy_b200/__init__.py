"""ruy_b200: ruy's matrix-multiplication hot path on NVIDIA B200 (sm_100a).

The product is the C-ABI shared library built from ruy_b200/csrc (declared in
include/ruy_b200.h) and the ruy-compatible C++ headers under include/ruy/.
This Python package is the host-side mirror of ruy's API used by the tests and
the benchmark.
"""
from .api import (  # noqa: F401
    CachePolicy, ChannelDimension, Context, Layout, Matrix, MulParams, Order, Path,
    PerformanceAdvisory, Plan, Rounding, RuyError, kAllPaths, kDefaultPaths,
    make_desc, make_simple_layout, mul, mul_async, mul_noalloc, validate,
)
