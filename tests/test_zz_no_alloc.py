"""ruyb200_mul_noalloc, the entry point for callers that cannot allocate device memory when they
multiply (their own pool owns the device, they run under a fixed memory budget, or they cannot afford
the synchronisation an allocation implies).  It works out of a static device array instead of a
context's arena, so the check is simply: through the C ABI, on two calls in a row that reuse that
array with different shapes, zero points and destination types, it must produce exactly what the
regular entry point (ruyb200_mul) produces.  Collected last on purpose: a run that stops at the first
failure has then already run every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

import ruy_b200
import util
from ruy_b200 import _abi, cases
from ruy_b200._lib import lib
from ruy_b200.api import ChannelDimension, Rounding

pytestmark = pytest.mark.gpu


def _both(case, ctx):
    """Runs `case` through ruyb200_mul and through ruyb200_mul_noalloc on separate destinations."""
    dev = torch.device("cuda", 0)
    want, _ = util.run_gpu(case, ctx, where="device", rounding=Rounding.kReference)
    dst = torch.from_numpy(case.new_dst(fill=-3 if case.dst_dtype != "uint8" else 200)).to(dev)
    lhs, rhs, p, d, keep = case.bind(dst, device=dev, rounding=Rounding.kReference)
    torch.cuda.synchronize()
    ruy_b200.mul_noalloc(lhs, rhs, p, d)
    got = case.dst_view(dst.cpu().numpy()).copy()
    return want, got


def test_noalloc_matches_regular_entry_point_twice_in_a_row():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.init()
    torch.cuda.set_device(0)
    ctx = ruy_b200.Context(0)
    try:
        # first call: asymmetric uint8, both zero points non-zero (both sums in the scratch), wide shape
        first = cases.random_case(700, 208, 512, "uint8", "uint8", "uint8", orders="RCC", perchannel=True, symmetric=False,
                                  seed=71)
        # second call: smaller, other types, other storage order of the destination, per-column channels:
        # anything stale left in the array by the first call would show
        second = cases.random_case(130, 64, 257, "int8", "uint8", "int16", orders="RCR", perchannel=True,
                                   channel=ChannelDimension.kCol, symmetric=False, seed=72)
        third = cases.config0(dst="int32")
        for case in (first, second, third):
            want, got = _both(case, ctx)
            assert np.array_equal(got, want), f"{case.name}: {(got != want).sum()} mismatches"
            assert np.array_equal(want, util.run_oracle(case, Rounding.kReference))
    finally:
        ctx.close()


def test_noalloc_refuses_what_it_cannot_do():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    dev = torch.device("cuda", 0)
    # beyond the static scratch: 16385 destination rows
    big = cases.random_case(16385, 16, 8, "int8", "int8", "int8", seed=73)
    dst = torch.zeros(big.dst_storage_elems(), dtype=torch.int8, device=dev)
    lhs, rhs, p, d, keep = big.bind(dst, device=dev)
    desc = ruy_b200.make_desc(lhs, rhs, p, d)
    assert lib().ruyb200_mul_noalloc(C.byref(desc), None) == _abi.ERR_INVALID
    assert b"16384" in lib().ruyb200_last_error()
    # a layout that would need repacking, and host pointers
    c = cases.random_case(32, 48, 16, "int8", "int8", "int8", orders="CCC", seed=74)
    dst = torch.zeros(c.dst_storage_elems(), dtype=torch.int8, device=dev)
    lhs, rhs, p, d, keep = c.bind(dst, device=dev)
    desc = ruy_b200.make_desc(lhs, rhs, p, d)
    assert lib().ruyb200_mul_noalloc(C.byref(desc), None) == _abi.ERR_UNSUPPORTED
    c = cases.config0()
    lhs, rhs, p, d, keep = c.bind(c.new_dst())
    desc = ruy_b200.make_desc(lhs, rhs, p, d)
    assert lib().ruyb200_mul_noalloc(C.byref(desc), None) == _abi.ERR_INVALID
