"""Parity of the CUDA library (through the C ABI) with the oracle and the golden reference outputs.
Integer results must be bit-exact; float results within 1e-5 relative of a double-accumulated
reference (|gpu - ref| <= 1e-5 * max(|ref|, 1))."""
import os

import numpy as np
import pytest
import torch

import ruy_b200
import util
from golden_cases import golden_cases, requant_extreme_cases
from ruy_b200 import cases
from ruy_b200.api import CachePolicy, ChannelDimension, Order, Path, PerformanceAdvisory, Rounding

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FLOAT_RTOL = 1e-5


@pytest.fixture(scope="module")
def generic_ctx(gpu_ctx):
    """A context whose muls are all served by the CUDA-core kernel."""
    os.environ["RUYB200_FORCE_KERNEL"] = "generic"
    try:
        ctx = ruy_b200.Context(0)
    finally:
        del os.environ["RUYB200_FORCE_KERNEL"]
    yield ctx
    ctx.close()


def assert_float_close(got, case):
    wide = util.run_oracle(case, wide_float=True).astype(np.float64)
    err = np.abs(got.astype(np.float64) - wide)
    assert np.all(err <= FLOAT_RTOL * np.maximum(np.abs(wide), 1.0)), float(err.max())


def assert_double_close(got, case):
    """Double accumulation in depth order on both sides; only fused against separate multiply-add can differ."""
    want = util.run_oracle(case).astype(np.float64)
    tol = 1e-6 if case.dst_dtype == "float32" else 1e-13
    err = np.abs(got.astype(np.float64) - want)
    assert np.all(err <= tol * np.maximum(np.abs(want), 1.0)), float(err.max())


def check_case(case, ctx, where="device", sentinel=None):
    got, storage = util.run_gpu(case, ctx, where=where, rounding=Rounding.kReference, sentinel=sentinel)
    if case.accum == "float64":
        assert_double_close(got, case)
    elif case.accum == "float32":
        assert_float_close(got, case)
    else:
        want = util.run_oracle(case, Rounding.kReference)
        assert np.array_equal(got, want), f"{case.name}: {(got != want).sum()} mismatches"
        gx, _ = util.run_gpu(case, ctx, where=where, rounding=Rounding.kX86)
        wx = util.run_oracle(case, util.x86_rounding_for(case))
        assert np.array_equal(gx, wx), f"{case.name} (x86 rounding): {(gx != wx).sum()} mismatches"
    if sentinel is not None:
        assert util.padding_untouched(case, storage, sentinel), "wrote outside the logical destination"


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c.name)
def test_golden_cases_default_kernels(case, gpu_ctx):
    g = np.load(os.path.join(GOLDEN, "ruy_reference_outputs.npz"))
    got, _ = util.run_gpu(case, gpu_ctx, rounding=Rounding.kReference)
    want = g[case.name + "/reference_mul"]
    if case.accum == "float64":
        assert_double_close(got, case)
        tol = 1e-6 if case.dst_dtype == "float32" else 1e-13
        assert np.all(np.abs(got.astype(np.float64) - want) <= tol * np.maximum(np.abs(want), 1.0))
        return
    if case.accum == "float32":
        assert_float_close(got, case)
        assert np.all(np.abs(got - want) <= 1e-4 * np.maximum(np.abs(want), 1.0))
        return
    assert np.array_equal(got, want), f"{(got != want).sum()} mismatches vs ruy::ReferenceMul"
    avx = g[case.name + "/avx512"]
    avx = want if avx.size == 0 else avx
    gx, _ = util.run_gpu(case, gpu_ctx, rounding=Rounding.kX86)
    assert np.array_equal(gx, avx), f"{(gx != avx).sum()} mismatches vs ruy::Mul on kAvx512"


@pytest.mark.parametrize("case", golden_cases()[::3], ids=lambda c: c.name)
def test_golden_cases_generic_kernel(case, generic_ctx):
    check_case(case, generic_ctx)
    assert generic_ctx.counters()["last_kernel"] == "generic"


@pytest.mark.parametrize("types", [("float64", "float32", "float32"), ("float32", "float64", "float64"),
                                   ("float64", "float64", "float64"), ("float32", "float32", "float64"),
                                   ("float64", "float64", "float32")])
def test_double_accumulation_mixes(types, gpu_ctx):
    """ruy's mixed floating-point cases (ruy/BUILD:1195-1207) and the other float/double mixes with a double accumulator:
    every storage order, padded strides, bias on either dimension, device and host operands, cache policies ignored."""
    l, r, d = types
    for s, (rows, depth, cols) in enumerate([(1, 1, 1), (7, 9, 5), (33, 70, 17), (64, 100, 48), (130, 257, 67)]):
        for o, ords in enumerate(["RCC", "CRR", "CCC", "RRR", "RCR", "CRC"]):
            c = cases.random_case(rows, depth, cols, l, r, d, orders=ords, extra_stride=o % 2, seed=4000 + s * 8 + o,
                                  channel=ChannelDimension.kCol if o % 2 else ChannelDimension.kRow,
                                  lhs_cache=CachePolicy.kAlwaysCache if o == 2 else CachePolicy.kNeverCache)
            assert c.accum == "float64"
            check_case(c, gpu_ctx, where="host" if o == 3 else "device", sentinel=7.0)
            assert gpu_ctx.counters()["last_kernel"] == "generic"
    c = cases.random_case(8, 16, 8, "float64", "float32", "float32", bias=False, seed=1)
    c.clamp = (-np.inf, np.inf)
    check_case(c, gpu_ctx)


def test_dispatch_uses_the_tensor_core_kernel_for_8bit(gpu_ctx):
    c = cases.config0()
    util.run_gpu(c, gpu_ctx)
    assert gpu_ctx.counters()["last_kernel"] == "tc_i8"
    util.run_gpu(cases.config1((50, 50, 50)), gpu_ctx)
    assert gpu_ctx.counters()["last_kernel"] == "sgemm"


@pytest.fixture(scope="module")
def single_cta_ctx(gpu_ctx):
    """A context that keeps the tensor-core kernel on one CTA per tile (no CTA pairs)."""
    os.environ["RUYB200_NO_PAIR"] = "1"
    try:
        ctx = ruy_b200.Context(0)
    finally:
        del os.environ["RUYB200_NO_PAIR"]
    yield ctx
    ctx.close()


PAIR_SHAPES = [(256, 128, 256), (512, 384, 640), (300, 208, 700), (1024, 4096, 512), (257, 64, 511), (768, 32, 256)]


@pytest.mark.parametrize("shape", PAIR_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_large_tiles_cta_pairs_and_single_cta(shape, gpu_ctx, single_cta_ctx):
    """Shapes with both destination dimensions >= 256 run on two-CTA (256 x 256) tiles; the same
    cases must also be exact on the one-CTA kernel."""
    rows, depth, cols = shape
    combos = [("int8", "int8", "int8", "RCC"), ("uint8", "uint8", "uint8", "RCR"), ("int8", "uint8", "int32", "RCC"),
              ("uint8", "int8", "int16", "RCR")]
    for i, (l, r, d, orders) in enumerate(combos):
        c = cases.random_case(rows, depth, cols, l, r, d, orders=orders, perchannel=bool(i % 2),
                              channel=ChannelDimension.kCol if i >= 2 else ChannelDimension.kRow, seed=900 + i,
                              symmetric=False if i % 2 else None)
        check_case(c, gpu_ctx)
        assert gpu_ctx.counters()["last_kernel"] == "tc_i8"
        check_case(c, single_cta_ctx)


# ruy/test_fast.cc:31-107 shape lists
SQUARES = list(range(1, 11)) + [15, 16, 17, 31, 32, 33, 63, 64, 65, 48]


@pytest.mark.parametrize("n", SQUARES)
def test_squares_all_orders(n, gpu_ctx):
    # ruy/test.h:481-498 (TestLinearAllOrders): 8 order combinations, strides one larger than minimal
    for o, orders in enumerate(["RCC", "CCC", "RRC", "CRC", "RCR", "CCR", "RRR", "CRR"]):
        c = cases.random_case(n, n, n, "int8", "int8", "int8", orders=orders, extra_stride=1, perchannel=bool(o % 2),
                              channel=ChannelDimension.kCol if o % 4 >= 2 else ChannelDimension.kRow, seed=n * 8 + o)
        check_case(c, gpu_ctx, sentinel=-77)


@pytest.mark.parametrize("types", [("uint8", "uint8", "uint8"), ("int8", "int8", "uint8"), ("int8", "uint8", "int8"),
                                   ("uint8", "int8", "int8"), ("uint8", "uint8", "int16"), ("int8", "int8", "int32"),
                                   ("int8", "uint8", "int32"), ("int8", "int16", "int16"), ("int16", "int8", "int16"),
                                   ("float32", "float32", "float32")], ids=lambda t: "x".join(t))
def test_type_matrix(types, gpu_ctx):
    # ruy/BUILD:1195-1207
    l, r, d = types
    shapes = [(3, 5, 78), (4, 5, 6), (65, 33, 17), (16, 160, 128), (130, 48, 257)]
    for s, (rows, depth, cols) in enumerate(shapes):
        for orders in (["RCC", "CRR"] if s % 2 else ["RCC", "CCC", "RRR"]):
            c = cases.random_case(rows, depth, cols, l, r, d, orders=orders, extra_stride=s % 2, perchannel=bool(s % 2),
                                  channel=ChannelDimension.kCol if s == 3 else ChannelDimension.kRow, seed=500 + s)
            check_case(c, gpu_ctx, sentinel=None if d == "float32" else 99)


@pytest.mark.parametrize("shape", [(1, 32767, 1), (5, 5001, 4), (2, 45984, 3), (8, 1024, 8), (8, 4096, 8)])
def test_deep(shape, gpu_ctx):
    # ruy/test_fast.cc:76-81, ruy/test_slow.cc:29-68 (incl. the row-sums overflow depth)
    for l, r, d in (("int8", "int8", "int8"), ("uint8", "uint8", "uint8")):
        check_case(cases.random_case(*shape, l, r, d, seed=31), gpu_ctx)
        check_case(cases.random_case(*shape, l, r, d, seed=32, symmetric=False), gpu_ctx)


@pytest.mark.parametrize("depth", [1, 2, 3, 4])
def test_shallow(depth, gpu_ctx):
    # ruy/test_fast.cc:83-88
    for n in (1, 7, 64, 100):
        check_case(cases.random_case(n, depth, n, "uint8", "uint8", "uint8", seed=n), gpu_ctx)


@pytest.mark.parametrize("width", [1, 2, 3, 4, 5, 8])
def test_narrow_and_gemv(width, gpu_ctx):
    # ruy/test_fast.cc:90-107
    for rows, depth in ((100, 50), (8, 64), (1000, 33)):
        check_case(cases.random_case(rows, depth, width, "int8", "int8", "int8", seed=width), gpu_ctx)
        check_case(cases.random_case(width, depth, rows, "uint8", "uint8", "uint8", orders="RCR", seed=width), gpu_ctx)
        check_case(cases.random_case(rows, depth, width, "float32", "float32", "float32", seed=width), gpu_ctx)


def test_host_pointers_are_staged_and_padding_preserved(gpu_ctx):
    before = gpu_ctx.counters()
    for c in (cases.config0(), cases.random_case(37, 100, 23, "uint8", "uint8", "uint8", orders="CRC", extra_stride=3, seed=2),
              cases.random_case(37, 100, 23, "int8", "int8", "int32", orders="RCR", extra_stride=2, seed=3),
              cases.config1((17, 301, 9))):
        check_case(c, gpu_ctx, where="host", sentinel=None if c.accum == "float32" else 55)
    after = gpu_ctx.counters()
    assert after["h2d_bytes"] > before["h2d_bytes"] and after["d2h_bytes"] > before["d2h_bytes"]


def test_large_host_operands_take_the_chunked_path(gpu_ctx):
    """Synchronous muls whose wide operand and destination are host memory are cut into chunks along the destination's
    outer dimension (copies in both directions overlapping the kernels): more launches than one, same results, padding
    untouched.  Column-major destination (the RHS is chunked, channels on the other dimension) and row-major destination
    (the LHS is chunked and the per-channel buffers move with the chunks)."""
    for shape, orders, lhs, rhs, dst in (((64, 2048, 2176), "RCC", "uint8", "uint8", "uint8"),
                                         ((2176, 2048, 40), "RCR", "int8", "int8", "int8")):
        c = cases.random_case(*shape, lhs, rhs, dst, orders=orders, extra_stride=16, perchannel=True,
                              symmetric=False if lhs == "uint8" else None, seed=5)
        before = gpu_ctx.counters()["launches"]
        got, storage = util.run_gpu(c, gpu_ctx, where="host", rounding=Rounding.kReference, sentinel=55)
        assert gpu_ctx.counters()["launches"] - before >= 3   # 2176 m indices in chunks of 768: three kernels
        want = util.run_oracle(c, Rounding.kReference)
        assert np.array_equal(got, want), f"{c.name}: {(got != want).sum()} mismatches"
        assert util.padding_untouched(c, storage, 55)


def test_chunked_path_with_only_one_side_on_the_host(gpu_ctx):
    """The same chunking when only the destination, or only the wide operand, is host memory."""
    dev = torch.device("cuda", 0)
    # device operands, large host destination
    c = cases.random_case(2048, 64, 2176, "uint8", "uint8", "uint8", orders="RCC", extra_stride=16, perchannel=True,
                          symmetric=False, seed=6)
    lhs, rhs, p, d, keep = c.bind(torch.zeros(c.dst_storage_elems(), dtype=torch.uint8, device=dev), device=dev,
                                  rounding=Rounding.kReference)
    host_dst = c.new_dst()
    d.data = host_dst
    before = gpu_ctx.counters()["launches"]
    ruy_b200.mul(lhs, rhs, p, gpu_ctx, d)
    assert gpu_ctx.counters()["launches"] - before >= 4
    assert np.array_equal(c.dst_view(host_dst), util.run_oracle(c, Rounding.kReference))
    # large host right-hand side (the chunked operand), device destination
    c = cases.random_case(64, 2048, 2176, "uint8", "uint8", "uint8", orders="RCC", extra_stride=16, perchannel=True,
                          symmetric=False, seed=6)
    dst_dev = torch.zeros(c.dst_storage_elems(), dtype=torch.uint8, device=dev)
    lhs, rhs, p, d, keep = c.bind(dst_dev, device=dev, rounding=Rounding.kReference)
    rhs.data = c.rhs
    before = gpu_ctx.counters()["launches"]
    ruy_b200.mul(lhs, rhs, p, gpu_ctx, d)
    assert gpu_ctx.counters()["launches"] - before >= 4
    assert np.array_equal(c.dst_view(dst_dev.cpu().numpy()), util.run_oracle(c, Rounding.kReference))


def test_mul_async_on_device_operands(gpu_ctx):
    c = cases.config0(exps=(-17, -13))
    got, _ = util.run_gpu(c, gpu_ctx, rounding=Rounding.kReference, use_async=True)
    assert np.array_equal(got, util.run_oracle(c))
    # host pointers are refused by the stream-ordered entry point
    lhs, rhs, p, dst, keep = c.bind(c.new_dst())
    with pytest.raises(ruy_b200.RuyError):
        ruy_b200.mul_async(lhs, rhs, p, gpu_ctx, dst)


def test_empty_and_degenerate_shapes(gpu_ctx):
    for rows, depth, cols in ((0, 5, 4), (4, 5, 0), (3, 0, 4)):
        c = cases.random_case(max(rows, 0), depth, max(cols, 0), "int8", "int8", "int8", seed=1)
        got, _ = util.run_gpu(c, gpu_ctx, rounding=Rounding.kReference)
        assert np.array_equal(got, util.run_oracle(c))


def test_default_multiplier_is_zero(gpu_ctx):
    # ruy/mul_params.h:259,264: an unset multiplier is 0, so every output is clamp(dst zero point)
    c = cases.random_case(9, 9, 9, "int8", "int8", "int8", seed=4)
    c.mfp, c.mexp, c.dst_zp = 0, 0, 7
    got, _ = util.run_gpu(c, gpu_ctx)
    assert (got == 7).all()


@pytest.mark.parametrize("dst,zp,cols", [("int8", 1, 1), ("int8", 1, 8), ("int8", -1, 8), ("uint8", 1, 8),
                                         ("int16", 1, 1), ("int16", -1, 8)])
def test_dst_zero_point_addition_saturates(dst, zp, cols, gpu_ctx):
    # ruy/test_overflow_dst_zero_point.cc:46-125
    from ruy_b200.api import Layout
    bias_v = 32767 if zp > 0 else -32768
    want = np.iinfo(dst).max if zp > 0 else np.iinfo(dst).min
    c = cases.MulCase("ovf", np.zeros(1, np.int8), Layout(1, 1, 1, Order.kColMajor), 0, np.zeros(cols, np.int8),
                      Layout(1, cols, 1, Order.kColMajor), 0, dst, Layout(1, cols, 1, Order.kColMajor), zp,
                      np.array([bias_v], np.int32), 2**31 - 1, 0)
    got, _ = util.run_gpu(c, gpu_ctx)
    assert (got == want).all()


def test_examples_known_answers(gpu_ctx):
    # example/example.cc:21-182: the tiny deterministic inputs, expected values from the oracle
    from ruy_b200.api import Layout
    rm, cm = Layout(2, 2, 2, Order.kRowMajor), Layout(2, 2, 2, Order.kColMajor)
    f = np.array([1, 2, 3, 4], np.float32)
    c = cases.MulCase("ex_float", f, rm, 0, f.copy(), cm, 0, "float32", cm, 0, np.array([1, 0], np.float32), clamp=(0.0, 15.0))
    got, _ = util.run_gpu(c, gpu_ctx)
    assert np.array_equal(got, np.array([[6, 12], [11, 15]], np.float32))
    c = cases.MulCase("ex_u8", np.array([124, 125, 126, 127], np.uint8), rm, 125, np.array([129, 130, 131, 132], np.uint8),
                      cm, 132, "uint8", cm, 129, None, 1 << 30, 0)
    got, _ = util.run_gpu(c, gpu_ctx)
    assert np.array_equal(got, util.run_oracle(c))
    i = np.array([1, 2, 3, 4], np.int8)
    c = cases.MulCase("ex_pc", i, rm, 0, i.copy(), cm, 0, "int8", cm, 0, None, np.array([3 << 28, 5 << 28], np.int32),
                      np.array([1, -2], np.int32))
    got, _ = util.run_gpu(c, gpu_ctx)
    assert np.array_equal(got, util.run_oracle(c))
    c = cases.MulCase("ex_raw", i, rm, 0, i.copy(), cm, 0, "int32", cm, 0)
    got, _ = util.run_gpu(c, gpu_ctx)
    assert np.array_equal(got, np.array([[5, 11], [11, 25]], np.int32))
    c = cases.MulCase("ex_i16", i, rm, 0, np.array([1000, 2000, 3000, 4000], np.int16), cm, 0, "int16", cm, 0, None,
                      np.array([3 << 28, 5 << 28], np.int32), np.array([1, -2], np.int32))
    got, _ = util.run_gpu(c, gpu_ctx)
    assert np.array_equal(got, util.run_oracle(c))


def test_paths_select_the_rounding_contract(gpu_ctx):
    # ruy/ctx.cc:67-76,150-178: last_used_path = most significant enabled path
    c = cases.config0(exps=(-17, -13))
    ref, x86 = util.run_oracle(c, Rounding.kReference), util.run_oracle(c, Rounding.kX86)
    assert (ref != x86).any()
    try:
        got, _ = util.run_gpu(c, gpu_ctx)  # nothing set explicitly: the normative reference rounding
        assert np.array_equal(got, ref)
        assert gpu_ctx.last_used_path() == Path.kAvx512
        gpu_ctx.set_runtime_enabled_paths(Path.kAvx512)
        assert gpu_ctx.get_runtime_enabled_paths() == Path.kAvx512 | Path.kStandardCpp
        got, _ = util.run_gpu(c, gpu_ctx)
        assert np.array_equal(got, x86) and gpu_ctx.last_used_path() == Path.kAvx512
        gpu_ctx.set_runtime_enabled_paths(Path.kAvx2Fma)
        got, _ = util.run_gpu(c, gpu_ctx)
        assert np.array_equal(got, x86) and gpu_ctx.last_used_path() == Path.kAvx2Fma
        gpu_ctx.set_runtime_enabled_paths(Path.kStandardCpp)
        got, _ = util.run_gpu(c, gpu_ctx)
        assert np.array_equal(got, ref) and gpu_ctx.last_used_path() == Path.kStandardCpp
    finally:
        gpu_ctx.set_runtime_enabled_paths(Path.kNone)


def test_context_defaults_and_advisory(gpu_ctx):
    # ruy/context_test.cc:27-44, ruy/perchannel_buffers_reallocation_test.cc:43-98
    assert gpu_ctx.max_num_threads == 1
    gpu_ctx.set_max_num_threads(4)
    assert gpu_ctx.max_num_threads == 4
    gpu_ctx.set_max_num_threads(1)
    c = cases.random_case(7, 8, 9, "int8", "int8", "int8", perchannel=True, seed=6)
    util.run_gpu(c, gpu_ctx)
    assert gpu_ctx.performance_advisory(PerformanceAdvisory.kReallocatedPerChannelBuffer)
    c2 = cases.random_case(16, 8, 9, "int8", "int8", "int8", perchannel=True, seed=6)
    util.run_gpu(c2, gpu_ctx)
    assert not gpu_ctx.performance_advisory(PerformanceAdvisory.kReallocatedPerChannelBuffer)


def test_prepacked_cache(gpu_ctx):
    # ruy/prepacked_cache_test.cc:39-285: miss then hit, key distinctness, policies, eviction, clear
    import torch
    ctx = ruy_b200.Context(0)
    try:
        c = cases.config0(64, 96, 32, exps=(-17, -13), lhs_cache=CachePolicy.kAlwaysCache)
        want = util.run_oracle(c)
        dev = torch.device("cuda", 0)
        dst = torch.zeros(c.dst_storage_elems(), dtype=torch.int8, device=dev)
        lhs, rhs, p, d, keep = c.bind(dst, device=dev, rounding=Rounding.kReference)
        torch.cuda.synchronize()
        ruy_b200.mul(lhs, rhs, p, ctx, d)
        k0 = ctx.counters()
        assert (k0["cache_misses"], k0["cache_hits"], ctx.prepacked_cache_entries()) == (1, 0, 1)
        assert np.array_equal(c.dst_view(dst.cpu().numpy()), want)
        dst.zero_()
        torch.cuda.synchronize()
        ruy_b200.mul(lhs, rhs, p, ctx, d)
        k1 = ctx.counters()
        assert (k1["cache_misses"], k1["cache_hits"], ctx.prepacked_cache_entries()) == (1, 1, 1)
        assert np.array_equal(c.dst_view(dst.cpu().numpy()), want)
        size_one = ctx.prepacked_cache_bytes()
        assert size_one >= 64 * 96
        # same pointer, different zero point => a different entry (ruy/prepacked_cache.h:68-80)
        lhs.zero_point = 1
        torch.cuda.synchronize()
        ruy_b200.mul(lhs, rhs, p, ctx, d)
        assert ctx.prepacked_cache_entries() == 2
        lhs.zero_point = 0
        # kNeverCache never inserts; kCacheIfLargeSpeedup caches only when the other side is narrow
        lhs.cache_policy = CachePolicy.kNeverCache
        ctx.clear_prepacked_cache()
        assert (ctx.prepacked_cache_entries(), ctx.prepacked_cache_bytes()) == (0, 0)
        torch.cuda.synchronize()
        ruy_b200.mul(lhs, rhs, p, ctx, d)
        assert ctx.prepacked_cache_entries() == 0
        lhs.cache_policy = CachePolicy.kCacheIfLargeSpeedup
        ruy_b200.mul(lhs, rhs, p, ctx, d)   # rhs has 32 columns: narrow
        assert ctx.prepacked_cache_entries() == 1
        wide = cases.config0(64, 96, 1024, lhs_cache=CachePolicy.kCacheIfLargeSpeedup)
        util.run_gpu(wide, ctx)
        assert ctx.prepacked_cache_entries() == 1  # 1024 columns: not worth caching under this policy
        # eviction: a budget of two entries keeps the most recently used ones
        ctx.clear_prepacked_cache()
        ctx.set_prepacked_cache_budget(2 * size_one + 64)
        mats = []
        for s in range(3):
            cs = cases.config0(64, 96, 32, exps=(-17, -13), seed=40 + s, lhs_cache=CachePolicy.kAlwaysCache)
            ds = torch.zeros(cs.dst_storage_elems(), dtype=torch.int8, device=dev)
            bound = cs.bind(ds, device=dev, rounding=Rounding.kReference)
            mats.append((cs, ds, bound))
            torch.cuda.synchronize()
            ruy_b200.mul(bound[0], bound[1], bound[2], ctx, bound[3])
            assert np.array_equal(cs.dst_view(ds.cpu().numpy()), util.run_oracle(cs))
        assert ctx.prepacked_cache_entries() == 2
        misses = ctx.counters()["cache_misses"]
        cs, ds, bound = mats[2]
        torch.cuda.synchronize()
        ruy_b200.mul(bound[0], bound[1], bound[2], ctx, bound[3])   # newest: still cached
        assert ctx.counters()["cache_misses"] == misses
        cs, ds, bound = mats[0]
        torch.cuda.synchronize()
        ruy_b200.mul(bound[0], bound[1], bound[2], ctx, bound[3])   # oldest: was evicted, packed again
        assert ctx.counters()["cache_misses"] == misses + 1
        assert np.array_equal(cs.dst_view(ds.cpu().numpy()), util.run_oracle(cs))
    finally:
        ctx.close()


def test_cached_host_weights_stay_resident(gpu_ctx):
    ctx = ruy_b200.Context(0)
    try:
        c = cases.config0(128, 256, 64, exps=(-17, -13), lhs_cache=CachePolicy.kAlwaysCache)
        want = util.run_oracle(c)
        dst = c.new_dst()
        lhs, rhs, p, d, keep = c.bind(dst, rounding=Rounding.kReference)
        k0 = ctx.counters()["h2d_bytes"]
        torch.cuda.synchronize()
        ruy_b200.mul(lhs, rhs, p, ctx, d)
        k1 = ctx.counters()["h2d_bytes"]
        assert np.array_equal(c.dst_view(dst), want)
        dst[:] = 0
        torch.cuda.synchronize()
        ruy_b200.mul(lhs, rhs, p, ctx, d)
        k2 = ctx.counters()["h2d_bytes"]
        # the second call with the same weight pointer does not upload the weights again
        assert k1 - k0 >= 128 * 256 + 64 * 256
        assert k2 - k1 == (k1 - k0) - 128 * 256
        assert np.array_equal(c.dst_view(dst), want)
    finally:
        ctx.close()


def test_pack_entry_point(gpu_ctx):
    import ctypes as C
    import torch
    from ruy_b200._lib import lib
    c = cases.random_case(45, 70, 21, "uint8", "int8", "int32", orders="CRC", extra_stride=1, seed=12)
    lhs, rhs, p, d, keep = c.bind(c.new_dst())
    for side, m in ((0, lhs), (1, rhs)):
        desc = m.to_desc()
        width = m.layout.rows if side == 0 else m.layout.cols
        depth = m.layout.cols if side == 0 else m.layout.rows
        pd = (depth + 15) // 16 * 16
        packed = torch.full((width * pd,), 7, dtype=torch.uint8, device="cuda")
        sums = torch.zeros(width, dtype=torch.int32, device="cuda")
        got_pd = C.c_int32()
        rc = lib().ruyb200_pack(gpu_ctx._h, C.byref(desc), side, packed.data_ptr(), packed.numel(), sums.data_ptr(),
                                C.byref(got_pd))
        assert rc == 0 and got_pd.value == pd
        logical = c.lhs if side == 0 else c.rhs
        lay = m.layout
        if lay.order == Order.kColMajor:
            mat = logical.reshape(lay.cols, lay.stride)[:, :lay.rows].T
        else:
            mat = logical.reshape(lay.rows, lay.stride)[:, :lay.cols]
        wk = mat if side == 0 else mat.T          # width x depth
        out = packed.cpu().numpy().view(logical.dtype).reshape(width, pd)
        assert np.array_equal(out[:, :depth], wk) and (out[:, depth:] == 0).all()
        assert np.array_equal(sums.cpu().numpy(), wk.astype(np.int64).sum(axis=1))


def test_config1_float_shapes(gpu_ctx):
    for shape in cases.CONFIG1_SHAPES:
        c = cases.config1(shape)
        got, _ = util.run_gpu(c, gpu_ctx)
        assert_float_close(got, c)


def test_config4_layers_batch1(gpu_ctx):
    for layer in range(len(cases.CONFIG4_LAYERS)):
        c = cases.config4(layer, batch=1)
        got, _ = util.run_gpu(c, gpu_ctx, rounding=Rounding.kReference)
        want = util.run_oracle(c)
        assert np.array_equal(got, want), (layer, int((got != want).sum()))
        assert 0.02 < (got == got.max()).mean() + (got == got.min()).mean() < 0.98  # outputs span the range


def test_config2_plan(gpu_ctx):
    import torch
    n = 48
    cs = cases.config2(n=16384, seed=0, first=100, count=n)
    dev = torch.device("cuda", 0)
    bound, descs = [], []
    for c in cs:
        dst = torch.zeros(c.dst_storage_elems(), dtype=torch.int8, device=dev)
        b = c.bind(dst, device=dev, rounding=Rounding.kReference)
        bound.append((c, dst, b))
        descs.append(ruy_b200.make_desc(b[0], b[1], b[2], b[3]))
    plan = ruy_b200.Plan(gpu_ctx, descs)
    nbytes, ops = plan.stats()
    assert ops == sum(c.ops for c in cs) and nbytes == sum(c.algorithmic_bytes() for c in cs)
    for _ in range(2):
        torch.cuda.synchronize()
        before = gpu_ctx.counters()["launches"]
        plan.run()
        gpu_ctx.sync()
        assert gpu_ctx.counters()["launches"] - before == 1          # all 48 muls in one persistent launch
        assert gpu_ctx.counters()["last_kernel"] == "batch_i8"
        for c, dst, b in bound:
            assert np.array_equal(c.dst_view(dst.cpu().numpy()), util.run_oracle(c)), c.name
            dst.zero_()
    plan.close()


def test_mirrored_destination_and_step_flags(gpu_ctx):
    """ruyb200_mul_async_mirrored on one GPU: the mirrors are two more buffers on the same device, so they must end
    up byte-identical to the destination (one-CTA and two-CTA tiles, ragged edges).  The flag pair is exercised in
    stream order: the signal precedes the wait, which therefore returns at once (a peer that never signals is a
    host-side concern and is not provoked on a GPU)."""
    import ctypes as C
    from ruy_b200 import peer
    from ruy_b200._lib import lib
    dev = torch.device("cuda", 0)
    # destination strides that are / are not multiples of 16 bytes, ragged ends in both dimensions
    for shape, extra in (((300, 208, 700), 0), ((64, 96, 40), 0), ((512, 128, 520), 0), ((300, 60, 270), 4), ((1024, 256, 600), 0),
                         ((384, 4096, 512), 16)):
        c = cases.random_case(*shape, "uint8", "int8", "uint8", orders="RCC", perchannel=True, symmetric=False, seed=77,
                              extra_stride=extra)
        want = util.run_oracle(c, Rounding.kReference)
        bufs = [torch.full((c.dst_storage_elems(),), 9, dtype=torch.uint8, device=dev) for _ in range(3)]
        lhs, rhs, p, d, keep = c.bind(bufs[0], device=dev, rounding=Rounding.kReference)
        torch.cuda.synchronize()
        peer.mul_async_mirrored(lhs, rhs, p, gpu_ctx, d, [bufs[1].data_ptr(), bufs[2].data_ptr()])
        gpu_ctx.sync()
        for b in bufs:
            assert np.array_equal(c.dst_view(b.cpu().numpy()), want)
            assert util.padding_untouched(c, b.cpu().numpy(), 9)
        # the same with the mirrored epilogue kept on store instructions (no copy-engine stores)
        os.environ["RUYB200_NO_STORE_MAPS"] = "1"
        try:
            plain = ruy_b200.Context(0)
        finally:
            del os.environ["RUYB200_NO_STORE_MAPS"]
        try:
            for b in bufs:
                b.fill_(9)
            torch.cuda.synchronize()
            peer.mul_async_mirrored(lhs, rhs, p, plain, d, [bufs[1].data_ptr(), bufs[2].data_ptr()])
            plain.sync()
            for b in bufs:
                assert np.array_equal(c.dst_view(b.cpu().numpy()), want)
                assert util.padding_untouched(c, b.cpu().numpy(), 9)
        finally:
            plain.close()
    flag_words = torch.zeros(8, dtype=torch.int32, device=dev)
    targets = torch.tensor([flag_words.data_ptr(), flag_words.data_ptr() + 4], dtype=torch.int64, device=dev)
    torch.cuda.synchronize()
    assert lib().ruyb200_peer_signal(gpu_ctx._h, C.c_void_p(targets.data_ptr()), 2, 5) == 0
    assert lib().ruyb200_peer_wait(gpu_ctx._h, C.c_void_p(flag_words.data_ptr()), 2, 5) == 0
    gpu_ctx.sync()
    assert flag_words.cpu().tolist()[:3] == [5, 5, 0]
    # both in one launch: every thread raises its flag first and then finds it raised
    assert lib().ruyb200_peer_exchange(gpu_ctx._h, C.c_void_p(targets.data_ptr()), C.c_void_p(flag_words.data_ptr()), 2, 6) == 0
    gpu_ctx.sync()
    assert flag_words.cpu().tolist()[:3] == [6, 6, 0]
    # float muls cannot be mirrored
    fc = cases.config1((50, 50, 50))
    dst = torch.zeros(fc.dst_storage_elems(), dtype=torch.float32, device=dev)
    lhs, rhs, p, d, keep = fc.bind(dst, device=dev)
    with pytest.raises(ruy_b200.RuyError):
        peer.mul_async_mirrored(lhs, rhs, p, gpu_ctx, d, [dst.data_ptr()])


def test_plan_mixed_items(gpu_ctx):
    """A plan with every kind of item: asymmetric uint8 (both zero-point sums computed while packing), int16 and
    int32 destinations, row-major destinations, per-column channels, depths that are not multiples of 8 or 32,
    a cached LHS, and muls too large for the batched kernel (replayed through the single-mul dispatch)."""
    import torch
    dev = torch.device("cuda", 0)
    specs = [
        dict(rows=16, depth=16, cols=16, lhs="uint8", rhs="uint8", dst="uint8", orders="RCC", symmetric=False),
        dict(rows=24, depth=40, cols=128, lhs="int8", rhs="uint8", dst="int8", orders="RCR", symmetric=False, perchannel=True),
        dict(rows=128, depth=128, cols=128, lhs="uint8", rhs="int8", dst="int16", orders="RCC", symmetric=False,
             perchannel=True, channel=ChannelDimension.kCol),
        dict(rows=97, depth=50, cols=33, lhs="int8", rhs="int8", dst="int32", orders="RCC"),
        dict(rows=5, depth=7, cols=3, lhs="uint8", rhs="uint8", dst="uint8", orders="RCR", symmetric=False, extra_stride=1),
        dict(rows=64, depth=96, cols=48, lhs="int8", rhs="int8", dst="int8", orders="RCC", perchannel=True,
             lhs_cache=CachePolicy.kAlwaysCache),
        dict(rows=64, depth=96, cols=48, lhs="int8", rhs="int8", dst="int8", orders="CRC", perchannel=True,
             lhs_cache=CachePolicy.kAlwaysCache),                       # column-major LHS: packed through the cache
        dict(rows=200, depth=64, cols=64, lhs="int8", rhs="int8", dst="int8", orders="RCC"),     # too many rows
        dict(rows=64, depth=300, cols=64, lhs="uint8", rhs="uint8", dst="uint8", orders="RCC", symmetric=False),  # too deep
        dict(rows=32, depth=32, cols=32, lhs="int8", rhs="int16", dst="int16", orders="RCC"),    # 16-bit operand
    ]
    ctx = ruy_b200.Context(0)
    try:
        bound, descs = [], []
        for i, sp in enumerate(specs):
            sp = dict(sp)
            c = cases.random_case(sp.pop("rows"), sp.pop("depth"), sp.pop("cols"), sp.pop("lhs"), sp.pop("rhs"), sp.pop("dst"),
                                  seed=300 + i, **sp)
            host = c.new_dst(fill=0)
            dst = torch.from_numpy(host).to(dev)
            b = c.bind(dst, device=dev, rounding=Rounding.kReference)
            bound.append((c, dst, b))
            descs.append(ruy_b200.make_desc(b[0], b[1], b[2], b[3]))
        plan = ruy_b200.Plan(ctx, descs)
        assert ctx.prepacked_cache_entries() == 2
        for rep in range(2):
            torch.cuda.synchronize()
            launches = ctx.counters()["launches"]
            plan.run()
            ctx.sync()
            assert ctx.counters()["launches"] - launches >= 1 + 3   # one batched launch + the three singles (+ helpers)
            for c, dst, b in bound:
                got = c.dst_view(dst.cpu().numpy())
                want = util.run_oracle(c, Rounding.kReference)
                assert np.array_equal(got, want), f"{c.name}: {(got != want).sum()} mismatches (replay {rep})"
                dst.zero_()
        # a live plan pins its cache entries
        ctx.clear_prepacked_cache()
        assert ctx.prepacked_cache_entries() == 2
        plan.close()
        ctx.clear_prepacked_cache()
        assert ctx.prepacked_cache_entries() == 0
    finally:
        ctx.close()


def _sampled_block_check(c, out, rows_sel, cols_sel):
    """Bit-exact check of a sampled rows x cols sub-block of a big result against numpy int64 dots."""
    L = c.lhs.reshape(c.rows, c.depth).astype(np.int64)[rows_sel]
    R = c.rhs.reshape(c.cols, c.depth).astype(np.int64)[cols_sel]      # col-major depth x cols
    acc = (L - c.lhs_zp) @ (R - c.rhs_zp).T
    if c.bias is not None:
        acc = acc + c.bias.astype(np.int64)[rows_sel][:, None]
    if c.dst_dtype != "int32":
        m = c.mfp.astype(np.int64)[rows_sel][:, None]
        e = c.mexp.astype(np.int64)[rows_sel][:, None]
        acc = (acc * m + (1 << (30 - e))) >> (31 - e)
        acc = np.clip(acc + c.dst_zp, c.clamp[0], c.clamp[1])
    got = out[np.ix_(rows_sel, cols_sel)].astype(np.int64)
    assert np.array_equal(got, acc), int((got != acc).sum())


def test_config3_full_size_properties(gpu_ctx):
    """4096 x 4096 x 8192: too big for the scalar oracle, so (1) a random 96 x 96 sub-block of the
    result is checked bit-exactly against 64-bit numpy dot products, (2) the sum of all raw
    accumulators equals the dot product of the operands' depth-wise sums (a checksum of checksums),
    (3) the int8 result equals the requantized int32 result element for element."""
    import torch
    rng = np.random.default_rng(1)
    c32 = cases.config3(dst="int32")
    dev = torch.device("cuda", 0)
    d32 = torch.zeros(c32.dst_storage_elems(), dtype=torch.int32, device=dev)
    b = c32.bind(d32, device=dev)
    torch.cuda.synchronize()
    ruy_b200.mul(b[0], b[1], b[2], gpu_ctx, b[3])
    assert gpu_ctx.counters()["last_kernel"] == "tc_i8"
    raw = c32.dst_view(d32.cpu().numpy())
    rows_sel = np.sort(rng.choice(c32.rows, 96, replace=False))
    cols_sel = np.sort(rng.choice(c32.cols, 96, replace=False))
    rows_sel[0], rows_sel[-1], cols_sel[0], cols_sel[-1] = 0, c32.rows - 1, 0, c32.cols - 1
    _sampled_block_check(c32, raw, rows_sel, cols_sel)
    lsum = c32.lhs.reshape(c32.rows, c32.depth).astype(np.int64).sum(axis=0)
    rsum = c32.rhs.reshape(c32.cols, c32.depth).astype(np.int64).sum(axis=0)
    assert int(raw.astype(np.int64).sum()) == int(lsum @ rsum)
    c8 = cases.config3(dst="int8")
    d8 = torch.zeros(c8.dst_storage_elems(), dtype=torch.int8, device=dev)
    b8 = c8.bind(d8, device=dev, rounding=Rounding.kReference)
    torch.cuda.synchronize()
    ruy_b200.mul(b8[0], b8[1], b8[2], gpu_ctx, b8[3])
    out8 = c8.dst_view(d8.cpu().numpy())
    _sampled_block_check(c8, out8, rows_sel, cols_sel)
    acc = raw.astype(np.int64) + c8.bias.astype(np.int64)[:, None]
    m, e = c8.mfp.astype(np.int64)[:, None], c8.mexp.astype(np.int64)[:, None]
    want = np.clip(((acc * m + (1 << (30 - e))) >> (31 - e)) + c8.dst_zp, -128, 127).astype(np.int8)
    assert np.array_equal(out8, want)


def test_decision_trace_line(capfd, monkeypatch):
    """RUYB200_TRACE=1 (read when the context is created) logs one line per mul with the decisions taken, in the spirit
    of ruy's RUY_TRACE (ruy/trace.h)."""
    monkeypatch.setenv("RUYB200_TRACE", "1")
    with ruy_b200.Context(0) as ctx:
        c = cases.config0()
        got, _ = util.run_gpu(c, ctx, rounding=Rounding.kReference)
        assert np.array_equal(got, util.run_oracle(c))
    err = capfd.readouterr().err
    assert "ruy_b200: mul 256x512x128 kernel=tc_i8" in err and "rounding=reference" in err


def test_plan_replay_inside_a_cuda_graph():
    """A plan whose muls all fit the batched kernel is one kernel launch per replay with no allocation, so it can be
    captured into a CUDA graph by a caller that keeps activations on the device (the library itself does not capture)."""
    dev = torch.device("cuda", 0)
    stream = torch.cuda.Stream(device=dev)
    with ruy_b200.Context(0, stream=stream.cuda_stream) as ctx:
        cs = [cases.random_case(r, d, c, "int8", "int8", "int8", perchannel=True, seed=11 + i)
              for i, (r, d, c) in enumerate(((16, 32, 48), (64, 64, 64), (128, 96, 24), (24, 128, 128)))]
        bound, descs = [], []
        for c in cs:
            dst = torch.zeros(c.dst_storage_elems(), dtype=torch.int8, device=dev)
            lhs, rhs, p, d, keep = c.bind(dst, device=dev, rounding=Rounding.kReference)
            bound.append((c, dst, keep))
            descs.append(ruy_b200.make_desc(lhs, rhs, p, d))
        plan = ruy_b200.Plan(ctx, descs)
        with torch.cuda.stream(stream):
            plan.run()                      # warm-up outside the capture (sets the kernel's attributes)
            stream.synchronize()
            for _, dst, _ in bound:
                dst.zero_()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                plan.run()
            stream.synchronize()
            for _, dst, _ in bound:
                assert not dst.any()        # capture records, it does not execute
            graph.replay()
            torch.cuda.synchronize()
        for c, dst, _ in bound:
            assert np.array_equal(c.dst_view(dst.cpu().numpy()), util.run_oracle(c)), c.name
        plan.close()


@pytest.mark.parametrize("orders", ["RCC", "CRC", "RCR", "CCR"])
def test_float_few_outputs_long_depth(orders, gpu_ctx):
    """Few destination elements with a long depth take the warp-per-element fp32 kernel: every storage order and
    padded strides, within 1e-5 of a double-accumulated reference (assert_float_close)."""
    for shape in ((9, 200, 7), (1, 1000, 1), (31, 128, 33)):
        c = cases.random_case(*shape, "float32", "float32", "float32", orders=orders, extra_stride=3, seed=21)
        check_case(c, gpu_ctx)


def test_requantization_extremes_single_muls(gpu_ctx):
    for c in requant_extreme_cases():
        check_case(c, gpu_ctx)


def test_requantization_extremes_in_a_plan(gpu_ctx):
    dev = torch.device("cuda", 0)
    for rounding in (Rounding.kReference, Rounding.kX86):
        bound, descs = [], []
        for c in requant_extreme_cases():
            dst = torch.zeros(c.dst_storage_elems(), dtype=getattr(torch, c.dst_dtype), device=dev)
            lhs, rhs, p, d, keep = c.bind(dst, device=dev, rounding=rounding)
            bound.append((c, dst, keep))
            descs.append(ruy_b200.make_desc(lhs, rhs, p, d))
        plan = ruy_b200.Plan(gpu_ctx, descs)
        plan.run()
        gpu_ctx.sync()
        assert gpu_ctx.counters()["last_kernel"] == "batch_i8"
        for c, dst, _ in bound:
            want = util.run_oracle(c, Rounding.kReference if rounding == Rounding.kReference else util.x86_rounding_for(c))
            got = c.dst_view(dst.cpu().numpy())
            assert np.array_equal(got, want), f"{c.name} ({rounding.name}): {(got != want).sum()} mismatches"
        plan.close()


def test_one_context_per_thread_runs_concurrently():
    """ruy's threading contract (ruy/ruy.h:84-87): a Context belongs to one thread, several threads may multiply at the same
    time each with its own.  Four host threads, four contexts (each with its own stream), mixed kernels."""
    import threading
    todo = [cases.config0(), cases.config1((100, 100, 100)),
            cases.random_case(70, 200, 90, "uint8", "uint8", "uint8", symmetric=False, perchannel=True, seed=31),
            cases.random_case(33, 65, 17, "int8", "int16", "int16", seed=32)]
    want = [util.run_oracle(c, wide_float=True) if c.accum == "float32" else util.run_oracle(c, Rounding.kReference) for c in todo]
    errors = []

    def work(i):
        try:
            with ruy_b200.Context(0) as ctx:
                for rep in range(10):
                    got, _ = util.run_gpu(todo[i], ctx, where="host" if rep % 2 else "device", rounding=Rounding.kReference)
                    if todo[i].accum == "float32":
                        ok = np.all(np.abs(got.astype(np.float64) - want[i]) <= FLOAT_RTOL * np.maximum(np.abs(want[i]), 1.0))
                    else:
                        ok = np.array_equal(got, want[i])
                    if not ok:
                        errors.append((todo[i].name, rep))
        except Exception as e:   # noqa: BLE001 - reported through the list
            errors.append((todo[i].name, repr(e)))

    threads = [threading.Thread(target=work, args=(i,)) for i in range(len(todo))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_two_devices_in_one_process():
    """Contexts on two GPUs of one process: each kernel's shared-memory opt-in, caches and plans are per device."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    for dev_index in (1, 0, 1):
        dev = torch.device("cuda", dev_index)
        with ruy_b200.Context(dev_index) as ctx:
            for c in (cases.config0(), cases.random_case(300, 208, 700, "uint8", "int8", "uint8", symmetric=False, seed=41)):
                dst = torch.zeros(c.dst_storage_elems(), dtype=getattr(torch, c.dst_dtype), device=dev)
                lhs, rhs, p, d, keep = c.bind(dst, device=dev, rounding=Rounding.kReference)
                ruy_b200.mul(lhs, rhs, p, ctx, d)
                assert np.array_equal(c.dst_view(dst.cpu().numpy()), util.run_oracle(c, Rounding.kReference)), (dev_index, c.name)
            small = [cases.random_case(r, k, n, "int8", "int8", "int8", perchannel=True, seed=50 + i)
                     for i, (r, k, n) in enumerate(((16, 32, 48), (64, 64, 64), (128, 96, 24)))]
            bound, descs = [], []
            for c in small:
                dst = torch.zeros(c.dst_storage_elems(), dtype=torch.int8, device=dev)
                lhs, rhs, p, d, keep = c.bind(dst, device=dev, rounding=Rounding.kReference)
                bound.append((c, dst, keep))
                descs.append(ruy_b200.make_desc(lhs, rhs, p, d))
            plan = ruy_b200.Plan(ctx, descs)
            plan.run()
            ctx.sync()
            for c, dst, _ in bound:
                assert np.array_equal(c.dst_view(dst.cpu().numpy()), util.run_oracle(c)), (dev_index, c.name)
            plan.close()
