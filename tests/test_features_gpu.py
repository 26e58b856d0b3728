"""GPU tests of the parts around the main kernels: the narrow-mul kernel and its dispatch, the tile-shape
choice of the tensor-core kernel (every candidate shape must give the same bits), persistence of prepacked
cache entries, the bounded peer wait, and plans that share a cached source pointer."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import ruy_b200
import util
from ruy_b200 import _abi, cases
from ruy_b200._lib import lib
from ruy_b200.api import CachePolicy, ChannelDimension, Rounding

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def ctx_with_env(**env):
    """A context created while the given environment variables are set (they are read at creation)."""
    old = {k: os.environ.get(k) for k in env}
    os.environ.update(env)
    try:
        return ruy_b200.Context(0)
    finally:
        for k, v in old.items():
            if v is None:
                del os.environ[k]
            else:
                os.environ[k] = v


def exact(case, ctx, **kw):
    got, _ = util.run_gpu(case, ctx, rounding=Rounding.kReference, **kw)
    want = util.run_oracle(case, Rounding.kReference)
    assert np.array_equal(got, want), f"{case.name}: {(got != want).sum()} mismatches"
    gx, _ = util.run_gpu(case, ctx, rounding=Rounding.kX86, **kw)
    wx = util.run_oracle(case, util.x86_rounding_for(case))
    assert np.array_equal(gx, wx), f"{case.name} (x86 rounding): {(gx != wx).sum()} mismatches"


# ---- narrow muls ---------------------------------------------------------------------------------

NARROW = [(256, 64, 1), (1, 64, 256), (4096, 512, 1), (300, 1000, 3), (5, 777, 130), (8, 4096, 8), (1000, 33, 8),
          (7, 5, 2), (1, 32767, 1), (2, 45984, 3),
          # two and four wide rows per warp, with rows left over at the end
          (2051, 100, 3), (9000, 96, 1), (4, 130, 8195), (16386, 64, 8)]


@pytest.mark.parametrize("shape", NARROW, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("types", [("int8", "int8", "int8"), ("uint8", "uint8", "uint8"), ("int8", "uint8", "int16"),
                                   ("uint8", "int8", "int32")], ids=lambda t: "-".join(t))
def test_narrow_8bit_muls_take_the_gemv_kernel(shape, types, gpu_ctx):
    for orders, ch in (("RCC", ChannelDimension.kRow), ("RCR", ChannelDimension.kCol)):
        c = cases.random_case(*shape, *types, orders=orders, perchannel=True, channel=ch, symmetric=False, seed=sum(shape))
        exact(c, gpu_ctx)
        assert gpu_ctx.counters()["last_kernel"] == "gemv"


# a wide side of 1024 rows or more, 2 to 16 narrow rows and a depth that is a multiple of 16: the form of the kernel
# that feeds 16 wide rows per CTA to register-level MMAs.  Depths of one partial step (64), whole steps plus a tail
# (4112 = 16 steps of 256 and 16 bytes), several rounds of the CTA's 8 warps; wide rows left over past the last 16;
# one or two tiles of 8 narrow rows; the narrow side as either operand.
NARROW_MMA = [(1030, 4112, 5), (3, 2064, 1100), (2048, 96, 9), (1024, 64, 16), (1500, 784, 13), (10, 272, 1024),
              (1040, 16, 2), (4099, 2304, 15)]


@pytest.mark.parametrize("shape", NARROW_MMA, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("types", [("int8", "int8", "int8"), ("uint8", "uint8", "uint8"), ("int8", "uint8", "int16"),
                                   ("uint8", "int8", "int32")], ids=lambda t: "-".join(t))
def test_up_to_16_narrow_rows_on_a_wide_operand_take_the_gemv_kernel(shape, types, gpu_ctx):
    narrow_is_rhs = shape[2] < shape[0]
    for symmetric in (False, True):
        # depth-contiguous operands: a row-major LHS and a column-major RHS
        for dst_order, ch in (("C", ChannelDimension.kRow), ("R", ChannelDimension.kCol)):
            c = cases.random_case(*shape, *types, orders="RC" + dst_order, perchannel=True, channel=ch, symmetric=symmetric,
                                  seed=sum(shape) + int(symmetric))
            exact(c, gpu_ctx)
            assert gpu_ctx.counters()["last_kernel"] == "gemv", (shape, narrow_is_rhs)


def test_more_than_8_narrow_rows_need_aligned_rows_for_the_gemv_kernel(gpu_ctx):
    # a depth that is not a multiple of 16, or rows off the 16-byte grid: packing and the tensor core
    c = cases.random_case(2048, 100, 12, "int8", "int8", "int8", orders="RCC", perchannel=True, seed=21)
    exact(c, gpu_ctx)
    assert gpu_ctx.counters()["last_kernel"] == "tc_i8"
    c = cases.random_case(2048, 128 + 16, 12, "int8", "int8", "int8", orders="RCC", extra_stride=3, seed=22)
    exact(c, gpu_ctx)
    assert gpu_ctx.counters()["last_kernel"] == "tc_i8"
    # a cached weight matrix is read in its packed form, whose rows are aligned
    c = cases.random_case(2048, 640, 12, "int8", "int8", "int8", orders="RCC", perchannel=True, seed=23, lhs_cache=CachePolicy.kAlwaysCache)
    exact(c, gpu_ctx, where="host")
    assert gpu_ctx.counters()["last_kernel"] == "gemv"
    # under 1024 wide rows, and from 17 narrow rows on, the tensor-core kernels keep the mul
    for shape in ((1000, 256, 12), (2048, 256, 17)):
        c = cases.random_case(*shape, "int8", "int8", "int8", orders="RCC", perchannel=True, seed=24)
        exact(c, gpu_ctx)
        assert gpu_ctx.counters()["last_kernel"] != "gemv"


def test_narrow_muls_other_layouts_and_host_operands(gpu_ctx):
    # operands that are not depth-contiguous cannot be streamed: they go through packing and the tensor core
    c = cases.random_case(300, 200, 4, "int8", "int8", "int8", orders="CRC", perchannel=True, seed=3)
    exact(c, gpu_ctx)
    assert gpu_ctx.counters()["last_kernel"] == "tc_i8"
    # odd strides: depth-contiguous but not 16-byte aligned, the kernel walks them bytewise
    c = cases.random_case(300, 203, 4, "uint8", "int8", "uint8", orders="RCC", extra_stride=3, symmetric=False, seed=4)
    exact(c, gpu_ctx)
    assert gpu_ctx.counters()["last_kernel"] == "gemv"
    # host operands are staged as they are; a cached weight matrix is read in its packed form
    c = cases.random_case(512, 640, 2, "int8", "int8", "int8", orders="RCC", perchannel=True, seed=5, lhs_cache=CachePolicy.kAlwaysCache)
    exact(c, gpu_ctx, where="host")
    assert gpu_ctx.counters()["last_kernel"] == "gemv"


def test_few_wide_rows_with_a_very_deep_depth_go_to_the_tensor_core(gpu_ctx):
    c = cases.random_case(64, 16384, 4, "int8", "int8", "int8", orders="RCC", perchannel=True, seed=12)
    exact(c, gpu_ctx)
    assert gpu_ctx.counters()["last_kernel"] == "tc_i8"
    c = cases.random_case(64, 16384, 1, "int8", "int8", "int8", orders="RCC", perchannel=True, seed=13)
    exact(c, gpu_ctx)
    assert gpu_ctx.counters()["last_kernel"] == "gemv"


def test_narrow_muls_can_stay_on_the_tensor_core():
    ctx = ctx_with_env(RUYB200_FORCE_KERNEL="tc_i8")
    try:
        for shape in ((256, 64, 1), (5, 777, 130), (1000, 33, 8)):
            c = cases.random_case(*shape, "int8", "uint8", "int8", orders="RCC", perchannel=True, symmetric=False, seed=9)
            exact(c, ctx)
            assert ctx.counters()["last_kernel"] == "tc_i8"
    finally:
        ctx.close()


@pytest.mark.parametrize("shape", [(256, 64, 1), (1, 64, 256), (1000, 1000, 1), (3, 32767, 2), (500, 301, 8), (64, 7, 5),
                                   (2051, 100, 3), (8195, 68, 4), (7, 50, 8201)],
                         ids=lambda s: "x".join(map(str, s)))
def test_narrow_float_muls(shape, gpu_ctx):
    for orders, extra in (("RCC", 0), ("RCR", 0), ("RCC", 1)):
        c = cases.random_case(*shape, "float32", "float32", "float32", orders=orders, extra_stride=extra, seed=sum(shape))
        got, _ = util.run_gpu(c, gpu_ctx)
        wide = util.run_oracle(c, wide_float=True).astype(np.float64)
        err = np.abs(got.astype(np.float64) - wide)
        assert np.all(err <= 1e-5 * np.maximum(np.abs(wide), 1.0)), float(err.max())
        assert gpu_ctx.counters()["last_kernel"] == "gemv"


# ---- tile shapes ---------------------------------------------------------------------------------

TILES = ["single:256", "single:192", "single:128", "single:64", "single:32", "pair:256", "pair:192", "pair:128", "pair:64"]


@pytest.mark.parametrize("tile", TILES)
def test_every_tile_shape_gives_the_same_bits(tile):
    """The tile-shape choice is free to pick any candidate, so each of them is forced in turn on shapes with ragged
    edges in every dimension (one- and two-CTA tiles, 8-, 16- and 32-bit destinations, fused and cached sums)."""
    ctx = ctx_with_env(RUYB200_TILE=tile)
    try:
        for shape, types in (((700, 208, 520), ("uint8", "uint8", "uint8")), ((512, 1024, 300), ("int8", "int8", "int8")),
                             ((300, 96, 260), ("int8", "uint8", "int16")), ((260, 40, 1100), ("int8", "int8", "int32"))):
            for orders in ("RCC", "RCR"):
                c = cases.random_case(*shape, *types, orders=orders, perchannel=True, symmetric=False, seed=len(tile))
                exact(c, ctx)
                assert ctx.counters()["last_kernel"] == "tc_i8"
        c = cases.config0(512, 512, 512, lhs_cache=CachePolicy.kAlwaysCache)
        exact(c, ctx)
    finally:
        ctx.close()


def test_tile_shape_choice_is_logged(capfd):
    ctx = ctx_with_env(RUYB200_TRACE="1")
    try:
        c = cases.config3(rows=1024, depth=512, cols=1024, dst="int8")
        got, _ = util.run_gpu(c, ctx, rounding=Rounding.kReference)
    finally:
        ctx.close()
    err = capfd.readouterr().err
    assert "kernel=tc_i8 tiles=" in err and "estimated" in err


# ---- persistence of prepacked weights --------------------------------------------------------------

def test_cache_export_import_round_trip():
    """Export the cached form of the weights from one context, import it into a fresh one: the next mul is a cache
    hit, launches no packing kernel and gives the same bits."""
    for c in (cases.config0(lhs_cache=CachePolicy.kAlwaysCache),
              cases.config3(rows=512, depth=1000, cols=384, dst="int8"),
              cases.random_case(200, 333, 64, "uint8", "uint8", "uint8", orders="CCC", symmetric=False, seed=8,
                                lhs_cache=CachePolicy.kAlwaysCache)):
        want = util.run_oracle(c, Rounding.kReference)
        dst = torch.zeros(c.dst_storage_elems(), dtype=getattr(torch, c.dst_dtype), device=DEV)
        lhs, rhs, p, d, keep = c.bind(dst, device=DEV, rounding=Rounding.kReference)
        with ruy_b200.Context(0) as a:
            ruy_b200.mul(lhs, rhs, p, a, d)
            assert a.counters()["cache_misses"] == 1
            blob = a.cache_export(lhs, 0)
            with pytest.raises(ruy_b200.RuyError):
                a.cache_export(rhs, 1)   # not cached
        info = ruy_b200.api.cache_blob_info(blob)
        assert info["width"] == c.rows and info["depth"] == c.depth and info["side"] == 0 and info["zero_point"] == c.lhs_zp
        assert info["format"] == _abi.CACHE_FORMAT_ROWS16 and info["has_sums"] == 1
        with ruy_b200.Context(0) as b:
            b.cache_import(lhs, 0, blob)
            assert b.prepacked_cache_entries() == 1
            before = b.counters()
            dst.zero_()
            ruy_b200.mul(lhs, rhs, p, b, d)
            after = b.counters()
            assert after["cache_hits"] - before["cache_hits"] == 1 and after["cache_misses"] == before["cache_misses"]
            # the mul itself is the only launch (plus the activation sums when the kernel cannot fuse them)
            assert after["launches"] - before["launches"] <= 2
            assert np.array_equal(c.dst_view(dst.cpu().numpy()), want)
            # a blob for another matrix is refused and leaves the cache alone
            other = cases.config0(128, 512, 64, lhs_cache=CachePolicy.kAlwaysCache)
            ol, _, _, _, okeep = other.bind(torch.zeros(other.dst_storage_elems(), dtype=torch.int8, device=DEV), device=DEV)
            with pytest.raises(ruy_b200.RuyError):
                b.cache_import(ol, 0, blob)
            bad = bytearray(blob)
            bad[100] ^= 0x5A
            b.clear_prepacked_cache()
            with pytest.raises(ruy_b200.RuyError):
                b.cache_import(lhs, 0, bytes(bad))
            assert b.prepacked_cache_entries() == 0


def test_blob_with_rows_padded_to_16_bytes_only_is_still_usable():
    """8-bit rows of 256 bytes and more are cached (and exported) padded to whole 128-byte lines.  A blob of the same
    weights with rows padded to 16 bytes only, as earlier versions wrote them, imports and multiplies to the same bits."""
    import struct
    from test_cache_blob import fnv1a
    c = cases.random_case(64, 300, 48, "int8", "int8", "int8", orders="RCC", perchannel=True, symmetric=False, seed=41,
                          lhs_cache=CachePolicy.kAlwaysCache)
    want = util.run_oracle(c, Rounding.kReference)
    dst = torch.zeros(c.dst_storage_elems(), dtype=torch.int8, device=DEV)
    lhs, rhs, p, d, keep = c.bind(dst, device=DEV, rounding=Rounding.kReference)
    with ruy_b200.Context(0) as a:
        ruy_b200.mul(lhs, rhs, p, a, d)
        blob = a.cache_export(lhs, 0)
    info = ruy_b200.api.cache_blob_info(blob)
    assert info["packed_depth"] == 384 and info["depth"] == 300
    rows = np.frombuffer(blob, dtype=np.int8, count=64 * 384, offset=64).reshape(64, 384)
    sums = blob[64 + 64 * 384:]
    payload = np.ascontiguousarray(rows[:, :304]).tobytes() + sums
    head = bytearray(blob[:56])
    struct.pack_into("<i", head, 28, 304)                  # packed depth
    struct.pack_into("<Q", head, 40, 64 * 304)             # data bytes
    old = bytes(head) + struct.pack("<Q", fnv1a(payload, fnv1a(bytes(head)))) + payload
    assert ruy_b200.api.cache_blob_info(old)["packed_depth"] == 304
    with ruy_b200.Context(0) as b:
        b.cache_import(lhs, 0, old)
        before = b.counters()
        dst.zero_()
        ruy_b200.mul(lhs, rhs, p, b, d)
        assert b.counters()["cache_hits"] - before["cache_hits"] == 1
        assert np.array_equal(c.dst_view(dst.cpu().numpy()), want)


# ---- bounded waits ------------------------------------------------------------------------------------

def test_peer_wait_gives_up_and_the_context_stays_usable():
    """A wait on a flag that nobody raises returns by itself after the configured limit; the next sync reports
    RUYB200_ERR_TIMEOUT, clears the status word, and the context computes correctly afterwards."""
    with ruy_b200.Context(0) as ctx:
        ctx.set_peer_wait_ms(5)
        flags = torch.zeros(8, dtype=torch.int32, device=DEV)
        torch.cuda.synchronize()
        assert lib().ruyb200_peer_wait(ctx._h, C.c_void_p(flags.data_ptr()), 2, 1) == 0
        with pytest.raises(ruy_b200.RuyError) as e:
            ctx.sync()
        assert e.value.status == _abi.ERR_TIMEOUT
        ctx.sync()    # the status word was cleared
        targets = torch.tensor([flags.data_ptr() + 16], dtype=torch.int64, device=DEV)   # raises word 4, waits on word 0
        assert lib().ruyb200_peer_exchange(ctx._h, C.c_void_p(targets.data_ptr()), C.c_void_p(flags.data_ptr()), 1, 3) == 0
        with pytest.raises(ruy_b200.RuyError) as e:
            ctx.sync()
        assert e.value.status == _abi.ERR_TIMEOUT
        assert flags.cpu().tolist()[4] == 3
        c = cases.config0()
        got, _ = util.run_gpu(c, ctx, rounding=Rounding.kReference)
        assert np.array_equal(got, util.run_oracle(c))


# ---- plans that share a cached source --------------------------------------------------------------------

def test_two_plans_pin_the_same_source_pointer_on_different_sides():
    """One square int8 matrix is the cached LHS of one plan's mul and the cached RHS of another's: two cache entries
    under one source pointer.  Destroying the first plan must release its own entry only."""
    n = 64
    rng = np.random.default_rng(5)
    shared = rng.integers(-127, 127, size=(n, n), endpoint=True).astype(np.int8)
    other = rng.integers(-127, 127, size=(n, n), endpoint=True).astype(np.int8)
    t_shared = torch.from_numpy(shared.reshape(-1)).to(DEV)
    t_other = torch.from_numpy(other.reshape(-1)).to(DEV)
    from ruy_b200.api import Matrix, MulParams, Order, make_simple_layout
    rm, cm = make_simple_layout(n, n, Order.kRowMajor), make_simple_layout(n, n, Order.kColMajor)
    with ruy_b200.Context(0) as ctx:
        def plan_for(lhs, rhs):
            dst = torch.zeros(n * n, dtype=torch.int32, device=DEV)
            p = MulParams("int32", "int32")
            return ruy_b200.Plan(ctx, [ruy_b200.make_desc(lhs, rhs, p, Matrix(dst, cm))]), dst
        # row-major n x n as LHS; the same bytes viewed col-major as RHS (i.e. its transpose)
        p1, d1 = plan_for(Matrix(t_shared, rm, 0, CachePolicy.kAlwaysCache), Matrix(t_other, cm))
        p2, d2 = plan_for(Matrix(t_other, rm), Matrix(t_shared, cm, 0, CachePolicy.kAlwaysCache))
        assert ctx.prepacked_cache_entries() == 2
        p1.close()
        ctx.clear_prepacked_cache()          # only the first plan's entry may go
        assert ctx.prepacked_cache_entries() == 1
        p2.run()
        ctx.sync()
        want2 = other.astype(np.int64) @ shared.astype(np.int64).T     # rhs(k, j) = shared[j, k]
        assert np.array_equal(d2.cpu().numpy().reshape(n, n).T, want2)
        p2.close()
        ctx.clear_prepacked_cache()
        assert ctx.prepacked_cache_entries() == 0


# ---- mirrored destination with the flag exchange inside the launch ------------------------------------------

def test_mirrored_mul_with_the_exchange_folded_in():
    """One GPU stands in for three ranks: two mirrors on the same device, and flag words that this launch raises
    itself (so its wait finds them raised).  Then a flag that nobody raises: the launch gives up after the
    context's wait limit, the result is still complete, and the next sync reports the timeout."""
    from ruy_b200 import peer
    with ruy_b200.Context(0) as ctx:
        for shape in ((512, 256, 520), (300, 1024, 700), (64, 96, 40)):
            c = cases.random_case(*shape, "int8", "int8", "int8", orders="RCC", perchannel=True, seed=21)
            want = util.run_oracle(c, Rounding.kReference)
            bufs = [torch.full((c.dst_storage_elems(),), 9, dtype=torch.int8, device=DEV) for _ in range(3)]
            lhs, rhs, p, d, keep = c.bind(bufs[0], device=DEV, rounding=Rounding.kReference)
            words = torch.zeros(8, dtype=torch.int32, device=DEV)
            targets = torch.tensor([words.data_ptr(), words.data_ptr() + 4, words.data_ptr() + 8], dtype=torch.int64, device=DEV)
            desc = ruy_b200.make_desc(lhs, rhs, p, d)
            mirrors = (C.c_void_p * 2)(bufs[1].data_ptr(), bufs[2].data_ptr())
            torch.cuda.synchronize()
            for step in (1, 2):
                assert lib().ruyb200_mul_async_mirrored_exchange(ctx._h, C.byref(desc), mirrors, 2, C.c_void_p(targets.data_ptr()),
                                                                 C.c_void_p(words.data_ptr()), 3, step) == 0
                ctx.sync()
                assert words.cpu().tolist()[:4] == [step, step, step, 0]
                for b in bufs:
                    assert np.array_equal(c.dst_view(b.cpu().numpy()), want)
                    b.fill_(9)
        # rank 1 "never signals": its target is null, its word stays at 0
        ctx.set_peer_wait_ms(5)
        words.zero_()
        targets = torch.tensor([words.data_ptr(), 0], dtype=torch.int64, device=DEV)
        torch.cuda.synchronize()
        assert lib().ruyb200_mul_async_mirrored_exchange(ctx._h, C.byref(desc), mirrors, 2, C.c_void_p(targets.data_ptr()),
                                                         C.c_void_p(words.data_ptr()), 2, 7) == 0
        with pytest.raises(ruy_b200.RuyError) as e:
            ctx.sync()
        assert e.value.status == _abi.ERR_TIMEOUT
        assert np.array_equal(c.dst_view(bufs[2].cpu().numpy()), want)
        # and the finished-CTA counter was rewound: the next exchange works
        words.zero_()
        targets = torch.tensor([words.data_ptr(), words.data_ptr() + 4], dtype=torch.int64, device=DEV)
        torch.cuda.synchronize()
        assert lib().ruyb200_mul_async_mirrored_exchange(ctx._h, C.byref(desc), mirrors, 2, C.c_void_p(targets.data_ptr()),
                                                         C.c_void_p(words.data_ptr()), 2, 8) == 0
        ctx.sync()
        assert words.cpu().tolist()[:2] == [8, 8]


# ---- fp32 on the tensor core ------------------------------------------------------------------------------

TF32_SHAPES = [(1024, 1024, 1024), (200, 333, 130), (64, 512, 64), (129, 2048, 96), (640, 32, 257), (300, 1500, 520)]


@pytest.mark.parametrize("shape", TF32_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_float_muls_on_the_tensor_core(shape, gpu_ctx):
    """3 x TF32 with 32-deep accumulation chains must meet the same bound as the FFMA kernel:
    |gpu - ref64| <= 1e-5 * max(|ref64|, 1) against a double-accumulated reference, for every storage order."""
    for orders, ch in (("RCC", ChannelDimension.kRow), ("CRC", ChannelDimension.kRow), ("RCR", ChannelDimension.kCol),
                       ("CCR", ChannelDimension.kRow)):
        c = cases.random_case(*shape, "float32", "float32", "float32", orders=orders, channel=ch, seed=sum(shape),
                              extra_stride=0 if orders != "CCR" else 3)
        got, _ = util.run_gpu(c, gpu_ctx)
        assert gpu_ctx.counters()["last_kernel"] == "tc_f32"
        wide = util.run_oracle(c, wide_float=True).astype(np.float64)
        err = np.abs(got.astype(np.float64) - wide)
        assert np.all(err <= 1e-5 * np.maximum(np.abs(wide), 1.0)), (orders, float(err.max()))


@pytest.mark.parametrize("shape", [(129, 4100, 96), (96, 16384, 72)], ids=lambda s: "x".join(map(str, s)))
def test_very_deep_float_muls(shape, gpu_ctx):
    """Depth does not change the fp32 dispatch: both fp32 kernels add 32-deep chains into a compensated total, and
    the tensor-core kernel is the closer one to double precision.  The 1e-5 bound is the benchmark's (depth up to 1024)
    and still holds at 4100; at depth 16384 plain fp32 products leave about 1e-5 themselves, so the bound checked there
    is 3e-5, on either kernel."""
    c = cases.random_case(*shape, "float32", "float32", "float32", orders="RCC", seed=sum(shape))
    wide = util.run_oracle(c, wide_float=True).astype(np.float64)
    tol = 1e-5 if shape[1] <= 4100 else 3e-5
    got, _ = util.run_gpu(c, gpu_ctx)
    assert gpu_ctx.counters()["last_kernel"] == "tc_f32"
    err = np.abs(got.astype(np.float64) - wide)
    assert np.all(err <= tol * np.maximum(np.abs(wide), 1.0)), float(err.max())
    ffma = ctx_with_env(RUYB200_FORCE_KERNEL="sgemm")
    try:
        got, _ = util.run_gpu(c, ffma)
        assert ffma.counters()["last_kernel"] == "sgemm"
    finally:
        ffma.close()
    err = np.abs(got.astype(np.float64) - wide)
    assert np.all(err <= tol * np.maximum(np.abs(wide), 1.0)), float(err.max())


def test_float_tensor_core_and_ffma_kernels_agree():
    """Benchmark config 1's large shape on both fp32 kernels: each within 1e-5 of the double-precision reference, hence
    within 2e-5 of each other; small shapes stay on the FFMA kernel."""
    c = cases.config1((1024, 1024, 1024))
    wide = util.run_oracle(c, wide_float=True).astype(np.float64)
    ffma = ctx_with_env(RUYB200_FORCE_KERNEL="sgemm")
    try:
        a, _ = util.run_gpu(c, ffma)
        assert ffma.counters()["last_kernel"] == "sgemm"
    finally:
        ffma.close()
    with ruy_b200.Context(0) as ctx:
        b, _ = util.run_gpu(c, ctx)
        assert ctx.counters()["last_kernel"] == "tc_f32"
        small = cases.config1((100, 100, 100))
        util.run_gpu(small, ctx)
        assert ctx.counters()["last_kernel"] == "sgemm"
    for got in (a, b):
        assert np.all(np.abs(got - wide) <= 1e-5 * np.maximum(np.abs(wide), 1.0))
