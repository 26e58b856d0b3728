"""The benchmark configurations at their full sizes, every output compared.

The scalar C oracle is too slow for these sizes, so the checker is the compiled, unmodified reference
(ruy::Mul on all host threads: Path::kStandardCpp for the reference rounding, the widest x86 path for the
x86 rounding), exactly as ruy's own tests compare every path with the reference on the same inputs
(ruy/test.h:2222-2270).  Where the compiled reference is not available the same cases are checked on sampled
sub-blocks against 64-bit numpy arithmetic."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import oracle
import ruy_b200
import util
from ruy_b200 import _abi, cases
from ruy_b200.api import CachePolicy, Matrix, MulParams, Rounding

pytestmark = pytest.mark.gpu
THREADS = os.cpu_count() or 1


def numpy_block(c, rows_sel, cols_sel):
    """Reference-rounding result of the sampled rows x cols of case `c` in 64-bit numpy (ruy/kernel.h:213-237,
    ruy/apply_multiplier.cc:53-64); row-major LHS and column-major RHS storage without padding."""
    L = c.lhs.reshape(c.rows, c.depth).astype(np.int64)[rows_sel]
    R = c.rhs.reshape(c.cols, c.depth).astype(np.int64)[cols_sel]
    acc = (L - c.lhs_zp) @ (R - c.rhs_zp).T
    if c.bias is not None:
        acc = acc + c.bias.astype(np.int64)[rows_sel][:, None]
    if c.dst_dtype != "int32":
        if isinstance(c.mfp, np.ndarray):
            m = c.mfp.astype(np.int64)[rows_sel][:, None]
            e = c.mexp.astype(np.int64)[rows_sel][:, None]
        else:
            m, e = np.int64(c.mfp), np.int64(c.mexp)
        acc = (acc * m + (np.int64(1) << (30 - e))) >> (31 - e)
        acc = np.clip(acc + c.dst_zp, c.clamp[0], c.clamp[1])
    return acc


def check_against_reference(c, ctx, sample_seed=0):
    """Bit-exact comparison of the whole result in both rounding modes; returns how it was checked."""
    ref = oracle.reference()
    got, _ = util.run_gpu(c, ctx, rounding=Rounding.kReference)
    if ref is not None:
        want = util.run_reference(c, path=_abi.PATH_STANDARD_CPP, threads=THREADS)
        assert np.array_equal(got, want), f"{c.name}: {(got != want).sum()} mismatches (reference rounding)"
        simd = oracle.host_simd_path()
        if simd != _abi.PATH_STANDARD_CPP:
            gx, _ = util.run_gpu(c, ctx, rounding=Rounding.kX86)
            wx = util.run_reference(c, path=simd, threads=THREADS)
            assert np.array_equal(gx, wx), f"{c.name}: {(gx != wx).sum()} mismatches (x86 rounding)"
            return "compiled reference, both roundings"
        return "compiled reference, reference rounding"
    rng = np.random.default_rng(sample_seed)
    rows_sel = np.sort(rng.choice(c.rows, min(c.rows, 64), replace=False))
    cols_sel = np.sort(rng.choice(c.cols, min(c.cols, 256), replace=False))
    rows_sel[0], rows_sel[-1], cols_sel[0], cols_sel[-1] = 0, c.rows - 1, 0, c.cols - 1
    want = numpy_block(c, rows_sel, cols_sel)
    sub = got[np.ix_(rows_sel, cols_sel)].astype(np.int64)
    assert np.array_equal(sub, want), f"{c.name}: {(sub != want).sum()} mismatches in the sampled block"
    return "sampled blocks against numpy"


@pytest.mark.parametrize("layer", range(len(cases.CONFIG4_LAYERS)))
def test_config4_layers_batch64(layer, gpu_ctx):
    """The uint8 pointwise-conv layers at batch 64 (up to 802816 columns, 6272 tiles in one launch)."""
    c = cases.config4(layer, batch=64)
    how = check_against_reference(c, gpu_ctx, sample_seed=layer)
    got, _ = util.run_gpu(c, gpu_ctx, rounding=Rounding.kReference)
    assert 0.02 < (got == got.max()).mean() + (got == got.min()).mean() < 0.98, how   # outputs span the range


def test_config2_full_plan(gpu_ctx):
    """All 16384 muls of the batched small-mul configuration in one plan, run twice, every destination compared
    (the cost-sorted schedule and the accumulator ring over ~110 items per CTA are only exercised at this size)."""
    dev = torch.device("cuda", 0)
    n = 16384
    cs = cases.config2(n=n, seed=0)

    def pool(arrays, dtype):
        offs, total = [], 0
        item = np.dtype(dtype).itemsize
        for a in arrays:
            offs.append(total)
            total += (a.size * item + 255) // 256 * 256 // item
        host = np.zeros(max(total, 1), dtype=dtype)
        for a, o in zip(arrays, offs):
            host[o:o + a.size] = a
        return torch.from_numpy(host).to(dev), offs

    lhs_buf, lhs_off = pool([c.lhs for c in cs], np.int8)
    rhs_buf, rhs_off = pool([c.rhs for c in cs], np.int8)
    bias_buf, vec_off = pool([c.bias for c in cs], np.int32)
    mfp_buf, _ = pool([c.mfp for c in cs], np.int32)
    mexp_buf, _ = pool([c.mexp for c in cs], np.int32)
    dst_buf, dst_off = pool([c.new_dst() for c in cs], np.int8)
    descs = []
    for i, c in enumerate(cs):
        lhs = Matrix(lhs_buf[lhs_off[i]:], c.lhs_layout, c.lhs_zp, CachePolicy.kAlwaysCache)
        rhs = Matrix(rhs_buf[rhs_off[i]:], c.rhs_layout, c.rhs_zp)
        dst = Matrix(dst_buf[dst_off[i]:], c.dst_layout, c.dst_zp)
        p = MulParams("int32", "int8")
        p.bias = bias_buf[vec_off[i]:]
        p.multiplier_fixedpoint_perchannel = mfp_buf[vec_off[i]:]
        p.multiplier_exponent_perchannel = mexp_buf[vec_off[i]:]
        p.clamp_min, p.clamp_max = c.clamp
        p.rounding = Rounding.kReference
        descs.append(ruy_b200.make_desc(lhs, rhs, p, dst))
    # the expected results: the compiled reference when present (about 10 ms of AVX-512 work), else the C oracle
    ref = oracle.reference()
    want = []
    if ref is not None:
        rctx = ref.ruy_ref_ctx_create(_abi.PATH_STANDARD_CPP, 1)
        try:
            for c in cs:
                want.append(util.run_reference(c, ctx=rctx))
        finally:
            ref.ruy_ref_ctx_destroy(rctx)
    else:
        want = [util.run_oracle(c) for c in cs]
    with ruy_b200.Context(0) as ctx:
        plan = ruy_b200.Plan(ctx, descs)
        try:
            for rep in range(2):
                torch.cuda.synchronize()
                before = ctx.counters()["launches"]
                plan.run()
                ctx.sync()
                assert ctx.counters()["launches"] - before == 1
                host = dst_buf.cpu().numpy()
                bad = [i for i, c in enumerate(cs)
                       if not np.array_equal(c.dst_view(host[dst_off[i]:dst_off[i] + c.dst_storage_elems()]), want[i])]
                assert not bad, f"replay {rep}: {len(bad)} of {n} muls differ, first {bad[:5]}"
                dst_buf.zero_()
        finally:
            plan.close()


def test_config3_full_against_compiled_reference(gpu_ctx):
    """4096 x 4096 x 8192 int8 -> int8, all 33.5 M outputs against ruy's own AVX-512 path (x86 rounding), which does
    this mul in a fraction of a second on the host cores.  The reference rounding of the same mul is covered by
    test_config3_full_size_properties (int8 result == requantised int32 result, int32 checked by checksums)."""
    ref = oracle.reference()
    simd = oracle.host_simd_path()
    if ref is None or simd == _abi.PATH_STANDARD_CPP:
        pytest.skip("needs the compiled reference and an x86 SIMD path on the host")
    c = cases.config3(dst="int8")
    gx, _ = util.run_gpu(c, gpu_ctx, rounding=Rounding.kX86)
    wx = util.run_reference(c, path=simd, threads=THREADS)
    assert np.array_equal(gx, wx), f"{(gx != wx).sum()} of {gx.size} outputs differ"
    # the two rounding contracts differ on a small fraction of the outputs, never by more than one
    gr, _ = util.run_gpu(c, gpu_ctx, rounding=Rounding.kReference)
    diff = np.abs(gr.astype(np.int32) - gx.astype(np.int32))
    assert diff.max() <= 1 and 0 < (diff != 0).mean() < 0.02


SHALLOW = [  # (rows, depth, cols, lhs, rhs, dst, per-channel, channel dimension)
    (64, 32, 151552 + 4 * 37, "uint8", "uint8", "uint8", False, "row"),     # ragged last tile
    (40, 32, 160000, "int8", "uint8", "int8", True, "row"),                 # n not a multiple of 16, per-row multipliers
    (128, 64, 75776 + 2 * 51, "int8", "uint8", "int8", True, "col"),        # depth 64, per-column (activation side) channels
    (100, 64, 80000, "int8", "int8", "int8", False, "row"),
    (256, 128, 37888 + 77, "uint8", "uint8", "uint8", False, "row"),        # depth 128: one row per line, 256 columns shared by two warps per quarter
    (200, 128, 40000, "int8", "uint8", "int8", True, "row"),                # an odd number of 32-column chunks, per-row multipliers
    (96, 128, 38000, "int8", "int8", "int8", True, "col"),
]


@pytest.mark.parametrize("spec", SHALLOW, ids=lambda s: "x".join(map(str, s[:3])) + "_" + s[7])
def test_shallow_depth_kernel(spec, capfd):
    """Depth 32 / 64 / 128 with contiguous activation rows takes the kernel that fetches 128-byte lines of whole rows;
    the same cases on the general kernel (RUYB200_NO_SHALLOW=1) must give the same bits."""
    from ruy_b200.api import ChannelDimension
    rows, depth, cols, lt, rt, dt, pc, ch = spec
    c = cases.random_case(rows, depth, cols, lt, rt, dt, orders="RCC", perchannel=pc, symmetric=False, seed=rows + depth,
                          channel=ChannelDimension.kRow if ch == "row" else ChannelDimension.kCol,
                          lhs_cache=CachePolicy.kAlwaysCache)
    os.environ["RUYB200_TRACE"] = "1"
    try:
        ctx = ruy_b200.Context(0)
    finally:
        del os.environ["RUYB200_TRACE"]
    try:
        check_against_reference(c, ctx, sample_seed=rows)
        assert "shallow depth" in capfd.readouterr().err
        got, _ = util.run_gpu(c, ctx, rounding=Rounding.kReference)
    finally:
        ctx.close()
    os.environ["RUYB200_NO_SHALLOW"] = "1"
    try:
        plain = ruy_b200.Context(0)
    finally:
        del os.environ["RUYB200_NO_SHALLOW"]
    try:
        want, _ = util.run_gpu(c, plain, rounding=Rounding.kReference)
    finally:
        plain.close()
    assert np.array_equal(got, want)


def test_shallow_depth_kernel_clamp_forms(gpu_ctx):
    """The shallow-depth kernel applies the clamp while narrowing: a clamp that is the whole range of the destination
    type (saturating narrowing only), an ordinary one, and a degenerate one whose lower bound exceeds the upper
    (ruy takes the minimum with the upper bound first, then the maximum with the lower: every output is the lower)."""
    for dt, clamp in (("uint8", (0, 255)), ("int8", (-128, 127)), ("uint8", (17, 201)), ("int8", (50, 10))):
        c = cases.random_case(48, 64, 75776, "int8" if dt == "int8" else "uint8", "uint8", dt, orders="RCC", symmetric=False, seed=9,
                              lhs_cache=CachePolicy.kAlwaysCache)
        c.clamp = clamp
        check_against_reference(c, gpu_ctx, sample_seed=3)
        got, _ = util.run_gpu(c, gpu_ctx, rounding=Rounding.kReference)
        if clamp[0] > clamp[1]:
            assert np.all(got == clamp[0])
        else:
            assert got.min() >= clamp[0] and got.max() <= clamp[1]


def test_general_kernel_clamp_forms(gpu_ctx):
    """The same three clamp forms on the general tensor-core kernel (depth 512 keeps it off the shallow-depth one)."""
    for dt, clamp in (("uint8", (0, 255)), ("int8", (-128, 127)), ("uint8", (17, 201)), ("int8", (50, 10))):
        c = cases.random_case(200, 512, 1000, "int8" if dt == "int8" else "uint8", "uint8", dt, orders="RCC", symmetric=False, seed=10)
        c.clamp = clamp
        check_against_reference(c, gpu_ctx, sample_seed=4)
