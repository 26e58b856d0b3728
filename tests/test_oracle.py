"""Pins the C restatement (oracle/ruy_oracle.c): against the reference's own known-answer tests,
against golden outputs produced by the compiled reference, and against the compiled reference
itself when it is available on this machine.  No GPU needed."""
import os
import re

import numpy as np
import pytest

import oracle
import util
from golden_cases import golden_cases, requant_extreme_cases
from ruy_b200 import cases
from ruy_b200.api import ChannelDimension, Order, Rounding

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = os.path.join(HERE, "golden")
REF_TESTS = os.path.join(oracle.REFERENCE_DIR, "ruy")


def _golden_outputs():
    return np.load(os.path.join(GOLDEN, "ruy_reference_outputs.npz"))


def test_requant_known_answers_from_reference_test_source():
    """ruy/apply_multiplier_test.cc:39-94: every TestMultiplyByQuantizedMultiplier(...) line is
    parsed from the reference's test source and replayed on the oracle."""
    path = os.path.join(REF_TESTS, "apply_multiplier_test.cc")
    if not os.path.exists(path):
        pytest.skip("reference checkout not present on this machine")
    text = open(path).read()
    env = {"max_int32": 2**31 - 1}
    rows = re.findall(r"TestMultiplyByQuantizedMultiplier\(([^;]+)\);", text)
    checked = 0
    for row in rows:
        parts = [p.strip() for p in row.replace("\n", " ").split(",")]
        if len(parts) != 4 or "input" in parts[0]:
            continue
        x, m, e, want = (int(eval(p, {"__builtins__": {}}, env)) for p in parts)
        assert oracle.oracle().oracle_requant_reference(x, m, e) == want, row
        checked += 1
    assert checked >= 30


def test_requant_per_channel_dispatch_known_answers():
    """ruy/apply_multiplier_test.cc:105-124: uniform vs per-channel multiplier selection, driven
    through the whole oracle mul (accumulator = bias, zero operands)."""
    bias = np.full(4, 1000, dtype=np.int32)
    mfp = np.array([2**31 - 1, 1 << 30, 2**31 - 1, 1 << 30], dtype=np.int32)
    mexp = np.array([0, 0, -1, -1], dtype=np.int32)
    from ruy_b200.api import Layout, Order
    c = cases.MulCase("pc", np.zeros(4, np.int8), Layout(4, 1, 1, Order.kRowMajor), 0, np.zeros(1, np.int8),
                      Layout(1, 1, 1, Order.kColMajor), 0, "int16", Layout(4, 1, 4, Order.kColMajor), 0, bias, mfp, mexp)
    assert util.run_oracle(c)[:, 0].tolist() == [1000, 500, 500, 250]
    c.mfp, c.mexp = 1 << 30, -1
    assert util.run_oracle(c)[:, 0].tolist() == [250] * 4


@pytest.mark.parametrize("dst,zp,cols", [("int8", 1, 1), ("int8", 1, 8), ("int8", -1, 8), ("uint8", 1, 8),
                                         ("int16", 1, 1), ("int16", -1, 8)])
def test_dst_zero_point_addition_saturates(dst, zp, cols):
    """ruy/test_overflow_dst_zero_point.cc:46-125: bias at the int16 limit plus the destination
    zero point must clamp, not wrap."""
    from ruy_b200.api import Layout, Order
    bias_v = 32767 if zp > 0 else -32768
    want = np.iinfo(dst).max if zp > 0 else np.iinfo(dst).min
    c = cases.MulCase("ovf", np.zeros(1, np.int8), Layout(1, 1, 1, Order.kColMajor), 0, np.zeros(cols, np.int8),
                      Layout(1, cols, 1, Order.kColMajor), 0, dst, Layout(1, cols, 1, Order.kColMajor), zp,
                      np.array([bias_v], np.int32), 2**31 - 1, 0)
    assert (util.run_oracle(c) == want).all()


def test_requant_golden_rows():
    g = np.load(os.path.join(GOLDEN, "ruy_requant.npz"))
    o = oracle.oracle()
    got = np.array([o.oracle_requant_reference(int(a), int(b), int(c)) for a, b, c in zip(g["x"], g["m"], g["e"])])
    assert np.array_equal(got, g["multiply_by_quantized_multiplier"])
    sat = lambda v: np.clip(v, -32768, 32767).astype(np.int16)  # noqa: E731  (dst int16, clamp full range)
    assert np.array_equal(sat(got), g["standard_cpp_int16"])
    gx = np.array([o.oracle_requant_x86(int(a), int(b), int(c)) for a, b, c in zip(g["x"], g["m"], g["e"])])
    assert np.array_equal(sat(gx), g["avx512_int16"])
    assert (g["standard_cpp_int16"] != g["avx512_int16"]).sum() > 0  # the two contracts really differ


@pytest.mark.parametrize("case", golden_cases(), ids=lambda c: c.name)
def test_oracle_matches_golden_reference_outputs(case):
    g = _golden_outputs()
    import sys
    sys.path.insert(0, GOLDEN)
    from make_golden import input_digest
    assert input_digest(case) == g[case.name + "/digest"], "generator drifted; regenerate the golden files"
    want = g[case.name + "/reference_mul"]
    std = g[case.name + "/standard_cpp"]
    avx = g[case.name + "/avx512"]
    std = want if std.size == 0 else std
    avx = want if avx.size == 0 else avx
    if case.accum == "float64":
        # double sums in depth order on both sides; only the contraction of a*b+c may differ between compilers
        tol = 1e-6 if case.dst_dtype == "float32" else 1e-13
        got = util.run_oracle(case).astype(np.float64)
        for other in (want, std, avx):
            assert np.all(np.abs(got - other) <= tol * np.maximum(np.abs(other), 1.0))
    elif case.accum == "float32":
        wide = util.run_oracle(case, wide_float=True).astype(np.float64)
        got = util.run_oracle(case)
        assert np.array_equal(got, want)  # same summation order as ReferenceMul<float>
        for other in (std, avx):
            assert np.all(np.abs(other - wide) <= 1e-5 * np.maximum(np.abs(wide), 1.0))
    else:
        assert np.array_equal(util.run_oracle(case, Rounding.kReference), want)
        assert np.array_equal(std, want)  # kStandardCpp == ReferenceMul
        assert np.array_equal(util.run_oracle(case, util.x86_rounding_for(case)), avx)


def _live_cases():
    out = []
    sizes = [(1, 1, 1), (2, 3, 4), (7, 9, 5), (15, 16, 17), (31, 32, 33), (63, 64, 65), (48, 48, 48), (9, 300, 11),
             (128, 16, 1), (1, 200, 64)]
    types = [("int8", "int8", "int8"), ("uint8", "uint8", "uint8"), ("int8", "int8", "int32"),
             ("uint8", "uint8", "int16"), ("int8", "int16", "int16"), ("int8", "uint8", "int8")]
    for s, (r, d, c) in enumerate(sizes):
        l, rr, dd = types[s % len(types)]
        for o, ords in enumerate(["RCC", "CRR", "CCC", "RRR"]):
            out.append(cases.random_case(r, d, c, l, rr, dd, orders=ords, extra_stride=o % 2, perchannel=bool(o % 2),
                                         channel=ChannelDimension.kCol if o >= 2 else ChannelDimension.kRow,
                                         seed=1000 + s * 4 + o))
    return out


@pytest.mark.parametrize("case", _live_cases(), ids=lambda c: c.name)
def test_oracle_matches_compiled_reference(case):
    if oracle.reference() is None:
        pytest.skip("compiled reference not built on this machine")
    ref = util.run_reference(case, reference_mul=True)
    assert np.array_equal(util.run_oracle(case, Rounding.kReference), ref)
    assert np.array_equal(util.run_reference(case, path=0x1), ref)
    simd = oracle.host_simd_path()
    if simd in (0x20, 0x40):
        assert np.array_equal(util.run_oracle(case, util.x86_rounding_for(case)),
                              util.run_reference(case, path=simd, threads=2))


@pytest.mark.parametrize("case", requant_extreme_cases(), ids=lambda c: c.name)
def test_oracle_matches_compiled_reference_on_requantization_extremes(case):
    """Exponents from +7 to -30, multipliers at both ends of their range, biases that wrap, degenerate clamps: the C
    restatement against ruy's own ReferenceMul, kStandardCpp and widest x86 path, compiled from the reference."""
    if oracle.reference() is None:
        pytest.skip("compiled reference not built on this machine")
    ref = util.run_reference(case, reference_mul=True)
    assert np.array_equal(util.run_oracle(case, Rounding.kReference), ref)
    assert np.array_equal(util.run_reference(case, path=0x1), ref)
    simd = oracle.host_simd_path()
    if simd in (0x20, 0x40):
        assert np.array_equal(util.run_oracle(case, util.x86_rounding_for(case)),
                              util.run_reference(case, path=simd, threads=2))


def test_sums_oracle():
    import ctypes as C
    c = cases.random_case(13, 77, 9, "uint8", "int8", "int32", orders="CRC", extra_stride=1, seed=5)
    lhs, rhs, p, d, keep = c.bind(c.new_dst())
    for side, m, width in ((0, lhs, 13), (1, rhs, 9)):
        desc = m.to_desc()
        sums = np.zeros(width, np.int32)
        oracle.oracle().ruy_oracle_sums(C.byref(desc), side, sums.ctypes.data)
        logical = np.asarray(m.data)
        lay = m.layout
        from ruy_b200.api import Order
        if lay.order == Order.kColMajor:
            mat = logical.reshape(lay.cols, lay.stride)[:, :lay.rows].T
        else:
            mat = logical.reshape(lay.rows, lay.stride)[:, :lay.cols]
        want = mat.astype(np.int64).sum(axis=1 if side == 0 else 0)
        assert np.array_equal(sums, want)


def _f64_mix_cases():
    # the two mixed floating-point cases ruy's own tests instantiate (ruy/BUILD:1195-1207)
    out = []
    for s, (r, d, c) in enumerate([(1, 1, 1), (7, 9, 5), (31, 32, 33), (64, 100, 48), (9, 300, 11)]):
        for o, ords in enumerate(["RCC", "CRR", "CCC", "RRR"]):
            for l, rr, dd in (("float64", "float32", "float32"), ("float32", "float64", "float64")):
                out.append(cases.random_case(r, d, c, l, rr, dd, orders=ords, extra_stride=o % 2,
                                             channel=ChannelDimension.kCol if o >= 2 else ChannelDimension.kRow,
                                             seed=3000 + s * 4 + o))
    return out


@pytest.mark.parametrize("case", _f64_mix_cases(), ids=lambda c: c.name)
def test_oracle_matches_compiled_reference_on_double_accumulation(case):
    """(f64, f32, f64, f32) and (f32, f64, f64, f64): the restatement against ReferenceMul and kStandardCpp.  The sums are
    double in depth order on both sides; the compiler may or may not contract a*b+c, hence a bound of a few ulps of the
    destination type instead of equality."""
    if oracle.reference() is None:
        pytest.skip("compiled reference not built on this machine")
    assert case.accum == "float64"
    ref = util.run_reference(case, reference_mul=True).astype(np.float64)
    got = util.run_oracle(case).astype(np.float64)
    tol = 1e-6 if case.dst_dtype == "float32" else 1e-13
    assert np.all(np.abs(got - ref) <= tol * np.maximum(np.abs(ref), 1.0))
    std = util.run_reference(case, path=0x1).astype(np.float64)
    assert np.all(np.abs(std - ref) <= tol * np.maximum(np.abs(ref), 1.0))
    # and against numpy's own double product, bias and clamp
    def logical(storage, lay):
        if lay.order == Order.kColMajor:
            return storage.reshape(lay.cols, lay.stride)[:, :lay.rows].T
        return storage.reshape(lay.rows, lay.stride)[:, :lay.cols]
    want = logical(case.lhs, case.lhs_layout).astype(np.float64) @ logical(case.rhs, case.rhs_layout).astype(np.float64)
    want = want + (case.bias[:, None] if case.channel == ChannelDimension.kRow else case.bias[None, :])
    want = np.clip(want, *case.clamp)
    assert np.all(np.abs(want - ref) <= tol * np.maximum(np.abs(want), 1.0))
