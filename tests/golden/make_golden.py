"""Generates tests/golden/*.npz by running the compiled, unmodified reference
(oracle/_ref/libruy_ref.so, built by oracle/Makefile from the reference checkout).

For every case of tests/golden_cases.py it records the destination produced by
ruy::ReferenceMul, by ruy::Mul on Path::kStandardCpp and by ruy::Mul on Path::kAvx512, plus
a checksum of the inputs so a changed generator is noticed.  It also records
ruy::detail::MultiplyByQuantizedMultiplier on random and edge inputs, and the same inputs
pushed through the AVX-512 kernel's requantization (accumulator = bias, all-zero operands).

Run from the repository root, on a machine with AVX-512 and the reference checkout:
    python tests/golden/make_golden.py
"""
import ctypes as C
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
import util  # noqa: E402
from golden_cases import golden_cases  # noqa: E402
from ruy_b200 import cases  # noqa: E402
from ruy_b200.api import Layout, Order  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def input_digest(case):
    h = hashlib.sha256()
    for a in (case.lhs, case.rhs, case.bias, case.mfp if isinstance(case.mfp, np.ndarray) else None,
              case.mexp if isinstance(case.mexp, np.ndarray) else None):
        if a is not None:
            h.update(np.ascontiguousarray(a).tobytes())
    h.update(repr((case.lhs_zp, case.rhs_zp, case.dst_zp, case.clamp, int(case.channel),
                   case.mfp if not isinstance(case.mfp, np.ndarray) else None,
                   case.mexp if not isinstance(case.mexp, np.ndarray) else None)).encode())
    return np.frombuffer(h.digest()[:8], dtype=np.uint64)[0]


def requant_inputs():
    rng = np.random.Generator(np.random.Philox(key=20240611))
    n = 4096
    x = rng.integers(-(1 << 24), 1 << 24, size=n).astype(np.int32)
    x[:64] = rng.integers(-(1 << 31), (1 << 31) - 1, size=64).astype(np.int32)
    m = rng.integers(1 << 30, (1 << 31) - 1, size=n, endpoint=True).astype(np.int32)
    e = rng.integers(-20, 3, size=n, endpoint=True).astype(np.int32)
    # keep x * 2^e * m/2^31 inside int32 so the reference's own range assertion holds
    big = np.abs(x.astype(np.int64)) << np.maximum(e, 0).astype(np.int64)
    e = np.where(big >= (1 << 30), np.minimum(e, 0), e).astype(np.int32)
    # exact ties: x odd multiples of 2^(k-1) with m = 2^30 ("one half")
    x[64:128] = (2 * rng.integers(-500, 500, size=64) + 1).astype(np.int32)
    m[64:128] = 1 << 30
    e[64:128] = 0
    x[128:192] = (2 * rng.integers(-500, 500, size=64) + 1).astype(np.int32) * 8
    m[128:192] = (1 << 31) - 1
    e[128:192] = -4
    return x, m, e


def requant_case(x, m, e):
    """acc = bias (operands all zero): pushes x through a path's requantization, dst int16 zp 0."""
    n = len(x)
    lhs = np.zeros(n * 4, dtype=np.int8)
    rhs = np.zeros(4 * 16, dtype=np.int8)
    return cases.MulCase("requant", lhs, Layout(n, 4, 4, Order.kRowMajor), 0, rhs, Layout(4, 16, 4, Order.kColMajor), 0,
                         "int16", Layout(n, 16, n, Order.kColMajor), 0, x.copy(), m.copy(), e.copy(), (-32768, 32767))


def main():
    ref = oracle.reference()
    if ref is None:
        oracle.build()
        ref = oracle.reference()
    assert ref is not None, "the compiled reference is needed to generate golden vectors"
    assert oracle.host_simd_path() == 0x40, "generate on a host with AVX-512"
    outs = {}
    for case in golden_cases():
        outs[case.name + "/digest"] = input_digest(case)
        base = util.run_reference(case, reference_mul=True)
        outs[case.name + "/reference_mul"] = base
        # the other two are stored only where they differ from ReferenceMul (an empty array = identical)
        for key, got in (("standard_cpp", util.run_reference(case, path=0x1)),
                         ("avx512", util.run_reference(case, path=0x40, threads=3))):
            outs[case.name + "/" + key] = got if not np.array_equal(got, base) else np.zeros(0, dtype=base.dtype)
    np.savez_compressed(os.path.join(HERE, "ruy_reference_outputs.npz"), **outs)

    x, m, e = requant_inputs()
    want = np.array([ref.ruy_ref_multiply_by_quantized_multiplier(int(a), int(b), int(c)) for a, b, c in zip(x, m, e)],
                    dtype=np.int64)
    rc = requant_case(x, m, e)
    std = util.run_reference(rc, path=0x1)[:, 0]
    avx = util.run_reference(rc, path=0x40)[:, 0]
    np.savez_compressed(os.path.join(HERE, "ruy_requant.npz"), x=x, m=m, e=e, multiply_by_quantized_multiplier=want,
                        standard_cpp_int16=std, avx512_int16=avx)
    print("wrote", len(golden_cases()), "cases;", "requant rows:", len(x),
          "; reference vs avx512 requant rows differing:", int((std != avx).sum()))


if __name__ == "__main__":
    main()
