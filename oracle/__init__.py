"""TEST INFRASTRUCTURE: Python loaders for the CPU checkers under oracle/.

`oracle()` loads the plain-C restatement (oracle/liboracle.so); `reference()`
loads the compiled, unmodified reference (oracle/_ref/libruy_ref.so) when it has
been built, else returns None.  Only tests, the smoke test and the benchmark's
CPU-baseline legs may import this package; the product never does.
"""
import ctypes as C
import os
import subprocess

from ruy_b200 import _abi

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libruy_ref.so")
# Where the reference checkout lies: RUY_REFERENCE_DIR, else a directory named "reference" beside this repository.
REFERENCE_DIR = os.environ.get("RUY_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
_oracle = None
_ref = None


def build(want_reference=True):
    """Compiles liboracle.so and, when the reference checkout is present, _ref/libruy_ref.so."""
    subprocess.check_call(["make", "-s", "-C", _HERE, "oracle"])
    if want_reference and os.path.isdir(os.path.join(REFERENCE_DIR, "ruy")):
        import torch
        torch_dir = os.path.dirname(torch.__file__)
        subprocess.check_call(["make", "-s", "-j8", "-C", _HERE, "ref", f"REF={REFERENCE_DIR}",
                               f"TORCH_DIR={torch_dir}"])


def oracle():
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_SO):
            build(want_reference=False)
        h = C.CDLL(ORACLE_SO)
        h.oracle_requant_reference.restype = C.c_int32
        h.oracle_requant_reference.argtypes = [C.c_int32, C.c_int32, C.c_int]
        h.oracle_requant_x86.restype = C.c_int32
        h.oracle_requant_x86.argtypes = [C.c_int32, C.c_int32, C.c_int]
        h.ruy_oracle_validate.restype = C.c_int
        h.ruy_oracle_validate.argtypes = [C.POINTER(_abi.MulDesc)]
        h.ruy_oracle_mul.restype = C.c_int
        h.ruy_oracle_mul.argtypes = [C.POINTER(_abi.MulDesc), C.c_int, C.c_int]
        h.ruy_oracle_sums.restype = C.c_int
        h.ruy_oracle_sums.argtypes = [C.POINTER(_abi.MatrixDesc), C.c_int, C.c_void_p]
        _oracle = h
    return _oracle


def reference():
    """The compiled reference, or None when it is not available on this machine."""
    global _ref
    if _ref is None:
        if not os.path.exists(REF_SO):
            return None
        try:
            import torch  # noqa: F401  (puts libc10.so, which carries cpuinfo, in the process)
            h = C.CDLL(REF_SO)
        except OSError:
            return None
        h.ruy_ref_ctx_create.restype = C.c_void_p
        h.ruy_ref_ctx_create.argtypes = [C.c_int, C.c_int]
        h.ruy_ref_ctx_destroy.restype = None
        h.ruy_ref_ctx_destroy.argtypes = [C.c_void_p]
        h.ruy_ref_last_used_path.restype = C.c_int
        h.ruy_ref_last_used_path.argtypes = [C.c_void_p]
        h.ruy_ref_clear_cache.restype = None
        h.ruy_ref_clear_cache.argtypes = [C.c_void_p]
        h.ruy_ref_mul.restype = C.c_int
        h.ruy_ref_mul.argtypes = [C.c_void_p, C.POINTER(_abi.MulDesc)]
        h.ruy_ref_reference_mul.restype = C.c_int
        h.ruy_ref_reference_mul.argtypes = [C.POINTER(_abi.MulDesc)]
        h.ruy_ref_multiply_by_quantized_multiplier.restype = C.c_int32
        h.ruy_ref_multiply_by_quantized_multiplier.argtypes = [C.c_int32, C.c_int32, C.c_int]
        h.ruy_ref_time_mul.restype = C.c_double
        h.ruy_ref_time_mul.argtypes = [C.c_void_p, C.POINTER(_abi.MulDesc), C.c_int, C.c_double]
        h.ruy_ref_time_batch.restype = C.c_double
        h.ruy_ref_time_batch.argtypes = [C.POINTER(_abi.MulDesc), C.c_int, C.c_int, C.c_int, C.c_int]
        _ref = h
    return _ref


def host_simd_path():
    """The widest ruy x86 path this host can execute (bit value of ruy::Path), from /proc/cpuinfo."""
    try:
        flags = open("/proc/cpuinfo").read()
    except OSError:
        return _abi.PATH_STANDARD_CPP
    need512 = ["avx512f", "avx512vl", "avx512cd", "avx512bw", "avx512dq"]
    if all(f" {f}" in flags for f in need512):
        return _abi.PATH_AVX512
    if " avx2" in flags and " fma" in flags:
        return _abi.PATH_AVX2_FMA
    if " avx" in flags:
        return _abi.PATH_AVX
    return _abi.PATH_STANDARD_CPP
