"""ctypes mirror of include/ruy_b200.h (structs, enums and function prototypes).

Every structure here must stay field-for-field identical to the C header; the
test-suite checks sizes and the exported symbol list against the header text.
"""
import ctypes as C

ABI_VERSION = 2

# ruyb200_status
OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_NO_DEVICE, ERR_CUDA, ERR_TIMEOUT, ERR_OOM = 0, -1, -2, -3, -4, -5, -6
STATUS_NAMES = {
    OK: "OK", ERR_INVALID: "ERR_INVALID", ERR_UNSUPPORTED: "ERR_UNSUPPORTED",
    ERR_NO_DEVICE: "ERR_NO_DEVICE", ERR_CUDA: "ERR_CUDA", ERR_TIMEOUT: "ERR_TIMEOUT", ERR_OOM: "ERR_OOM",
}

# ruyb200_dtype
I8, U8, I16, I32, F32, F64 = 0, 1, 2, 3, 4, 5
DTYPE_SIZE = {I8: 1, U8: 1, I16: 2, I32: 4, F32: 4, F64: 8}
NUMPY_DTYPE = {I8: "int8", U8: "uint8", I16: "int16", I32: "int32", F32: "float32", F64: "float64"}
DTYPE_OF_NUMPY = {v: k for k, v in NUMPY_DTYPE.items()}

COL_MAJOR, ROW_MAJOR = 0, 1
NEVER_CACHE, CACHE_IF_LARGE_SPEEDUP, CACHE_IF_SIGNIFICANT_SPEEDUP, ALWAYS_CACHE = 0, 1, 2, 3
CHANNEL_ROW, CHANNEL_COL = 0, 1
ROUNDING_FROM_PATH, ROUNDING_REFERENCE, ROUNDING_X86 = 0, 1, 2
PATH_NONE, PATH_STANDARD_CPP = 0, 0x1
PATH_INTERNAL_VARIANT1, PATH_INTERNAL_VARIANT2, PATH_INTERNAL_VARIANT3 = 0x2, 0x4, 0x8
PATH_AVX, PATH_AVX2_FMA, PATH_AVX512 = 0x10, 0x20, 0x40
ADVISORY_NONE, ADVISORY_REALLOCATED_PERCHANNEL_BUFFER = 0, 1
KERNEL_NONE, KERNEL_GENERIC, KERNEL_TC_I8, KERNEL_SGEMM, KERNEL_GEMV, KERNEL_BATCH_I8, KERNEL_TC_F32 = 0, 1, 2, 3, 4, 5, 6
KERNEL_NAMES = {0: "none", 1: "generic", 2: "tc_i8", 3: "sgemm", 4: "gemv", 5: "batch_i8", 6: "tc_f32"}


class MatrixDesc(C.Structure):
    """ruyb200_matrix."""
    _fields_ = [
        ("data", C.c_void_p),
        ("rows", C.c_int32),
        ("cols", C.c_int32),
        ("stride", C.c_int32),
        ("zero_point", C.c_int32),
        ("order", C.c_uint8),
        ("dtype", C.c_uint8),
        ("cache_policy", C.c_uint8),
        ("reserved", C.c_uint8),
    ]


class Scalar(C.Union):
    """ruyb200_scalar."""
    _fields_ = [("i", C.c_int32), ("f", C.c_float), ("d", C.c_double)]


class MulParamsDesc(C.Structure):
    """ruyb200_mul_params."""
    _fields_ = [
        ("bias", C.c_void_p),
        ("multiplier_fixedpoint_perchannel", C.c_void_p),
        ("multiplier_exponent_perchannel", C.c_void_p),
        ("multiplier_fixedpoint", C.c_int32),
        ("multiplier_exponent", C.c_int32),
        ("clamp_min", Scalar),
        ("clamp_max", Scalar),
        ("channel_dimension", C.c_uint8),
        ("perchannel_buffers_capacity_rounding_log2", C.c_uint8),
        ("accum_dtype", C.c_uint8),
        ("rounding_mode", C.c_uint8),
    ]


class MulDesc(C.Structure):
    """ruyb200_mul_desc."""
    _fields_ = [
        ("lhs", MatrixDesc),
        ("rhs", MatrixDesc),
        ("dst", MatrixDesc),
        ("params", MulParamsDesc),
    ]


class CacheBlob(C.Structure):
    """ruyb200_cache_blob."""
    _fields_ = [
        ("abi_version", C.c_uint32),
        ("format", C.c_uint32),
        ("dtype", C.c_uint8),
        ("side", C.c_uint8),
        ("has_sums", C.c_uint8),
        ("reserved", C.c_uint8),
        ("width", C.c_int32),
        ("depth", C.c_int32),
        ("packed_depth", C.c_int32),
        ("zero_point", C.c_int32),
        ("data_bytes", C.c_uint64),
        ("sums_bytes", C.c_uint64),
    ]


CACHE_FORMAT_ROWS16 = 1

_P = C.POINTER

# name -> (restype, argtypes); the authoritative list of exported entry points.
PROTOTYPES = {
    "ruyb200_abi_version": (C.c_int, []),
    "ruyb200_device_count": (C.c_int, []),
    "ruyb200_last_error": (C.c_char_p, []),
    "ruyb200_ctx_create": (C.c_int, [C.c_int, _P(C.c_void_p)]),
    "ruyb200_ctx_create_on_stream": (C.c_int, [C.c_int, C.c_void_p, _P(C.c_void_p)]),
    "ruyb200_ctx_destroy": (C.c_int, [C.c_void_p]),
    "ruyb200_ctx_set_max_num_threads": (C.c_int, [C.c_void_p, C.c_int]),
    "ruyb200_ctx_get_max_num_threads": (C.c_int, [C.c_void_p]),
    "ruyb200_ctx_set_runtime_enabled_paths": (C.c_int, [C.c_void_p, C.c_uint32]),
    "ruyb200_ctx_get_runtime_enabled_paths": (C.c_uint32, [C.c_void_p]),
    "ruyb200_ctx_last_used_path": (C.c_uint32, [C.c_void_p]),
    "ruyb200_ctx_performance_advisory": (C.c_int, [C.c_void_p, C.c_int]),
    "ruyb200_ctx_clear_prepacked_cache": (C.c_int, [C.c_void_p]),
    "ruyb200_ctx_set_prepacked_cache_budget": (C.c_int, [C.c_void_p, C.c_size_t]),
    "ruyb200_ctx_prepacked_cache_bytes": (C.c_size_t, [C.c_void_p]),
    "ruyb200_ctx_prepacked_cache_entries": (C.c_int, [C.c_void_p]),
    "ruyb200_ctx_counters": (C.c_int, [C.c_void_p, _P(C.c_uint64)]),
    "ruyb200_ctx_stream": (C.c_void_p, [C.c_void_p]),
    "ruyb200_ctx_sync": (C.c_int, [C.c_void_p]),
    "ruyb200_mul": (C.c_int, [C.c_void_p, _P(MulDesc)]),
    "ruyb200_mul_async": (C.c_int, [C.c_void_p, _P(MulDesc)]),
    "ruyb200_validate": (C.c_int, [_P(MulDesc)]),
    "ruyb200_mul_async_mirrored": (C.c_int, [C.c_void_p, _P(MulDesc), _P(C.c_void_p), C.c_int]),
    "ruyb200_mul_async_mirrored_exchange": (C.c_int, [C.c_void_p, _P(MulDesc), _P(C.c_void_p), C.c_int, C.c_void_p, C.c_void_p,
                                                      C.c_int, C.c_uint32]),
    "ruyb200_mul_async_multicast_exchange": (C.c_int, [C.c_void_p, _P(MulDesc), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                                       C.c_uint32]),
    "ruyb200_peer_alloc": (C.c_int, [C.c_size_t, _P(C.c_void_p)]),
    "ruyb200_peer_free": (C.c_int, [C.c_void_p]),
    "ruyb200_peer_export": (C.c_int, [C.c_void_p, C.c_char_p]),
    "ruyb200_peer_open": (C.c_int, [C.c_char_p, _P(C.c_void_p)]),
    "ruyb200_peer_close": (C.c_int, [C.c_void_p]),
    "ruyb200_peer_signal": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_uint32]),
    "ruyb200_peer_wait": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_uint32]),
    "ruyb200_peer_exchange": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_uint32]),
    "ruyb200_ctx_set_peer_wait_ms": (C.c_int, [C.c_void_p, C.c_uint32]),
    "ruyb200_cache_blob_info": (C.c_int, [C.c_void_p, C.c_size_t, _P(CacheBlob)]),
    "ruyb200_cache_export": (C.c_int, [C.c_void_p, _P(MatrixDesc), C.c_int, C.c_void_p, _P(C.c_size_t)]),
    "ruyb200_cache_import": (C.c_int, [C.c_void_p, _P(MatrixDesc), C.c_int, C.c_void_p, C.c_size_t]),
    "ruyb200_mul_noalloc": (C.c_int, [_P(MulDesc), C.c_void_p]),
    "ruyb200_plan_create": (C.c_int, [C.c_void_p, _P(MulDesc), C.c_int, _P(C.c_void_p)]),
    "ruyb200_plan_run": (C.c_int, [C.c_void_p]),
    "ruyb200_plan_destroy": (C.c_int, [C.c_void_p]),
    "ruyb200_plan_stats": (C.c_int, [C.c_void_p, _P(C.c_uint64), _P(C.c_uint64)]),
    "ruyb200_pack": (C.c_int, [C.c_void_p, _P(MatrixDesc), C.c_int, C.c_void_p, C.c_size_t,
                               C.c_void_p, _P(C.c_int32)]),
}
