"""Python mirror of ruy's public API over the C ABI of libruy_b200.so.

Names, argument meaning and defaults follow ruy's C++ headers so that tests read
like ruy's own: `Matrix` / `Layout` / `make_simple_layout` (ruy/matrix.h:30-172),
`MulParams` (ruy/mul_params.h:102-223), `Context` (ruy/context.h:38-112), `Path`
(ruy/path.h:55-90) and `mul` (ruy/ruy.h:98-104).  The objects only hold views:
matrix data is a numpy array (host memory) or a torch CUDA tensor (device
memory) owned by the caller, exactly as ruy::Matrix owns nothing.

This module never computes anything itself; every `mul` goes to the CUDA
library, and loading fails loudly if the library has not been built.
"""
import ctypes as C
import enum

import numpy as np

from . import _abi
from ._lib import lib


class Order(enum.IntEnum):
    kColMajor = _abi.COL_MAJOR
    kRowMajor = _abi.ROW_MAJOR


class CachePolicy(enum.IntEnum):
    kNeverCache = _abi.NEVER_CACHE
    kCacheIfLargeSpeedup = _abi.CACHE_IF_LARGE_SPEEDUP
    kCacheIfSignificantSpeedup = _abi.CACHE_IF_SIGNIFICANT_SPEEDUP
    kAlwaysCache = _abi.ALWAYS_CACHE


class ChannelDimension(enum.IntEnum):
    kRow = _abi.CHANNEL_ROW
    kCol = _abi.CHANNEL_COL


class Path(enum.IntFlag):
    kNone = 0
    kStandardCpp = 0x1
    kInternalStandardCppVariant1 = 0x2
    kInternalStandardCppVariant2 = 0x4
    kInternalStandardCppVariant3 = 0x8
    kAvx = 0x10
    kAvx2Fma = 0x20
    kAvx512 = 0x40


kDefaultPaths = Path.kStandardCpp | Path.kAvx | Path.kAvx2Fma | Path.kAvx512
kAllPaths = kDefaultPaths


class PerformanceAdvisory(enum.IntEnum):
    kNone = 0
    kReallocatedPerChannelBuffer = 1


class Rounding(enum.IntEnum):
    kFromPath = _abi.ROUNDING_FROM_PATH
    kReference = _abi.ROUNDING_REFERENCE
    kX86 = _abi.ROUNDING_X86


class RuyError(RuntimeError):
    def __init__(self, status, where):
        msg = lib().ruyb200_last_error().decode("utf-8", "replace")
        super().__init__(f"{where}: {_abi.STATUS_NAMES.get(status, status)} ({msg})")
        self.status = status


def _check(status, where):
    if status != _abi.OK:
        raise RuyError(status, where)


class Layout:
    """ruy::Layout (ruy/matrix.h:33-51)."""

    def __init__(self, rows=0, cols=0, stride=0, order=Order.kColMajor):
        self.rows, self.cols, self.stride, self.order = rows, cols, stride, Order(order)


def make_simple_layout(rows, cols, order):
    """ruy::MakeSimpleLayout (ruy/matrix.h:167-172): stride = the contiguous dimension."""
    order = Order(order)
    return Layout(rows, cols, rows if order == Order.kColMajor else cols, order)


def _is_torch(x):
    return type(x).__module__.startswith("torch")


def _ptr_and_dtype(data):
    if data is None:
        return None, None
    if _is_torch(data):
        import torch
        names = {torch.int8: "int8", torch.uint8: "uint8", torch.int16: "int16",
                 torch.int32: "int32", torch.float32: "float32", torch.float64: "float64"}
        return data.data_ptr(), _abi.DTYPE_OF_NUMPY[names[data.dtype]]
    a = data
    return a.ctypes.data, _abi.DTYPE_OF_NUMPY[a.dtype.name]


class Matrix:
    """ruy::Matrix<Scalar> (ruy/matrix.h:132-165): a non-owning view plus zero point and
    cache policy.  `data` is a flat or 2-D numpy array / torch tensor holding the storage."""

    def __init__(self, data=None, layout=None, zero_point=0, cache_policy=CachePolicy.kNeverCache):
        self.data = data
        self.layout = layout if layout is not None else Layout()
        self.zero_point = zero_point
        self.cache_policy = CachePolicy(cache_policy)

    def to_desc(self):
        ptr, dt = _ptr_and_dtype(self.data)
        d = _abi.MatrixDesc()
        d.data = ptr
        d.rows, d.cols, d.stride = self.layout.rows, self.layout.cols, self.layout.stride
        d.zero_point = int(self.zero_point)
        d.order = int(self.layout.order)
        d.dtype = dt if dt is not None else 0
        d.cache_policy = int(self.cache_policy)
        return d


class MulParams:
    """ruy::MulParams<AccumScalar, DstScalar> (ruy/mul_params.h:102-223).

    `accum` / `dst` are numpy dtype names.  Defaults match ruy: no bias, multiplier 0 with
    exponent 0, clamp = the full range of the destination type (+-inf for float), channel
    dimension kRow (ruy/mul_params.h:228-299)."""

    def __init__(self, accum="int32", dst="int8"):
        self.accum = np.dtype(accum).name
        self.dst = np.dtype(dst).name
        self.bias = None
        self.multiplier_fixedpoint = 0
        self.multiplier_exponent = 0
        self.multiplier_fixedpoint_perchannel = None
        self.multiplier_exponent_perchannel = None
        if self.accum in ("float32", "float64"):
            self.clamp_min, self.clamp_max = -np.inf, np.inf
        else:
            info = np.iinfo(self.dst)
            self.clamp_min, self.clamp_max = int(info.min), int(info.max)
        self.channel_dimension = ChannelDimension.kRow
        self.perchannel_buffers_capacity_rounding = 1
        self.rounding = Rounding.kFromPath

    def to_desc(self):
        p = _abi.MulParamsDesc()
        p.bias = _ptr_and_dtype(self.bias)[0]
        p.multiplier_fixedpoint_perchannel = _ptr_and_dtype(self.multiplier_fixedpoint_perchannel)[0]
        p.multiplier_exponent_perchannel = _ptr_and_dtype(self.multiplier_exponent_perchannel)[0]
        p.multiplier_fixedpoint = int(self.multiplier_fixedpoint)
        p.multiplier_exponent = int(self.multiplier_exponent)
        if self.accum == "float64":
            p.clamp_min.d = float(self.clamp_min)
            p.clamp_max.d = float(self.clamp_max)
        elif self.accum == "float32":
            p.clamp_min.f = float(self.clamp_min)
            p.clamp_max.f = float(self.clamp_max)
        else:
            p.clamp_min.i = int(self.clamp_min)
            p.clamp_max.i = int(self.clamp_max)
        p.channel_dimension = int(self.channel_dimension)
        p.perchannel_buffers_capacity_rounding_log2 = int(self.perchannel_buffers_capacity_rounding).bit_length() - 1
        p.accum_dtype = _abi.DTYPE_OF_NUMPY[self.accum]
        p.rounding_mode = int(self.rounding)
        return p


def make_desc(lhs, rhs, mul_params, dst):
    d = _abi.MulDesc()
    d.lhs, d.rhs, d.dst, d.params = lhs.to_desc(), rhs.to_desc(), dst.to_desc(), mul_params.to_desc()
    return d


class Context:
    """ruy::Context (ruy/context.h:38-112) backed by one CUDA device and stream."""

    def __init__(self, device=-1, stream=None):
        self._h = C.c_void_p()
        if stream is None:
            _check(lib().ruyb200_ctx_create(device, C.byref(self._h)), "ruyb200_ctx_create")
        else:
            _check(lib().ruyb200_ctx_create_on_stream(device, C.c_void_p(stream), C.byref(self._h)),
                   "ruyb200_ctx_create_on_stream")

    def close(self):
        if getattr(self, "_h", None) is not None and self._h:
            lib().ruyb200_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def max_num_threads(self):
        return lib().ruyb200_ctx_get_max_num_threads(self._h)

    def set_max_num_threads(self, value):
        _check(lib().ruyb200_ctx_set_max_num_threads(self._h, value), "set_max_num_threads")

    def set_runtime_enabled_paths(self, paths):
        _check(lib().ruyb200_ctx_set_runtime_enabled_paths(self._h, int(paths)), "set_runtime_enabled_paths")

    def get_runtime_enabled_paths(self):
        return Path(lib().ruyb200_ctx_get_runtime_enabled_paths(self._h))

    def last_used_path(self):
        return Path(lib().ruyb200_ctx_last_used_path(self._h))

    def performance_advisory(self, advisory):
        return bool(lib().ruyb200_ctx_performance_advisory(self._h, int(advisory)))

    def clear_prepacked_cache(self):
        _check(lib().ruyb200_ctx_clear_prepacked_cache(self._h), "clear_prepacked_cache")

    ClearPrepackedCache = clear_prepacked_cache

    def set_prepacked_cache_budget(self, nbytes):
        _check(lib().ruyb200_ctx_set_prepacked_cache_budget(self._h, nbytes), "set_prepacked_cache_budget")

    def prepacked_cache_bytes(self):
        return lib().ruyb200_ctx_prepacked_cache_bytes(self._h)

    def prepacked_cache_entries(self):
        return lib().ruyb200_ctx_prepacked_cache_entries(self._h)

    def counters(self):
        out = (C.c_uint64 * 6)()
        _check(lib().ruyb200_ctx_counters(self._h, out), "counters")
        return {"launches": out[0], "cache_hits": out[1], "cache_misses": out[2],
                "h2d_bytes": out[3], "d2h_bytes": out[4], "last_kernel": _abi.KERNEL_NAMES.get(out[5], out[5])}

    def stream(self):
        return lib().ruyb200_ctx_stream(self._h)

    def set_peer_wait_ms(self, ms):
        _check(lib().ruyb200_ctx_set_peer_wait_ms(self._h, int(ms)), "ruyb200_ctx_set_peer_wait_ms")

    def cache_export(self, matrix, side):
        """The cached (prepacked) form of `matrix` as a bytes blob (see ruyb200_cache_export).  side: 0 = LHS, 1 = RHS."""
        m = matrix.to_desc()
        n = C.c_size_t(0)
        _check(lib().ruyb200_cache_export(self._h, C.byref(m), side, None, C.byref(n)), "ruyb200_cache_export")
        buf = C.create_string_buffer(n.value)
        _check(lib().ruyb200_cache_export(self._h, C.byref(m), side, buf, C.byref(n)), "ruyb200_cache_export")
        return buf.raw[:n.value]

    def cache_import(self, matrix, side, blob):
        """Installs a blob made by cache_export as the cache entry of `matrix` (see ruyb200_cache_import)."""
        m = matrix.to_desc()
        _check(lib().ruyb200_cache_import(self._h, C.byref(m), side, blob, len(blob)), "ruyb200_cache_import")

    def sync(self):
        _check(lib().ruyb200_ctx_sync(self._h), "ruyb200_ctx_sync")


def mul(lhs, rhs, mul_params, context, dst):
    """ruy::Mul(lhs, rhs, mul_params, context, &dst) (ruy/ruy.h:98-104): synchronous."""
    d = make_desc(lhs, rhs, mul_params, dst)
    _check(lib().ruyb200_mul(context._h, C.byref(d)), "ruyb200_mul")


def mul_async(lhs, rhs, mul_params, context, dst):
    """Stream-ordered variant for device-resident operands (no synchronization)."""
    d = make_desc(lhs, rhs, mul_params, dst)
    _check(lib().ruyb200_mul_async(context._h, C.byref(d)), "ruyb200_mul_async")


def mul_noalloc(lhs, rhs, mul_params, dst, stream=None):
    """ruyb200_mul_noalloc: the 8-bit mul for callers that must not allocate (no context, static scratch,
    device-resident depth-contiguous operands, at most 16384 x 16384 destinations).  Synchronous."""
    d = make_desc(lhs, rhs, mul_params, dst)
    _check(lib().ruyb200_mul_noalloc(C.byref(d), C.c_void_p(stream) if stream else None), "ruyb200_mul_noalloc")


def cache_blob_info(blob):
    """Host-side validation and description of a prepacked-cache blob (no device needed); raises RuyError if unusable."""
    info = _abi.CacheBlob()
    _check(lib().ruyb200_cache_blob_info(blob, len(blob), C.byref(info)), "ruyb200_cache_blob_info")
    return {name: getattr(info, name) for name, _ in _abi.CacheBlob._fields_ if name != "reserved"}


def validate(lhs, rhs, mul_params, dst):
    d = make_desc(lhs, rhs, mul_params, dst)
    return lib().ruyb200_validate(C.byref(d))


class Plan:
    """Many independent muls replayed with one persistent launch (see ruyb200_plan_create)."""

    def __init__(self, context, descs):
        n = len(descs)
        arr = (_abi.MulDesc * n)(*descs)
        self._h = C.c_void_p()
        self._ctx = context
        _check(lib().ruyb200_plan_create(context._h, arr, n, C.byref(self._h)), "ruyb200_plan_create")

    def run(self):
        _check(lib().ruyb200_plan_run(self._h), "ruyb200_plan_run")

    def stats(self):
        b, o = C.c_uint64(), C.c_uint64()
        _check(lib().ruyb200_plan_stats(self._h, C.byref(b), C.byref(o)), "ruyb200_plan_stats")
        return b.value, o.value

    def close(self):
        if getattr(self, "_h", None) is not None and self._h:
            lib().ruyb200_plan_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
