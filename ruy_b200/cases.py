"""Seeded synthetic workloads: the five benchmark configurations and ruy-style random cases.

A `MulCase` holds host (numpy) storage for one ruy::Mul call.  `bind()` turns it into the
`Matrix` / `MulParams` views of ruy_b200.api over either the host arrays or device copies
(torch CUDA tensors), so the same bytes can be given to the CUDA library, to the C oracle
and to the compiled reference.

Value distributions follow the benchmark definition: int8 weights uniform in [-127,127],
activations uniform in [-128,127] (or a clipped normal for the large projection), int32 bias
uniform in [-1000,1000], per-channel fixed-point multipliers uniform in [2^30, 2^31-1] with
exponents uniform in a small negative range.  Random test cases mimic the distributions of
ruy's own harness (ruy/test.h:233-353,1590-1659,1719-1783): zero points over the full range
but symmetric half of the time, a multiplier chosen so that outputs span the destination
range, clamps one step inside the destination range.
"""
import hashlib

import numpy as np

from .api import (CachePolicy, ChannelDimension, Layout, Matrix, MulParams, Order, Rounding)


def _rng(*key):
    """Counter-based generator keyed by the (config, index, tensor) tuple; stable across processes."""
    digest = hashlib.sha256(repr(key).encode()).digest()
    return np.random.Generator(np.random.Philox(key=int.from_bytes(digest[:16], "little")))


def quantize_multiplier(real):
    """real > 0 -> (fixedpoint in [2^30, 2^31), exponent) with real ~= fixedpoint * 2^(exponent-31).
    Same decomposition as ruy/test.h:1608-1626 (frexp then round to 31 bits)."""
    if real == 0:
        return 0, 0
    frac, exp = np.frexp(real)
    q = int(round(float(frac) * (1 << 31)))
    if q == (1 << 31):
        q //= 2
        exp += 1
    return q, int(exp)


class MulCase:
    def __init__(self, name, lhs, lhs_layout, lhs_zp, rhs, rhs_layout, rhs_zp, dst_dtype, dst_layout,
                 dst_zp=0, bias=None, mfp=0, mexp=0, clamp=None, channel=ChannelDimension.kRow,
                 lhs_cache=CachePolicy.kNeverCache, rhs_cache=CachePolicy.kNeverCache):
        self.name = name
        self.lhs, self.lhs_layout, self.lhs_zp = lhs, lhs_layout, lhs_zp
        self.rhs, self.rhs_layout, self.rhs_zp = rhs, rhs_layout, rhs_zp
        self.dst_dtype = np.dtype(dst_dtype).name
        self.dst_layout, self.dst_zp = dst_layout, dst_zp
        self.bias, self.mfp, self.mexp = bias, mfp, mexp
        if np.float64 in (lhs.dtype, rhs.dtype) or np.dtype(dst_dtype) == np.float64:
            self.accum = "float64"      # ruy's mixed cases (f64, f32, f64, f32) and (f32, f64, f64, f64)
        else:
            self.accum = "float32" if lhs.dtype == np.float32 else "int32"
        if clamp is None:
            if self.accum in ("float32", "float64"):
                clamp = (-np.inf, np.inf)
            else:
                info = np.iinfo(self.dst_dtype)
                clamp = (int(info.min), int(info.max))
        self.clamp = clamp
        self.channel = ChannelDimension(channel)
        self.lhs_cache, self.rhs_cache = CachePolicy(lhs_cache), CachePolicy(rhs_cache)

    # shapes -----------------------------------------------------------------
    @property
    def rows(self):
        return self.lhs_layout.rows

    @property
    def depth(self):
        return self.lhs_layout.cols

    @property
    def cols(self):
        return self.rhs_layout.cols

    @property
    def ops(self):
        return 2 * self.rows * self.depth * self.cols

    def algorithmic_bytes(self):
        """Each logical operand read once + dst written once + per-channel parameters."""
        es = np.dtype(self.lhs.dtype).itemsize
        n = self.rows * self.depth * es + self.depth * self.cols * np.dtype(self.rhs.dtype).itemsize
        n += self.rows * self.cols * np.dtype(self.dst_dtype).itemsize
        nch = self.rows if self.channel == ChannelDimension.kRow else self.cols
        if self.bias is not None:
            n += 4 * nch
        if isinstance(self.mfp, np.ndarray):
            n += 8 * nch
        return n

    def dst_storage_elems(self):
        lay = self.dst_layout
        outer = lay.cols if lay.order == Order.kColMajor else lay.rows
        return lay.stride * outer

    def new_dst(self, fill=None):
        a = np.zeros(self.dst_storage_elems(), dtype=self.dst_dtype)
        if fill is not None:
            a[:] = fill
        return a

    def dst_view(self, storage):
        """Logical rows x cols view (numpy) of a dst storage array."""
        lay = self.dst_layout
        s = np.asarray(storage)
        if lay.order == Order.kColMajor:
            return s.reshape(lay.cols, lay.stride)[:, :lay.rows].T
        return s.reshape(lay.rows, lay.stride)[:, :lay.cols]

    # binding ----------------------------------------------------------------
    def bind(self, dst_storage, device=None, rounding=Rounding.kFromPath):
        """Returns (lhs, rhs, params, dst, keepalive).  With device=None the views are over the
        host arrays; otherwise inputs are copied to that torch device and dst_storage must be a
        tensor there."""
        keep = []

        def put(a):
            if a is None or device is None:
                return a
            import torch
            t = torch.from_numpy(np.ascontiguousarray(a)).to(device)
            keep.append(t)
            return t

        lhs = Matrix(put(self.lhs), self.lhs_layout, self.lhs_zp, self.lhs_cache)
        rhs = Matrix(put(self.rhs), self.rhs_layout, self.rhs_zp, self.rhs_cache)
        dst = Matrix(dst_storage, self.dst_layout, self.dst_zp)
        p = MulParams(self.accum, self.dst_dtype)
        p.bias = put(self.bias)
        if isinstance(self.mfp, np.ndarray):
            p.multiplier_fixedpoint_perchannel = put(self.mfp)
            p.multiplier_exponent_perchannel = put(self.mexp)
        else:
            p.multiplier_fixedpoint, p.multiplier_exponent = self.mfp, self.mexp
        p.clamp_min, p.clamp_max = self.clamp
        p.channel_dimension = self.channel
        p.rounding = rounding
        keep.extend([lhs, rhs, dst, p])
        return lhs, rhs, p, dst, keep


def _layout(rows, cols, order, extra_stride=0):
    order = Order(order)
    inner = rows if order == Order.kColMajor else cols
    return Layout(rows, cols, inner + extra_stride, order)


def _storage(logical, layout):
    """Lays a logical rows x cols array out per `layout` (padding elements are left as noise)."""
    rows, cols = logical.shape
    if layout.order == Order.kColMajor:
        buf = np.zeros((cols, layout.stride), dtype=logical.dtype)
        buf[:, :rows] = logical.T
    else:
        buf = np.zeros((rows, layout.stride), dtype=logical.dtype)
        buf[:, :cols] = logical
    return np.ascontiguousarray(buf.reshape(-1))


def _perchannel(rng, n, exp_lo, exp_hi):
    mfp = rng.integers(1 << 30, (1 << 31) - 1, size=n, endpoint=True, dtype=np.int64).astype(np.int32)
    mexp = rng.integers(exp_lo, exp_hi, size=n, endpoint=True, dtype=np.int64).astype(np.int32)
    return mfp, mexp


def config0(rows=256, depth=512, cols=128, exps=(-10, -4), seed=0, dst="int8", lhs_cache=CachePolicy.kNeverCache):
    """Single int8 x int8 -> int8 mul: row-major weights (zp 0), col-major activations (zp -3),
    per-row multipliers, dst zp 5.  exps=(-17,-13) gives the non-saturating variant."""
    rng = _rng("c0", rows, depth, cols, seed, exps)
    L = rng.integers(-127, 127, size=(rows, depth), endpoint=True).astype(np.int8)
    R = rng.integers(-128, 127, size=(depth, cols), endpoint=True).astype(np.int8)
    bias = rng.integers(-1000, 1000, size=rows, endpoint=True).astype(np.int32)
    ll, rl = _layout(rows, depth, Order.kRowMajor), _layout(depth, cols, Order.kColMajor)
    dl = _layout(rows, cols, Order.kColMajor)
    if np.dtype(dst).name == "int32":
        return MulCase(f"c0_{rows}x{depth}x{cols}_i32", _storage(L, ll), ll, 0, _storage(R, rl), rl, -3,
                       "int32", dl, 0, bias, lhs_cache=lhs_cache)
    mfp, mexp = _perchannel(rng, rows, *exps)
    return MulCase(f"c0_{rows}x{depth}x{cols}_e{exps[0]}", _storage(L, ll), ll, 0, _storage(R, rl), rl, -3,
                   dst, dl, 5, bias, mfp, mexp, (-128, 127), lhs_cache=lhs_cache)


CONFIG1_SHAPES = [(50, 50, 50), (100, 100, 100), (17, 301, 9), (256, 64, 1), (1024, 1024, 1024)]


def config1(shape, seed=0):
    """fp32 mul: row-major LHS, col-major RHS, values in [-1,1], bias per row, clamp [-6,6]."""
    rows, depth, cols = shape
    rng = _rng("c1", rows, depth, cols, seed)
    L = rng.uniform(-1, 1, size=(rows, depth)).astype(np.float32)
    R = rng.uniform(-1, 1, size=(depth, cols)).astype(np.float32)
    bias = rng.uniform(-1, 1, size=rows).astype(np.float32)
    ll, rl = _layout(rows, depth, Order.kRowMajor), _layout(depth, cols, Order.kColMajor)
    dl = _layout(rows, cols, Order.kColMajor)
    return MulCase(f"c1_{rows}x{depth}x{cols}", _storage(L, ll), ll, 0, _storage(R, rl), rl, 0, "float32", dl,
                   0, bias, clamp=(-6.0, 6.0))


CONFIG2_DIMS = (16, 24, 32, 48, 64, 96, 128)


def config2_shapes(n=16384, seed=0):
    rng = _rng("c2shapes", n, seed)
    return rng.choice(np.array(CONFIG2_DIMS), size=(n, 3))


def config2(n=16384, seed=0, first=0, count=None):
    """Batched small int8 muls; values as config0, LHS marked kAlwaysCache.  `first`/`count`
    select the shard of the mul index range (the shapes are drawn for the whole job)."""
    shapes = config2_shapes(n, seed)
    count = n - first if count is None else count
    out = []
    for idx in range(first, first + count):
        r, d, c = (int(v) for v in shapes[idx])
        out.append(config0(r, d, c, exps=(-10, -4), seed=(seed, idx), lhs_cache=CachePolicy.kAlwaysCache))
    return out


def config3(rows=4096, depth=4096, cols=8192, dst="int32", seed=0, col_begin=0, col_count=None):
    """Large projection: int8 weights U[-127,127] zp 0 (kAlwaysCache), activations round(N(0,40^2))
    clipped to int8, zp 0.  dst int32 raw accumulators, or int8 with per-row multipliers, bias and
    dst zp 5.  col_begin/col_count select a column shard; every shard sees the same weights."""
    col_count = cols - col_begin if col_count is None else col_count
    rng = _rng("c3w", rows, depth, seed)
    L = rng.integers(-127, 127, size=(rows, depth), endpoint=True).astype(np.int8)
    rngp = _rng("c3p", rows, seed)
    bias = rngp.integers(-1000, 1000, size=rows, endpoint=True).astype(np.int32)
    mfp, mexp = _perchannel(rngp, rows, -10, -4)
    # activations are generated per 256-column block so that a shard equals the slice of the whole
    blocks = []
    b0, b1 = col_begin // 256, (col_begin + col_count + 255) // 256
    for b in range(b0, b1):
        rb = _rng("c3a", depth, seed, b)
        blk = np.clip(np.rint(rb.normal(0.0, 40.0, size=(256, depth))), -128, 127).astype(np.int8)
        blocks.append(blk)
    Rt = np.concatenate(blocks, axis=0)[col_begin - b0 * 256: col_begin - b0 * 256 + col_count]
    ll = _layout(rows, depth, Order.kRowMajor)
    rl = _layout(depth, col_count, Order.kColMajor)
    dl = _layout(rows, col_count, Order.kColMajor)
    rhs_storage = np.ascontiguousarray(Rt.reshape(-1))  # col-major depth x cols == row-major cols x depth
    if np.dtype(dst).name == "int32":
        return MulCase(f"c3_{rows}x{depth}x{col_count}_i32", _storage(L, ll), ll, 0, rhs_storage, rl, 0,
                       "int32", dl, 0, None, lhs_cache=CachePolicy.kAlwaysCache)
    return MulCase(f"c3_{rows}x{depth}x{col_count}_i8", _storage(L, ll), ll, 0, rhs_storage, rl, 0, "int8", dl,
                   5, bias, mfp, mexp, (-128, 127), lhs_cache=CachePolicy.kAlwaysCache)


CONFIG4_LAYERS = [(64, 32, 12544), (128, 64, 3136), (256, 128, 784), (512, 256, 196), (1024, 512, 49),
                  (1024, 1024, 49)]
CONFIG4_DST_SCALE = 6.0 / 255.0  # synthetic output scale: the ReLU6 range spans the uint8 range


def config4(layer, batch=1, seed=0):
    """uint8 pointwise-conv layer with asymmetric quantization: LHS zp 128, RHS zp drawn per layer,
    one per-tensor multiplier chosen so the accumulators span the output range, ReLU6 clamp."""
    rows, depth, cols = CONFIG4_LAYERS[layer]
    cols *= batch
    rng = _rng("c4", layer, seed)
    L = rng.integers(0, 255, size=(rows, depth), endpoint=True).astype(np.uint8)
    rhs_zp = int(rng.integers(0, 255, endpoint=True))
    Rt = _rng("c4a", layer, batch, seed).integers(0, 255, size=(cols, depth), endpoint=True).astype(np.uint8)
    bias = rng.integers(-1000, 1000, size=rows, endpoint=True).astype(np.int32)
    # accumulators are ~ N(0, depth * var_l * var_r); map 3 sigma onto the 6.0 range
    sigma = np.sqrt(depth * (256 ** 2 / 12.0) ** 2)
    mfp, mexp = quantize_multiplier(255.0 / (3.0 * sigma))
    dst_zp = 0
    clamp = (dst_zp, min(255, dst_zp + int(round(6.0 / CONFIG4_DST_SCALE))))
    ll = _layout(rows, depth, Order.kRowMajor)
    rl = _layout(depth, cols, Order.kColMajor)
    dl = _layout(rows, cols, Order.kColMajor)
    return MulCase(f"c4_l{layer}_b{batch}", _storage(L, ll), ll, 128, np.ascontiguousarray(Rt.reshape(-1)), rl,
                   rhs_zp, "uint8", dl, dst_zp, bias, mfp, mexp, clamp, lhs_cache=CachePolicy.kAlwaysCache)


_INT_RANGE = {"int8": (-128, 127), "uint8": (0, 255), "int16": (-32768, 32767)}


def random_case(rows, depth, cols, lhs="int8", rhs="int8", dst="int8", orders="RCC", extra_stride=0,
                perchannel=False, channel=ChannelDimension.kRow, seed=0, bias=True, symmetric=None,
                lhs_cache=CachePolicy.kNeverCache, rhs_cache=CachePolicy.kNeverCache):
    """A ruy-test-style random case.  orders: three letters R/C for lhs, rhs, dst storage order.
    extra_stride adds that many elements to every minimal stride (ruy/test.h:481-498)."""
    rng = _rng("rand", rows, depth, cols, lhs, rhs, dst, orders, extra_stride, perchannel, int(channel), seed)
    o = [Order.kRowMajor if ch == "R" else Order.kColMajor for ch in orders]
    ll, rl, dl = (_layout(rows, depth, o[0], extra_stride), _layout(depth, cols, o[1], extra_stride),
                  _layout(rows, cols, o[2], extra_stride))
    if lhs in ("float32", "float64"):
        L = rng.uniform(-1, 1, size=(rows, depth)).astype(lhs)
        R = rng.uniform(-1, 1, size=(depth, cols)).astype(rhs)
        nch = rows if channel == ChannelDimension.kRow else cols
        wide = "float64" in (lhs, rhs, dst)       # the bias has the accumulator's type
        b = rng.uniform(-1, 1, size=nch).astype(np.float64 if wide else np.float32) if bias else None
        lo = float(-0.25 * np.sqrt(depth))
        name = f"f32_{rows}x{depth}x{cols}_{orders}" if not wide else f"{lhs}x{rhs}_{dst}_{rows}x{depth}x{cols}_{orders}"
        return MulCase(name, _storage(L, ll), ll, 0, _storage(R, rl), rl, 0,
                       dst if wide else "float32", dl, 0, b, clamp=(lo, -lo * 0.9), channel=channel,
                       lhs_cache=lhs_cache, rhs_cache=rhs_cache)
    (llo, lhi), (rlo, rhi) = _INT_RANGE[lhs], _INT_RANGE[rhs]
    # LHS avoids the minimum value, as ruy's harness does (kOffCenterAvoidMinValue)
    L = rng.integers(llo + 1, lhi, size=(rows, depth), endpoint=True).astype(lhs)
    R = rng.integers(rlo, rhi, size=(depth, cols), endpoint=True).astype(rhs)
    has16 = "int16" in (lhs, rhs)
    if symmetric is None:
        symmetric = bool(rng.integers(0, 2))
    if has16:
        lzp = rzp = 0
    elif symmetric:
        lzp, rzp = (llo + lhi + 1) // 2, (rlo + rhi + 1) // 2
    else:
        lzp, rzp = int(rng.integers(llo + 1, lhi, endpoint=True)), int(rng.integers(rlo, rhi, endpoint=True))
    nch = rows if channel == ChannelDimension.kRow else cols
    b = rng.integers(-10000, 10000, size=nch, endpoint=True).astype(np.int32) if bias else None
    if dst == "int32":
        return MulCase(f"{lhs}x{rhs}_i32_{rows}x{depth}x{cols}_{orders}", _storage(L, ll), ll, lzp,
                       _storage(R, rl), rl, rzp, "int32", dl, 0, b, channel=channel,
                       lhs_cache=lhs_cache, rhs_cache=rhs_cache)
    dlo, dhi = _INT_RANGE[dst]
    dzp = 0 if has16 else int(rng.integers(dlo + (dhi - dlo) * 2 // 5, dlo + (dhi - dlo) * 3 // 5, endpoint=True))
    lstd = np.sqrt(((lhi - llo) ** 2) / 12.0 + ((llo + lhi) / 2.0 - lzp) ** 2)
    rstd = np.sqrt(((rhi - rlo) ** 2) / 12.0 + ((rlo + rhi) / 2.0 - rzp) ** 2)
    mag = max(1.0, 2.0 * np.sqrt(depth) * lstd * rstd)
    real = (dhi - dlo) / 2.0 / mag
    if perchannel:
        pairs = [quantize_multiplier(real * float(rng.uniform(0.5, 1.5))) for _ in range(nch)]
        mfp = np.array([p[0] for p in pairs], dtype=np.int32)
        mexp = np.array([p[1] for p in pairs], dtype=np.int32)
    else:
        mfp, mexp = quantize_multiplier(real)
    return MulCase(f"{lhs}x{rhs}_{dst}_{rows}x{depth}x{cols}_{orders}_s{extra_stride}", _storage(L, ll), ll, lzp,
                   _storage(R, rl), rl, rzp, dst, dl, dzp, b, mfp, mexp, (dlo + 1, dhi - 1), channel,
                   lhs_cache=lhs_cache, rhs_cache=rhs_cache)
