// CUDA-core kernels: the any-type / any-layout matmul (the role Path::kStandardCpp's
// Kernel plays in ruy, ruy/kernel.h:176-241), the zero-point sums, and the packing kernel
// (ruy/pack.h:105-151).
#include "common.cuh"

namespace ruyb200 {

namespace {

__device__ __forceinline__ int32_t load_as_int(const void* p, uint8_t dtype, int64_t idx) {
  switch (dtype) {
    case RUYB200_I8: return ((const int8_t*)p)[idx];
    case RUYB200_U8: return ((const uint8_t*)p)[idx];
    case RUYB200_I16: return ((const int16_t*)p)[idx];
    default: return ((const int32_t*)p)[idx];
  }
}

constexpr int kTile = 32;    // dst tile edge per block
constexpr int kChunk = 32;   // depth chunk staged in shared memory

// One block computes a kTile x kTile destination tile; operands are staged through shared
// memory in depth chunks with loads coalesced along whichever dimension is contiguous.
// Accumulates (m - zp_m) * (n - zp_n) directly, as ReferenceMul does, so no sums are needed.
template <bool kFloat>
__global__ void __launch_bounds__(256) generic_mul_kernel(SideView ms, SideView ns, DstView dst, Epilogue ep) {
  __shared__ int32_t sm[kTile][kChunk + 1];
  __shared__ int32_t sn[kTile][kChunk + 1];
  const int m0 = blockIdx.y * kTile;
  const int n0 = blockIdx.x * kTile;
  const int tx = threadIdx.x % 32;   // n within tile
  const int ty = threadIdx.x / 32;   // 8 groups, 4 m each
  int32_t iacc[4] = {0, 0, 0, 0};
  float facc[4] = {0.f, 0.f, 0.f, 0.f};
  float fcomp[4] = {0.f, 0.f, 0.f, 0.f};  // float sums are folded chunk by chunk with compensation
  for (int k0 = 0; k0 < ep.depth; k0 += kChunk) {
    // stage: thread t loads 4 elements per side
    for (int e = threadIdx.x; e < kTile * kChunk; e += 256) {
      // choose the fast-varying index along the contiguous dimension of each side
      int wm, km, wn, kn;
      if (ms.stride_k == 1) { km = e % kChunk; wm = e / kChunk; } else { wm = e % kTile; km = e / kTile; }
      if (ns.stride_k == 1) { kn = e % kChunk; wn = e / kChunk; } else { wn = e % kTile; kn = e / kTile; }
      int32_t vm = 0, vn = 0;
      if (m0 + wm < ms.width && k0 + km < ep.depth) {
        const int64_t idx = (int64_t)(m0 + wm) * ms.stride_w + (int64_t)(k0 + km) * ms.stride_k;
        vm = kFloat ? __float_as_int(((const float*)ms.data)[idx]) : load_as_int(ms.data, ms.dtype, idx) - ms.zero_point;
      }
      if (n0 + wn < ns.width && k0 + kn < ep.depth) {
        const int64_t idx = (int64_t)(n0 + wn) * ns.stride_w + (int64_t)(k0 + kn) * ns.stride_k;
        vn = kFloat ? __float_as_int(((const float*)ns.data)[idx]) : load_as_int(ns.data, ns.dtype, idx) - ns.zero_point;
      }
      sm[wm][km] = vm;
      sn[wn][kn] = vn;
    }
    __syncthreads();
    float fpart[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
    for (int k = 0; k < kChunk; k++) {
      const int32_t bn = sn[tx][k];
#pragma unroll
      for (int r = 0; r < 4; r++) {
        const int32_t am = sm[ty * 4 + r][k];
        if (kFloat) {
          fpart[r] = fmaf(__int_as_float(am), __int_as_float(bn), fpart[r]);
        } else {
          iacc[r] = (int32_t)((uint32_t)iacc[r] + (uint32_t)(am * bn));
        }
      }
    }
    if (kFloat) {
#pragma unroll
      for (int r = 0; r < 4; r++) {
        const float y = fpart[r] - fcomp[r];
        const float t = facc[r] + y;
        fcomp[r] = (t - facc[r]) - y;
        facc[r] = t;
      }
    }
    __syncthreads();
  }
  Epilogue e2 = ep;
  e2.zp_m = 0;  // zero points were already subtracted while staging
  e2.zp_n = 0;
  const int n = n0 + tx;
#pragma unroll
  for (int r = 0; r < 4; r++) {
    const int m = m0 + ty * 4 + r;
    if (m < dst.size_m && n < dst.size_n) {
      if (kFloat) {
        ((float*)dst.data)[(int64_t)m * dst.stride_m + n] = finish_float(facc[r], m, n, e2);
      } else {
        store_int(dst, ep.dst_dtype, m, n, finish_int(iacc[r], m, n, e2));
      }
    }
  }
}

// Double accumulation over float or double operands (ruy's type mixes (f64, f32, f64, f32) and (f32, f64, f64, f64),
// ruy/BUILD:1195-1207, served in ruy by the standard C++ kernel, ruy/kernel.h:176-241).  Same tiling as above; the
// products and the sum are double, in depth order, which is the order ruy's kernel adds in.
template <typename TM, typename TN, typename TD>
__global__ void __launch_bounds__(256) generic_f64_kernel(SideView ms, SideView ns, DstView dst, Epilogue ep, double clamp_min,
                                                          double clamp_max) {
  __shared__ double sm[kTile][kChunk + 1];
  __shared__ double sn[kTile][kChunk + 1];
  const int m0 = blockIdx.y * kTile;
  const int n0 = blockIdx.x * kTile;
  const int tx = threadIdx.x % 32;
  const int ty = threadIdx.x / 32;
  double acc[4] = {0.0, 0.0, 0.0, 0.0};
  for (int k0 = 0; k0 < ep.depth; k0 += kChunk) {
    for (int e = threadIdx.x; e < kTile * kChunk; e += 256) {
      int wm, km, wn, kn;
      if (ms.stride_k == 1) { km = e % kChunk; wm = e / kChunk; } else { wm = e % kTile; km = e / kTile; }
      if (ns.stride_k == 1) { kn = e % kChunk; wn = e / kChunk; } else { wn = e % kTile; kn = e / kTile; }
      double vm = 0.0, vn = 0.0;
      if (m0 + wm < ms.width && k0 + km < ep.depth) {
        vm = (double)((const TM*)ms.data)[(int64_t)(m0 + wm) * ms.stride_w + (int64_t)(k0 + km) * ms.stride_k];
      }
      if (n0 + wn < ns.width && k0 + kn < ep.depth) {
        vn = (double)((const TN*)ns.data)[(int64_t)(n0 + wn) * ns.stride_w + (int64_t)(k0 + kn) * ns.stride_k];
      }
      sm[wm][km] = vm;
      sn[wn][kn] = vn;
    }
    __syncthreads();
#pragma unroll 4
    for (int k = 0; k < kChunk; k++) {
      const double bn = sn[tx][k];
#pragma unroll
      for (int r = 0; r < 4; r++) acc[r] = fma(sm[ty * 4 + r][k], bn, acc[r]);
    }
    __syncthreads();
  }
  const int n = n0 + tx;
#pragma unroll
  for (int r = 0; r < 4; r++) {
    const int m = m0 + ty * 4 + r;
    if (m < dst.size_m && n < dst.size_n) {
      double v = acc[r];
      if (ep.bias) v += ((const double*)ep.bias)[ep.channel_on_n ? n : m];
      v = fmin(v, clamp_max);
      v = fmax(v, clamp_min);
      ((TD*)dst.data)[(int64_t)m * dst.stride_m + n] = (TD)v;
    }
  }
}

// Sum of the 16 bytes of q, each taken as signed or unsigned.
__device__ __forceinline__ uint32_t sum16(const uint4 q, bool is_signed) {
  if (is_signed) {
    int a = 0;
    a = __dp4a((int)q.x, 0x01010101, a);
    a = __dp4a((int)q.y, 0x01010101, a);
    a = __dp4a((int)q.z, 0x01010101, a);
    a = __dp4a((int)q.w, 0x01010101, a);
    return (uint32_t)a;
  }
  unsigned a = 0;
  a = __dp4a(q.x, 0x01010101u, a);
  a = __dp4a(q.y, 0x01010101u, a);
  a = __dp4a(q.z, 0x01010101u, a);
  a = __dp4a(q.w, 0x01010101u, a);
  return a;
}

// kThreadsPerRow threads (a warp, or the whole CTA of 256) per width-row, striding over depth.  A CTA per row is for
// operands of few rows: with one warp per row a 16-row operand of depth 16384 is a chain of 32 dependent-latency
// trips on 16 warps (about 45 us); 256 threads with four loads in flight each finish it in a few microseconds.
template <int kThreadsPerRow>
__global__ void __launch_bounds__(256) sums_kernel(SideView s, int depth, int32_t* sums) {
  __shared__ uint32_t warp_sums[8];
  const int w = kThreadsPerRow == 256 ? blockIdx.x : blockIdx.x * 8 + threadIdx.x / 32;
  const int lane = threadIdx.x % kThreadsPerRow;
  uint32_t acc = 0;
  if (w < s.width) {
    const bool is_signed = s.dtype == RUYB200_I8;
    const bool vec = s.stride_k == 1 && (s.dtype == RUYB200_I8 || s.dtype == RUYB200_U8) &&
                     (((uintptr_t)s.data + (uint64_t)w * s.stride_w) % 16 == 0);
    int k = 0;
    if (vec) {
      const uint4* row = (const uint4*)((const char*)s.data + (int64_t)w * s.stride_w);
      const int nvec = depth / 16;
      int v = lane;
      for (; v + 3 * kThreadsPerRow < nvec; v += 4 * kThreadsPerRow) {
        uint4 q[4];
#pragma unroll
        for (int u = 0; u < 4; u++) q[u] = row[v + u * kThreadsPerRow];
#pragma unroll
        for (int u = 0; u < 4; u++) acc += sum16(q[u], is_signed);
      }
      for (; v < nvec; v += kThreadsPerRow) acc += sum16(row[v], is_signed);
      k = nvec * 16;
    }
    for (int kk = k + lane; kk < depth; kk += kThreadsPerRow) {
      acc += (uint32_t)load_as_int(s.data, s.dtype, (int64_t)w * s.stride_w + (int64_t)kk * s.stride_k);
    }
  }
  acc = __reduce_add_sync(0xffffffffu, acc);
  if (kThreadsPerRow == 32) {
    if (w < s.width && lane == 0) sums[w] = (int32_t)acc;
    return;
  }
  if (threadIdx.x % 32 == 0) warp_sums[threadIdx.x / 32] = acc;
  __syncthreads();
  if (threadIdx.x == 0 && w < s.width) {
    uint32_t total = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) total += warp_sums[i];
    sums[w] = (int32_t)total;
  }
}

// Packing: out[w][k] (depth-contiguous, packed_depth elements per row, zero padded) and sums.
// Block = 32 x 8 threads handling 32 widths; loops over depth in chunks of 32 through a
// shared-memory tile so that both the read and the write are coalesced for either source order.
template <typename T>
__global__ void __launch_bounds__(256) pack_kernel(SideView s, int depth, int packed_depth, T* out, int32_t* sums) {
  __shared__ T tile[32][33];
  const int tx = threadIdx.x % 32;
  const int ty = threadIdx.x / 32;
  const int w0 = blockIdx.x * 32;
  uint32_t acc[4] = {0, 0, 0, 0};
  const T* src = (const T*)s.data;
  for (int k0 = 0; k0 < packed_depth; k0 += 32) {
    // load tile[w][k]
    for (int r = 0; r < 4; r++) {
      int w, k;
      if (s.stride_k == 1) { k = tx; w = ty + 8 * r; } else { w = tx; k = ty + 8 * r; }
      T v = 0;
      if (w0 + w < s.width && k0 + k < depth) {
        v = src[(int64_t)(w0 + w) * s.stride_w + (int64_t)(k0 + k) * s.stride_k];
      }
      tile[w][k] = v;
    }
    __syncthreads();
    for (int r = 0; r < 4; r++) {
      const int w = ty + 8 * r;
      const int k = tx;
      const T v = tile[w][k];
      if (w0 + w < s.width && k0 + k < packed_depth) {
        out[(int64_t)(w0 + w) * packed_depth + k0 + k] = v;
      }
      acc[r] += (uint32_t)(int32_t)v;
    }
    __syncthreads();
  }
  if (sums) {
    for (int r = 0; r < 4; r++) {
      const uint32_t t = __reduce_add_sync(0xffffffffu, acc[r]);
      if (tx == 0 && w0 + ty + 8 * r < s.width) sums[w0 + ty + 8 * r] = (int32_t)t;
    }
  }
}

// 16 bytes from any address, of which the first n_valid (1 or more) exist; the rest read as zero.  One or two aligned
// 16-byte loads (only of 16-byte granules that hold at least one existing byte), then word selects and funnel shifts:
// consecutive lanes reading consecutive pieces stay fully coalesced whatever the alignment.
__device__ __forceinline__ uint4 load16_any(const uint8_t* p, int n_valid) {
  const uintptr_t addr = (uintptr_t)p;
  const int nv = n_valid < 16 ? n_valid : 16;
  const int sh = (int)(addr & 15);
  const uint4* base = reinterpret_cast<const uint4*>(addr - sh);
  const uint4 a = base[0];
  if (sh == 0 && nv == 16) return a;
  uint4 b = make_uint4(0u, 0u, 0u, 0u);
  if (sh + nv > 16) b = base[1];
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  const int wo = sh >> 2, bits = 8 * (sh & 3);
  uint32_t x[5];
#pragma unroll
  for (int i = 0; i < 5; i++) x[i] = wo == 0 ? w[i] : (wo == 1 ? w[i + 1] : (wo == 2 ? w[i + 2] : w[i + 3 < 8 ? i + 3 : 7]));
  uint32_t o[4];
#pragma unroll
  for (int i = 0; i < 4; i++) {
    o[i] = __funnelshift_r(x[i], x[i + 1], bits);
    const int keep = nv - 4 * i;   // bytes of this word that exist
    if (keep <= 0) o[i] = 0u;
    else if (keep < 4) o[i] &= (1u << (8 * keep)) - 1u;
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// 8-bit operands stored depth-contiguous whose rows are not on 16-byte boundaries (or not as long as the packed
// depth): a warp per row and slab of depth, every lane 16 packed bytes per trip, sums on the way.  With more than one
// slab (gridDim.y) the sums are added atomically to a zeroed buffer.
__global__ void __launch_bounds__(256) pack8_rows_kernel(SideView s, int depth, int packed_depth, uint8_t* out, int32_t* sums,
                                                         int slab) {
  const int lane = threadIdx.x % 32;
  const long long w = (long long)blockIdx.x * 8 + threadIdx.x / 32;
  if (w >= s.width) return;
  const bool is_signed = s.dtype == RUYB200_I8;
  const uint8_t* row = (const uint8_t*)s.data + w * s.stride_w;
  uint8_t* orow = out + w * packed_depth;
  const int k_begin = blockIdx.y * slab;
  const int k_end = k_begin + slab < packed_depth ? k_begin + slab : packed_depth;
  uint32_t acc = 0;
  int k = k_begin + 16 * lane;
  for (; k + 512 < k_end; k += 1024) {   // two pieces per trip: more loads in flight
    const uint4 q0 = depth - k > 0 ? load16_any(row + k, depth - k) : make_uint4(0u, 0u, 0u, 0u);
    const uint4 q1 = depth - k - 512 > 0 ? load16_any(row + k + 512, depth - k - 512) : make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(orow + k) = q0;
    *reinterpret_cast<uint4*>(orow + k + 512) = q1;
    acc += sum16(q0, is_signed) + sum16(q1, is_signed);
  }
  for (; k < k_end; k += 512) {
    const uint4 q = depth - k > 0 ? load16_any(row + k, depth - k) : make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(orow + k) = q;
    acc += sum16(q, is_signed);
  }
  if (sums) {
    acc = __reduce_add_sync(0xffffffffu, acc);
    if (lane == 0) {
      if (gridDim.y == 1) sums[w] = (int32_t)acc;
      else atomicAdd(&sums[w], (int32_t)acc);
    }
  }
}

// 8-bit operands stored width-contiguous (a column-major LHS, a row-major RHS): tiles of 64 widths x 64 of depth are
// read as 16-byte runs along the width, turned in shared memory, and written as 16-byte runs along the depth.
__global__ void __launch_bounds__(256) pack8_transpose_kernel(SideView s, int depth, int packed_depth, uint8_t* out,
                                                              int32_t* sums, int slab) {
  __shared__ uint32_t tile[64][17];   // [depth][width / 4], one word of padding per row
  const bool is_signed = s.dtype == RUYB200_I8;
  const int t = threadIdx.x;
  const long long w0 = (long long)blockIdx.x * 64;
  const int k_begin = blockIdx.y * slab;
  const int k_end = k_begin + slab < packed_depth ? k_begin + slab : packed_depth;
  const uint8_t* src = (const uint8_t*)s.data;
  const uint8_t* tile_bytes = reinterpret_cast<const uint8_t*>(&tile[0][0]);
  uint32_t acc = 0;
  for (int k0 = k_begin; k0 < k_end; k0 += 64) {
    {
      const int k = k0 + t / 4, seg = t % 4;
      const long long n_valid = s.width - (w0 + 16 * seg);
      uint4 q = make_uint4(0u, 0u, 0u, 0u);
      if (k < depth && n_valid > 0) q = load16_any(src + (int64_t)k * s.stride_k + w0 + 16 * seg, n_valid > 16 ? 16 : (int)n_valid);
      tile[t / 4][4 * seg + 0] = q.x;
      tile[t / 4][4 * seg + 1] = q.y;
      tile[t / 4][4 * seg + 2] = q.z;
      tile[t / 4][4 * seg + 3] = q.w;
    }
    __syncthreads();
    {
      const int w = t / 4, kseg = t % 4;
      uint32_t o[4];
#pragma unroll
      for (int i = 0; i < 4; i++) {
        uint32_t v = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) v |= (uint32_t)tile_bytes[(16 * kseg + 4 * i + b) * 68 + w] << (8 * b);
        o[i] = v;
      }
      const uint4 q = make_uint4(o[0], o[1], o[2], o[3]);
      if (w0 + w < s.width && k0 + 16 * kseg < k_end) {
        *reinterpret_cast<uint4*>(out + (w0 + w) * packed_depth + k0 + 16 * kseg) = q;
        acc += sum16(q, is_signed);
      }
    }
    __syncthreads();
  }
  if (sums) {
    acc += __shfl_xor_sync(0xffffffffu, acc, 1);
    acc += __shfl_xor_sync(0xffffffffu, acc, 2);
    const long long w = w0 + t / 4;
    if (t % 4 == 0 && w < s.width) {
      if (gridDim.y == 1) sums[w] = (int32_t)acc;
      else atomicAdd(&sums[w], (int32_t)acc);
    }
  }
}

}  // namespace

cudaError_t launch_generic(const SideView& m_side, const SideView& n_side, const DstView& dst,
                           const Epilogue& ep, cudaStream_t stream) {
  if (dst.size_m <= 0 || dst.size_n <= 0) return cudaSuccess;
  dim3 grid((dst.size_n + kTile - 1) / kTile, (dst.size_m + kTile - 1) / kTile);
  if (grid.y > 65535) return cudaErrorInvalidConfiguration;
  if (ep.is_float) {
    generic_mul_kernel<true><<<grid, 256, 0, stream>>>(m_side, n_side, dst, ep);
  } else {
    generic_mul_kernel<false><<<grid, 256, 0, stream>>>(m_side, n_side, dst, ep);
  }
  return cudaGetLastError();
}

cudaError_t launch_generic_f64(const SideView& m_side, const SideView& n_side, const DstView& dst, const Epilogue& ep,
                               double clamp_min, double clamp_max, cudaStream_t stream) {
  if (dst.size_m <= 0 || dst.size_n <= 0) return cudaSuccess;
  dim3 grid((dst.size_n + kTile - 1) / kTile, (dst.size_m + kTile - 1) / kTile);
  if (grid.y > 65535) return cudaErrorInvalidConfiguration;
  const int code = (m_side.dtype == RUYB200_F64 ? 4 : 0) | (n_side.dtype == RUYB200_F64 ? 2 : 0) | (ep.dst_dtype == RUYB200_F64 ? 1 : 0);
#define RUYB200_F64_CASE(c, TM, TN, TD) \
  case c: generic_f64_kernel<TM, TN, TD><<<grid, 256, 0, stream>>>(m_side, n_side, dst, ep, clamp_min, clamp_max); break;
  switch (code) {
    RUYB200_F64_CASE(0, float, float, float)
    RUYB200_F64_CASE(1, float, float, double)
    RUYB200_F64_CASE(2, float, double, float)
    RUYB200_F64_CASE(3, float, double, double)
    RUYB200_F64_CASE(4, double, float, float)
    RUYB200_F64_CASE(5, double, float, double)
    RUYB200_F64_CASE(6, double, double, float)
    RUYB200_F64_CASE(7, double, double, double)
  }
#undef RUYB200_F64_CASE
  return cudaGetLastError();
}

cudaError_t launch_sums(const SideView& side, int depth, int32_t* sums, cudaStream_t stream) {
  if (side.width <= 0) return cudaSuccess;
  // a CTA per row while that still leaves every SM several rows' worth of loads in flight
  if (side.width <= 2048 && depth >= 2048) {
    sums_kernel<256><<<side.width, 256, 0, stream>>>(side, depth, sums);
  } else {
    sums_kernel<32><<<(side.width + 7) / 8, 256, 0, stream>>>(side, depth, sums);
  }
  return cudaGetLastError();
}

cudaError_t launch_pack(const SideView& side, int depth, int packed_depth, void* packed,
                        int32_t* sums, cudaStream_t stream) {
  if (side.width <= 0) return cudaSuccess;
  const bool is8 = side.dtype == RUYB200_I8 || side.dtype == RUYB200_U8;
  if (is8 && (side.stride_k == 1 || side.stride_w == 1) && ((uintptr_t)packed & 15) == 0 && packed_depth % 16 == 0) {
    // the vector kernels; the depth is cut into slabs (gridDim.y) until the launch has a few thousand warps
    const bool rows = side.stride_k == 1;
    const int unit = rows ? 512 : 64;                     // depth bytes per trip
    const long long blocks_x = rows ? ((long long)side.width + 7) / 8 : ((long long)side.width + 63) / 64;
    const long long want = (1024 + blocks_x - 1) / blocks_x;
    const int max_slabs = (packed_depth + unit - 1) / unit;
    const int n_slabs = (int)(want < 1 ? 1 : (want > max_slabs ? max_slabs : want));
    const int slab = ((packed_depth + n_slabs - 1) / n_slabs + unit - 1) / unit * unit;
    const int blocks_y = (packed_depth + slab - 1) / slab;
    if (blocks_x <= 0x7fffffffLL && blocks_y <= 65535) {
      if (sums && blocks_y > 1) {
        cudaError_t ce = cudaMemsetAsync(sums, 0, sizeof(int32_t) * (size_t)side.width, stream);
        if (ce != cudaSuccess) return ce;
      }
      const dim3 grid((unsigned)blocks_x, (unsigned)blocks_y);
      if (rows) pack8_rows_kernel<<<grid, 256, 0, stream>>>(side, depth, packed_depth, (uint8_t*)packed, sums, slab);
      else pack8_transpose_kernel<<<grid, 256, 0, stream>>>(side, depth, packed_depth, (uint8_t*)packed, sums, slab);
      return cudaGetLastError();
    }
  }
  const int grid = (side.width + 31) / 32;
  switch (side.dtype) {
    case RUYB200_I8:
      pack_kernel<int8_t><<<grid, 256, 0, stream>>>(side, depth, packed_depth, (int8_t*)packed, sums);
      break;
    case RUYB200_U8:
      pack_kernel<uint8_t><<<grid, 256, 0, stream>>>(side, depth, packed_depth, (uint8_t*)packed, sums);
      break;
    case RUYB200_I16:
      pack_kernel<int16_t><<<grid, 256, 0, stream>>>(side, depth, packed_depth, (int16_t*)packed, sums);
      break;
    case RUYB200_F32:
      // floats are moved as 32-bit patterns; no sums
      pack_kernel<int32_t><<<grid, 256, 0, stream>>>(side, depth, packed_depth, (int32_t*)packed, nullptr);
      break;
    default:
      return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace ruyb200
