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

// One warp per width-row; lanes stride over depth.
__global__ void sums_kernel(SideView s, int depth, int32_t* sums) {
  const int w = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (w >= s.width) return;
  const int lane = threadIdx.x % 32;
  uint32_t acc = 0;
  const bool vec = s.stride_k == 1 && (s.dtype == RUYB200_I8 || s.dtype == RUYB200_U8) &&
                   (((uintptr_t)s.data + (uint64_t)w * s.stride_w) % 16 == 0);
  int k = 0;
  if (vec) {
    const uint4* row = (const uint4*)((const char*)s.data + (int64_t)w * s.stride_w);
    const int nvec = depth / 16;
    for (int v = lane; v < nvec; v += 32) {
      const uint4 q = row[v];
      if (s.dtype == RUYB200_I8) {
        int a = 0;
        a = __dp4a((int)q.x, 0x01010101, a);
        a = __dp4a((int)q.y, 0x01010101, a);
        a = __dp4a((int)q.z, 0x01010101, a);
        a = __dp4a((int)q.w, 0x01010101, a);
        acc += (uint32_t)a;
      } else {
        unsigned a = 0;
        a = __dp4a(q.x, 0x01010101u, a);
        a = __dp4a(q.y, 0x01010101u, a);
        a = __dp4a(q.z, 0x01010101u, a);
        a = __dp4a(q.w, 0x01010101u, a);
        acc += a;
      }
    }
    k = nvec * 16;
  }
  for (int kk = k + lane; kk < depth; kk += 32) {
    acc += (uint32_t)load_as_int(s.data, s.dtype, (int64_t)w * s.stride_w + (int64_t)kk * s.stride_k);
  }
  acc = __reduce_add_sync(0xffffffffu, acc);
  if (lane == 0) sums[w] = (int32_t)acc;
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
  const int warps_per_block = 8;
  const int grid = (side.width + warps_per_block - 1) / warps_per_block;
  sums_kernel<<<grid, warps_per_block * 32, 0, stream>>>(side, depth, sums);
  return cudaGetLastError();
}

cudaError_t launch_pack(const SideView& side, int depth, int packed_depth, void* packed,
                        int32_t* sums, cudaStream_t stream) {
  if (side.width <= 0) return cudaSuccess;
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
