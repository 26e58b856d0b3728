// Narrow muls: one side of the product has at most eight rows (matrix times vector, or times a handful of
// vectors).  ruy has dedicated kernels for the single-column case, Kernel8bitAvx512SingleCol
// (ruy/kernel_avx512.cc:628-870) and KernelFloatAvx512SingleCol (ruy/kernel_avx512.cc:1238-1320), because a
// 16-wide kernel wastes fifteen sixteenths of its work there; a 128-lane tensor-core tile would waste even more.
// Such a mul is a stream over the wide operand: HBM-bound, one pass, no packing, no tensor core.
//
// One warp per row of the wide side.  The lanes stride over 16-byte pieces of the depth; every piece of the wide
// row is multiplied (dp4a for 8-bit, FFMA for fp32) with the same piece of each narrow row, which the whole grid
// shares through L1/L2.  The zero-point sums of both sides (ruy/pack.h:117-129) come out of the same pass.  A
// butterfly reduction leaves the totals in every lane and lane j finishes and stores output j with the epilogue
// of ruy/kernel.h:213-237.
#include "common.cuh"

#include <atomic>
#include <type_traits>

namespace ruyb200 {

namespace {

constexpr int kWarpsPerBlock = 8;


template <bool kASigned, bool kBSigned>
__device__ __forceinline__ int32_t dot4(uint32_t a, uint32_t b, int32_t c) {
  int32_t d;
  if (kASigned && kBSigned) {
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  } else if (kASigned) {
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  } else if (kBSigned) {
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  } else {
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  }
  return d;
}

template <bool kSigned>
__device__ __forceinline__ int32_t sum4(uint32_t a, int32_t c) {
  return dot4<kSigned, false>(a, 0x01010101u, c);
}

template <bool kSigned>
__device__ __forceinline__ int32_t load8(const uint8_t* p) {
  return kSigned ? (int32_t)(int8_t)*p : (int32_t)*p;
}

struct GemvArgs {
  SideView wide;      // one warp per row of this side
  SideView narrow;    // at most kGemvMaxNarrow rows
  DstView dst;
  Epilogue ep;
  int wide_is_m;      // 1: the wide side indexes the destination's m dimension, 0: its n (contiguous) dimension
  int vec;            // both sides: 16-byte aligned base and row stride
  int need_wsum;      // the narrow side's zero point is not 0: the sums over depth of the wide rows are needed
  int need_nsum;      // the wide side's zero point is not 0: the sums of the narrow rows are needed
};

// Finishes one output from its raw dot product and the two sums over depth (ruy/kernel.h:213-237).
__device__ __forceinline__ int32_t finish_with_sums(int32_t raw, int32_t sum_m, int32_t sum_n, int m, int n, const Epilogue& ep) {
  uint32_t acc = (uint32_t)raw;
  const int ch = ep.channel_on_n ? n : m;
  if (ep.bias) acc += (uint32_t)((const int32_t*)ep.bias)[ch];
  acc -= (uint32_t)ep.zp_m * (uint32_t)sum_n;
  acc -= (uint32_t)ep.zp_n * (uint32_t)sum_m;
  acc += (uint32_t)ep.zp_m * (uint32_t)ep.zp_n * (uint32_t)ep.depth;
  int32_t v = (int32_t)acc;
  if (ep.dst_dtype != RUYB200_I32) {
    const int32_t mult = ep.mfp_pc ? ep.mfp_pc[ch] : ep.mfp;
    const int e = ep.mexp_pc ? ep.mexp_pc[ch] : ep.mexp;
    v = ep.rounding_x86 ? requant_x86(v, mult, e) : requant_reference(v, mult, e);
  }
  v = (int32_t)((uint32_t)v + (uint32_t)ep.dst_zp);
  if (ep.dst_dtype != RUYB200_I32) {
    v = min(v, ep.clamp_max);
    v = max(v, ep.clamp_min);
  }
  return v;
}

template <int kNarrow, bool kWideSigned, bool kNarrowSigned>
__global__ void __launch_bounds__(32 * kWarpsPerBlock) gemv_i8_kernel(const GemvArgs a) {
  const int lane = threadIdx.x % 32;
  const long long w = (long long)blockIdx.x * kWarpsPerBlock + threadIdx.x / 32;
  if (w >= a.wide.width) return;
  const int depth = a.ep.depth;
  const uint8_t* wrow = (const uint8_t*)a.wide.data + w * a.wide.stride_w;
  const uint8_t* nbase = (const uint8_t*)a.narrow.data;
  const int64_t nstride = a.narrow.stride_w;
  int32_t acc[kNarrow], nsum[kNarrow];
#pragma unroll
  for (int j = 0; j < kNarrow; j++) acc[j] = nsum[j] = 0;
  int32_t wsum = 0;
  int k = 0;
  if (a.vec) {
    const int pieces = depth / 16;
    int c = lane;
    // four pieces per lane and trip, all loads of the wide row first: more bytes in flight per warp
    for (; c + 96 < pieces; c += 128) {
      uint4 x[4];
#pragma unroll
      for (int u = 0; u < 4; u++) x[u] = __ldcs(reinterpret_cast<const uint4*>(wrow) + c + 32 * u);
      if (a.need_wsum) {
#pragma unroll
        for (int u = 0; u < 4; u++) {
          wsum = sum4<kWideSigned>(x[u].x, wsum);
          wsum = sum4<kWideSigned>(x[u].y, wsum);
          wsum = sum4<kWideSigned>(x[u].z, wsum);
          wsum = sum4<kWideSigned>(x[u].w, wsum);
        }
      }
#pragma unroll
      for (int j = 0; j < kNarrow; j++) {
        if (j < a.narrow.width) {
          uint4 y[4];
#pragma unroll
          for (int u = 0; u < 4; u++) y[u] = __ldg(reinterpret_cast<const uint4*>(nbase + j * nstride) + c + 32 * u);
#pragma unroll
          for (int u = 0; u < 4; u++) {
            acc[j] = dot4<kWideSigned, kNarrowSigned>(x[u].x, y[u].x, acc[j]);
            acc[j] = dot4<kWideSigned, kNarrowSigned>(x[u].y, y[u].y, acc[j]);
            acc[j] = dot4<kWideSigned, kNarrowSigned>(x[u].z, y[u].z, acc[j]);
            acc[j] = dot4<kWideSigned, kNarrowSigned>(x[u].w, y[u].w, acc[j]);
            if (a.need_nsum) {
              nsum[j] = sum4<kNarrowSigned>(y[u].x, nsum[j]);
              nsum[j] = sum4<kNarrowSigned>(y[u].y, nsum[j]);
              nsum[j] = sum4<kNarrowSigned>(y[u].z, nsum[j]);
              nsum[j] = sum4<kNarrowSigned>(y[u].w, nsum[j]);
            }
          }
        }
      }
    }
    for (; c < pieces; c += 32) {
      const uint4 x = __ldcs(reinterpret_cast<const uint4*>(wrow) + c);   // streamed: read exactly once
      if (a.need_wsum) {
        wsum = sum4<kWideSigned>(x.x, wsum);
        wsum = sum4<kWideSigned>(x.y, wsum);
        wsum = sum4<kWideSigned>(x.z, wsum);
        wsum = sum4<kWideSigned>(x.w, wsum);
      }
#pragma unroll
      for (int j = 0; j < kNarrow; j++) {
        if (j < a.narrow.width) {
          const uint4 y = __ldg(reinterpret_cast<const uint4*>(nbase + j * nstride) + c);
          acc[j] = dot4<kWideSigned, kNarrowSigned>(x.x, y.x, acc[j]);
          acc[j] = dot4<kWideSigned, kNarrowSigned>(x.y, y.y, acc[j]);
          acc[j] = dot4<kWideSigned, kNarrowSigned>(x.z, y.z, acc[j]);
          acc[j] = dot4<kWideSigned, kNarrowSigned>(x.w, y.w, acc[j]);
          if (a.need_nsum) {
            nsum[j] = sum4<kNarrowSigned>(y.x, nsum[j]);
            nsum[j] = sum4<kNarrowSigned>(y.y, nsum[j]);
            nsum[j] = sum4<kNarrowSigned>(y.z, nsum[j]);
            nsum[j] = sum4<kNarrowSigned>(y.w, nsum[j]);
          }
        }
      }
    }
    k = pieces * 16;
  }
  // what the 16-byte pieces do not cover (all of it for unaligned operands), one byte per lane and step
  for (int kk = k + lane; kk < depth; kk += 32) {
    const int32_t x = load8<kWideSigned>(wrow + kk);
    wsum += x;
#pragma unroll
    for (int j = 0; j < kNarrow; j++) {
      if (j < a.narrow.width) {
        const int32_t y = load8<kNarrowSigned>(nbase + j * nstride + kk);
        acc[j] = (int32_t)((uint32_t)acc[j] + (uint32_t)(x * y));   // accumulators wrap, as ruy's do
        nsum[j] += y;
      }
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    wsum += __shfl_xor_sync(0xffffffffu, wsum, d);
#pragma unroll
    for (int j = 0; j < kNarrow; j++) {
      acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], d);
      nsum[j] += __shfl_xor_sync(0xffffffffu, nsum[j], d);
    }
  }
  int32_t my_acc = 0, my_nsum = 0;
#pragma unroll
  for (int j = 0; j < kNarrow; j++) {
    if (lane == j) {
      my_acc = acc[j];
      my_nsum = nsum[j];
    }
  }
  if (lane < a.narrow.width) {
    const int m = a.wide_is_m ? (int)w : lane;
    const int n = a.wide_is_m ? lane : (int)w;
    const int32_t sum_m = a.wide_is_m ? wsum : my_nsum;
    const int32_t sum_n = a.wide_is_m ? my_nsum : wsum;
    store_int(a.dst, a.ep.dst_dtype, m, n, finish_with_sums(my_acc, sum_m, sum_n, m, n, a.ep));
  }
}

// m16n8k32 integer MMA on the warp's registers (the legacy tensor-core path): d += a (16 x 32 bytes) * b (32 x 8).
template <bool kASigned, bool kBSigned>
__device__ __forceinline__ void mma_16x8x32(int32_t (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  if (kASigned && kBSigned) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else if (kASigned) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else if (kBSigned) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}

// Two to eight narrow rows against a wide operand of thousands of rows: dp4a runs at a quarter of the integer rate on
// this part, and with four of them per narrow row and 16-byte piece the kernel above is bound by them, not by HBM
// (16384 x 16384 x 8: 215 us against 41 us for the stream).  Here a CTA takes 16 wide rows; its warps take turns on
// steps of 256 bytes of depth, each step feeding eight m16n8k32 MMAs: lane (g, t) (g = lane / 4, t = lane % 4) loads
// the 16-byte pieces t, t + 4, t + 8, t + 12 of the step from wide rows g and g + 8 and, for each tile of 8 narrow
// rows (one or two tiles), from narrow row g of the tile; the MMA's k
// index is a permutation of the byte index, the same for both operands, so the sums over k are unchanged.  The
// zero-point sums still use dp4a, one per loaded word.  The warps' partial sums meet in shared memory and warp 0
// finishes.  Needs 16-byte aligned rows and a depth that is a multiple of 16.
template <bool kWideSigned, bool kNarrowSigned, int kTiles, int kWarps>
__global__ void __launch_bounds__(32 * kWarps, kWarps == 2 ? 8 : (kTiles == 2 ? 16 : 24) / kWarps) gemv_i8_mma_kernel(const GemvArgs a) {
  constexpr int kPart = 5 * kTiles + 2;  // per lane: 4 accumulators and a narrow sum per tile of 8 narrow rows, 2 wide sums
  __shared__ int32_t part[kWarps - 1][kPart][32];
  const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
  const int g = lane >> 2, t = lane & 3;
  const long long w0 = (long long)blockIdx.x * 16;
  const int depth = a.ep.depth;
  const long long last = a.wide.width - 1;
  const long long r0 = w0 + g, r1 = w0 + g + 8;
  const uint4* row0 = reinterpret_cast<const uint4*>((const uint8_t*)a.wide.data + (r0 < last ? r0 : last) * a.wide.stride_w);
  const uint4* row1 = reinterpret_cast<const uint4*>((const uint8_t*)a.wide.data + (r1 < last ? r1 : last) * a.wide.stride_w);
  const uint4* nrow[kTiles];
  bool have_n[kTiles];
#pragma unroll
  for (int j = 0; j < kTiles; j++) {
    have_n[j] = 8 * j + g < a.narrow.width;
    nrow[j] = reinterpret_cast<const uint4*>((const uint8_t*)a.narrow.data + (have_n[j] ? 8 * j + g : 0) * a.narrow.stride_w);
  }
  int32_t c[kTiles][4];
  int32_t nsum[kTiles];
#pragma unroll
  for (int j = 0; j < kTiles; j++) {
    nsum[j] = 0;
#pragma unroll
    for (int i = 0; i < 4; i++) c[j][i] = 0;
  }
  int32_t wsum0 = 0, wsum1 = 0;
  const int pieces = depth / 16;
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  // one step: all of its loads first (8 of the wide rows, 4 per tile of narrow rows), then the MMAs and the sums
  struct Frag {
    uint4 xa[4], xb[4], y[kTiles][4];
  };
  auto load = [&](Frag& f, const int base, auto whole_tag) {
    constexpr bool kWhole = decltype(whole_tag)::value;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int p = base + t + 4 * i;
      f.xa[i] = (kWhole || p < pieces) ? __ldcs(row0 + p) : zero;
      f.xb[i] = (kWhole || p < pieces) ? __ldcs(row1 + p) : zero;
    }
#pragma unroll
    for (int j = 0; j < kTiles; j++) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        const int p = base + t + 4 * i;
        f.y[j][i] = (have_n[j] && (kWhole || p < pieces)) ? __ldg(nrow[j] + p) : zero;
      }
    }
  };
  auto compute = [&](const Frag& f) {
#pragma unroll
    for (int j = 0; j < kTiles; j++) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        mma_16x8x32<kWideSigned, kNarrowSigned>(c[j], f.xa[i].x, f.xb[i].x, f.xa[i].y, f.xb[i].y, f.y[j][i].x, f.y[j][i].y);
        mma_16x8x32<kWideSigned, kNarrowSigned>(c[j], f.xa[i].z, f.xb[i].z, f.xa[i].w, f.xb[i].w, f.y[j][i].z, f.y[j][i].w);
      }
      if (a.need_nsum) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
          nsum[j] = sum4<kNarrowSigned>(f.y[j][i].x, nsum[j]);
          nsum[j] = sum4<kNarrowSigned>(f.y[j][i].y, nsum[j]);
          nsum[j] = sum4<kNarrowSigned>(f.y[j][i].z, nsum[j]);
          nsum[j] = sum4<kNarrowSigned>(f.y[j][i].w, nsum[j]);
        }
      }
    }
    if (a.need_wsum) {
#pragma unroll
      for (int i = 0; i < 4; i++) {
        wsum0 = sum4<kWideSigned>(f.xa[i].x, wsum0);
        wsum0 = sum4<kWideSigned>(f.xa[i].y, wsum0);
        wsum0 = sum4<kWideSigned>(f.xa[i].z, wsum0);
        wsum0 = sum4<kWideSigned>(f.xa[i].w, wsum0);
        wsum1 = sum4<kWideSigned>(f.xb[i].x, wsum1);
        wsum1 = sum4<kWideSigned>(f.xb[i].y, wsum1);
        wsum1 = sum4<kWideSigned>(f.xb[i].z, wsum1);
        wsum1 = sum4<kWideSigned>(f.xb[i].w, wsum1);
      }
    }
  };
  int base = warp * 16;
  if (kWarps <= 2 && kTiles == 1) {
    // few warps per CTA (all CTAs resident at once, about 14 warps per SM): two steps' loads in flight per warp
    for (; base + kWarps * 16 + 16 <= pieces; base += 2 * kWarps * 16) {
      Frag f0, f1;
      load(f0, base, std::true_type{});
      load(f1, base + kWarps * 16, std::true_type{});
      compute(f0);
      compute(f1);
    }
  }
  for (; base + 16 <= pieces; base += kWarps * 16) {
    Frag f;
    load(f, base, std::true_type{});
    compute(f);
  }
  if (base < pieces) {
    Frag f;
    load(f, base, std::false_type{});
    compute(f);
  }
  if (warp > 0) {
#pragma unroll
    for (int j = 0; j < kTiles; j++) {
#pragma unroll
      for (int i = 0; i < 4; i++) part[warp - 1][5 * j + i][lane] = c[j][i];
      part[warp - 1][5 * j + 4][lane] = nsum[j];
    }
    part[warp - 1][5 * kTiles][lane] = wsum0;
    part[warp - 1][5 * kTiles + 1][lane] = wsum1;
  }
  __syncthreads();
  if (warp > 0) return;
#pragma unroll
  for (int w = 0; w < kWarps - 1; w++) {
#pragma unroll
    for (int j = 0; j < kTiles; j++) {
#pragma unroll
      for (int i = 0; i < 4; i++) c[j][i] += part[w][5 * j + i][lane];
      nsum[j] += part[w][5 * j + 4][lane];
    }
    wsum0 += part[w][5 * kTiles][lane];
    wsum1 += part[w][5 * kTiles + 1][lane];
  }
  // the four lanes of a quad hold the four quarters of each step
#pragma unroll
  for (int d = 1; d <= 2; d <<= 1) {
    wsum0 += __shfl_xor_sync(0xffffffffu, wsum0, d);
    wsum1 += __shfl_xor_sync(0xffffffffu, wsum1, d);
#pragma unroll
    for (int j = 0; j < kTiles; j++) nsum[j] += __shfl_xor_sync(0xffffffffu, nsum[j], d);
  }
#pragma unroll
  for (int j = 0; j < kTiles; j++) {
    // this lane's outputs of the tile: wide rows r0 and r1, narrow rows 8 j + 2 t and 8 j + 2 t + 1, whose sums sit in
    // quads 2 t and 2 t + 1
    const int32_t nsum_a = __shfl_sync(0xffffffffu, nsum[j], (2 * t) * 4);
    const int32_t nsum_b = __shfl_sync(0xffffffffu, nsum[j], (2 * t + 1) * 4);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const long long w = i < 2 ? r0 : r1;
      const int col = 8 * j + 2 * t + (i & 1);
      if (w < a.wide.width && col < a.narrow.width) {
        const int m = a.wide_is_m ? (int)w : col;
        const int n = a.wide_is_m ? col : (int)w;
        const int32_t ws = i < 2 ? wsum0 : wsum1, ns = (i & 1) ? nsum_b : nsum_a;
        const int32_t sum_m = a.wide_is_m ? ws : ns;
        const int32_t sum_n = a.wide_is_m ? ns : ws;
        store_int(a.dst, a.ep.dst_dtype, m, n, finish_with_sums(c[j][i], sum_m, sum_n, m, n, a.ep));
      }
    }
  }
}

template <int kTiles, int kWarps>
cudaError_t launch_i8_mma_warps(const GemvArgs& a, cudaStream_t stream) {
  const unsigned grid = (unsigned)(((long long)a.wide.width + 15) / 16);
  const bool ws = a.wide.dtype == RUYB200_I8, ns = a.narrow.dtype == RUYB200_I8;
  if (ws && ns) gemv_i8_mma_kernel<true, true, kTiles, kWarps><<<grid, 32 * kWarps, 0, stream>>>(a);
  else if (ws) gemv_i8_mma_kernel<true, false, kTiles, kWarps><<<grid, 32 * kWarps, 0, stream>>>(a);
  else if (ns) gemv_i8_mma_kernel<false, true, kTiles, kWarps><<<grid, 32 * kWarps, 0, stream>>>(a);
  else gemv_i8_mma_kernel<false, false, kTiles, kWarps><<<grid, 32 * kWarps, 0, stream>>>(a);
  return cudaGetLastError();
}

// Warps per CTA of the MMA form.  The grid is one CTA per 16 wide rows whatever their number, so what can be chosen is
// how many CTAs an SM holds at once (24 warps' worth with one tile of narrow rows, 16 with two): with 8 warps per CTA,
// 16384 rows are 1024 CTAs on 444 places, 2.3 waves of which the last runs on a third of the machine (measured 50.9 us
// where one narrow row, which has no such tail, takes 40.7 us); with 2 warps per CTA all 1024 are resident at once.
// Taken: the largest CTA among those that waste the least of their last wave.
int mma_form_warps(long long ctas, int sm_count, int tiles) {
  int best = 8;
  double best_eff = 0.0;
  for (int w = 8; w >= 2; w /= 2) {
    const long long places = (long long)sm_count * (w == 2 ? 8 : (tiles == 2 ? 16 : 24) / w);   // the kernel's launch bounds
    const long long waves = (ctas + places - 1) / places;
    const double eff = waves <= 1 ? 1.0 : (double)ctas / (double)(waves * places);
    if (eff > best_eff + 0.02) {
      best = w;
      best_eff = eff;
    }
  }
  return best;
}

template <int kTiles>
cudaError_t launch_i8_mma(const GemvArgs& a, cudaStream_t stream) {
  // per device, filled on first use; contexts on several threads may get here together, hence atomic
  static std::atomic<int> sm_counts[64];
  int dev = 0;
  cudaGetDevice(&dev);
  int sms = dev >= 0 && dev < 64 ? sm_counts[dev].load(std::memory_order_relaxed) : 0;
  if (sms == 0) {
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    if (dev >= 0 && dev < 64) sm_counts[dev].store(sms, std::memory_order_relaxed);
  }
  switch (mma_form_warps(((long long)a.wide.width + 15) / 16, sms, kTiles)) {
    case 2: return launch_i8_mma_warps<kTiles, 2>(a, stream);
    case 4: return launch_i8_mma_warps<kTiles, 4>(a, stream);
    default: return launch_i8_mma_warps<kTiles, 8>(a, stream);
  }
}

// Compensated (Kahan) running sum: folds y into (sum, comp).
__device__ __forceinline__ void kahan_add(float& sum, float& comp, float y) {
  const float yy = y - comp;
  const float t = sum + yy;
  comp = (t - sum) - yy;
  sum = t;
}

// fp32: the same walk with FFMA.  Each lane folds four products at a time into a compensated sum and the lane tree
// is compensated as well, so that a long depth with cancellation stays within 1e-5 of a double-precision sum.
template <int kNarrow>
__global__ void __launch_bounds__(32 * kWarpsPerBlock) gemv_f32_kernel(const GemvArgs a) {
  const int lane = threadIdx.x % 32;
  const long long w = (long long)blockIdx.x * kWarpsPerBlock + threadIdx.x / 32;
  if (w >= a.wide.width) return;
  const int depth = a.ep.depth;
  const float* wrow = (const float*)a.wide.data + w * a.wide.stride_w;
  const float* nbase = (const float*)a.narrow.data;
  const int64_t nstride = a.narrow.stride_w;
  float sum[kNarrow], comp[kNarrow];
#pragma unroll
  for (int j = 0; j < kNarrow; j++) sum[j] = comp[j] = 0.f;
  int k = 0;
  if (a.vec) {
    const int pieces = depth / 4;
    int c = lane;
    // one narrow row: four pieces per lane and trip, all loads of the wide row first, for more bytes in flight per warp
    // (8192 x 8192 x 1: 67.6 -> 58.4 us; with four narrow rows the same loop was 5 % slower, so they keep single pieces)
    for (; kNarrow == 1 && c + 96 < pieces; c += 128) {
      float4 x[4];
#pragma unroll
      for (int u = 0; u < 4; u++) x[u] = __ldcs(reinterpret_cast<const float4*>(wrow) + c + 32 * u);
#pragma unroll
      for (int j = 0; j < kNarrow; j++) {
        if (j < a.narrow.width) {
          float4 y[4];
#pragma unroll
          for (int u = 0; u < 4; u++) y[u] = __ldg(reinterpret_cast<const float4*>(nbase + j * nstride) + c + 32 * u);
#pragma unroll
          for (int u = 0; u < 4; u++) {
            float part = x[u].x * y[u].x;
            part = fmaf(x[u].y, y[u].y, part);
            part = fmaf(x[u].z, y[u].z, part);
            part = fmaf(x[u].w, y[u].w, part);
            kahan_add(sum[j], comp[j], part);
          }
        }
      }
    }
    for (; c < pieces; c += 32) {
      const float4 x = __ldcs(reinterpret_cast<const float4*>(wrow) + c);
#pragma unroll
      for (int j = 0; j < kNarrow; j++) {
        if (j < a.narrow.width) {
          const float4 y = __ldg(reinterpret_cast<const float4*>(nbase + j * nstride) + c);
          float part = x.x * y.x;
          part = fmaf(x.y, y.y, part);
          part = fmaf(x.z, y.z, part);
          part = fmaf(x.w, y.w, part);
          kahan_add(sum[j], comp[j], part);
        }
      }
    }
    k = pieces * 4;
  }
  for (int kk = k + lane; kk < depth; kk += 32) {
    const float x = wrow[kk];
#pragma unroll
    for (int j = 0; j < kNarrow; j++) {
      if (j < a.narrow.width) kahan_add(sum[j], comp[j], x * nbase[j * nstride + kk]);
    }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
#pragma unroll
    for (int j = 0; j < kNarrow; j++) {
      const float other = __shfl_xor_sync(0xffffffffu, sum[j], d);
      const float other_c = __shfl_xor_sync(0xffffffffu, comp[j], d);
      const float y = other - (comp[j] + other_c);
      const float t = sum[j] + y;
      comp[j] = (t - sum[j]) - y;
      sum[j] = t;
    }
  }
  float mine = 0.f;
#pragma unroll
  for (int j = 0; j < kNarrow; j++) {
    if (lane == j) mine = sum[j];
  }
  if (lane < a.narrow.width) {
    const int m = a.wide_is_m ? (int)w : lane;
    const int n = a.wide_is_m ? lane : (int)w;
    ((float*)a.dst.data)[(int64_t)m * a.dst.stride_m + n] = finish_float(mine, m, n, a.ep);
  }
}

template <int kNarrow>
cudaError_t launch_i8(const GemvArgs& a, unsigned grid, cudaStream_t stream) {
  const bool ws = a.wide.dtype == RUYB200_I8, ns = a.narrow.dtype == RUYB200_I8;
  if (ws && ns) gemv_i8_kernel<kNarrow, true, true><<<grid, 32 * kWarpsPerBlock, 0, stream>>>(a);
  else if (ws) gemv_i8_kernel<kNarrow, true, false><<<grid, 32 * kWarpsPerBlock, 0, stream>>>(a);
  else if (ns) gemv_i8_kernel<kNarrow, false, true><<<grid, 32 * kWarpsPerBlock, 0, stream>>>(a);
  else gemv_i8_kernel<kNarrow, false, false><<<grid, 32 * kWarpsPerBlock, 0, stream>>>(a);
  return cudaGetLastError();
}

}  // namespace

static bool rows_16_byte_aligned(const SideView& x, const SideView& y) {
  return (((uintptr_t)x.data | (uintptr_t)y.data | (uintptr_t)x.stride_w | (uintptr_t)y.stride_w) & 15) == 0;
}

bool gemv_eligible(const SideView& m_side, const SideView& n_side, int depth, bool is_float) {
  const int narrow = m_side.width < n_side.width ? m_side.width : n_side.width;
  if (narrow < 1 || narrow > kGemvMmaMaxNarrow) return false;
  if (m_side.stride_k != 1 || n_side.stride_k != 1) return false;
  const long long wide = m_side.width < n_side.width ? n_side.width : m_side.width;
  if ((wide + kWarpsPerBlock - 1) / kWarpsPerBlock > 0x7fffffffLL) return false;
  if (is_float) return narrow <= kGemvMaxNarrow && m_side.dtype == RUYB200_F32 && n_side.dtype == RUYB200_F32;
  const bool m8 = m_side.dtype == RUYB200_I8 || m_side.dtype == RUYB200_U8;
  const bool n8 = n_side.dtype == RUYB200_I8 || n_side.dtype == RUYB200_U8;
  if (!(m8 && n8)) return false;
  return narrow <= kGemvMaxNarrow || (gemv_mma_shape(narrow, wide, depth) && rows_16_byte_aligned(m_side, n_side));
}

cudaError_t launch_gemv(const SideView& m_side, const SideView& n_side, const DstView& dst, const Epilogue& ep,
                        cudaStream_t stream) {
  if (dst.size_m <= 0 || dst.size_n <= 0) return cudaSuccess;
  GemvArgs a;
  a.wide_is_m = m_side.width >= n_side.width ? 1 : 0;
  a.wide = a.wide_is_m ? m_side : n_side;
  a.narrow = a.wide_is_m ? n_side : m_side;
  a.dst = dst;
  a.ep = ep;
  const size_t esz = ep.is_float ? 4 : 1;
  a.vec = (((uintptr_t)a.wide.data | (uintptr_t)a.narrow.data | (uintptr_t)(a.wide.stride_w * esz) |
            (uintptr_t)(a.narrow.stride_w * esz)) & 15) == 0;
  a.need_wsum = a.narrow.zero_point != 0;
  a.need_nsum = a.wide.zero_point != 0;
  const unsigned grid = (unsigned)(((long long)a.wide.width + kWarpsPerBlock - 1) / kWarpsPerBlock);
  const int narrow = a.narrow.width;
  if (ep.is_float) {
    if (narrow <= 1) gemv_f32_kernel<1><<<grid, 32 * kWarpsPerBlock, 0, stream>>>(a);
    else if (narrow <= 4) gemv_f32_kernel<4><<<grid, 32 * kWarpsPerBlock, 0, stream>>>(a);
    else gemv_f32_kernel<kGemvMaxNarrow><<<grid, 32 * kWarpsPerBlock, 0, stream>>>(a);
    return cudaGetLastError();
  }
  if (a.vec && gemv_mma_shape(narrow, a.wide.width, ep.depth)) {
    if (narrow <= 8) return launch_i8_mma<1>(a, stream);
    return launch_i8_mma<2>(a, stream);
  }
  if (narrow <= 1) return launch_i8<1>(a, grid, stream);
  if (narrow <= 4) return launch_i8<4>(a, grid, stream);
  return launch_i8<kGemvMaxNarrow>(a, grid, stream);
}

}  // namespace ruyb200
