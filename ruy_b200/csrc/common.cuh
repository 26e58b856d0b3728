// Internal declarations shared by the CUDA translation units of libruy_b200.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/ruy_b200.h"

namespace ruyb200 {

// One side of the "TrMul" view (ruy/create_trmul_params.h:465-480): a width x depth matrix
// addressed as data[w * stride_w + k * stride_k] (in elements).  The LHS is width = rows,
// the RHS is width = cols; a depth-contiguous ("K-major") side has stride_k == 1.
struct SideView {
  const void* data;
  int64_t stride_w;
  int64_t stride_k;
  int32_t width;
  int32_t zero_point;
  uint8_t dtype;
};

// Everything the fused epilogue needs (ruy/kernel.h:213-237, ruy/kernel_common.h:94-213).
// "n" indexes the destination's contiguous dimension, "m" the other one; which of them is
// the row index depends on the destination's storage order.
struct Epilogue {
  const void* bias;            // int32 or float, indexed by channel
  const int32_t* mfp_pc;       // per-channel fixed-point multipliers or nullptr
  const int32_t* mexp_pc;      // per-channel exponents or nullptr
  const int32_t* sums_m;       // sum over depth of the m-side operand, per m (needed when zp_n != 0)
  const int32_t* sums_n;       // sum over depth of the n-side operand, per n (needed when zp_m != 0)
  int32_t mfp;
  int32_t mexp;
  int32_t clamp_min;           // int32, or float bits when is_float
  int32_t clamp_max;
  int32_t zp_m;                // zero point of the m-side operand
  int32_t zp_n;                // zero point of the n-side operand
  int32_t dst_zp;
  int32_t depth;
  uint8_t channel_on_n;        // 1: per-channel buffers are indexed by n, 0: by m
  uint8_t rounding_x86;        // 1: two-step x86 rounding, 0: reference rounding
  uint8_t dst_dtype;           // ruyb200_dtype
  uint8_t is_float;
};

// Destination addressing: element (m, n) lives at dst[m * stride_m + n] (n contiguous).
struct DstView {
  void* data;
  int64_t stride_m;
  int32_t size_m;
  int32_t size_n;
};

// ruy::detail::MultiplyByQuantizedMultiplier (ruy/apply_multiplier.cc:48-65).
__device__ __forceinline__ int32_t requant_reference(int32_t x, int32_t m, int e) {
  const int total_shift = 31 - e;
  const long long round = 1ll << (total_shift - 1);
  const long long r = (long long)x * (long long)m + round;
  return (int32_t)(r >> total_shift);
}

// The rounding of ruy's x86 kernels (ruy/kernel_avx512.cc:340-465): wrapping left shift,
// rounding doubling high multiply, then rounding right shift with an overflow guard.
__device__ __forceinline__ int32_t requant_x86(int32_t x, int32_t m, int e) {
  const int ls = e > 0 ? e : 0;
  const int rs = e < 0 ? -e : 0;
  const int32_t a = (int32_t)((uint32_t)x << ls);
  const int32_t t = (int32_t)(((long long)a * (long long)m + (1ll << 30)) >> 31);
  const int32_t nudge = rs > 0 ? (int32_t)(1u << (rs - 1)) : 0;
  if (t > 0x7fffffff - nudge) return (int32_t)(1u << (31 - rs));
  return (t + nudge) >> rs;
}

// Raw int32 dot product -> final int32 value before the narrowing cast.
// `raw` is sum_k M[m,k]*N[n,k] over the stored (not zero-point-shifted) values.
__device__ __forceinline__ int32_t finish_int(int32_t raw, int m, int n, const Epilogue& ep) {
  uint32_t acc = (uint32_t)raw;
  const int ch = ep.channel_on_n ? n : m;
  if (ep.bias) acc += (uint32_t)((const int32_t*)ep.bias)[ch];
  if (ep.zp_m) acc -= (uint32_t)ep.zp_m * (uint32_t)ep.sums_n[n];
  if (ep.zp_n) acc -= (uint32_t)ep.zp_n * (uint32_t)ep.sums_m[m];
  if (ep.zp_m && ep.zp_n) acc += (uint32_t)ep.zp_m * (uint32_t)ep.zp_n * (uint32_t)ep.depth;
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

__device__ __forceinline__ float finish_float(float acc, int m, int n, const Epilogue& ep) {
  const int ch = ep.channel_on_n ? n : m;
  if (ep.bias) acc += ((const float*)ep.bias)[ch];
  acc = fminf(acc, __int_as_float(ep.clamp_max));
  acc = fmaxf(acc, __int_as_float(ep.clamp_min));
  return acc;
}

__device__ __forceinline__ void store_int(const DstView& d, uint8_t dtype, int m, int n, int32_t v) {
  const int64_t off = (int64_t)m * d.stride_m + n;
  switch (dtype) {
    case RUYB200_I8: ((int8_t*)d.data)[off] = (int8_t)v; break;
    case RUYB200_U8: ((uint8_t*)d.data)[off] = (uint8_t)v; break;
    case RUYB200_I16: ((int16_t*)d.data)[off] = (int16_t)v; break;
    default: ((int32_t*)d.data)[off] = v; break;
  }
}

// ---- launchers (host side); each enqueues on `stream` and returns a cudaError_t ----------

// CUDA-core kernel for any supported type combination, order and stride.
cudaError_t launch_generic(const SideView& m_side, const SideView& n_side, const DstView& dst,
                           const Epilogue& ep, cudaStream_t stream);

// The same for ruy's mixed floating-point cases: float or double operands and destination (the dtype fields say
// which), double accumulation, double bias and clamp bounds.
cudaError_t launch_generic_f64(const SideView& m_side, const SideView& n_side, const DstView& dst, const Epilogue& ep,
                               double clamp_min, double clamp_max, cudaStream_t stream);

// Sum over depth of every width-row of a side (int32, wrap-around).
cudaError_t launch_sums(const SideView& side, int depth, int32_t* sums, cudaStream_t stream);

// PackImpl analogue: writes the side as [width][packed_depth] depth-contiguous with zero
// padding and (for integer types, when sums != nullptr) its per-width sums.
cudaError_t launch_pack(const SideView& side, int depth, int packed_depth, void* packed,
                        int32_t* sums, cudaStream_t stream);

// tcgen05 kind::i8 GEMM.  Both sides must be 8-bit, depth-contiguous, with 16-byte aligned
// base and stride_w (bytes).  `status` is a device word that receives a non-zero code if a
// bounded wait gives up.
// What launch_tc_i8 decided, for the decision log.
struct TcI8Info {
  int pair, block_n, tiles, fused_sums, row_pitch, grid;
  double est_cycles;   // the tile-shape choice's estimate for the launch, in SM cycles
  int shallow;         // > 0: served by the shallow-depth kernel, that many activation rows per 128-byte line
};
struct TcI8Launch {
  SideView m_side;
  SideView n_side;
  DstView dst;
  Epilogue ep;
  int depth;
  int sm_count;
  int* status;
  bool allow_pair;   // permit the two-CTA (cta_group::2) variant
  void* mirrors[7];  // addresses in peers' buffers that correspond to dst.data; every destination store is repeated there
  int n_mirrors;
  // Address that corresponds to dst.data in an NVLink multicast mapping bound to every rank's copy of the destination
  // (this rank's included): when set, each piece of the destination is stored there once (multimem.st; the switch
  // delivers it to all copies) instead of to dst.data and the mirrors.  8-bit destinations with a 16-byte aligned base
  // and stride and a contiguous dimension that is a multiple of 16 only.
  void* multicast = nullptr;
  // Device array of 1 + n_mirrors tensor maps made by make_i8_store_map over dst.data and the mirrors, or null: with
  // them the copy engine writes each staged half tile to every copy (no store instruction crosses NVLink).
  const void* store_maps = nullptr;
  TcI8Info* info = nullptr;   // filled in when not null
  bool fuse_sums_m;  // if ep.zp_n != 0 and ep.sums_m == nullptr, let the kernel produce the m-side sums itself
  // Overrides of the tile-shape choice (tests and measurements): force_pair -1 = free, 0 = one-CTA tiles only,
  // 1 = two-CTA tiles when possible; force_block_n 0 = free, else the widest n tile of at most that many columns.
  int force_pair = -1;
  int force_block_n = 0;
  bool allow_shallow = true;   // permit the shallow-depth kernel (depth 32, 64 or 128, contiguous activation rows)
  // Optional step-end flag exchange done by the launch itself (see ruyb200_mul_async_mirrored_exchange).
  uint32_t* const* xchg_remote = nullptr;
  const uint32_t* xchg_local = nullptr;
  int n_xchg = 0;
  uint32_t xchg_value = 0;
  unsigned int* xchg_counter = nullptr;
  unsigned long long xchg_limit_ns = 0;
};
cudaError_t launch_tc_i8(const TcI8Launch& args, cudaStream_t stream);
// Encodes (on the host, 128 bytes at map_out) the tensor map the mirrored epilogue's copy-engine stores use for an
// 8-bit destination whose element (m, n) lives at base + m * stride_m + n.  False when base or stride_m is not a
// multiple of 16 bytes.
constexpr size_t kStoreMapBytes = 128;
bool make_i8_store_map(void* map_out, void* base, int size_n, int size_m, int64_t stride_m);
// True when the operands satisfy launch_tc_i8's requirements.
bool tc_i8_eligible(const SideView& m_side, const SideView& n_side);
// The shallow-depth variant (shallow_i8.cu); launch_tc_i8 hands eligible launches over to it.
bool shallow_i8_eligible(const TcI8Launch& args);
cudaError_t launch_shallow_i8(const TcI8Launch& args, cudaStream_t stream);

// Narrow muls (one side has at most kGemvMaxNarrow rows): one pass over the wide operand, no packing, no sums
// needed from the caller.  Both sides must be depth-contiguous; 8-bit x 8-bit or fp32.
constexpr int kGemvMaxNarrow = 8;
bool gemv_eligible(const SideView& m_side, const SideView& n_side, int depth, bool is_float);
// 8-bit muls with 2 to kGemvMmaMaxNarrow narrow rows on a wide operand of 1024 rows or more and a depth that is a
// multiple of 16 run in the MMA form of the narrow kernel (16 wide rows per CTA, register-level m16n8k32 MMAs), which
// also needs every row of both operands on a 16-byte boundary.
constexpr int kGemvMmaMaxNarrow = 16;
inline bool gemv_mma_shape(int narrow, long long wide, int depth) {
  return narrow >= 2 && narrow <= kGemvMmaMaxNarrow && wide >= 1024 && depth >= 16 && (depth & 15) == 0;
}
cudaError_t launch_gemv(const SideView& m_side, const SideView& n_side, const DstView& dst, const Epilogue& ep,
                        cudaStream_t stream);

// fp32 on the tensor core (3 x TF32 with short accumulation chains, see tc_f32.cu).  scratch_m / scratch_n receive
// the hi/lo split of each side: tc_f32_scratch_bytes(width, depth) bytes each, 256-byte aligned.
size_t tc_f32_scratch_bytes(int width, int depth);
cudaError_t launch_tc_f32(const SideView& m_side, const SideView& n_side, const DstView& dst, const Epilogue& ep, void* scratch_m,
                          void* scratch_n, int sm_count, int* status, cudaStream_t stream);

// fp32 kernels.
cudaError_t launch_sgemm(const SideView& m_side, const SideView& n_side, const DstView& dst,
                         const Epilogue& ep, cudaStream_t stream);

}  // namespace ruyb200
