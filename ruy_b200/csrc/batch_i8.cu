// Many small 8-bit muls in one persistent launch: what TrMul's "simple loop" (pack LHS, pack RHS, one
// kernel call, ruy/trmul.cc:339-356) does for one small mul, pipelined across thousands of them.
//
// Each work item is one whole mul whose dimensions all fit one tensor-core tile (<= 128 x 128 x 128).
// Every SM runs one persistent CTA that walks a static, size-balanced list of items through a ring of
// shared-memory slots:
//
//   * warps 0-3  : pack.  Read both operands from HBM (8-byte units, several in flight per lane) and
//                  write them into the slot in the tensor core's depth-major core-matrix layout,
//                  zero-padding depth to a multiple of 32 and accumulating the zero-point sums of the
//                  rows they touch (ruy/pack.h:105-132) on the way.  Runs up to kSlots items ahead, which
//                  is what keeps enough bytes in flight to use the HBM bandwidth.
//   * warp 4     : one elected lane issues the item's tcgen05.mma kind::i8 (M=128, N<=128, K=32) into one
//                  of four tensor-memory accumulators.
//   * warps 5-12 : epilogue.  Stage the per-column terms in shared memory, read the accumulators
//                  (tcgen05.ld), apply bias, zero-point terms, fixed-point multiplier, zero point, clamp
//                  (ruy/kernel.h:213-237) and store.  The destination's contiguous dimension sits on the
//                  TMEM lanes, so the 32 lanes of a warp write 32 consecutive elements.
//
// All mbarrier waits are bounded; a wait that gives up sets a status word and an abort flag and every
// role leaves its loop, so tensor memory is always released and the kernel always returns.
#include <cuda_runtime.h>

#include <cstring>

#include "batch_i8.h"
#include "common.cuh"

namespace ruyb200 {

namespace {

constexpr int kSlots = 6;
constexpr int kTileBytes = 16 * 1024;             // one operand: up to 128 rows x 128 bytes of depth
constexpr int kSlotBytes = 2 * kTileBytes;
constexpr int kAccBuffers = 4;
constexpr int kAccCols = 128;
constexpr int kPackWarps = 4;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 32 * (kPackWarps + 1 + kEpiWarps);
constexpr int kSmemBytes = kSlots * kSlotBytes + 1024;
constexpr uint32_t kSpinLimit = 4u << 20;

struct NTerm {
  int32_t add;
  int32_t mul;
  int32_t exp;
  int32_t pad;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait by one lane, result broadcast to the (converged) warp.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) {
    ok = 0;
    for (uint32_t i = 0; i < kSpinLimit; i++) {
      if (mbar_try_wait(bar, parity)) { ok = 1; break; }
      if (i >= 64) {
        if (*abort_flag) break;
        __nanosleep(64);
      }
    }
  }
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// AND-reduction over the epilogue threads (named barrier 1).
__device__ __forceinline__ bool epilogue_all(bool ok) {
  uint32_t res;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(res)
      : "r"((uint32_t)ok), "n"(32 * kEpiWarps)
      : "memory");
  return res != 0;
}
// AND-reduction over the pack threads (named barrier 2); doubles as their per-item barrier.
__device__ __forceinline__ bool pack_all(bool ok) {
  uint32_t res;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 2, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(res)
      : "r"((uint32_t)ok), "n"(32 * kPackWarps)
      : "memory");
  return res != 0;
}

// One K=32 MMA on core-matrix (no swizzle) depth-major tiles: 8 rows x 16 bytes per core matrix, the two
// 16-byte depth chunks of an MMA 128 bytes apart (leading byte offset), 8-row groups `sbo` bytes apart.
__device__ __forceinline__ void mma_i8_nosw(uint32_t tmem_d, uint32_t addr_a, uint32_t addr_b, uint32_t sbo, uint32_t idesc,
                                            uint32_t accumulate) {
  const uint32_t hi = (sbo >> 4) | (1u << 14);   // stride byte offset at bits 32..45, descriptor version 1 at bit 46
  const uint32_t lo_a = ((addr_a & 0x3FFFF) >> 4) | ((128u >> 4) << 16);
  const uint32_t lo_b = ((addr_b & 0x3FFFF) >> 4) | ((128u >> 4) << 16);
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.u32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(lo_a), "r"(lo_b), "r"(idesc), "r"(accumulate), "r"(hi)
      : "memory");
}

// Packs one operand (width x depth, depth-contiguous rows `stride` bytes apart) into the core-matrix
// layout at `tile`, zero-padding depth up to kpad, and adds each row's byte sum into sums[] if wanted.
// Lanes map to (row within a group of 8, 8-byte unit) so shared-memory stores are conflict-free.
__device__ __forceinline__ void pack_operand(const uint8_t* __restrict__ src, int width, int depth, int stride, int kpad,
                                             bool is_signed, uint8_t* tile, int32_t* sums, int ptid) {
  const int units = kpad / 8;                  // 8-byte units per row, padding included
  const uint32_t sbo = (uint32_t)(kpad / 16) * 128;
  const int groups = (width + 7) / 8;
  const int total = groups * 8 * units;        // (group, unit, row in group) with the row fastest
  constexpr int kBatch = 4;
  for (int base = ptid; base < total; base += 128 * kBatch) {
    uint2 v[kBatch];
    int row[kBatch], unit[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; b++) {
      const int e = base + b * 128;
      v[b] = make_uint2(0u, 0u);
      row[b] = -1;
      if (e < total) {
        const int r8 = e & 7;
        const int u = (e >> 3) % units;
        const int g = (e >> 3) / units;
        const int r = g * 8 + r8;
        row[b] = r;
        unit[b] = u;
        const int k0 = u * 8;
        if (r < width && k0 < depth) {
          const uint8_t* p = src + (int64_t)r * stride + k0;
          if (k0 + 8 <= depth) {
            v[b] = *reinterpret_cast<const uint2*>(p);
          } else {
            uint32_t w[2] = {0u, 0u};
            for (int t = 0; t < depth - k0; t++) w[t >> 2] |= (uint32_t)p[t] << (8 * (t & 3));
            v[b] = make_uint2(w[0], w[1]);
          }
        }
      }
    }
#pragma unroll
    for (int b = 0; b < kBatch; b++) {
      if (row[b] < 0) continue;
      const int r = row[b], u = unit[b];
      uint8_t* dst = tile + (uint32_t)(r >> 3) * sbo + (uint32_t)(u >> 1) * 128 + (uint32_t)(r & 7) * 16 + (uint32_t)(u & 1) * 8;
      *reinterpret_cast<uint2*>(dst) = v[b];
      if (sums && r < width) {
        int s;
        if (is_signed) {
          s = __dp4a((int)v[b].x, 0x01010101, 0);
          s = __dp4a((int)v[b].y, 0x01010101, s);
        } else {
          s = (int)__dp4a(v[b].x, 0x01010101u, 0u);
          s = (int)__dp4a(v[b].y, 0x01010101u, (unsigned)s);
        }
        if (s) atomicAdd(&sums[r], s);
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
batch_i8_kernel(const BatchItem* __restrict__ items, const int32_t* __restrict__ order, int num_items, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kSlots];     // packed data of a slot is in place
  __shared__ __align__(8) uint64_t empty_bar[kSlots];    // MMAs have read the slot and the epilogue has read its header
  __shared__ __align__(8) uint64_t acc_full_bar[kAccBuffers];
  __shared__ __align__(8) uint64_t acc_empty_bar[kAccBuffers];
  __shared__ __align__(16) BatchItem slot_item[kSlots];
  __shared__ int32_t slot_sums[kSlots][256];             // [0,128): m side rows, [128,256): n side rows
  __shared__ __align__(16) NTerm n_terms[kAccBuffers][kAccCols];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; s++) {
      mbar_init(&full_bar[s], 32 * kPackWarps);
      mbar_init(&empty_bar[s], 1 + kEpiWarps);
    }
    for (int b = 0; b < kAccBuffers; b++) {
      mbar_init(&acc_full_bar[b], 1);
      mbar_init(&acc_empty_bar[b], kEpiWarps);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kPackWarps) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kAccBuffers * kAccCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;
  const int my_count = (num_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;   // items of this CTA

  if (warp < kPackWarps) {
    // ---------------- pack: HBM -> shared memory, zero-point sums on the way ----------------
    const int ptid = threadIdx.x;
    uint32_t s = 0, ph = 0;
    for (int it = 0; it < my_count; it++) {
      bool ok = mbar_wait_warp(&empty_bar[s], ph ^ 1, abortp);
      if (!ok && lane == 0) { if (!*abortp) atomicCAS(status, 0, 1); *abortp = 1; }
      const int idx = order[blockIdx.x + it * gridDim.x];
      const BatchItem* gi = items + idx;
      if (ok) {
        // header: the item descriptor travels with the slot (8 lanes x 16 bytes)
        if (ptid < (int)(sizeof(BatchItem) / 16)) {
          reinterpret_cast<uint4*>(&slot_item[s])[ptid] = reinterpret_cast<const uint4*>(gi)[ptid];
        }
        slot_sums[s][ptid] = 0;
        slot_sums[s][ptid + 128] = 0;
      }
      // collective continue/abort decision; also: the sums are zero before anybody adds to them
      if (!pack_all(ok)) break;
      const BatchItem item = *gi;
      const int kpad = (item.depth + 31) & ~31;
      uint8_t* tile_m = smem + s * kSlotBytes;
      uint8_t* tile_n = tile_m + kTileBytes;
      pack_operand(item.m_ptr, item.size_m, item.depth, item.stride_m, kpad, (item.flags & kItemMSigned) != 0, tile_m,
                   item.zp_n ? &slot_sums[s][0] : nullptr, ptid);
      pack_operand(item.n_ptr, item.size_n, item.depth, item.stride_n, kpad, (item.flags & kItemNSigned) != 0, tile_n,
                   item.zp_m ? &slot_sums[s][128] : nullptr, ptid);
      // make this thread's generic-proxy writes visible to the tensor core's async-proxy reads, then signal
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(&full_bar[s]);
      if (++s == kSlots) { s = 0; ph ^= 1; }
    }
  } else if (warp == kPackWarps) {
    // ---------------- MMA issue ----------------
    uint32_t s = 0, ph = 0;
    for (int it = 0; it < my_count; it++) {
      const int buf = it % kAccBuffers;
      const uint32_t aph = (it / kAccBuffers) & 1;
      bool ok = mbar_wait_warp(&acc_empty_bar[buf], aph ^ 1, abortp);
      ok = ok && mbar_wait_warp(&full_bar[s], ph, abortp);
      if (!ok) {
        if (lane == 0) { if (!*abortp) atomicCAS(status, 0, 2); *abortp = 1; }
        break;
      }
      tc_fence_after();
      const int depth = slot_item[s].depth;
      const int size_n = slot_item[s].size_n;
      const uint32_t flags = slot_item[s].flags;
      const int kpad = (depth + 31) & ~31;
      const int nmma = (size_n + 15) & ~15;
      const uint32_t idesc = (2u << 4) | ((flags & kItemMSigned ? 1u : 0u) << 7) | ((flags & kItemNSigned ? 1u : 0u) << 10) |
                             ((uint32_t)(nmma >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t sbo = (uint32_t)(kpad / 16) * 128;
      const uint32_t addr_m = smem_u32(smem + s * kSlotBytes);
      const uint32_t addr_n = addr_m + kTileBytes;
      const uint32_t tmem_d = tmem_base + (uint32_t)(buf * kAccCols);
      if (elect_one()) {
        for (int k = 0; k < kpad / 32; k++) {
          mma_i8_nosw(tmem_d, addr_m + k * 256, addr_n + k * 256, sbo, idesc, k != 0);
        }
        mma_commit(&empty_bar[s]);
        mma_commit(&acc_full_bar[buf]);
      }
      __syncwarp();
      if (++s == kSlots) { s = 0; ph ^= 1; }
    }
  } else {
    // ---------------- epilogue ----------------
    const int ew = warp - (kPackWarps + 1);
    const int quarter = warp % 4;          // TMEM lane quarter this warp may read
    const int chunk_parity = ew / 4;       // the two warps of a quarter alternate 16-column chunks
    const int etid = threadIdx.x - 32 * (kPackWarps + 1);
    uint32_t s = 0;
    bool ok = true;
    for (int it = 0; it < my_count && ok; it++) {
      const int buf = it % kAccBuffers;
      const uint32_t aph = (it / kAccBuffers) & 1;
      if (!mbar_wait_warp(&acc_full_bar[buf], aph, abortp)) {
        if (lane == 0) { if (!*abortp) atomicCAS(status, 0, 3); *abortp = 1; }
        ok = false;
      }
      // collective decision; also orders the previous item's reads of n_terms[] before this item's writes
      ok = epilogue_all(ok);
      if (!ok) break;
      tc_fence_after();
      const BatchItem item = slot_item[s];
      const bool ch_n = (item.flags & kItemChannelOnN) != 0;
      const bool x86 = (item.flags & kItemX86) != 0;
      const int dst_dtype = (int)((item.flags >> kItemDstShift) & 7u);
      const int32_t zz = item.zp_m * item.zp_n * item.depth;
      NTerm* nt = n_terms[buf];
      if (etid < kAccCols) {
        const int n = etid;
        NTerm t;
        t.add = zz;
        t.mul = item.mfp;
        t.exp = item.mexp;
        t.pad = 0;
        if (n < item.size_n) {
          if (item.zp_m) t.add -= item.zp_m * slot_sums[s][128 + n];
          if (ch_n) {
            if (item.bias) t.add += item.bias[n];
            if (item.mfp_pc) t.mul = item.mfp_pc[n];
            if (item.mexp_pc) t.exp = item.mexp_pc[n];
          }
        }
        nt[n] = t;
      }
      const int m = quarter * 32 + lane;
      const bool m_ok = m < item.size_m;
      int32_t add_m = 0, mul_m = item.mfp, exp_m = item.mexp;
      if (m_ok) {
        if (item.zp_n) add_m -= item.zp_n * slot_sums[s][m];
        if (!ch_n) {
          if (item.bias) add_m += item.bias[m];
          if (item.mfp_pc) mul_m = item.mfp_pc[m];
          if (item.mexp_pc) exp_m = item.mexp_pc[m];
        }
      }
      epilogue_all(true);                  // n_terms[] staged, slot header and sums consumed by everybody
      if (lane == 0) mbar_arrive(&empty_bar[s]);
      const bool quarter_used = quarter * 32 < item.size_m;
      if (quarter_used) {
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * kAccCols);
        const int esz = dst_dtype == RUYB200_I32 ? 4 : (dst_dtype == RUYB200_I16 ? 2 : 1);
        for (int c = chunk_parity * 16; c < item.size_n; c += 32) {
          uint32_t r[16];
          tmem_ld_16(taddr + c, r);
          tmem_ld_wait();
          if (m_ok) {
#pragma unroll
            for (int q = 0; q < 16; q++) {
              const int n = c + q;
              if (n < item.size_n) {
                const NTerm t = nt[n];
                int32_t x = (int32_t)(r[q] + (uint32_t)t.add + (uint32_t)add_m);
                if (dst_dtype != RUYB200_I32) {
                  const int32_t mul = ch_n ? t.mul : mul_m;
                  const int e = ch_n ? t.exp : exp_m;
                  x = x86 ? requant_x86(x, mul, e) : requant_reference(x, mul, e);
                  x = (int32_t)((uint32_t)x + (uint32_t)item.dst_zp);
                  x = max(min(x, item.clamp_max), item.clamp_min);
                } else {
                  x = (int32_t)((uint32_t)x + (uint32_t)item.dst_zp);
                }
                uint8_t* p = item.dst + ((int64_t)n * item.dst_stride + m) * esz;
                if (esz == 1) *p = (uint8_t)x;
                else if (esz == 2) *reinterpret_cast<int16_t*>(p) = (int16_t)x;
                else *reinterpret_cast<int32_t*>(p) = x;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty_bar[buf]);
      if (++s == kSlots) s = 0;
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kPackWarps) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kAccBuffers * kAccCols)
                 : "memory");
  }
}

}  // namespace

bool batch_i8_fits(const SideView& m_side, const SideView& n_side, int depth) {
  const SideView* sides[2] = {&m_side, &n_side};
  for (const SideView* s : sides) {
    if (s->dtype != RUYB200_I8 && s->dtype != RUYB200_U8) return false;
    if (s->stride_k != 1 || s->width < 1 || s->width > 128) return false;
    if (((uintptr_t)s->data & 7) != 0 || (s->stride_w & 7) != 0 || s->stride_w > (1 << 30)) return false;
  }
  return depth >= 1 && depth <= 128;
}

cudaError_t launch_batch_i8(const BatchItem* items, const int32_t* order, int num_items, int sm_count, int* status,
                            cudaStream_t stream) {
  if (num_items <= 0) return cudaSuccess;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(batch_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  const int grid = num_items < sm_count ? num_items : sm_count;
  batch_i8_kernel<<<grid, kThreads, kSmemBytes, stream>>>(items, order, num_items, status);
  return cudaGetLastError();
}

}  // namespace ruyb200
