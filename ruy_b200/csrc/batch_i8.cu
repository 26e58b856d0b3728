// Many small 8-bit muls in one persistent launch: what TrMul's "simple loop" (pack LHS, pack RHS, one
// kernel call, ruy/trmul.cc:339-356) does for one small mul, pipelined across thousands of them.
//
// Each work item is one whole mul whose dimensions all fit one tensor-core tile (<= 128 x 128 x 128).
// Every SM runs one persistent CTA that walks a static, size-balanced list of items through a ring of
// shared-memory slots:
//
//   * warps 0-5  : pack (ruy/pack.h:105-132).  Each warp owns one slot and one item at a time and never waits
//                  for its copies.  An operand whose rows are 16-byte aligned is fetched by ONE tensor-map
//                  copy (the plan holds a map per operand) that lands as 128-byte rows with the 128-byte
//                  swizzle, zero-filled past depth; any other operand is scattered by cp.async (8 or 16
//                  bytes each) into the unswizzled core-matrix layout.  The per-channel vectors and the
//                  cached zero-point sums ride along as bulk copies (or cp.async).  Six whole items are in
//                  flight per SM, which is what keeps enough bytes outstanding to use the HBM bandwidth.
//   * warps 6-7  : alternate items; one elected lane issues the item's tcgen05.mma kind::i8 (M=128, N<=128,
//                  K=32) from descriptors the pack warp left in the slot, into the item's accumulator: one
//                  or two of eight 64-column units of tensor memory, handed out by the plan as a ring, so
//                  up to eight items can sit between MMA and epilogue.
//   * warps 8-23 : epilogue, four groups of four warps; group g drains accumulator g.  Zero-point sums
//                  are taken from the packed tile, per-column terms are staged in shared memory, then
//                  tcgen05.ld, bias, zero-point terms, fixed-point multiplier, zero point, clamp
//                  (ruy/kernel.h:213-237) and store.  The destination's contiguous dimension sits on the
//                  TMEM lanes, so the 32 lanes of a warp write 32 consecutive elements.
//
// All mbarrier waits are bounded; a wait that gives up sets a status word and an abort flag and every
// role leaves its loop, so tensor memory is always released and the kernel always returns.
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "batch_i8.h"
#include "common.cuh"

namespace ruyb200 {

namespace {

constexpr int kSlots = 6;                          // one per pack warp
constexpr int kTileBytes = 16 * 1024;             // one operand: up to 128 rows x 128 bytes of depth
constexpr int kSlotBytes = 2 * kTileBytes;
constexpr int kAccUnits = kBatchAccUnits;        // 64-column accumulator units; an item takes one or two (assigned by the plan)
constexpr int kUnitCols = 64;
constexpr int kAccCols = 128;                     // most columns one item can use
constexpr int kTmemCols = 512;                     // allocation must be a power of two
constexpr int kPackWarps = kSlots;
constexpr int kEpiGroups = 4;
constexpr int kEpiWarps = 4 * kEpiGroups;         // each group covers the four TMEM lane quarters
constexpr int kMmaWarp = kPackWarps;                // warps 6 and 7 issue the MMAs of alternate items
constexpr int kMmaWarps = 2;
constexpr int kFirstEpiWarp = 8;                  // a multiple of 4, so that (warp % 4) is the lane quarter within a group
constexpr int kThreads = 32 * (kFirstEpiWarp + kEpiWarps);
constexpr int kSmemBytes = kSlots * kSlotBytes + 1024;
constexpr uint32_t kSpinLimit = 1u << 24;   // probes per wait before it gives up

// What the MMA warp needs for one item, prepared by the pack warp: descriptor halves and K steps of both tiles.
struct alignas(16) MmaCmd {
  uint32_t lo_m, hi_m, lo_n, hi_n;
  uint32_t kstep_m, kstep_n, idesc, nk_fence;   // nk_fence: K=32 steps (bits 0-7), BatchItem::acc (bits 8-13), bit 31 = a tile was written by cp.async
};

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
// One potentially blocking probe: returns early when the phase completes, otherwise after a short
// implementation-defined time.
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
// Bounded wait of a (converged) warp.  Every lane probes and nothing sleeps in between: measured on this
// kernel, a wake-up costs about 125 cycles this way, 200 with one probing lane plus a broadcast, 350 with a
// suspend-time hint and far more with nanosleep back-off, and every item passes through four such hand-offs.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  int ok = 0;
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) { ok = 1; break; }
    if ((i & 15) == 15 && *abort_flag) break;
  }
  return __all_sync(0xffffffffu, ok) != 0;
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
// AND-reduction over the 128 threads of one epilogue group (named barrier 1 + group).
__device__ __forceinline__ bool group_all(bool ok, int group) {
  uint32_t res;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, %2, 128, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(res)
      : "r"((uint32_t)ok), "r"(1 + group)
      : "memory");
  return res != 0;
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_tile(uint32_t smem_dst, const CUtensorMap* map, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %2}], [%3];"
      ::"r"(smem_dst), "l"(map), "r"(0), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// Untiled bulk copy global -> shared; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_dst), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Shared-memory matrix descriptor halves for the two tile layouts.  Swizzled rows of 128 bytes: 8-row groups
// 1024 bytes apart, swizzle mode 2 at bits 61..63, one K=32 step = 32 bytes.  Unswizzled core matrices (8 rows x
// 16 bytes): the two 16-byte depth chunks of an MMA 128 bytes apart (leading byte offset), 8-row groups `sbo`
// bytes apart, one K=32 step = 256 bytes.  Version 1 at bit 46 in both.
struct TileDesc {
  uint32_t lo, hi, kstep;
};
__device__ __forceinline__ TileDesc tile_desc(bool swizzled, uint32_t addr, uint32_t sbo) {
  TileDesc d;
  if (swizzled) {
    d.lo = ((addr & 0x3FFFF) >> 4) | (1u << 16);
    d.hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    d.kstep = 32 >> 4;
  } else {
    d.lo = ((addr & 0x3FFFF) >> 4) | ((128u >> 4) << 16);
    d.hi = (sbo >> 4) | (1u << 14);
    d.kstep = 256 >> 4;
  }
  return d;
}
__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint32_t lo_a, uint32_t hi_a, uint32_t lo_b, uint32_t hi_b, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "setp.ne.u32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %6};\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(lo_a), "r"(lo_b), "r"(idesc), "r"(accumulate), "r"(hi_a), "r"(hi_b)
      : "memory");
}

// cp.async of `bytes` (4, 8 or 16) of which only the first src_bytes are read; the rest is zero-filled.
template <int kBytes>
__device__ __forceinline__ void cp_async_zfill(uint32_t dst_smem, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(dst_smem), "l"(src), "n"(kBytes), "r"(src_bytes) : "memory");
}

// Issues the copies that pack one operand (width x depth, depth-contiguous rows `stride` bytes apart)
// into the core-matrix layout at `tile` (shared-memory address), starting at tile row `row_off` (a
// multiple of 8): 8 rows x 16 bytes per core matrix, consecutive 16-byte depth chunks 128 bytes apart,
// 8-row groups `sbo` bytes apart; depth is zero-filled up to kpad.  One warp; lane = (row within a group
// of 8, one of 4 interleaved units), so one warp instruction covers 8 rows x (32 or 64) contiguous bytes.
template <int kUnit>   // 8 or 16 bytes per copy
__device__ __forceinline__ void issue_pack(const uint8_t* __restrict__ src, int width, int depth, int stride, int kpad,
                                           uint32_t tile, int row_off, int lane) {
  const int units = kpad / kUnit;
  const uint32_t sbo = (uint32_t)(kpad >> 4) * 128;
  const int groups = (width + 7) >> 3;
  const int r8 = lane & 7;
  const int ul = lane >> 3;
  for (int g = 0; g < groups; g++) {
    const int r = g * 8 + r8;
    if (r >= width) continue;        // rows past the end stay as they are: their results are never stored
    const uint8_t* rowp = src + (int64_t)r * stride;
    const int tr = r + row_off;
    const uint32_t rowdst = tile + (uint32_t)(tr >> 3) * sbo + (uint32_t)(tr & 7) * 16;
    for (int u = ul; u < units; u += 4) {
      const int k0 = u * kUnit;
      int nbytes = depth - k0;
      nbytes = nbytes < 0 ? 0 : (nbytes > kUnit ? kUnit : nbytes);
      const uint32_t dst = kUnit == 16 ? rowdst + (uint32_t)u * 128 : rowdst + (uint32_t)(u >> 1) * 128 + (uint32_t)(u & 1) * 8;
      cp_async_zfill<kUnit>(dst, nbytes ? rowp + k0 : rowp, nbytes);
    }
  }
}

// Sum of the bytes of one packed tile row (kpad bytes, padding is zero).
__device__ __forceinline__ int32_t tile_row_sum(const uint8_t* tile, int tr, int kpad, bool is_signed) {
  const uint32_t sbo = (uint32_t)(kpad >> 4) * 128;
  const uint8_t* p = tile + (uint32_t)(tr >> 3) * sbo + (uint32_t)(tr & 7) * 16;
  int s = 0;
  for (int q = 0; q < (kpad >> 4); q++) {
    const uint4 v = *reinterpret_cast<const uint4*>(p + q * 128);
    if (is_signed) {
      s = __dp4a((int)v.x, 0x01010101, s);
      s = __dp4a((int)v.y, 0x01010101, s);
      s = __dp4a((int)v.z, 0x01010101, s);
      s = __dp4a((int)v.w, 0x01010101, s);
    } else {
      s = (int)__dp4a(v.x, 0x01010101u, (unsigned)s);
      s = (int)__dp4a(v.y, 0x01010101u, (unsigned)s);
      s = (int)__dp4a(v.z, 0x01010101u, (unsigned)s);
      s = (int)__dp4a(v.w, 0x01010101u, (unsigned)s);
    }
  }
  return s;
}

// The same for a swizzled tile: row tr is 128 bytes at tr * 128, its 16-byte chunk c stored at position c ^ (tr & 7).
__device__ __forceinline__ int32_t tile_row_sum_swizzled(const uint8_t* tile, int tr, int kpad, bool is_signed) {
  const uint8_t* p = tile + tr * 128;
  int s = 0;
  for (int q = 0; q < (kpad >> 4); q++) {
    const uint4 v = *reinterpret_cast<const uint4*>(p + ((q ^ (tr & 7)) << 4));
    if (is_signed) {
      s = __dp4a((int)v.x, 0x01010101, s);
      s = __dp4a((int)v.y, 0x01010101, s);
      s = __dp4a((int)v.z, 0x01010101, s);
      s = __dp4a((int)v.w, 0x01010101, s);
    } else {
      s = (int)__dp4a(v.x, 0x01010101u, (unsigned)s);
      s = (int)__dp4a(v.y, 0x01010101u, (unsigned)s);
      s = (int)__dp4a(v.z, 0x01010101u, (unsigned)s);
      s = (int)__dp4a(v.w, 0x01010101u, (unsigned)s);
    }
  }
  return s;
}

// Requantize with per-call constants hoisted: rnd = 2^(30-e) (64 bit), sh = 31-e.
__device__ __forceinline__ int32_t requant_ref_fast(int32_t x, int32_t mul, long long rnd, int sh) {
  const long long p = (long long)x * (long long)mul + rnd;
  return (int32_t)(p >> sh);
}

__global__ void __launch_bounds__(kThreads, 1)
batch_i8_kernel(const BatchItem* __restrict__ items, const CUtensorMap* __restrict__ maps, int num_items, int* status, int debug) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kSlots];     // packed data of a slot is in place
  __shared__ __align__(8) uint64_t empty_bar[kSlots];    // MMAs have read the slot and the epilogue has read its header
  __shared__ __align__(8) uint64_t acc_full_bar[kAccUnits];
  __shared__ __align__(8) uint64_t acc_empty_bar[kAccUnits];
  __shared__ __align__(16) BatchItem slot_item[kSlots];
  __shared__ MmaCmd slot_cmd[kSlots];
  __shared__ __align__(16) int32_t slot_vec[kSlots][4][128];   // the item's bias / multiplier / exponent vectors and cached m-side sums
  __shared__ __align__(16) NTerm n_terms[kEpiGroups][kAccCols];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  // the tensor maps of this CTA's first items start their way from HBM while the barriers and tensor memory are set up
  if (warp < kPackWarps && lane < 2 && (int)blockIdx.x + warp * (int)gridDim.x < num_items) {
    prefetch_map(maps + 2 * (size_t)(blockIdx.x + warp * gridDim.x) + lane);
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kSlots; s++) {
      mbar_init(&full_bar[s], 32 + 1);       // every pack lane's copies + the header
      mbar_init(&empty_bar[s], 1 + 4);       // the MMA commit + the four warps of the epilogue group
    }
    for (int b = 0; b < kAccUnits; b++) {
      mbar_init(&acc_full_bar[b], 1);
      mbar_init(&acc_empty_bar[b], 4);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;
  // This CTA's items are items[blockIdx.x + k * gridDim.x], k = 0 .. my_count-1, in that order.
  const int my_count = (num_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

  if (warp < kPackWarps) {
    // ---------------- pack: HBM -> shared memory, zero-point sums on the way ----------------
    // Pack warp w owns slot w and handles items k = w, w + kSlots, ...: kSlots items are being packed at any
    // time, each by its own warp, which is what keeps enough loads in flight.
    const int s = warp;
    uint32_t ph = 0;
    // The descriptor travels global -> register (one 16-byte piece in each of 8 lanes, fetched one item
    // ahead) -> the slot header in shared memory, from where every role reads the fields it needs.
    uint4 next_piece = make_uint4(0u, 0u, 0u, 0u);
    const bool piece_lane = lane < (int)(sizeof(BatchItem) / 16);
    if (s < my_count && piece_lane) next_piece = reinterpret_cast<const uint4*>(items + blockIdx.x + s * gridDim.x)[lane];
#ifdef RUYB200_DEBUG_CLOCKS
    long long dbg_wait = 0, dbg_work = 0, dbg_tma = 0, dbg_scatter = 0, dbg_t0 = clock64();
    int dbg_ntma = 0;
#endif
    for (int k = s; k < my_count; k += kSlots, ph ^= 1) {
      const uint4 piece = next_piece;
      if (k + kSlots < my_count && piece_lane) {
        next_piece = reinterpret_cast<const uint4*>(items + blockIdx.x + (k + kSlots) * gridDim.x)[lane];
      }
#ifdef RUYB200_DEBUG_CLOCKS
      long long dbg_a = clock64();
#endif
      if (!mbar_wait_warp(&empty_bar[s], ph ^ 1, abortp)) {
        if (lane == 0) { if (!*abortp) atomicCAS(status, 0, 1); *abortp = 1; }
        break;
      }
#ifdef RUYB200_DEBUG_CLOCKS
      long long dbg_b = clock64();
      dbg_wait += dbg_b - dbg_a;
#endif
      if (piece_lane) reinterpret_cast<uint4*>(&slot_item[s])[lane] = piece;
      __syncwarp();
      const BatchItem& item = slot_item[s];
      const int kpad = (item.depth + 31) & ~31;
      const uint32_t tile_m = smem_u32(smem + s * kSlotBytes);
      const uint32_t tile_n = tile_m + kTileBytes;
      const uint8_t* m_ptr = item.m_ptr;
      const uint8_t* n_ptr = item.n_ptr;
      const int size_m = item.size_m, size_n = item.size_n, depth = item.depth, stride_m = item.stride_m,
                stride_n = item.stride_n, m_off = item.m_off;
      const uint32_t flags = item.flags;
      const CUtensorMap* item_maps = maps + 2 * (size_t)(blockIdx.x + k * gridDim.x);
      uint32_t tx = 0;     // bytes the bulk / tensor copies will report on full_bar[s] (the same value in every lane)
#ifdef RUYB200_DEBUG_CLOCKS
      long long dbg_c = clock64();
#endif
      if (flags & kItemMTma) {
#ifdef RUYB200_DEBUG_KNOBS
        if (!(debug & 4))
#endif
        {
        if (lane == 0) tma_load_tile(tile_m + (uint32_t)m_off * 128, item_maps, &full_bar[s]);
        tx += 128u * (uint32_t)((size_m + 7) & ~7);
        }
      }
#ifdef RUYB200_DEBUG_KNOBS
      else if (debug & 16384) {
      }
#endif
      else if ((((uintptr_t)m_ptr | (uint32_t)stride_m) & 15) == 0) {
        issue_pack<16>(m_ptr, size_m, depth, stride_m, kpad, tile_m, m_off, lane);
      } else {
        issue_pack<8>(m_ptr, size_m, depth, stride_m, kpad, tile_m, m_off, lane);
      }
      if (flags & kItemNTma) {
#ifdef RUYB200_DEBUG_KNOBS
        if (!(debug & 4))
#endif
        {
        if (lane == 0) tma_load_tile(tile_n, item_maps + 1, &full_bar[s]);
        tx += 128u * (uint32_t)((size_n + 15) & ~15);
        }
      }
#ifdef RUYB200_DEBUG_KNOBS
      else if (debug & 16384) {
      }
#endif
      else if ((((uintptr_t)n_ptr | (uint32_t)stride_n) & 15) == 0) {
        issue_pack<16>(n_ptr, size_n, depth, stride_n, kpad, tile_n, 0, lane);
      } else {
        issue_pack<8>(n_ptr, size_n, depth, stride_n, kpad, tile_n, 0, lane);
      }
#ifdef RUYB200_DEBUG_CLOCKS
      if ((flags & (kItemMTma | kItemNTma)) == (kItemMTma | kItemNTma)) { dbg_tma += clock64() - dbg_c; dbg_ntma++; }
      else { dbg_scatter += clock64() - dbg_c; }
#endif
      // the next item's maps are on their way while this one's data moves
#ifdef RUYB200_DEBUG_KNOBS
      if (!(debug & 1))
#endif
      if (k + kSlots < my_count && lane < 2) prefetch_map(item_maps + 2 * (size_t)kSlots * gridDim.x + lane);
      // per-channel vectors (indexed along m or along n) and the cached m-side sums ride along
      const int nch = (flags & kItemChannelOnN) ? size_n : size_m;
      const int32_t* v0 = item.bias;
      const int32_t* v1 = item.mfp_pc;
      const int32_t* v2 = item.mexp_pc;
      const int32_t* v3 = item.sums_m;
#ifdef RUYB200_DEBUG_KNOBS
      if (debug & 2) {
      } else
#endif
      if (flags & kItemVecBulk) {
        const int32_t* vp = lane == 0 ? v0 : (lane == 1 ? v1 : (lane == 2 ? v2 : v3));
        const uint32_t vbytes = 4u * (uint32_t)(lane == 3 ? size_m : nch);
        if (lane < 4 && vp) bulk_load(smem_u32(&slot_vec[s][lane][0]), vp, vbytes, &full_bar[s]);
        tx += 4u * (uint32_t)nch * ((v0 ? 1u : 0u) + (v1 ? 1u : 0u) + (v2 ? 1u : 0u)) + (v3 ? 4u * (uint32_t)size_m : 0u);
      } else {
        if (v0) for (int i = lane; i < nch; i += 32) cp_async_zfill<4>(smem_u32(&slot_vec[s][0][i]), v0 + i, 4);
        if (v1) for (int i = lane; i < nch; i += 32) cp_async_zfill<4>(smem_u32(&slot_vec[s][1][i]), v1 + i, 4);
        if (v2) for (int i = lane; i < nch; i += 32) cp_async_zfill<4>(smem_u32(&slot_vec[s][2][i]), v2 + i, 4);
        if (v3) for (int i = lane; i < size_m; i += 32) cp_async_zfill<4>(smem_u32(&slot_vec[s][3][i]), v3 + i, 4);
      }
      // full_bar[s] completes when every lane's cp.async copies have landed (32 deferred arrivals), lane 0 has
      // arrived (which publishes the header written above) and the bulk / tensor copies have delivered `tx` bytes
      asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full_bar[s])) : "memory");
      if (lane == 0) {
        const uint32_t sbo = (uint32_t)(kpad >> 4) * 128;
        const TileDesc dm = tile_desc((flags & kItemMTma) != 0, tile_m, sbo);
        const TileDesc dn = tile_desc((flags & kItemNTma) != 0, tile_n, sbo);
        MmaCmd cmd;
        cmd.lo_m = dm.lo; cmd.hi_m = dm.hi; cmd.kstep_m = dm.kstep;
        cmd.lo_n = dn.lo; cmd.hi_n = dn.hi; cmd.kstep_n = dn.kstep;
        cmd.idesc = (2u << 4) | ((flags & kItemMSigned ? 1u : 0u) << 7) | ((flags & kItemNSigned ? 1u : 0u) << 10) |
                    ((uint32_t)(((size_n + 15) & ~15) >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        cmd.nk_fence = (uint32_t)(kpad >> 5) | ((item.acc & 0x3fu) << 8) | (((flags & (kItemMTma | kItemNTma)) != (kItemMTma | kItemNTma)) ? 0x80000000u : 0u);
        slot_cmd[s] = cmd;
      }
      __syncwarp();
      if (lane == 0) {
        if (tx) mbar_arrive_expect_tx(&full_bar[s], tx); else mbar_arrive(&full_bar[s]);
      }
#ifdef RUYB200_DEBUG_CLOCKS
      dbg_work += clock64() - dbg_b;
#endif
    }
#ifdef RUYB200_DEBUG_CLOCKS
    if (blockIdx.x == 0 && threadIdx.x == 0)
      printf("pack warp 0: total %lld cycles, waiting for its slot %lld, issuing copies %lld (operands: %lld in %d items by tensor map, %lld otherwise), items %d\n",
             clock64() - dbg_t0, dbg_wait, dbg_work, dbg_tma, dbg_ntma, dbg_scatter, (my_count + kSlots - 1) / kSlots);
#endif
  } else if (warp < kMmaWarp + kMmaWarps) {
    // ---------------- MMA issue: this warp takes items mw, mw + 2, ... ----------------
    const int mw = warp - kMmaWarp;
#ifdef RUYB200_DEBUG_CLOCKS
    long long dbg_acc = 0, dbg_full = 0, dbg_t0 = clock64();
#endif
    for (int it = mw; it < my_count; it += kMmaWarps) {
      const int s = it % kSlots;
      const uint32_t ph = (it / kSlots) & 1;
#ifdef RUYB200_DEBUG_CLOCKS
      long long dbg_a = clock64();
#endif
      // the packed data first (the slot also says which accumulator units the item takes), then the units
      bool ok = mbar_wait_warp(&full_bar[s], ph, abortp);
#ifdef RUYB200_DEBUG_CLOCKS
      long long dbg_b = clock64();
      dbg_full += dbg_b - dbg_a;
#endif
      uint4 c0 = make_uint4(0u, 0u, 0u, 0u), c1 = c0;
      int unit = 0;
      bool two = false;
      if (ok) {
        c0 = reinterpret_cast<const uint4*>(&slot_cmd[s])[0];   // lo_m, hi_m, lo_n, hi_n
        c1 = reinterpret_cast<const uint4*>(&slot_cmd[s])[1];   // kstep_m, kstep_n, idesc, nk_fence
        const uint32_t acc = (c1.w >> 8) & 0x3fu;
        unit = (int)(acc & 7u);
        two = (acc & 8u) != 0;
        ok = mbar_wait_warp(&acc_empty_bar[unit], ((acc >> 4) & 1u) ^ 1u, abortp);
        if (ok && two) ok = mbar_wait_warp(&acc_empty_bar[unit + 1], ((acc >> 5) & 1u) ^ 1u, abortp);
      }
#ifdef RUYB200_DEBUG_CLOCKS
      dbg_acc += clock64() - dbg_b;
#endif
      if (!ok) {
        if (lane == 0) { if (!*abortp) atomicCAS(status, 0, 2); *abortp = 1; }
        break;
      }
      // a tile filled by cp.async was written through the generic proxy; the tensor core reads through the async proxy
      if (c1.w & 0x80000000u) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + (uint32_t)(unit * kUnitCols);
      const int nk = (int)(c1.w & 0xffu);
      if (elect_one()) {
#ifdef RUYB200_DEBUG_KNOBS
        if (!(debug & 32))
#endif
        for (int k = 0; k < nk; k++) {
          mma_i8(tmem_d, c0.x + k * c1.x, c0.y, c0.z + k * c1.y, c0.w, c1.z, k != 0);
        }
#ifdef RUYB200_DEBUG_KNOBS
        if (debug & 4096) {
          mbar_arrive(&empty_bar[s]);
          mbar_arrive(&acc_full_bar[unit]);
          if (two) mbar_arrive(&acc_full_bar[unit + 1]);
        } else
#endif
        {
          mma_commit(&empty_bar[s]);
          mma_commit(&acc_full_bar[unit]);
          if (two) mma_commit(&acc_full_bar[unit + 1]);   // keeps the second unit's barrier phases in step with its use count
        }
      }
      __syncwarp();
    }
#ifdef RUYB200_DEBUG_CLOCKS
    if (blockIdx.x == 0 && lane == 0)
      printf("mma warp %d: total %lld cycles, waiting for an accumulator %lld, waiting for packed data %lld, items %d\n", mw,
             clock64() - dbg_t0, dbg_acc, dbg_full, my_count);
#endif
  } else if (warp >= kFirstEpiWarp) {
    // ---------------- epilogue: group g drains items g, g + 4, ... from whichever accumulator units they were given ----------------
    const int group = (warp - kFirstEpiWarp) / 4;
    const int quarter = warp % 4;          // TMEM lane quarter this warp may read
    const int gtid = (warp - kFirstEpiWarp) % 4 * 32 + lane;
    NTerm* nt = n_terms[group];
#ifdef RUYB200_DEBUG_CLOCKS
    long long dbg_wait = 0, dbg_stage = 0, dbg_work = 0, dbg_t0 = clock64();
#endif
    for (int it = group; it < my_count; it += kEpiGroups) {
      const int s = it % kSlots;
#ifdef RUYB200_DEBUG_CLOCKS
      long long dbg_a = clock64();
#endif
      // Only the group's first warp probes barriers; the group barrier below releases the others.  It waits for the
      // slot's data first, because the slot's header says which accumulator unit (and which of its phases) to wait for.
      bool ok = true;
      if (quarter == 0) {
        ok = mbar_wait_warp(&full_bar[s], (uint32_t)(it / kSlots) & 1u, abortp);
        if (ok) {
          const uint32_t a = slot_item[s].acc;
          ok = mbar_wait_warp(&acc_full_bar[a & 7u], (a >> 4) & 1u, abortp);
        }
      }
#ifdef RUYB200_DEBUG_CLOCKS
      long long dbg_b = clock64();
      dbg_wait += dbg_b - dbg_a;
#endif
      if (!ok && lane == 0) { if (!*abortp) atomicCAS(status, 0, 3); *abortp = 1; }
      // collective decision; also orders the previous item's reads of n_terms[] before this item's writes
      if (!group_all(ok, group)) break;
      tc_fence_after();
#ifdef RUYB200_DEBUG_KNOBS
      if (debug & 8192) {
        __syncwarp();
        const uint32_t a = slot_item[s].acc;
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&empty_bar[s]);
          mbar_arrive(&acc_empty_bar[a & 7u]);
          if (a & 8u) mbar_arrive(&acc_empty_bar[(a & 7u) + 1]);
        }
        continue;
      }
#endif
      const BatchItem& item = slot_item[s];   // valid until this group has arrived on empty_bar[s]
      const uint32_t acc = item.acc;
      const int unit = (int)(acc & 7u);
      const bool two_units = (acc & 8u) != 0;
      const bool ch_n = (item.flags & kItemChannelOnN) != 0;
      const bool x86 = (item.flags & kItemX86) != 0;
      const int dst_dtype = (int)((item.flags >> kItemDstShift) & 7u);
      const bool per_n = ch_n || item.zp_m != 0;   // some term varies along n
      const int kpad = (item.depth + 31) & ~31;
      const uint8_t* tile_m = smem + s * kSlotBytes;
      const uint8_t* tile_n = tile_m + kTileBytes;
      const int32_t* vbias = item.bias ? slot_vec[s][0] : nullptr;
      const int32_t* vmfp = item.mfp_pc ? slot_vec[s][1] : nullptr;
      const int32_t* vmexp = item.mexp_pc ? slot_vec[s][2] : nullptr;
      if (per_n) {
        const int n = gtid;
        NTerm t;
        t.add = item.zp_m * item.zp_n * item.depth;
        t.mul = item.mfp;
        t.exp = item.mexp;
        t.pad = 0;
        if (n < item.size_n) {
          // zero-point term of this destination column: the sum over depth of the n-side row, taken from the packed tile
          if (item.zp_m) {
            const bool sg = (item.flags & kItemNSigned) != 0;
            t.add -= item.zp_m * ((item.flags & kItemNTma) ? tile_row_sum_swizzled(tile_n, n, kpad, sg) : tile_row_sum(tile_n, n, kpad, sg));
          }
          if (ch_n) {
            if (vbias) t.add += vbias[n];
            if (vmfp) t.mul = vmfp[n];
            if (vmexp) t.exp = vmexp[n];
          }
        }
        nt[n] = t;
      }
      const int m = quarter * 32 + lane - item.m_off;     // tile row -> destination index along m
      const bool m_ok = m >= 0 && m < item.size_m;
      int32_t add_m = 0, mul_m = item.mfp, exp_m = item.mexp;
      if (m_ok) {
        if (item.zp_n) {
          const bool sg = (item.flags & kItemMSigned) != 0;
          const int tr = quarter * 32 + lane;
          const int32_t sum = item.sums_m ? slot_vec[s][3][m]
                                          : ((item.flags & kItemMTma) ? tile_row_sum_swizzled(tile_m, tr, kpad, sg)
                                                                      : tile_row_sum(tile_m, tr, kpad, sg));
          add_m -= item.zp_n * sum;
        }
        if (!ch_n) {
          if (vbias) add_m += vbias[m];
          if (vmfp) mul_m = vmfp[m];
          if (vmexp) exp_m = vmexp[m];
        }
      }
      const int size_m = item.size_m, size_n = item.size_n, m_off = item.m_off;
      const int32_t cmin = item.clamp_min, cmax = item.clamp_max, dzp = item.dst_zp;
      uint8_t* const dst_base = item.dst;
      const int dst_stride = item.dst_stride;
      if (per_n) group_all(true, group);   // n_terms[] staged (uniform over the group: per_n comes from the header)
      __syncwarp();                        // this warp is done with the slot's header, vectors and tiles
      if (lane == 0) mbar_arrive(&empty_bar[s]);
#ifdef RUYB200_DEBUG_CLOCKS
      long long dbg_c = clock64();
      dbg_stage += dbg_c - dbg_b;
#endif
      const bool quarter_used = quarter * 32 + 32 > m_off && quarter * 32 < m_off + size_m;
      if (quarter_used) {
        const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(unit * kUnitCols);
        const int esz = dst_dtype == RUYB200_I32 ? 4 : (dst_dtype == RUYB200_I16 ? 2 : 1);
        const int64_t step = (int64_t)dst_stride * esz;
        uint8_t* out = dst_base + (int64_t)m * esz;
        const bool fast = !per_n && !x86 && dst_dtype != RUYB200_I32;
        const int sh = 31 - exp_m;
        const long long rnd = 1ll << (sh - 1);
        // With every shift of the warp at least 32, the result is the high word of the product shifted on.
        // With every shift of the warp at least 32 and the per-row addend small enough that accumulator + addend
        // cannot wrap (|accumulator| < 2^23 for depth <= 128), the whole requantization is one 64-bit multiply-add
        // and one shift of its high word: acc * mul + (addend * mul + rounding [+ zero point << shift]).
        const bool high_word = fast && esz == 1 && __all_sync(0xffffffffu, sh >= 32 && add_m > -(1 << 30) && add_m < (1 << 30));
        const int sh_hi = sh - 32;
        const bool fold_zp = __all_sync(0xffffffffu, sh <= 50) && dzp >= -256 && dzp <= 255;
        const long long c64 = (long long)add_m * (long long)mul_m + rnd + (fold_zp ? (long long)dzp * (1ll << (sh & 63)) : 0ll);
        const int32_t dzp_late = fold_zp ? 0 : dzp;
        // 16 columns: all values first (branch-free, so the sixteen dependency chains interleave), then the stores
        auto process = [&](uint32_t (&rr)[16], int c) {   // results replace the accumulators in rr[]
          const int lim = size_n - c;
          if (high_word) {
#pragma unroll
            for (int q = 0; q < 16; q++) {
              const long long p = (long long)(int32_t)rr[q] * (long long)mul_m + c64;
              rr[q] = (uint32_t)max(min(((int32_t)(p >> 32) >> sh_hi) + dzp_late, cmax), cmin);
            }
          } else if (fast) {
#pragma unroll
            for (int q = 0; q < 16; q++) {
              const int32_t x = requant_ref_fast((int32_t)(rr[q] + (uint32_t)add_m), mul_m, rnd, sh);
              rr[q] = (uint32_t)max(min(x + dzp, cmax), cmin);
            }
          } else {
#pragma unroll
            for (int q = 0; q < 16; q++) {
              int32_t x = (int32_t)(rr[q] + (uint32_t)add_m);
              int32_t mul = mul_m;
              int e = exp_m;
              if (per_n) {
                const NTerm t = nt[(c + q) & (kAccCols - 1)];
                x = (int32_t)((uint32_t)x + (uint32_t)t.add);
                if (ch_n) { mul = t.mul; e = t.exp; }
              }
              if (dst_dtype != RUYB200_I32) {
                x = x86 ? requant_x86(x, mul, e) : requant_reference(x, mul, e);
                x = (int32_t)((uint32_t)x + (uint32_t)dzp);
                x = max(min(x, cmax), cmin);
              } else {
                x = (int32_t)((uint32_t)x + (uint32_t)dzp);
              }
              rr[q] = (uint32_t)x;
            }
          }
          uint8_t* o = out + (int64_t)c * step;
#ifdef RUYB200_DEBUG_KNOBS
          if (debug & 16) {
            uint32_t acc = 0;
#pragma unroll
            for (int q = 0; q < 16; q++) acc ^= rr[q];
            if (acc == 0x12345678u) o[0] = 1;
          } else
#endif
          if (esz == 1) {
            if (lim >= 16) {
#pragma unroll
              for (int q = 0; q < 16; q++) o[q * step] = (uint8_t)rr[q];
            } else {
#pragma unroll
              for (int q = 0; q < 16; q++) if (q < lim) o[q * step] = (uint8_t)rr[q];
            }
          } else if (esz == 2) {
#pragma unroll
            for (int q = 0; q < 16; q++) if (q < lim) *reinterpret_cast<int16_t*>(o + q * step) = (int16_t)rr[q];
          } else {
#pragma unroll
            for (int q = 0; q < 16; q++) if (q < lim) *reinterpret_cast<int32_t*>(o + q * step) = (int32_t)rr[q];
          }
        };
        // two register buffers: the load of the next 16 columns is in flight while 16 are processed
        uint32_t ra[16], rb[16];
#ifdef RUYB200_DEBUG_KNOBS
        if (!(debug & 64))
#endif
        tmem_ld_16(taddr, ra);
#ifdef RUYB200_DEBUG_KNOBS
        if (debug & 8) {
          tmem_ld_wait();
        } else
#endif
        for (int c = 0; c < size_n; c += 32) {
          tmem_ld_wait();
          if (c + 16 < size_n) tmem_ld_16(taddr + c + 16, rb);
          if (m_ok) process(ra, c);
          if (c + 16 < size_n) {
            tmem_ld_wait();
            if (c + 32 < size_n) tmem_ld_16(taddr + c + 32, ra);
            if (m_ok) process(rb, c + 16);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&acc_empty_bar[unit]);
        if (two_units) mbar_arrive(&acc_empty_bar[unit + 1]);
      }
#ifdef RUYB200_DEBUG_CLOCKS
      dbg_work += clock64() - dbg_c;
#endif
    }
#ifdef RUYB200_DEBUG_CLOCKS
    if (blockIdx.x == 0 && lane == 0 && group == 0)
      printf("epilogue group 0 quarter %d: total %lld cycles, waiting for a tile %lld, staging %lld, working %lld\n", quarter,
             clock64() - dbg_t0, dbg_wait, dbg_stage, dbg_work);
#endif
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols)
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

cudaError_t launch_batch_i8(const BatchItem* items, const CUtensorMap* maps, int num_items, int grid, int* status,
                            cudaStream_t stream) {
  if (num_items <= 0) return cudaSuccess;
  // the opt-in to more than 48 KB of dynamic shared memory is per device; contexts on several threads may get here together
  static std::mutex mu;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= 64 || !attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(batch_i8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < 64) attr_set[dev] = true;
    }
  }
  int debug = 0;
#ifdef RUYB200_DEBUG_KNOBS
  if (getenv("RUYB200_DEBUG")) debug = atoi(getenv("RUYB200_DEBUG"));
#endif
  batch_i8_kernel<<<grid, kThreads, kSmemBytes, stream>>>(items, maps, num_items, status, debug);
  return cudaGetLastError();
}

}  // namespace ruyb200
