// The 8-bit tensor-core GEMM: ruy's Kernel8bit* (ruy/kernel_avx512.cc:55-626) and the packing
// that feeds it (ruy/pack_avx512.cc:840-1090), as one persistent warp-specialised sm_100a kernel.
//
//   * warp 0   : TMA producer.  Loads 128-byte-deep slabs of both operands straight from their
//                depth-contiguous source layout into 128B-swizzled shared-memory tiles
//                (cp.async.bulk.tensor, no cluster multicast); out-of-range rows and depth are
//                zero-filled by the TMA unit, which is what ruy's packing pads with.
//   * warp 1   : issues tcgen05.mma kind::i8 (M=128, N<=256, K=32 per instruction), int32
//                accumulators in tensor memory, two accumulator buffers so the epilogue of one
//                tile overlaps the main loop of the next.
//   * warps 2-9: epilogue, two groups of four warps that take tiles in turn.  Per tile the per-channel terms (bias, zero-point corrections,
//                multiplier, exponent) are staged once in shared memory; then tcgen05.ld brings
//                32 accumulator columns at a time into registers, the fixed-point multiplier,
//                destination zero point and clamp are applied (ruy/kernel.h:213-237), and the
//                results are narrowed and stored.  The destination's contiguous dimension is
//                mapped to the MMA N dimension, so each thread owns a run of consecutive
//                destination elements and writes them with 16-byte stores.
//
// Every wait on an mbarrier is bounded; a wait that gives up records a code in *status,
// raises a CTA-wide abort flag, and every role leaves its loops so that tensor memory is
// released and the kernel returns.
#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "batch_i8.h"
#include "common.cuh"

namespace ruyb200 {

namespace {

constexpr int kMaxDevices = 64;
constexpr int kBlockM = 128;          // TMEM lanes per tile
constexpr int kMaxBlockN = 256;       // accumulator columns per tile
constexpr int kBlockKBytes = 128;     // one swizzle atom of depth per stage
constexpr int kStages = 4;
constexpr int kABytes = kBlockM * kBlockKBytes;        // 16 KiB
constexpr int kBBytes = kMaxBlockN * kBlockKBytes;     // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;         // 48 KiB
// staging area used when the destination is mirrored into peers' memory: 128 rows x 128 bytes, pitch 144
constexpr int kMirrorPitch = 144;
// ... or, when the copy engine writes the tile out (tensor-map stores), 128 rows x 128 bytes in the 128-byte swizzle
// pattern (the same area: the kernel's static shared memory leaves no room for a second buffer)
constexpr int kMirrorStagingBytes = 128 * kMirrorPitch;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + kMirrorStagingBytes;  // + alignment slack
// two-CTA variant: each CTA stages 128 rows of each operand per stage
constexpr int kPairStages = 6;
constexpr int kPairStageBytes = kABytes + 128 * kBlockKBytes;   // 32 KiB
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + kMirrorStagingBytes;
constexpr int kEpilogueWarps = 8;
constexpr int kEpilogueGroups = kEpilogueWarps / 4;   // a group covers the four TMEM lane quarters and drains whole tiles
constexpr int kThreads = 64 + 32 * kEpilogueWarps;   // producer warp + MMA warp + epilogue warps
constexpr int kTmemCols = 512;
constexpr int kMaxAccBufs = 8;        // narrow tiles leave room for more accumulators, which hides the epilogue's latency
constexpr uint32_t kSpinFast = 2048;
constexpr uint32_t kSpinLimit = 4u << 20;  // with 100 ns sleeps: well under a second

enum StatusCode { kOk = 0, kTimeoutProducer = 1, kTimeoutMma = 2, kTimeoutEpilogue = 3 };

struct KernelArgs {
  DstView dst;
  Epilogue ep;
  int size_m;      // width of the m side (TMEM lanes)
  int size_n;      // width of the n side (TMEM columns)
  int depth;
  int block_n;     // multiple of 16, <= 256
  int tiles_m;
  int tiles_n;
  uint32_t idesc;
  int acc_bufs;    // accumulator buffers in tensor memory: 2, 4 or 8 (512 columns / columns per tile, as a power of two)
  int acc_shift;   // log2(acc_bufs)
  int epi_groups;  // 1: all eight epilogue warps drain each tile together; 2: two groups of four take tiles in turn
  int sums_col;    // >= 0: accumulator column that receives sum_k of the m-side row (an all-ones row of the n operand); -1: none
  int mma_n;       // N of the MMA: block_n, plus 16 when the sums column is appended
  int* status;
  void* mirror[7]; // peers' copies of the destination: same layout, every store is repeated there
  int n_mirror;
  void* multicast; // not null: the destination's address in a multicast mapping over every rank's copy; stores go there only
  // not null: 1 + n_mirror tensor maps in device memory over the destination and its mirrors (uint8, 128 x 128 boxes,
  // 128-byte swizzle): staged half tiles are written out by the copy engine instead of by store instructions
  const CUtensorMap* store_maps;
  int row_pitch;   // bytes per tile row in shared memory = width of the swizzle pattern: 128, or 64 / 32 for depth <= 64 / 32
  uint32_t desc_hi; // high word of the shared-memory matrix descriptors for that pattern
  int pack_clamps; // 8-bit destination: 1 = clamp range inside int16, values are clamped two at a time while being narrowed; 2 / 3 = the clamp is all of uint8 / int8 and the saturating narrowing applies it; 0 = each value is clamped first
  uint32_t clamp_lo2, clamp_hi2;   // the clamp bounds replicated in both 16-bit halves
  int tight_wait;  // shallow main loops: the epilogue probes its barrier without backing off
  int mirror_wide; // every destination base and the destination stride are multiples of 16 bytes
  int debug;       // profiling knobs (0 in production): 1 = epilogue skips its math and stores, 2 = producer skips the loads
  // Step-end flag exchange folded into this launch (mirrored destinations): the CTA that finishes last raises
  // xchg_remote[i] (one word per rank, in that rank's memory) to xchg_value and then waits, for at most
  // xchg_limit_ns, until xchg_local[i] (this rank's words) have all reached it.  n_xchg == 0: no exchange.
  uint32_t* const* xchg_remote;
  const uint32_t* xchg_local;
  int n_xchg;
  uint32_t xchg_value;
  unsigned int* xchg_counter;   // CTAs that have finished; zero between launches
  unsigned long long xchg_limit_ns;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
// Tensor-map store of one staged 128 x 128-byte tile: shared memory -> global (this GPU's or a peer's), part of the
// calling thread's current bulk group.  Rows and columns outside the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(map), "r"(x), "r"(y), "r"(smem_u32(smem_src))
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// until none of this thread's bulk groups is still reading its shared-memory source
__device__ __forceinline__ void bulk_wait_read_0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// until all of this thread's bulk groups have completed their writes
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

// A 16-byte store to a multicast address: NVSwitch writes it into the memory of every GPU bound to the mapping.
__device__ __forceinline__ void multimem_st_16(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(p), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
               : "memory");
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

// Non-blocking probe (try_wait may suspend the thread for a while before answering).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
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

// Bounded wait for the thread that feeds the tensor core: polls tightly (it is alone, and its
// latency is on the critical path).  Returns false if it gave up or if another role already raised
// the abort flag.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i >= kSpinFast) {
      if (*abort_flag) return false;
      __nanosleep(100);
    }
  }
  return false;
}

// Bounded wait that backs off almost immediately.  Every poll of an mbarrier is a shared-memory
// access that competes with the tensor core's operand fetches, so roles that wait for a long time
// (the producer on a free stage, the epilogue on a finished tile) sleep between polls.
__device__ __forceinline__ bool mbar_wait_relaxed(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i >= 4) {
      if ((i & 63) == 0 && *abort_flag) return false;
      __nanosleep(i < 64 ? 40 : 200);
    }
  }
  return false;
}

// The same for a whole warp: lane 0 polls, the result is broadcast.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait_relaxed(bar, parity, abort_flag) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}

// Bounded wait with every lane probing and no sleep: the shortest wake-up (about 125 cycles against several
// hundred with back-off).  Used by the epilogue when tiles are shallow, where every tile's hand-offs are exposed.
__device__ __forceinline__ bool mbar_wait_warp_tight(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  int ok = 0;
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) { ok = 1; break; }
    if ((i & 15) == 15 && *abort_flag) break;
  }
  return __all_sync(0xffffffffu, ok) != 0;
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptors describe a depth-contiguous tile stored as rows of 128 bytes with the
// 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset); the leading byte offset is
// unused for swizzled depth-major tiles.
// High 32 bits of the shared-memory matrix descriptor (constant for every tile of this kernel):
// stride byte offset 1024 >> 4 at bits 32..45, descriptor version 1 at bit 46, 128-byte swizzle at 61..63.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
// Low 32 bits: start address >> 4 at bits 0..13, leading byte offset (unused, 1) at bits 16..29.
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3FFFF) >> 4) | (1u << 16); }

// Issues the four K=32 MMAs of one 128-byte-deep stage.  The issuing thread is alone and the tensor
// core's instruction queue is shallow, so everything this thread executes between MMAs is on the
// critical path: descriptors are advanced with one 32-bit add each (+2 = 32 bytes along depth)
// inside a single asm block.  `first_accumulates` is 0 only for the first stage of a tile.
template <bool kPair>
__device__ __forceinline__ void mma_stage4(uint32_t tmem_d, uint32_t lo_a, uint32_t lo_b, uint32_t idesc,
                                           uint32_t first_accumulates) {
  if (kPair) {
    asm volatile(
        "{\n\t.reg .pred p, t;\n\t.reg .b64 da, db;\n\t.reg .b32 la, lb;\n\t"
        "setp.ne.u32 p, %4, 0;\n\t"
        "setp.eq.u32 t, 0, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %3, p;\n\t"
        "add.u32 la, %1, 2;\n\tadd.u32 lb, %2, 2;\n\tmov.b64 da, {la, %5};\n\tmov.b64 db, {lb, %5};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %3, t;\n\t"
        "add.u32 la, %1, 4;\n\tadd.u32 lb, %2, 4;\n\tmov.b64 da, {la, %5};\n\tmov.b64 db, {lb, %5};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %3, t;\n\t"
        "add.u32 la, %1, 6;\n\tadd.u32 lb, %2, 6;\n\tmov.b64 da, {la, %5};\n\tmov.b64 db, {lb, %5};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %3, t;\n\t}"
        ::"r"(tmem_d), "r"(lo_a), "r"(lo_b), "r"(idesc), "r"(first_accumulates), "r"(kDescHi)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p, t;\n\t.reg .b64 da, db;\n\t.reg .b32 la, lb;\n\t"
        "setp.ne.u32 p, %4, 0;\n\t"
        "setp.eq.u32 t, 0, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t"
        "add.u32 la, %1, 2;\n\tadd.u32 lb, %2, 2;\n\tmov.b64 da, {la, %5};\n\tmov.b64 db, {lb, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, t;\n\t"
        "add.u32 la, %1, 4;\n\tadd.u32 lb, %2, 4;\n\tmov.b64 da, {la, %5};\n\tmov.b64 db, {lb, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, t;\n\t"
        "add.u32 la, %1, 6;\n\tadd.u32 lb, %2, 6;\n\tmov.b64 da, {la, %5};\n\tmov.b64 db, {lb, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, t;\n\t}"
        ::"r"(tmem_d), "r"(lo_a), "r"(lo_b), "r"(idesc), "r"(first_accumulates), "r"(kDescHi)
        : "memory");
  }
}

// One K=32 MMA (used for a ragged last stage).
template <bool kPair>
__device__ __forceinline__ void mma_one(uint32_t tmem_d, uint32_t lo_a, uint32_t lo_b, uint32_t idesc, uint32_t accumulate,
                                        uint32_t desc_hi) {
  if (kPair) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.u32 p, %4, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(lo_a), "r"(lo_b), "r"(idesc), "r"(accumulate), "r"(desc_hi)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.u32 p, %4, 0;\n\t"
        "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(lo_a), "r"(lo_b), "r"(idesc), "r"(accumulate), "r"(desc_hi)
        : "memory");
  }
}

__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld_32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// AND-reduction of `ok` over the threads of one epilogue group through named barrier 1 + group.
__device__ __forceinline__ bool epilogue_all(bool ok, int group, int group_threads) {
  uint32_t res;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(res)
      : "r"((uint32_t)ok), "r"(1 + group), "r"(group_threads)
      : "memory");
  return res != 0;
}

// Per-destination-column (n) terms of one tile, staged in shared memory by the epilogue warps.
struct NTerms {
  int32_t add;   // bias (if the channel runs along n) and the zero-point corrections that depend on n
  int32_t mul;   // fixed-point multiplier (if the channel runs along n)
  int32_t exp;   // multiplier exponent (if the channel runs along n)
  int32_t pad;
};

// Narrows 32 int32 values to bytes (8 words).  With `clamp`, the values are first saturated to 16 bits two at a
// time, clamped to [lo2, hi2] per 16-bit half (bounds replicated in both halves) and then reduced to their low bytes:
// 7 instructions per 4 values instead of 14 for clamping and masking them one by one.
// `mode` (KernelArgs::pack_clamps): 0 = the values are already clamped, 1 = clamp two at a time in 16-bit halves,
// 2 / 3 = the clamp is the whole range of uint8 / int8, which the saturating narrowing applies by itself.
__device__ __forceinline__ void narrow_u8x32(const int32_t* v, int mode, uint32_t lo2, uint32_t hi2, uint32_t* w) {
  if (mode >= 2) {
#pragma unroll
    for (int q = 0; q < 8; q++) {
      uint32_t hi, d;
      if (mode == 2) {
        asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(v[4 * q + 3]), "r"(v[4 * q + 2]), "r"(0u));
        asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(v[4 * q + 1]), "r"(v[4 * q]), "r"(hi));
      } else {
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(v[4 * q + 3]), "r"(v[4 * q + 2]), "r"(0u));
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(v[4 * q + 1]), "r"(v[4 * q]), "r"(hi));
      }
      w[q] = d;
    }
  } else if (mode == 1) {
#pragma unroll
    for (int q = 0; q < 8; q++) {
      uint32_t a, b;
      asm("cvt.pack.sat.s16.s32 %0, %1, %2;" : "=r"(a) : "r"(v[4 * q + 1]), "r"(v[4 * q]));
      asm("cvt.pack.sat.s16.s32 %0, %1, %2;" : "=r"(b) : "r"(v[4 * q + 3]), "r"(v[4 * q + 2]));
      a = __vmaxs2(__vmins2(a, hi2), lo2);
      b = __vmaxs2(__vmins2(b, hi2), lo2);
      w[q] = __byte_perm(a, b, 0x6420);
    }
  } else {
#pragma unroll
    for (int q = 0; q < 8; q++) {
      w[q] = (uint32_t)(v[4 * q] & 0xff) | ((uint32_t)(v[4 * q + 1] & 0xff) << 8) |
             ((uint32_t)(v[4 * q + 2] & 0xff) << 16) | ((uint32_t)(v[4 * q + 3] & 0xff) << 24);
    }
  }
}

// Narrow and store 32 consecutive destination elements n0..n0+31 of row m.
template <int kDstBytes>
__device__ __forceinline__ void store_run32_at(char* dst_base, const KernelArgs& a, int m, int n0, int n_end, const int32_t* v) {
  char* base = dst_base + ((int64_t)m * a.dst.stride_m + n0) * kDstBytes;
  const bool full = n0 + 32 <= n_end;   // n_end: end of this tile's columns (and of the destination)
  if (full && (((uintptr_t)base) & 15) == 0) {
    // streaming stores: the destination is written once and never read here, it should not displace the operands in L2
    uint4* out = (uint4*)base;
    if (kDstBytes == 1) {
      uint32_t w[8];
      narrow_u8x32(v, a.pack_clamps, a.clamp_lo2, a.clamp_hi2, w);
      __stcs(&out[0], make_uint4(w[0], w[1], w[2], w[3]));
      __stcs(&out[1], make_uint4(w[4], w[5], w[6], w[7]));
    } else if (kDstBytes == 2) {
#pragma unroll
      for (int q = 0; q < 4; q++) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; t++) {
          w[t] = (uint32_t)(v[8 * q + 2 * t] & 0xffff) | ((uint32_t)(v[8 * q + 2 * t + 1] & 0xffff) << 16);
        }
        __stcs(&out[q], make_uint4(w[0], w[1], w[2], w[3]));
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; q++) {
        __stcs(&out[q], make_uint4((uint32_t)v[4 * q], (uint32_t)v[4 * q + 1], (uint32_t)v[4 * q + 2], (uint32_t)v[4 * q + 3]));
      }
    }
    return;
  }
  DstView d = a.dst;
  d.data = dst_base;
#pragma unroll
  for (int q = 0; q < 32; q++) {   // unrolled: v[] stays in registers
    const int32_t x = (kDstBytes == 1 && a.pack_clamps) ? max(min(v[q], a.ep.clamp_max), a.ep.clamp_min) : v[q];
    if (n0 + q < n_end) store_int(d, a.ep.dst_dtype, m, n0 + q, x);
  }
}

// Narrow and store 32 consecutive destination elements n0..n0+31 of row m: locally and, when the destination is
// mirrored into peer GPUs' memory, at the same place of every mirror.
template <int kDstBytes>
__device__ __forceinline__ void store_run32(const KernelArgs& a, int m, int n0, int n_end, const int32_t* v) {
  store_run32_at<kDstBytes>((char*)a.dst.data, a, m, n0, n_end, v);
  for (int i = 0; i < a.n_mirror; i++) store_run32_at<kDstBytes>((char*)a.mirror[i], a, m, n0, n_end, v);
}

// ---- helpers for the two-CTA (cta_group::2) variant -------------------------------------------

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// Address of the same shared-memory location in the CTA of the given cluster rank.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(cluster_addr), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// TMA load into this CTA's shared memory whose completion is signalled on a barrier that may live
// in the partner CTA of the pair (no multicast: each CTA fetches its own half).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
      : "memory");
}

// Arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs
// issued so far have completed.
__device__ __forceinline__ void mma_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}

// kDstBytes: 1 (int8/uint8), 2 (int16), 4 (int32: raw accumulators, no multiplier, no clamp).
// kX86: the two-step rounding of ruy's x86 kernels instead of the reference rounding.
// kPair: two CTAs on neighbouring SMs (a cluster of 2) share each 256 x 256 tile: one thread of the
//        even CTA issues cta_group::2 MMAs that read both CTAs' shared memory, every CTA loads its
//        own 128 rows of each operand, keeps its 128 accumulator rows in its own tensor memory and
//        runs its own epilogue.  Halves shared-memory fill per MMA and deepens the pipeline to 6 stages.
// kMirror: the destination is also written to peers' copies (or to a multicast mapping) and the launch may end with
//        the step's flag exchange.  A variant of its own: with that code compiled in, the plain kernel spilled
//        registers and took 2.5 % longer on the 4096 x 4096 x 8192 mul (90.3 against 88.0 us, alternating runs).
template <int kDstBytes, bool kX86, bool kPair, bool kMirror>
__global__ void __launch_bounds__(kThreads, 1)
tc_i8_kernel(const __grid_constant__ CUtensorMap map_m, const __grid_constant__ CUtensorMap map_n,
             const KernelArgs args) {
  constexpr int kNumStages = kPair ? kPairStages : kStages;
  constexpr int kStageSize = kPair ? kPairStageBytes : kStageBytes;
  constexpr int kUnitM = kPair ? 2 * kBlockM : kBlockM;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kNumStages];
  __shared__ __align__(8) uint64_t empty_bar[kNumStages];
  __shared__ __align__(8) uint64_t acc_full_bar[kMaxAccBufs];
  __shared__ __align__(8) uint64_t acc_empty_bar[kMaxAccBufs];
  // per-n terms of the tile being drained, one array per field so that the common paths fetch four addends per load
  __shared__ __align__(16) int32_t nt_add_s[kEpilogueGroups][kMaxBlockN];
  // {addend, multiplier, high word of the rounding term (+ destination zero point), shift - 32} per n, for
  // multipliers that vary along n: one 16-byte load per element
  __shared__ __align__(16) int4 nt4_s[kEpilogueGroups][kMaxBlockN];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int last_cta;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  const uint32_t rank = kPair ? cluster_ctarank() : 0;
  const int unit = kPair ? blockIdx.x / 2 : blockIdx.x;      // a CTA, or a pair of CTAs
  const int units = kPair ? gridDim.x / 2 : gridDim.x;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kNumStages; s++) {
      mbar_init(&full_bar[s], 1);   // pair: only the even CTA's barriers are used; its producer expects both CTAs' bytes
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < kMaxAccBufs; b++) {
      mbar_init(&acc_full_bar[b], 1);
      // the warps of the group that drained it (in both CTAs of a pair)
      mbar_init(&acc_empty_bar[b], (kEpilogueWarps / args.epi_groups) * (kPair ? 2 : 1));
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    if (kPair) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  if (!kPair && args.sums_col >= 0) {
    // Zero-point sums of the m-side operand for free: 16 rows of the n-side tile that no TMA box ever covers
    // are filled with 0x01 once, so accumulator column sums_col becomes sum_k m[.,k] (ruy/pack.h:117-129 computes
    // these sums while packing).  All bytes are equal, so the swizzle does not matter.
    for (int st = 0; st < kNumStages; st++) {
      uint32_t* ones = reinterpret_cast<uint32_t*>(smem + st * kStageSize + kABytes + args.sums_col * args.row_pitch);
      for (int i = threadIdx.x; i < 16 * args.row_pitch / 4; i += kThreads) ones[i] = 0x01010101u;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();   // the partner's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const int num_tiles = args.tiles_m * args.tiles_n;
  const int k_blocks = (args.depth + kBlockKBytes - 1) / kBlockKBytes;
  volatile int* abortp = &abort_flag;
  const int n_rows_per_cta = kPair ? args.block_n / 2 : args.block_n;   // rows of the n operand this CTA stages

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t s = 0, ph = 0;
      uint32_t issued = 0;
      const uint32_t stage_tx = (uint32_t)((kBlockM + n_rows_per_cta) * args.row_pitch);
      const uint32_t full0_cluster = kPair ? map_to_rank(smem_u32(&full_bar[0]), 0) : 0;
      bool ok = true;
      for (int tile = unit; tile < num_tiles && ok; tile += units) {
        const int tm = tile / args.tiles_n;
        const int tn = tile % args.tiles_n;
        const int row_m = tm * kUnitM + (int)rank * kBlockM;
        const int row_n = tn * args.block_n + (int)rank * n_rows_per_cta;
        for (int kb = 0; kb < k_blocks; kb++) {
          if (!mbar_try_wait(&empty_bar[s], ph ^ 1)) {
            if (!mbar_wait(&empty_bar[s], ph ^ 1, abortp)) {
              if (!*abortp) atomicCAS(args.status, 0, kTimeoutProducer);
              *abortp = 1;
              ok = false;
              break;
            }
          }
          uint8_t* sa = smem + s * kStageSize;
          uint8_t* sb = sa + kABytes;
          if (args.debug & 2) {   // profiling: signal the stage without fetching anything
            if (!kPair) mbar_arrive(&full_bar[s]); else if (rank == 0) mbar_arrive(&full_bar[s]);
          } else if (kPair) {
            // Both CTAs' copies complete on the even CTA's barrier.  Only that CTA arrives on it, expecting
            // the bytes of both; its partner's bytes may land first, which a transaction count tolerates
            // because the phase cannot complete before the one pending arrival has happened.
            const uint32_t bar = full0_cluster + s * 8;
            if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * stage_tx);
            tma_load_2d_pair(sa, &map_m, kb * kBlockKBytes, row_m, bar);
            tma_load_2d_pair(sb, &map_n, kb * kBlockKBytes, row_n, bar);
          } else {
            mbar_expect_tx(&full_bar[s], stage_tx);
            tma_load_2d(sa, &map_m, kb * kBlockKBytes, row_m, &full_bar[s]);
            tma_load_2d(sb, &map_n, kb * kBlockKBytes, row_n, &full_bar[s]);
          }
          issued++;
          if (++s == kNumStages) { s = 0; ph ^= 1; }
        }
      }
      if (!ok && issued > 0 && !kPair) {
        // give copies that are still in flight a bounded chance to land before the CTA exits
        const uint32_t last = issued - 1;
        for (uint32_t i = 0; i < kSpinLimit / 64; i++) {
          if (mbar_try_wait(&full_bar[last % kNumStages], (last / kNumStages) & 1)) break;
          __nanosleep(100);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (the even CTA of a pair issues for both) ----------------
    // The whole warp runs the loop converged and one elected lane issues the tensor-core
    // instructions: warp-uniform operands then live in uniform registers and the few instructions
    // between two MMAs stay short enough to keep the tensor core's shallow queue fed.
    if (rank == 0) {
      uint32_t s = 0, ph = 0;       // stage index and its phase, advanced incrementally
      uint32_t tcount = 0;
      bool ok = true;
      const uint32_t lo_a0 = desc_lo(smem_u32(smem));
      const uint32_t stage_step = (uint32_t)kStageSize >> 4;
      const uint32_t b_off = (uint32_t)kABytes >> 4;
      const int full_blocks = args.depth / kBlockKBytes;   // stages that hold a whole 128 bytes of depth
      const uint32_t idesc = args.idesc;
#ifdef RUYB200_DEBUG_KNOBS
      long long dbg_t0 = clock64(), dbg_full = 0, dbg_acc = 0;
#endif
      for (int tile = unit; tile < num_tiles && ok; tile += units, tcount++) {
        const int buf = (int)(tcount & (uint32_t)(args.acc_bufs - 1));
        const uint32_t aph = (tcount >> args.acc_shift) & 1;
#ifdef RUYB200_DEBUG_KNOBS
        long long dbg_a = clock64();
#endif
        if (!mbar_wait(&acc_empty_bar[buf], aph ^ 1, abortp)) {
          if (!*abortp) atomicCAS(args.status, 0, kTimeoutMma);
          *abortp = 1;
          break;
        }
        tc_fence_after();
#ifdef RUYB200_DEBUG_KNOBS
        dbg_acc += clock64() - dbg_a;
#endif
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * (kTmemCols >> args.acc_shift));
        for (int kb = 0; kb < k_blocks; kb++) {
#ifdef RUYB200_DEBUG_KNOBS
          const bool dbg_ready = (args.debug & 16) ? mbar_test_wait(&full_bar[s], ph) : mbar_try_wait(&full_bar[s], ph);
          if (!dbg_ready) {
            long long dbg_b = clock64();
#else
          if (!mbar_try_wait(&full_bar[s], ph)) {
#endif
            if (!mbar_wait(&full_bar[s], ph, abortp)) {
              if (!*abortp) atomicCAS(args.status, 0, kTimeoutMma);
              *abortp = 1;
              ok = false;
              break;
            }
#ifdef RUYB200_DEBUG_KNOBS
            dbg_full += clock64() - dbg_b;
#endif
          }
          tc_fence_after();
          const uint32_t lo_a = lo_a0 + s * stage_step;
          const uint32_t lo_b = lo_a + b_off;
          if (elect_one()) {
            if (kb < full_blocks) {
              mma_stage4<kPair>(tmem_d, lo_a, lo_b, idesc, kb != 0);
            } else {
              const int ksteps = (args.depth - kb * kBlockKBytes + 31) / 32;
              for (int k = 0; k < ksteps; k++) mma_one<kPair>(tmem_d, lo_a + 2 * k, lo_b + 2 * k, idesc, (kb | k) != 0, args.desc_hi);
            }
            // frees the stage (in both CTAs of a pair) once these MMAs have read it
            if (kPair) mma_commit_pair(&empty_bar[s]); else mma_commit(&empty_bar[s]);
          }
          __syncwarp();
          if (++s == kNumStages) { s = 0; ph ^= 1; }
        }
        if (ok) {
          if (elect_one()) {
            if (kPair) mma_commit_pair(&acc_full_bar[buf]); else mma_commit(&acc_full_bar[buf]);
          }
          __syncwarp();
        }
      }
#ifdef RUYB200_DEBUG_KNOBS
      if ((args.debug & 16) && blockIdx.x == 0 && lane == 0)
        printf("mma warp: total %lld cycles, waiting for data %lld, waiting for a free accumulator %lld, tiles %u\n",
               clock64() - dbg_t0, dbg_full, dbg_acc, tcount);
#endif
    }
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    const Epilogue& ep = args.ep;
    const int ew = warp - 2;
    const int lane_group = warp % 4;       // the TMEM lane quarter this warp may read
    // Deep main loops: all eight warps drain each tile together (two warps per lane quarter alternate 32-column
    // chunks), so the accumulator is free again as early as possible.  Shallow ones: two groups of four warps take
    // tiles in turn, so that the per-tile latencies (barrier, tensor-memory loads, stores) of two tiles overlap.
    const int groups = args.epi_groups;
    const int group = groups == 2 ? ew / 4 : 0;
    const int group_threads = 32 * kEpilogueWarps / groups;
    const int etid = groups == 2 ? (ew % 4) * 32 + lane : ew * 32 + lane;   // thread index within the group
    const int c_first = groups == 2 ? 0 : (ew / 4) * 32;
    const int c_step = groups == 2 ? 32 : 64;
    const bool ch_n = ep.channel_on_n != 0;
    const int32_t zz = ep.zp_m * ep.zp_n * ep.depth;
    uint32_t tcount = 0;
    bool ok = true;
    int staged_tn = -1;            // which n tile this group's staging buffer holds
    bool tile_fast = false;        // every n of that tile allows the short requantisation with per-n multipliers
#ifdef RUYB200_DEBUG_KNOBS
    long long dbg_wait = 0, dbg_busy = 0, dbg_stage = 0;
#endif
    for (int tile = unit; tile < num_tiles && ok; tile += units, tcount++) {
      const int tm = tile / args.tiles_n;
      const int tn = tile % args.tiles_n;
      const int buf = (int)(tcount & (uint32_t)(args.acc_bufs - 1));
      const uint32_t aph = (tcount >> args.acc_shift) & 1;
#ifdef RUYB200_DEBUG_KNOBS
      long long dbg_a = clock64();
#endif
      if (groups == 2 && (int)(tcount & 1) != group) continue;   // the other group's tile
      // stage the per-n terms of this tile (overlaps the tile's main loop) unless the group's buffer already holds
      // them (there is one n tile, or it did not change)
      int32_t* nt_add = nt_add_s[group];
      int4* nt4 = nt4_s[group];
      const bool restage = staged_tn != tn;
      if (restage) {
        // warps of this group may still be reading the buffer for the previous tile
        epilogue_all(true, group, group_threads);
        staged_tn = tn;
        bool my_fast = true;
        for (int i = etid; i < args.block_n; i += group_threads) {
          const int n = tn * args.block_n + i;
          NTerms t;
          t.add = zz;
          t.mul = ep.mfp;
          t.exp = ep.mexp;
          t.pad = 0;
          if (n < args.size_n) {
            if (ep.zp_m) t.add -= ep.zp_m * ep.sums_n[n];
            if (ch_n) {
              if (ep.bias) t.add += ((const int32_t*)ep.bias)[n];
              if (ep.mfp_pc) t.mul = ep.mfp_pc[n];
              if (ep.mexp_pc) t.exp = ep.mexp_pc[n];
            }
          }
          nt_add[i] = t.add;
          // total shift 33..45: the rounding term has no low word and the zero point fits beside it, so that
          // result = (mulhi(x, mul) + rnd_hi) >> (shift - 32); other shifts take the general path
          const int sh = 31 - t.exp;
          const bool n_fast = n >= args.size_n || (sh >= 33 && sh <= 45 && ep.dst_zp > -32768 && ep.dst_zp < 32768);
          my_fast = my_fast && n_fast;
          const int sh_hi = sh - 32;
          const int32_t rnd_hi = n_fast ? (int32_t)(1u << ((sh - 33) & 31)) + ep.dst_zp * (int32_t)(1u << (sh_hi & 31)) : 0;
          nt4[i] = make_int4(t.add, t.mul, rnd_hi, sh_hi);
        }
        // every n of the tile must qualify; the reduction also publishes the staged terms
        tile_fast = epilogue_all(my_fast, group, group_threads);
      }
      // per-m terms of this thread's row
      const int m = tm * kUnitM + (int)rank * kBlockM + lane_group * 32 + lane;
      const bool m_ok = m < args.size_m;
      int32_t add_m = 0, mul_m = ep.mfp, exp_m = ep.mexp;
      if (m_ok) {
        if (ep.zp_n && ep.sums_m) add_m -= ep.zp_n * ep.sums_m[m];
        if (!ch_n) {
          if (ep.bias) add_m += ((const int32_t*)ep.bias)[m];
          if (ep.mfp_pc) mul_m = ep.mfp_pc[m];
          if (ep.mexp_pc) exp_m = ep.mexp_pc[m];
        }
      }
#ifdef RUYB200_DEBUG_KNOBS
      long long dbg_b = clock64();
      dbg_stage += dbg_b - dbg_a;
#endif
      if (!(args.tight_wait ? mbar_wait_warp_tight(&acc_full_bar[buf], aph, abortp) : mbar_wait_warp(&acc_full_bar[buf], aph, abortp))) {
        if (!*abortp) atomicCAS(args.status, 0, kTimeoutEpilogue);
        *abortp = 1;
        ok = false;
      }
      // One named-barrier reduction over all epilogue threads: it publishes the staged terms and
      // makes the continue/abort decision collective, so no warp is ever left waiting for another
      // that has already left the loop.
      ok = epilogue_all(ok, group, group_threads);
      if (!ok) break;
      tc_fence_after();
#ifdef RUYB200_DEBUG_KNOBS
      long long dbg_c = clock64();
      dbg_wait += dbg_c - dbg_b;
#endif
      const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(buf * (kTmemCols >> args.acc_shift));
      const int n_end = min(args.size_n, (tn + 1) * args.block_n);   // a 32-column chunk may reach past the tile's columns
      const bool have_chunk = c_first < args.block_n && tn * args.block_n + c_first < args.size_n && !(args.debug & 1);
      uint32_t r[32];
      // the sums column and the first chunk are fetched together: one wait instead of two
      uint32_t row_sum = 0;
      if (!kPair && args.sums_col >= 0) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(row_sum) : "r"(taddr + (uint32_t)args.sums_col) : "memory");
      }
      if (have_chunk) tmem_ld_32(taddr + c_first, r);
      tmem_ld_wait();
      if (!kPair && args.sums_col >= 0) add_m -= ep.zp_n * (int32_t)row_sum;
      // When the multiplier does not vary along n (one multiplier for the whole matrix, or one per m), the
      // rounding term and the shift are per-thread constants.
      const bool mul_varies_with_n = ch_n && (ep.mfp_pc != nullptr || ep.mexp_pc != nullptr);
      const int sh_c = 31 - exp_m;
      const long long rnd_c = 1ll << (sh_c - 1);
      // With every shift of the warp at least 32 the result is the high word of the 64-bit product shifted on, and the
      // destination zero point can ride in the rounding term when it cannot overflow there.
      const bool high_word = kDstBytes != 4 && !kX86 && !mul_varies_with_n && __all_sync(0xffffffffu, sh_c >= 32);
      const bool fold_zp = sh_c <= 45 && ep.dst_zp > -32768 && ep.dst_zp < 32768;
      const long long rnd_hw = rnd_c + (fold_zp ? (long long)ep.dst_zp * (1ll << (sh_c & 63)) : 0ll);
      const int32_t zp_late = fold_zp ? 0 : ep.dst_zp;
      const int sh_hi = (sh_c - 32) & 31;
      // bias / zero-point terms, fixed-point multiplier, destination zero point and clamp for the 32 accumulators in r[]
      // 8-bit destinations leave the clamp to the narrowing step (two values per instruction there)
      const bool late_clamp = kDstBytes == 1 && args.pack_clamps;
      auto finish_chunk = [&](int c, int32_t (&v)[32]) {
        if (kDstBytes != 4 && !kX86 && mul_varies_with_n && tile_fast) {
#pragma unroll
          for (int q = 0; q < 32; q++) {
            const int4 t = nt4[c + q];
            const int32_t x = (int32_t)(r[q] + (uint32_t)t.x + (uint32_t)add_m);
            const int32_t y = (__mulhi(x, t.y) + t.z) >> t.w;
            v[q] = late_clamp ? y : max(min(y, ep.clamp_max), ep.clamp_min);
          }
        } else if (high_word || (kDstBytes != 4 && !kX86 && !mul_varies_with_n)) {
#pragma unroll
          for (int q4 = 0; q4 < 8; q4++) {
            const int4 ad = *reinterpret_cast<const int4*>(&nt_add[c + 4 * q4]);   // c is a multiple of 32
            const int32_t adds[4] = {ad.x, ad.y, ad.z, ad.w};
#pragma unroll
            for (int t = 0; t < 4; t++) {
              const int q = 4 * q4 + t;
              const int32_t x = (int32_t)(r[q] + (uint32_t)adds[t] + (uint32_t)add_m);
              int32_t y;
              if (high_word) {
                const long long p = (long long)x * (long long)mul_m + rnd_hw;
                y = (int32_t)((uint32_t)((int32_t)(p >> 32) >> sh_hi) + (uint32_t)zp_late);
              } else {
                y = (int32_t)((uint32_t)(int32_t)(((long long)x * (long long)mul_m + rnd_c) >> sh_c) + (uint32_t)ep.dst_zp);
              }
              v[q] = late_clamp ? y : max(min(y, ep.clamp_max), ep.clamp_min);
            }
          }
        } else {
#pragma unroll
          for (int q = 0; q < 32; q++) {
            int32_t x = (int32_t)(r[q] + (uint32_t)nt_add[c + q] + (uint32_t)add_m);
            if (kDstBytes != 4) {
              const int4 t = nt4[c + q];
              const int32_t mul = ch_n ? t.y : mul_m;
              const int e = ch_n ? -1 - t.w : exp_m;     // t.w holds 31 - e - 32
              x = kX86 ? requant_x86(x, mul, e) : requant_reference(x, mul, e);
              x = (int32_t)((uint32_t)x + (uint32_t)ep.dst_zp);
              if (!late_clamp) x = max(min(x, ep.clamp_max), ep.clamp_min);
            } else {
              x = (int32_t)((uint32_t)x + (uint32_t)ep.dst_zp);
            }
            v[q] = x;
          }
        }
      };
      if (kMirror && kDstBytes == 1 && (args.n_mirror > 0 || args.multicast != nullptr) && groups == 1) {
        // Mirrored 8-bit destination.  A thread owns 32 bytes of one destination column; written directly, a warp's
        // store would be 32 separate 32-byte pieces, which NVLink moves poorly.  So the tile is staged through
        // shared memory 128 columns at a time and written out with every warp instruction covering 128 contiguous
        // bytes, locally and to every peer.
        uint8_t* const stg0 = smem + kNumStages * kStageSize;
        const int ml = lane_group * 32 + lane;
        const int halves = (args.block_n + 127) / 128;
        const bool issuer = ew == 0 && lane == 0;            // the thread that owns this CTA's bulk groups
        for (int h = 0; h < halves; h++) {
          const int nh0 = tn * args.block_n + h * 128;       // first destination index of this half
          if (nh0 >= n_end) break;                           // uniform over the CTA
          // The copy engine writes the half out when it is a whole 128-byte box, or ends where the tensor ends on a
          // 16-byte boundary (rows and 16-byte pieces outside the tensor are not written; a tensor that ends inside a
          // piece gets the whole piece, measured, so such an edge is left to the store instructions below, like
          // any other width).
          const bool by_tma = args.store_maps != nullptr &&
                              (n_end - nh0 >= 128 || (n_end == args.size_n && (args.size_n & 15) == 0));
          if (by_tma) {
            // The first 32-column chunk is worked out before the wait, so that arithmetic overlaps the copy engine's reads
            // of the previous half; the second follows once the staging area is free (one chunk of results live across
            // the barrier, not two: the registers are short in this variant).
#pragma unroll
            for (int j = 0; j < 2; j++) {
              const int c = h * 128 + j * 64 + c_first;
              const bool have = !(c >= args.block_n || tn * args.block_n + c >= args.size_n);   // uniform across the warp
              uint32_t w[8];
              if (have) {
                if (c != c_first) {
                  tmem_ld_32(taddr + c, r);
                  tmem_ld_wait();
                }
                int32_t v[32];
                finish_chunk(c, v);
                narrow_u8x32(v, late_clamp ? 1 : 0, args.clamp_lo2, args.clamp_hi2, w);
              }
              if (j == 0) {
                if (issuer) bulk_wait_read_0();                // the stores that last read the staging area are done with it
                epilogue_all(true, group, group_threads);
              }
              if (have) {
                // row ml of the box; its 16-byte piece p sits at p ^ (ml & 7)
                const int p0 = (j * 64 + c_first) >> 4;
                uint8_t* row = stg0 + ml * 128;
                *reinterpret_cast<uint4*>(row + (((p0) ^ (ml & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(row + (((p0 + 1) ^ (ml & 7)) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
              }
            }
            fence_proxy_async();                             // these writes, before the copy engine reads them
            epilogue_all(true, group, group_threads);        // the half tile is staged
            if (issuer) {
              const int y = tm * kUnitM + (int)rank * kBlockM;
              for (int t = 0; t <= args.n_mirror; t++) tma_store_2d(args.store_maps + t, stg0, nh0, y);
              bulk_commit();
            }
            continue;
          }
          uint8_t* const stg = stg0;
          if (args.store_maps != nullptr) {
            if (issuer) bulk_wait_read_0();
            epilogue_all(true, group, group_threads);
          }
          for (int j = 0; j < 2; j++) {
            const int c = h * 128 + j * 64 + c_first;
            if (c >= args.block_n || tn * args.block_n + c >= args.size_n) continue;   // uniform across the warp
            if (c != c_first) {
              tmem_ld_32(taddr + c, r);
              tmem_ld_wait();
            }
            int32_t v[32];
            finish_chunk(c, v);
            uint32_t w[8];
            narrow_u8x32(v, late_clamp ? 1 : 0, args.clamp_lo2, args.clamp_hi2, w);
            uint4* sp = reinterpret_cast<uint4*>(stg + ml * kMirrorPitch + (c - h * 128));
            sp[0] = make_uint4(w[0], w[1], w[2], w[3]);
            sp[1] = make_uint4(w[4], w[5], w[6], w[7]);
          }
          epilogue_all(true, group, group_threads);          // the half tile is staged
          const int nb = min(128, n_end - nh0);
          if (args.mirror_wide && (nb & 15) == 0) {
            // 16 bytes per lane: one warp instruction moves four rows of 128 bytes
            const int c16 = (lane & 7) * 16;
            int rr = ew * 4 + (lane >> 3);
            int mm = tm * kUnitM + (int)rank * kBlockM + rr;
            int64_t off = (int64_t)mm * args.dst.stride_m + nh0 + c16;
            const uint8_t* sp = stg + rr * kMirrorPitch + c16;
            if (c16 < nb) {
#pragma unroll
              for (int it = 0; it < kBlockM / (4 * kEpilogueWarps); it++) {
                if (mm < args.size_m) {
                  const uint4 val = *reinterpret_cast<const uint4*>(sp);
                  if (args.multicast) {
                    multimem_st_16((uint8_t*)args.multicast + off, val);   // one store, delivered to every rank's copy
                  } else {
                    *reinterpret_cast<uint4*>((uint8_t*)args.dst.data + off) = val;
                    for (int t = 0; t < args.n_mirror; t++) *reinterpret_cast<uint4*>((uint8_t*)args.mirror[t] + off) = val;
                  }
                }
                mm += 4 * kEpilogueWarps;
                off += (int64_t)(4 * kEpilogueWarps) * args.dst.stride_m;
                sp += 4 * kEpilogueWarps * kMirrorPitch;
              }
            }
          } else {
            for (int rr = ew; rr < kBlockM; rr += kEpilogueWarps) {
              const int mm = tm * kUnitM + (int)rank * kBlockM + rr;
              if (mm >= args.size_m) break;                    // uniform across the warp
              if (lane * 4 < nb) {
                const uint32_t val = *reinterpret_cast<const uint32_t*>(stg + rr * kMirrorPitch + lane * 4);
                const int64_t off = (int64_t)mm * args.dst.stride_m + nh0 + lane * 4;
                for (int t = -1; t < args.n_mirror; t++) {
                  uint8_t* base = (uint8_t*)(t < 0 ? args.dst.data : args.mirror[t]) + off;
                  if (lane * 4 + 4 <= nb && (((uintptr_t)base) & 3) == 0) {
                    *reinterpret_cast<uint32_t*>(base) = val;
                  } else {
                    for (int b = 0; b < 4 && lane * 4 + b < nb; b++) base[b] = (uint8_t)(val >> (8 * b));
                  }
                }
              }
            }
          }
          epilogue_all(true, group, group_threads);          // the staging area may be overwritten
        }
      } else {
        for (int c = c_first; c < args.block_n; c += c_step) {
          const int n0 = tn * args.block_n + c;
          if (n0 >= args.size_n || (args.debug & 1)) break;   // uniform across the warp
          if (c != c_first) {
            tmem_ld_32(taddr + c, r);
            tmem_ld_wait();
          }
          if (m_ok) {
            int32_t v[32];
            finish_chunk(c, v);
            store_run32<kDstBytes>(args, m, n0, n_end, v);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (kPair) {
          mbar_arrive_cluster(map_to_rank(smem_u32(&acc_empty_bar[buf]), 0));   // the issuing CTA tracks both epilogues
        } else {
          mbar_arrive(&acc_empty_bar[buf]);
        }
      }
#ifdef RUYB200_DEBUG_KNOBS
      dbg_busy += clock64() - dbg_c;
#endif
    }
#ifdef RUYB200_DEBUG_KNOBS
    if ((args.debug & 16) && blockIdx.x == 0 && threadIdx.x == 64)
      printf("epilogue warp: staging %lld, waiting for a tile %lld, working %lld cycles over %u tiles\n", dbg_stage,
             dbg_wait, dbg_busy, tcount);
#endif
    if (kMirror && args.store_maps != nullptr && ew == 0 && lane == 0) {
      bulk_wait_all();          // the copy engine has written every tile of this CTA, here and in the peers' memory
      fence_proxy_async();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();   // neither CTA releases tensor memory or exits while its partner may still signal it
  tc_fence_after();
  if (warp == 0) {
    if (kPair) {
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    } else {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
  }
  if (kMirror && args.n_xchg > 0) {
    // The CTA that finishes last tells every rank that this rank's tiles have landed and waits (bounded) for the same
    // news from the others: the step's flag exchange without a launch of its own.  The peers run on other GPUs;
    // nothing here waits for another launch on this GPU.
    // Ordering: the CTA's stores (all its threads, joined by the barrier above; the copy engine's, completed by
    // their issuing thread) -> this fence at GPU scope -> the counter; the last CTA sees every count, and ONE
    // system-scope fence there, which is cumulative over everything that happened before it, puts all tiles before
    // the flags.  System-scope fences and acquire loads cost microseconds each on this part: a version with one per
    // epilogue thread, one per CTA, one per flag plus a release store and acquire polls measured 19 us for the exchange
    // on one GPU with local flags, this one 3.
    if (threadIdx.x == 0) {
      __threadfence();
      const unsigned int prev = atomicAdd(args.xchg_counter, 1u);
      last_cta = prev == gridDim.x - 1 ? 1 : 0;
      if (last_cta) {
        __threadfence();
        *args.xchg_counter = 0u;   // for the next launch, which follows in stream order
      }
    }
    __syncthreads();
    if (last_cta && (int)threadIdx.x < args.n_xchg) {
      const int i = threadIdx.x;
      __threadfence_system();
      if (args.xchg_remote[i]) {
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(args.xchg_remote[i]), "r"(args.xchg_value) : "memory");
      }
      // The peers' flags are polled with relaxed loads (an acquire load costs as much as a fence, every time); one
      // fence follows the loop.
      unsigned long long t0;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
      for (unsigned it = 0;; it++) {
        uint32_t v;
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(args.xchg_local + i) : "memory");
        if ((int32_t)(v - args.xchg_value) >= 0) break;
        if ((it & 15) == 15) {
          unsigned long long t;
          asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
          if (t - t0 > args.xchg_limit_ns) {
            atomicCAS(args.status, 0, 9);   // a peer never signalled: report, do not hang
            break;
          }
        }
      }
      __threadfence_system();   // the acquire side of the flags, once: what follows this launch reads the peers' tiles
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  // looked up once per process; initialisation of a function-local static is thread-safe
  static const EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      return (EncodeTiledFn)p;
    }
    return nullptr;
  }();
  return fn;
}

// 2-D map over a width x depth byte matrix: dim0 = depth (contiguous), dim1 = width.
// `pitch` (128, 64 or 32) is the box's depth extent in bytes and selects the matching swizzle pattern.
bool make_map(CUtensorMap* map, const SideView& s, int depth, int box_rows, int pitch = kBlockKBytes) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)depth, (cuuint64_t)s.width};
  cuuint64_t strides[1] = {(cuuint64_t)s.stride_w};
  cuuint32_t box[2] = {(cuuint32_t)pitch, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapSwizzle sw = pitch == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                            : (pitch == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(s.data), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool make_i8_store_map(void* map_out, void* base, int size_n, int size_m, int64_t stride_m) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn || ((uintptr_t)base & 15) != 0 || (stride_m & 15) != 0 || size_n <= 0 || size_m <= 0) return false;
  cuuint64_t dims[2] = {(cuuint64_t)size_n, (cuuint64_t)size_m};
  cuuint64_t strides[1] = {(cuuint64_t)stride_m};
  cuuint32_t box[2] = {128, 128};
  cuuint32_t estr[2] = {1, 1};
  return fn((CUtensorMap*)map_out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_i8_tile_map(CUtensorMap* map, const void* base, int depth, int width, int64_t stride_w, int box_rows) {
  SideView s;
  s.data = base;
  s.stride_w = stride_w;
  s.stride_k = 1;
  s.width = width;
  s.zero_point = 0;
  s.dtype = RUYB200_U8;
  return make_map(map, s, depth, box_rows);
}

namespace {

bool is_8bit(uint8_t dtype) { return dtype == RUYB200_I8 || dtype == RUYB200_U8; }

template <int kDstBytes, bool kX86, bool kPair, bool kMirror>
cudaError_t launch_variant(const CUtensorMap& map_m, const CUtensorMap& map_n, const KernelArgs& a, int grid,
                           cudaStream_t stream) {
  constexpr int smem = kPair ? kPairSmemBytes : kSmemBytes;
  // the opt-in to more than 48 KB of dynamic shared memory is per device and per kernel variant; contexts on
  // several threads may get here at the same time
  static std::mutex mu;
  static bool attr_set[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= kMaxDevices || !attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(tc_i8_kernel<kDstBytes, kX86, kPair, kMirror>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < kMaxDevices) attr_set[dev] = true;
    }
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kPair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, tc_i8_kernel<kDstBytes, kX86, kPair, kMirror>, map_m, map_n, a);
}

// How many 2-CTA clusters of this kernel can be resident at the same time on the current device.
int max_resident_pairs(int sm_count) {
  static std::mutex mu;
  static int cached[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> lock(mu);
  if (dev >= 0 && dev < kMaxDevices && cached[dev]) return cached[dev];
  int n = 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(sm_count / 2 * 2);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaFuncSetAttribute(tc_i8_kernel<1, false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes);
  if (cudaOccupancyMaxActiveClusters(&n, tc_i8_kernel<1, false, true, false>, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = sm_count / 2;
  }
  if (n > sm_count / 2) n = sm_count / 2;
  if (getenv("RUYB200_VERBOSE")) fprintf(stderr, "ruy_b200: %d resident CTA pairs on %d SMs\n", n, sm_count);
  if (dev >= 0 && dev < kMaxDevices) cached[dev] = n;
  return n;
}

template <bool kPair>
cudaError_t launch_by_type(const CUtensorMap& map_m, const CUtensorMap& map_n, const KernelArgs& a, int grid,
                           cudaStream_t stream) {
  const bool x86 = a.ep.rounding_x86 != 0;
  const bool mirror = a.n_mirror > 0 || a.multicast != nullptr || a.n_xchg > 0;
  switch (a.ep.dst_dtype) {
    case RUYB200_I8:
    case RUYB200_U8:
      if (mirror) {
        return x86 ? launch_variant<1, true, kPair, true>(map_m, map_n, a, grid, stream)
                   : launch_variant<1, false, kPair, true>(map_m, map_n, a, grid, stream);
      }
      return x86 ? launch_variant<1, true, kPair, false>(map_m, map_n, a, grid, stream)
                 : launch_variant<1, false, kPair, false>(map_m, map_n, a, grid, stream);
    case RUYB200_I16:
      if (mirror) {
        return x86 ? launch_variant<2, true, kPair, true>(map_m, map_n, a, grid, stream)
                   : launch_variant<2, false, kPair, true>(map_m, map_n, a, grid, stream);
      }
      return x86 ? launch_variant<2, true, kPair, false>(map_m, map_n, a, grid, stream)
                 : launch_variant<2, false, kPair, false>(map_m, map_n, a, grid, stream);
    default:
      return mirror ? launch_variant<4, false, kPair, true>(map_m, map_n, a, grid, stream)
                    : launch_variant<4, false, kPair, false>(map_m, map_n, a, grid, stream);
  }
}

// ---- tile-shape choice ---------------------------------------------------------------------------
//
// The part of ruy's MakeBlockMap that matters on this machine (ruy/block_map.cc:217-245 "multithreading
// score", :289-317 "kernel amortization score", :339-471 the choice): ruy scores power-of-two block sizes by
// how many blocks each thread gets and how well a block amortises the kernel's fixed costs, and takes the
// best.  Here a "thread" is a persistent CTA (or CTA pair) and the schedule is static, so a launch takes
// ceil(tiles / units) rounds of one tile each: the candidates are one-CTA tiles of 128 x bn and two-CTA tiles of
// 256 x bn for a handful of widths bn (multiples of 16, at most 256), and the score is the estimated duration
// rounds x cycles per tile.  Smaller tiles waste less of the last round and occupy more SMs when tiles are few,
// but cost more per multiply-add; the estimate weighs the two.
struct TileShape {
  bool pair;
  int block_n;
  double cycles;   // estimated SM cycles of the whole launch
};

// Constants of the estimate, in SM cycles, fitted to launches of this kernel with every candidate forced in turn
// (4096-deep shards of 1024 to 8192 columns; depth 128 to 1024 with 3136 to 50176 columns).  A 128-byte stage takes the
// longer of its four MMAs (N / 2 cycles each) and of a fill time that is mostly latency: about 330 cycles plus 0.8
// (two-CTA) or 1.05 (one-CTA) cycles per tile column, so narrow tiles cost almost as much per stage as wide ones and a
// deep mul wants the widest tile.  A 32-column chunk of the epilogue takes one warp about 900 cycles; with two warps
// per lane quarter a tile drains twice as fast, and with two epilogue groups (shallow depths) two tiles drain at once.
// The last tile's epilogue is not overlapped with anything, which is what makes narrower tiles win when a launch has
// only one or two rounds.
constexpr double kStageBaseCycles = 330.0;
constexpr double kStageCyclesPerColumnPair = 0.8;
constexpr double kStageCyclesPerColumnSingle = 1.05;
constexpr double kChunkCycles = 900.0;
constexpr double kHandoffCycles = 700.0;      // per tile: barrier round trips between producer, issuer and epilogue

// Estimated cycles of a launch that gives every unit `rounds` tiles of this shape.
double launch_cycles(long long rounds, int bn, bool pair, int depth, bool fuse, bool two_groups) {
  const int mma_n = bn + (fuse ? 16 : 0);
  const int k_blocks = (depth + kBlockKBytes - 1) / kBlockKBytes;
  const int last_steps = ((depth - (k_blocks - 1) * kBlockKBytes) + 31) / 32;   // K=32 steps of the last stage
  const double fill = kStageBaseCycles + (pair ? kStageCyclesPerColumnPair : kStageCyclesPerColumnSingle) * mma_n;
  const double mma_full = 4 * (mma_n / 2.0), mma_last = last_steps * (mma_n / 2.0);
  const double main_loop = (k_blocks - 1) * (mma_full > fill ? mma_full : fill) + (mma_last > fill ? mma_last : fill);
  const int chunks = (bn + 31) / 32;
  const double drain = two_groups ? chunks * kChunkCycles : chunks * kChunkCycles / 2.0;   // one tile, start to end
  const double drain_rate = two_groups ? drain / 2.0 : drain;                              // per tile in steady state
  const double steady = main_loop > drain_rate ? main_loop : drain_rate;
  return rounds * (steady + kHandoffCycles) + drain;
}

// force_pair: -1 = free choice, 0 = one-CTA tiles only, 1 = two-CTA tiles when the shape allows them.
// force_block_n: 0 = free choice, otherwise the widest candidate of at most that many columns is taken.
TileShape choose_tile_shape(int size_m, int size_n, int depth, bool fuse, bool pair_possible, int sm_count, int pairs_resident,
                            int force_pair, int force_block_n, bool two_groups) {
  TileShape best = {false, 0, 0.0};
  const int bn_cap = fuse ? kMaxBlockN - 16 : kMaxBlockN;
  const bool want_pair_only = force_pair > 0 && pair_possible;
  // widths tried: the cap, a few fixed steps below it, and the even split of the n dimension (256 columns as
  // 128 + 128 rather than 240 + 16 when the all-ones rows take 16 of the 256)
  const int even_tiles = (size_n + bn_cap - 1) / bn_cap;
  const int even_bn = ((size_n + even_tiles - 1) / even_tiles + 15) / 16 * 16;
  const int widths[] = {even_bn, 192, 128, 96, 64, 48, 32, 16};
  for (int p = 0; p < 2; p++) {
    const bool pair = p == 1;
    if (pair && (!pair_possible || force_pair == 0)) continue;
    if (!pair && want_pair_only) continue;
    const int units = pair ? pairs_resident : sm_count;
    const int unit_m = pair ? 2 * kBlockM : kBlockM;
    const long long tiles_m = (size_m + unit_m - 1) / unit_m;
    for (int bn : widths) {
      if (bn > even_bn) continue;                              // wider than the dimension needs
      if (pair && bn < 64) continue;                           // each CTA of a pair stages at least 32 rows
      if (force_block_n > 0 && bn > force_block_n && bn > 16) continue;
      const long long tiles = tiles_m * ((size_n + bn - 1) / bn);
      const long long rounds = (tiles + units - 1) / units;
      const double cycles = launch_cycles(rounds, bn, pair, depth, fuse, two_groups);
      // ties go to the larger tile, as in ruy (ruy/block_map.cc:410)
      if (best.block_n == 0 || cycles < best.cycles * 0.999) best = {pair, bn, cycles};
      if (force_block_n > 0) break;   // the widest admissible candidate of this kind
    }
  }
  return best;
}

}  // namespace

bool tc_i8_eligible(const SideView& m_side, const SideView& n_side) {
  const SideView* sides[2] = {&m_side, &n_side};
  for (const SideView* s : sides) {
    if (!is_8bit(s->dtype)) return false;
    if (s->stride_k != 1) return false;
    if (((uintptr_t)s->data & 15) != 0) return false;
    if (s->stride_w % 16 != 0 || s->stride_w <= 0) return false;
    if (s->width <= 0) return false;
  }
  return true;
}

cudaError_t launch_tc_i8(const TcI8Launch& L, cudaStream_t stream) {
  if (L.multicast) {
    const bool ok = (L.ep.dst_dtype == RUYB200_I8 || L.ep.dst_dtype == RUYB200_U8) && L.n_mirrors <= 0 &&
                    ((((uintptr_t)L.dst.data | (uintptr_t)L.multicast | (uintptr_t)L.dst.stride_m) & 15) == 0) &&
                    (L.dst.size_n & 15) == 0;
    if (!ok) return cudaErrorInvalidValue;
  }
  if (shallow_i8_eligible(L)) return launch_shallow_i8(L, stream);
  KernelArgs a;
  a.dst = L.dst;
  a.ep = L.ep;
  a.size_m = L.m_side.width;
  a.size_n = L.n_side.width;
  a.depth = L.depth;
  a.status = L.status;
  a.n_mirror = L.n_mirrors < 0 ? 0 : (L.n_mirrors > 7 ? 7 : L.n_mirrors);
  for (int i = 0; i < 7; i++) a.mirror[i] = i < a.n_mirror ? L.mirrors[i] : nullptr;
  a.multicast = L.multicast;
  a.store_maps = (L.store_maps != nullptr && a.n_mirror > 0 && L.multicast == nullptr && (L.ep.dst_dtype == RUYB200_I8 || L.ep.dst_dtype == RUYB200_U8))
                     ? (const CUtensorMap*)L.store_maps
                     : nullptr;
  a.mirror_wide = (((uintptr_t)L.dst.data | (uintptr_t)L.dst.stride_m) & 15) == 0;
  for (int i = 0; i < a.n_mirror; i++) a.mirror_wide = a.mirror_wide && ((uintptr_t)L.mirrors[i] & 15) == 0;
  a.debug = 0;
#ifdef RUYB200_DEBUG_KNOBS
  if (getenv("RUYB200_DEBUG")) a.debug = atoi(getenv("RUYB200_DEBUG"));
#endif
  a.n_xchg = L.n_xchg > 0 && L.xchg_remote && L.xchg_local && L.xchg_counter ? (L.n_xchg > 32 ? 32 : L.n_xchg) : 0;
  a.xchg_remote = L.xchg_remote;
  a.xchg_local = L.xchg_local;
  a.xchg_value = L.xchg_value;
  a.xchg_counter = L.xchg_counter;
  a.xchg_limit_ns = L.xchg_limit_ns;
  const uint32_t fmt_m = L.m_side.dtype == RUYB200_I8 ? 1u : 0u;
  const uint32_t fmt_n = L.n_side.dtype == RUYB200_I8 ? 1u : 0u;
  // The m-side zero-point sums can come out of the tensor core itself (an all-ones row appended to the n tile)
  // instead of a separate pass over the m operand; that variant runs with one CTA per tile.
  const bool fuse = L.fuse_sums_m && L.ep.zp_n != 0 && L.ep.sums_m == nullptr;
  const bool pair_possible = !fuse && L.allow_pair && a.size_m >= 256 && a.size_n >= 256 && L.sm_count >= 2;
  const int pairs_resident = pair_possible ? max_resident_pairs(L.sm_count) : 0;
  a.epi_groups = (L.depth <= 512 && L.n_mirrors <= 0 && !L.multicast) ? 2 : 1;
  const TileShape shape = choose_tile_shape(a.size_m, a.size_n, L.depth, fuse, pair_possible, L.sm_count, pairs_resident,
                                            L.force_pair, L.force_block_n, a.epi_groups == 2);
  const bool pair = shape.pair;
  const int bn = shape.block_n;
  a.block_n = bn;
  a.sums_col = fuse ? bn : -1;
  a.mma_n = fuse ? bn + 16 : bn;
  const int unit_m = pair ? 2 * kBlockM : kBlockM;
  a.tiles_m = (a.size_m + unit_m - 1) / unit_m;
  a.tiles_n = (a.size_n + bn - 1) / bn;
  a.acc_shift = a.mma_n <= 64 ? 3 : (a.mma_n <= 128 ? 2 : 1);
  a.acc_bufs = 1 << a.acc_shift;
  const bool dst8 = L.ep.dst_dtype == RUYB200_I8 || L.ep.dst_dtype == RUYB200_U8;
  a.pack_clamps = dst8 && L.ep.clamp_min >= -32768 && L.ep.clamp_max <= 32767 && L.ep.clamp_min <= L.ep.clamp_max;
  if (a.pack_clamps && L.ep.dst_dtype == RUYB200_U8 && L.ep.clamp_min == 0 && L.ep.clamp_max == 255) a.pack_clamps = 2;
  if (a.pack_clamps && L.ep.dst_dtype == RUYB200_I8 && L.ep.clamp_min == -128 && L.ep.clamp_max == 127) a.pack_clamps = 3;
  a.clamp_lo2 = ((uint32_t)L.ep.clamp_min & 0xffffu) * 0x10001u;
  a.clamp_hi2 = ((uint32_t)L.ep.clamp_max & 0xffffu) * 0x10001u;
  a.tight_wait = L.depth <= 512 ? 1 : 0;
#ifdef RUYB200_DEBUG_KNOBS
  if (getenv("RUYB200_TIGHT")) a.tight_wait = atoi(getenv("RUYB200_TIGHT"));
#endif
  // instruction descriptor: int32 accumulate, operand signedness, both operands depth-major,
  // N/8 at bit 17, M/16 at bit 24 (M spans both CTAs of a pair)
  a.idesc = (2u << 4) | (fmt_m << 7) | (fmt_n << 10) | ((uint32_t)(a.mma_n >> 3) << 17) | ((uint32_t)(unit_m >> 4) << 24);
  // Shallow operands use a narrower swizzle pattern: the copy engine then moves 32 or 64 bytes per row instead of
  // 128 (mostly out-of-range zero fill), which is what bounds tiles whose depth is a single MMA step or two.
  a.row_pitch = L.depth <= 32 ? 32 : (L.depth <= 64 ? 64 : 128);
#ifdef RUYB200_DEBUG_KNOBS
  const char* np_env = getenv("RUYB200_WIDE_ROWS");
  if (np_env && *np_env == '1') a.row_pitch = 128;
#endif
  // stride byte offset (8 rows) at bits 32..45, descriptor version 1 at bit 46, swizzle mode at bits 61..63 (2: 128 B, 4: 64 B, 6: 32 B)
  a.desc_hi = ((uint32_t)(8 * a.row_pitch) >> 4) | (1u << 14) | ((a.row_pitch == 128 ? 2u : (a.row_pitch == 64 ? 4u : 6u)) << 29);
  CUtensorMap map_m, map_n;
  if (!make_map(&map_m, L.m_side, L.depth, kBlockM, a.row_pitch) ||
      !make_map(&map_n, L.n_side, L.depth, pair ? bn / 2 : bn, a.row_pitch)) {
    return cudaErrorInvalidValue;
  }
  const long long tiles = (long long)a.tiles_m * a.tiles_n;
  if (L.info) {
    L.info->pair = pair;
    L.info->block_n = bn;
    L.info->tiles = (int)tiles;
    L.info->fused_sums = fuse;
    L.info->row_pitch = a.row_pitch;
    L.info->grid = 0;
    L.info->est_cycles = shape.cycles;
    L.info->shallow = 0;
  }
  if (pair) {
    // The tile schedule is static, so every pair must be resident from the start: size the grid
    // by the number of 2-CTA clusters the device can hold at once.
    int pairs = pairs_resident;
#ifdef RUYB200_DEBUG_KNOBS
    const char* env = getenv("RUYB200_PAIRS");
    if (env && atoi(env) > 0 && atoi(env) < pairs) pairs = atoi(env);
#endif
    const int grid = 2 * (int)(tiles < pairs ? tiles : pairs);
    return launch_by_type<true>(map_m, map_n, a, grid, stream);
  }
  const int grid = (int)(tiles < L.sm_count ? tiles : L.sm_count);
  return launch_by_type<false>(map_m, map_n, a, grid, stream);
}

}  // namespace ruyb200
