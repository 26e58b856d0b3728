// 8-bit muls with a very shallow depth (32, 64 or 128) and a long activation side: the first pointwise-convolution
// layers of a mobile network, e.g. 64 x 32 x 802816.  Same arithmetic as the general tensor-core kernel
// (ruy/kernel_avx512.cc:55-626, ruy/kernel.h:213-237); what differs is how the activations travel.
//
// With depth 32 a row of the activation operand is 32 bytes.  Fetched as 128 rows x 32 bytes per tile, the copy engine
// handles 128 tiny rows for 4 KB, and every 8 KB of output costs a full round of barrier hand-offs.  But the rows are
// contiguous in memory (row stride == depth), so the operand is also a plain array of 128-byte lines, each holding F =
// 128 / depth consecutive rows.  This kernel fetches 128 such lines per stage (16 KB, 128 x F rows, one copy of 128-byte
// rows) and issues F MMAs on it: MMA q reads bytes [q * depth, (q + 1) * depth) of every line as its K extent (a
// descriptor start offset, exactly like a K step), so accumulator q holds the rows F * line + q.  One hand-off then
// covers F times the output, the copy engine moves full 128-byte rows, and a thread's F results are F consecutive
// destination rows, which it writes as one contiguous run.
//
//   warp 0     : TMA producer: the weights once, then one 16 KB stage of activation lines per tile
//   warp 1     : F x (depth / 32) tcgen05.mma kind::i8 per tile into F accumulators (M = 128 lines, N = weight rows)
//   warps 2-   : two epilogue groups of four or eight warps that take tiles in turn (one or two warps per tensor-memory
//                lane quarter; two split the rows of a line).  The zero-point sums of the activation rows
//                (ruy/pack.h:117-129) are taken from the stage in shared memory (each thread sums its own line),
//                which is why the epilogue, not the MMA, releases the stage.
//
// The kernel is bound by the epilogue's integer work, so the copy and MMA warps park in their waits (a suspend-time
// hint) instead of probing: probing warps took a quarter of the issued instructions from the epilogue warps that share
// their schedulers.  No cluster multicast; all mbarrier waits are bounded as in the general kernel.
#include <cuda.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace ruyb200 {

namespace {

constexpr int kLines = 128;                    // 128-byte lines per tile = TMEM lanes
constexpr int kStageBytes = kLines * 128;      // 16 KiB
constexpr int kStages = 8;
constexpr int kWeightBytes = 256 * 128;        // at most 256 weight rows x 128 bytes
constexpr int kSmemBytes = kStages * kStageBytes + kWeightBytes + 1024;
// Threads of a CTA with kWpq epilogue warps per lane quarter in each of the two epilogue groups.
constexpr int threads_for(int wpq) { return 64 + 2 * 4 * wpq * 32; }
constexpr int kTmemCols = 512;                 // two buffers of 256 columns: F accumulators of N columns each
constexpr int kMaxN = 256;
constexpr uint32_t kSpinLimit = 4u << 20;
constexpr int kMaxDevices = 64;

struct ShallowArgs {
  DstView dst;
  Epilogue ep;
  int size_m, size_n;
  int pitch;         // bytes per activation row = depth: 32, 64 or 128
  int fold;          // rows per 128-byte line: 128 / pitch
  int n_cols;        // accumulator columns per sub-accumulator: size_n rounded up to 16
  int num_tiles;
  uint32_t idesc;
  uint32_t desc_hi_b;   // high word of the weights' shared-memory descriptor (32-, 64- or 128-byte swizzle)
  int split_cols;       // two warps per lane quarter: 1 = they take alternate 32-column chunks, 0 = alternate rows of the line
  int m_signed;      // activations are int8 (else uint8)
  uint32_t clamp_lo2, clamp_hi2;
  int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
// The same probe with a suspend-time hint: the warp may stay parked for up to `ns` nanoseconds or until the phase
// completes.  For the roles whose hand-offs are not on the critical path (copy and MMA issue run several tiles ahead
// of the epilogue): a parked warp leaves the issue slots of its scheduler to the epilogue warps that share it.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_parked(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit / 16; i++) {
    if (mbar_try_wait_parked(bar, parity, 2000)) return true;
    if (*abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kSpinLimit; i++) {
    if (mbar_try_wait(bar, parity)) return true;
    if (i >= 2048) {
      if (*abort_flag) return false;
      __nanosleep(100);
    }
  }
  return false;
}
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
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
// activation lines: 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart, descriptor version 1
constexpr uint32_t kDescHiA = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3FFFF) >> 4) | (1u << 16); }
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
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, with the 32 registers of an earlier load as in/out operands: code that reads them cannot be moved
// above the wait, which matters once a load stays in flight while other values are processed.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]), "+r"(r[9]),
                 "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]),
                 "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]),
                 "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Narrows 32 int32 values to bytes (8 words); with `clamp`, two values at a time are saturated to 16 bits and clamped.
__device__ __forceinline__ void narrow_u8x32(const uint32_t* v, bool clamp, uint32_t lo2, uint32_t hi2, uint32_t* w) {
  if (clamp) {
#pragma unroll
    for (int q = 0; q < 8; q++) {
      uint32_t a, b;
      asm("cvt.pack.sat.s16.s32 %0, %1, %2;" : "=r"(a) : "r"((int32_t)v[4 * q + 1]), "r"((int32_t)v[4 * q]));
      asm("cvt.pack.sat.s16.s32 %0, %1, %2;" : "=r"(b) : "r"((int32_t)v[4 * q + 3]), "r"((int32_t)v[4 * q + 2]));
      a = __vmaxs2(__vmins2(a, hi2), lo2);
      b = __vmaxs2(__vmins2(b, hi2), lo2);
      w[q] = __byte_perm(a, b, 0x6420);
    }
  } else {
#pragma unroll
    for (int q = 0; q < 8; q++) {
      w[q] = (v[4 * q] & 0xff) | ((v[4 * q + 1] & 0xff) << 8) | ((v[4 * q + 2] & 0xff) << 16) | ((v[4 * q + 3] & 0xff) << 24);
    }
  }
}

// kMulPerN: the multipliers vary along the accumulator columns (per-channel multipliers with the channels on n); a
// variant of its own because its column terms need many more registers.
// Narrows 32 int32 values to bytes with saturation to the destination type's range (two instructions per word).
__device__ __forceinline__ void narrow_sat_x32(const uint32_t* v, bool to_unsigned, uint32_t* w) {
#pragma unroll
  for (int q = 0; q < 8; q++) {
    uint32_t hi, d;
    if (to_unsigned) {
      asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"((int32_t)v[4 * q + 3]), "r"((int32_t)v[4 * q + 2]), "r"(0u));
      asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"((int32_t)v[4 * q + 1]), "r"((int32_t)v[4 * q]), "r"(hi));
    } else {
      asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"((int32_t)v[4 * q + 3]), "r"((int32_t)v[4 * q + 2]), "r"(0u));
      asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"((int32_t)v[4 * q + 1]), "r"((int32_t)v[4 * q]), "r"(hi));
    }
    w[q] = d;
  }
}

// kWpq: epilogue warps per lane quarter within a group (1 or 2); two split the rows of a line between them.  Measured
// on 64 x 32 x 802816 (four rows per line): 33.9 us with two, 37.1 us with one; on 128 x 64 x 200704 (two rows per
// line, five tiles per CTA): 21.4 against 20.7 us.  The launcher takes two when a line holds four rows.
template <bool kX86, bool kMulPerN, int kWpq>
__global__ void __launch_bounds__(threads_for(kWpq), 1)
shallow_i8_kernel(const __grid_constant__ CUtensorMap map_lines, const __grid_constant__ CUtensorMap map_w, const ShallowArgs args) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t acc_full_bar[2];
  __shared__ __align__(8) uint64_t acc_empty_bar[2];
  __shared__ __align__(8) uint64_t weights_bar;
  // per-n (weight row) terms: the addends alone (four per load on the common path), and {addend, multiplier, rounding
  // term of the short form (+ destination zero point), total shift - 32} for multipliers that vary along n
  __shared__ __align__(16) int32_t nt_add[kMaxN];
  __shared__ __align__(16) int4 nt4[kMaxN];
  __shared__ int all_n_fast;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  constexpr int kWarpsPerQuarter = kWpq;
  constexpr int kGroupWarps = 4 * kWpq;
  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* w_tile = smem + kStages * kStageBytes;
  const Epilogue& ep = args.ep;
  const bool ch_n = ep.channel_on_n != 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kGroupWarps);     // the warps of the epilogue group that drained the tile
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&acc_full_bar[b], 1);
      mbar_init(&acc_empty_bar[b], kGroupWarps);
    }
    mbar_init(&weights_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // the per-n terms are the same for every tile (there is one n tile): stage them once
  if (threadIdx.x == 0) all_n_fast = 1;
  __syncthreads();
  for (int n = threadIdx.x; n < kMaxN; n += threads_for(kWpq)) {
    int32_t add = ep.zp_m * ep.zp_n * ep.depth, mul = ep.mfp, e = ep.mexp;
    if (n < args.size_n) {
      if (ep.zp_m) add -= ep.zp_m * ep.sums_n[n];
      if (ch_n) {
        if (ep.bias) add += ((const int32_t*)ep.bias)[n];
        if (ep.mfp_pc) mul = ep.mfp_pc[n];
        if (ep.mexp_pc) e = ep.mexp_pc[n];
      }
    }
    const int sh = 31 - e;
    const bool fast = sh >= 33 && sh <= 45 && ep.dst_zp > -32768 && ep.dst_zp < 32768;
    if (!fast && n < args.size_n) all_n_fast = 0;
    nt_add[n] = add;
    nt4[n] = make_int4(add, mul, (int32_t)(1u << ((sh - 33) & 31)) + ep.dst_zp * (int32_t)(1u << ((sh - 32) & 31)), sh - 32);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;
  const int num_tiles = args.num_tiles;
  const int fold = args.fold, pitch = args.pitch, n_cols = args.n_cols;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      mbar_expect_tx(&weights_bar, (uint32_t)(n_cols * pitch));
      tma_load_2d(w_tile, &map_w, 0, 0, &weights_bar);
      uint32_t s = 0, ph = 0, issued = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait_parked(&empty_bar[s], ph ^ 1, abortp)) {
          if (!*abortp) atomicCAS(args.status, 0, 1);
          *abortp = 1;
          ok = false;
          break;
        }
        mbar_expect_tx(&full_bar[s], (uint32_t)kStageBytes);
        tma_load_2d(smem + s * kStageBytes, &map_lines, 0, tile * kLines, &full_bar[s]);
        issued++;
        if (++s == kStages) { s = 0; ph ^= 1; }
      }
      if (!ok && issued > 0) {
        const uint32_t last = issued - 1;
        for (uint32_t i = 0; i < kSpinLimit / 64; i++) {
          if (mbar_try_wait(&full_bar[last % kStages], (last / kStages) & 1)) break;
          __nanosleep(100);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    bool ok = mbar_wait(&weights_bar, 0, abortp);
    if (!ok && lane == 0) {
      if (!*abortp) atomicCAS(args.status, 0, 2);
      *abortp = 1;
    }
    uint32_t s = 0, ph = 0, tcount = 0;
    const uint32_t lo_a0 = desc_lo(smem_u32(smem));
    const uint32_t lo_b = desc_lo(smem_u32(w_tile));
    const int ksteps = pitch / 32;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tcount++) {
      const uint32_t buf = tcount & 1, aph = (tcount >> 1) & 1;
      if (!mbar_wait_parked(&acc_empty_bar[buf], aph ^ 1, abortp) || !mbar_wait_parked(&full_bar[s], ph, abortp)) {
        if (!*abortp) atomicCAS(args.status, 0, 2);
        *abortp = 1;
        break;
      }
      tc_fence_after();
      const uint32_t lo_a = lo_a0 + s * ((uint32_t)kStageBytes >> 4);
      if (elect_one()) {
        for (int q = 0; q < fold; q++) {
          const uint32_t tmem_d = tmem_base + buf * 256u + (uint32_t)(q * n_cols);
          for (int k = 0; k < ksteps; k++) {
            // row q of every line: its bytes start q * pitch into the line; a K step is another 32 bytes (+2 in the descriptor)
            mma_i8(tmem_d, lo_a + (uint32_t)((q * pitch) >> 4) + 2u * k, kDescHiA, lo_b + 2u * k, args.desc_hi_b, args.idesc, k != 0);
          }
        }
        mma_commit(&acc_full_bar[buf]);
      }
      __syncwarp();
      if (++s == kStages) { s = 0; ph ^= 1; }
    }
  } else {
    // ---------------- epilogue: two groups take tiles in turn ----------------
    const int ew = warp - 2;
    const int group = ew / kGroupWarps;
    const int quarter = warp % 4;             // TMEM lane quarter this warp may read
    const int half = (ew % kGroupWarps) / 4;  // which of the warps of this quarter in the group: it takes rows half, half + kWarpsPerQuarter, ...
    const int line_in_tile = quarter * 32 + lane;
    const int32_t cmin = ep.clamp_min, cmax = ep.clamp_max;
    // 8-bit destinations: the clamp bounds fit 16 bits, so the bounds are applied to two values at a time while narrowing
    // (min with the upper bound first, then max with the lower one: the order of ruy/kernel.h:232-233)
    constexpr bool late_clamp = true;
    constexpr bool mul_per_n = kMulPerN;
    const bool zp_small = ep.dst_zp > -32768 && ep.dst_zp < 32768;
    // clamp bounds equal to the destination type's range: the saturating narrowing alone applies them
    const bool full_range = ep.dst_dtype == RUYB200_U8 ? (cmin == 0 && cmax == 255) : (cmin == -128 && cmax == 127);
    const bool dst_unsigned = ep.dst_dtype == RUYB200_U8;
    const int chunks = (args.size_n + 31) / 32;
    const bool split_cols = kWpq > 1 && args.split_cols != 0;
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tcount++) {
      if ((int)(tcount & 1) != group) continue;        // the other group's tile
      const uint32_t buf = tcount & 1, aph = (tcount >> 1) & 1;
      const uint32_t s = tcount % kStages, sph = (tcount / kStages) & 1;
      if (!mbar_wait_warp(&acc_full_bar[buf], aph, abortp)) {
        if (lane == 0) {
          if (!*abortp) atomicCAS(args.status, 0, 3);
          *abortp = 1;
        }
        ok = false;
      }
      if (!ok) break;
      tc_fence_after();
      // the stage's bytes were written by the copy engine: observing its barrier orders them before these reads
      mbar_try_wait(&full_bar[s], sph);
      // (Keeping a second tensor-memory load in flight while a piece is processed was measured and dropped: 38.8 us
      // against 37.1 us on 64 x 32 x 802816; the registers it takes are worth more as a second warp per quarter.)
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * 256u;
      // this warp's pieces: with two warps per quarter either alternate rows of the line or alternate column chunks
      const int q_first = split_cols ? 0 : half, q_step = split_cols ? 1 : kWarpsPerQuarter;
      const int c_first = split_cols ? 32 * half : 0, c_step = split_cols ? 32 * kWarpsPerQuarter : 32;
      const int n_pieces = ((fold - q_first + q_step - 1) / q_step) * ((chunks * 32 - c_first + c_step - 1) / c_step);
      uint32_t ra[32];
      int q_ld = q_first, c_ld = c_first;      // the piece the next load fetches
      auto issue_load = [&](uint32_t* r) {
        tmem_ld_32(taddr + (uint32_t)(q_ld * n_cols + c_ld), r);
        c_ld += c_step;
        if (c_ld >= chunks * 32) { c_ld = c_first; q_ld += q_step; }
      };

      const long long line = (long long)tile * kLines + line_in_tile;
      const int m0 = (int)(line * fold);
      // Per-row terms of this thread's rows: the zero-point sum comes from the thread's own line in shared memory
      // (16-byte piece j of line r sits at j ^ (r & 7)); the multiplier is reduced to the constants of the short form
      // result = (mulhi(x, mul) + rnd) >> sh, valid for a total shift of 33..45 bits, where it is exact:
      // (x * mul + 2^(s-1)) >> s == (hi32(x * mul) + 2^(s-33)) >> (s - 32), and the zero point rides in rnd.
      int32_t add_q[4], mul_q[4], exp_q[4], rnd_q[4];
      bool fast_lane = !kX86 && zp_small;
      {
        const uint8_t* lp = smem + s * kStageBytes + line_in_tile * 128;
        const int per_row = pitch / 16;
#pragma unroll
        for (int q = 0; q < 4; q++) {
          add_q[q] = 0;
          mul_q[q] = ep.mfp;
          exp_q[q] = ep.mexp;
          if (q < fold && (split_cols || (q % kWarpsPerQuarter) == half)) {
            const int m = m0 + q;
            if (ep.zp_n) {
              int32_t sum = 0;
              for (int j = 0; j < per_row; j++) {
                const uint4 v = *reinterpret_cast<const uint4*>(lp + (((q * per_row + j) ^ (line_in_tile & 7)) << 4));
                if (args.m_signed) {
                  sum = __dp4a((int)v.x, 0x01010101, sum);
                  sum = __dp4a((int)v.y, 0x01010101, sum);
                  sum = __dp4a((int)v.z, 0x01010101, sum);
                  sum = __dp4a((int)v.w, 0x01010101, sum);
                } else {
                  sum = (int)__dp4a(v.x, 0x01010101u, (unsigned)sum);
                  sum = (int)__dp4a(v.y, 0x01010101u, (unsigned)sum);
                  sum = (int)__dp4a(v.z, 0x01010101u, (unsigned)sum);
                  sum = (int)__dp4a(v.w, 0x01010101u, (unsigned)sum);
                }
              }
              add_q[q] = -ep.zp_n * sum;
            }
            if (!ch_n && m < args.size_m) {
              if (ep.bias) add_q[q] += ((const int32_t*)ep.bias)[m];
              if (ep.mfp_pc) mul_q[q] = ep.mfp_pc[m];
              if (ep.mexp_pc) exp_q[q] = ep.mexp_pc[m];
            }
          }
          const int sh = 31 - exp_q[q];
          fast_lane = fast_lane && sh >= 33 && sh <= 45;
          rnd_q[q] = (int32_t)(1u << ((sh - 33) & 31)) + ep.dst_zp * (int32_t)(1u << ((sh - 32) & 31));
        }
      }
      const bool fast_m = __all_sync(0xffffffffu, fast_lane) != 0;
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);       // the stage may be refilled
      // The pieces of the tile in order (row q of the line, 32 columns from c), results replacing the accumulators
      // in the registers that held them.
      int q = q_first, c = c_first;
      auto process = [&](uint32_t* r) {
        const int m = m0 + q;
        const bool m_ok = m < args.size_m;
        int32_t addm = add_q[0], mulm = mul_q[0], expm = exp_q[0], rndm = rnd_q[0];
#pragma unroll
        for (int t = 1; t < 4; t++) {
          if (q == t) { addm = add_q[t]; mulm = mul_q[t]; expm = exp_q[t]; rndm = rnd_q[t]; }
        }
        if (m_ok) {
          if (!kX86 && (mul_per_n ? all_n_fast != 0 : fast_m)) {
            const int sh_hi = (31 - expm - 32) & 31;
#pragma unroll
            for (int j4 = 0; j4 < 8; j4++) {
              if (mul_per_n) {
#pragma unroll
                for (int t = 0; t < 4; t++) {
                  const int4 nt = nt4[c + 4 * j4 + t];
                  const int32_t x = (int32_t)(r[4 * j4 + t] + (uint32_t)nt.x + (uint32_t)addm);
                  const int32_t y = (__mulhi(x, nt.y) + nt.z) >> nt.w;
                  r[4 * j4 + t] = (uint32_t)(late_clamp ? y : max(min(y, cmax), cmin));
                }
              } else {
                const int4 ad = *reinterpret_cast<const int4*>(&nt_add[c + 4 * j4]);
                const int32_t adds[4] = {ad.x, ad.y, ad.z, ad.w};
#pragma unroll
                for (int t = 0; t < 4; t++) {
                  const int32_t x = (int32_t)(r[4 * j4 + t] + (uint32_t)adds[t] + (uint32_t)addm);
                  const int32_t y = (__mulhi(x, mulm) + rndm) >> sh_hi;
                  r[4 * j4 + t] = (uint32_t)(late_clamp ? y : max(min(y, cmax), cmin));
                }
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const int4 nt = nt4[c + j];
              int32_t x = (int32_t)(r[j] + (uint32_t)nt_add[c + j] + (uint32_t)addm);
              const int32_t mul = mul_per_n ? nt.y : mulm;
              const int e = mul_per_n ? -1 - nt.w : expm;     // nt.w holds 31 - e - 32
              x = kX86 ? requant_x86(x, mul, e) : requant_reference(x, mul, e);
              x = (int32_t)((uint32_t)x + (uint32_t)ep.dst_zp);
              r[j] = (uint32_t)(late_clamp ? x : max(min(x, cmax), cmin));
            }
          }
          uint8_t* out = (uint8_t*)args.dst.data + (int64_t)m * args.dst.stride_m + c;
          if (c + 32 <= args.size_n && (((uintptr_t)out) & 15) == 0) {
            uint32_t w[8];
            if (full_range) narrow_sat_x32(r, dst_unsigned, w);
            else narrow_u8x32(r, late_clamp, args.clamp_lo2, args.clamp_hi2, w);
            __stcs(reinterpret_cast<uint4*>(out), make_uint4(w[0], w[1], w[2], w[3]));
            __stcs(reinterpret_cast<uint4*>(out) + 1, make_uint4(w[4], w[5], w[6], w[7]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; j++) {
              if (c + j < args.size_n) out[j] = (uint8_t)(late_clamp ? max(min((int32_t)r[j], cmax), cmin) : (int32_t)r[j]);
            }
          }
        }
        c += c_step;
        if (c >= chunks * 32) { c = c_first; q += q_step; }
        __syncwarp();   // the next tensor-memory instruction is warp-wide
      };
      for (int piece = 0; piece < n_pieces; piece++) {
        issue_load(ra);
        tmem_ld_wait_for(ra);
        process(ra);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty_bar[buf]);
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
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

bool make_map(CUtensorMap* map, const void* base, uint64_t inner, uint64_t outer, uint64_t stride_bytes, uint32_t box_inner,
              uint32_t box_outer, CUtensorMapSwizzle swizzle) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool is_8bit(uint8_t dtype) { return dtype == RUYB200_I8 || dtype == RUYB200_U8; }

}  // namespace

bool shallow_i8_eligible(const TcI8Launch& L) {
  const int depth = L.depth;
  if (depth != 32 && depth != 64 && depth != 128) return false;
  if (L.n_mirrors > 0 || L.n_xchg > 0 || L.multicast != nullptr) return false;
  if (!is_8bit(L.m_side.dtype) || !is_8bit(L.n_side.dtype)) return false;
  if (L.ep.dst_dtype != RUYB200_I8 && L.ep.dst_dtype != RUYB200_U8) return false;
  // activation rows back to back, so that 128 bytes hold 128 / depth whole rows
  if (L.m_side.stride_k != 1 || L.m_side.stride_w != depth || ((uintptr_t)L.m_side.data & 15) != 0) return false;
  const int fold = 128 / depth;
  // whole lines only, and enough of them that every SM gets a few 128-line tiles (else the general kernel's smaller
  // tiles spread the work better)
  if (L.m_side.width % fold != 0 || (long long)L.m_side.width < 2ll * L.sm_count * kLines * fold) return false;
  if (!L.allow_shallow) return false;
  if (L.n_side.stride_k != 1 || (L.n_side.stride_w & 15) != 0 || ((uintptr_t)L.n_side.data & 15) != 0) return false;
  const int n_cols = (L.n_side.width + 15) / 16 * 16;
  if (L.n_side.width < 1 || n_cols > kMaxN || fold * n_cols > 256) return false;
  // the zero-point sums of the weights must come with the launch when the activations' zero point needs them
  if (L.ep.zp_m != 0 && L.ep.sums_n == nullptr) return false;
  return true;
}

cudaError_t launch_shallow_i8(const TcI8Launch& L, cudaStream_t stream) {
  ShallowArgs a;
  a.dst = L.dst;
  a.ep = L.ep;
  a.size_m = L.m_side.width;
  a.size_n = L.n_side.width;
  a.pitch = L.depth;
  a.fold = 128 / L.depth;
  a.n_cols = (a.size_n + 15) / 16 * 16;
  const long long lines = (long long)a.size_m / a.fold;
  a.num_tiles = (int)((lines + kLines - 1) / kLines);
  const uint32_t fmt_m = L.m_side.dtype == RUYB200_I8 ? 1u : 0u;
  const uint32_t fmt_n = L.n_side.dtype == RUYB200_I8 ? 1u : 0u;
  a.m_signed = (int)fmt_m;
  // int32 accumulate, operand signedness, both operands depth-major, N / 8 at bit 17, M / 16 at bit 24
  a.idesc = (2u << 4) | (fmt_m << 7) | (fmt_n << 10) | ((uint32_t)(a.n_cols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
  // weights: rows of `pitch` bytes with the matching swizzle (mode 4: 64 bytes, 6: 32 bytes), 8-row groups 8 * pitch apart
  a.desc_hi_b = ((uint32_t)(8 * a.pitch) >> 4) | (1u << 14) | ((a.pitch == 128 ? 2u : (a.pitch == 64 ? 4u : 6u)) << 29);
  a.clamp_lo2 = ((uint32_t)L.ep.clamp_min & 0xffffu) * 0x10001u;
  a.clamp_hi2 = ((uint32_t)L.ep.clamp_max & 0xffffu) * 0x10001u;
  a.status = L.status;
  CUtensorMap map_lines, map_w;
  if (!make_map(&map_lines, L.m_side.data, 128, (uint64_t)lines, 128, 128, kLines, CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_map(&map_w, L.n_side.data, (uint64_t)L.depth, (uint64_t)a.size_n, (uint64_t)L.n_side.stride_w, (uint32_t)a.pitch,
                (uint32_t)a.n_cols,
                a.pitch == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : (a.pitch == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B))) {
    return cudaErrorInvalidValue;
  }
  const bool x86 = L.ep.rounding_x86 != 0;
  const bool mul_per_n = L.ep.channel_on_n != 0 && (L.ep.mfp_pc != nullptr || L.ep.mexp_pc != nullptr);
  // two warps per lane quarter when a line holds four rows; the per-column-multiplier variant would spill at the 96
  // registers that 18 warps leave per thread and stays with one
  const int chunks = (a.size_n + 31) / 32;
  int wpq = (a.fold >= 4 && !mul_per_n) ? 2 : 1;
  a.split_cols = 0;
  if (a.fold == 1 && !mul_per_n && chunks >= 4 && chunks % 2 == 0) {   // one row per line: the two warps share its columns
    wpq = 2;
    a.split_cols = 1;
  }
  if (const char* env = getenv("RUYB200_SHALLOW_WPQ")) {               // measurement knob: 1 = one warp per quarter always
    if (atoi(env) == 1) { wpq = 1; a.split_cols = 0; }
  }
  typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const ShallowArgs);
  static const KernelFn kernels[2][3] = {
      {shallow_i8_kernel<false, false, 1>, shallow_i8_kernel<false, false, 2>, shallow_i8_kernel<false, true, 1>},
      {shallow_i8_kernel<true, false, 1>, shallow_i8_kernel<true, false, 2>, shallow_i8_kernel<true, true, 1>}};
  const int variant = mul_per_n ? 2 : wpq - 1;
  const KernelFn kernel = kernels[x86][variant];
  {
    static std::mutex mu;
    static bool attr_set[kMaxDevices][2][3] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= kMaxDevices || !attr_set[dev][x86][variant]) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < kMaxDevices) attr_set[dev][x86][variant] = true;
    }
  }
  const int grid = a.num_tiles < L.sm_count ? a.num_tiles : L.sm_count;
  if (L.info) {
    L.info->pair = 0;
    L.info->block_n = a.n_cols;
    L.info->tiles = a.num_tiles;
    L.info->fused_sums = 1;
    L.info->row_pitch = a.pitch;
    L.info->grid = grid;
    L.info->est_cycles = 0.0;
    L.info->shallow = a.fold;
  }
  kernel<<<grid, threads_for(wpq), kSmemBytes, stream>>>(map_lines, map_w, a);
  return cudaGetLastError();
}

}  // namespace ruyb200
