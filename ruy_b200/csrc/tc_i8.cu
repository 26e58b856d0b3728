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
//   * warps 2-9: epilogue.  Per tile the per-channel terms (bias, zero-point corrections,
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

#include "common.cuh"

namespace ruyb200 {

namespace {

constexpr int kBlockM = 128;          // TMEM lanes per tile
constexpr int kMaxBlockN = 256;       // accumulator columns per tile
constexpr int kBlockKBytes = 128;     // one swizzle atom of depth per stage
constexpr int kStages = 4;
constexpr int kABytes = kBlockM * kBlockKBytes;        // 16 KiB
constexpr int kBBytes = kMaxBlockN * kBlockKBytes;     // 32 KiB
constexpr int kStageBytes = kABytes + kBBytes;         // 48 KiB
constexpr int kSmemBytes = kStages * kStageBytes + 1024;  // + alignment slack
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;   // producer warp + MMA warp + epilogue warps
constexpr int kTmemCols = 512;
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
  int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
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

// Bounded wait.  Returns false if it gave up or if another role already raised the abort flag.
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

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
      : "memory");
}

// Shared-memory matrix descriptor for a depth-contiguous tile stored as rows of 128 bytes with
// the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte offset), the leading
// byte offset is unused for swizzled depth-major tiles, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void mma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.u32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
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

__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// AND-reduction of `ok` over the epilogue threads through named barrier 1.
__device__ __forceinline__ bool epilogue_all(bool ok) {
  uint32_t res;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(res)
      : "r"((uint32_t)ok), "n"(32 * kEpilogueWarps)
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

// Narrow and store 32 consecutive destination elements n0..n0+31 of row m.
template <int kDstBytes>
__device__ __forceinline__ void store_run32(const KernelArgs& a, int m, int n0, const int32_t* v) {
  char* base = (char*)a.dst.data + ((int64_t)m * a.dst.stride_m + n0) * kDstBytes;
  const bool full = n0 + 32 <= a.size_n;
  if (full && (((uintptr_t)base) & 15) == 0) {
    uint4* out = (uint4*)base;
    if (kDstBytes == 1) {
      uint32_t w[8];
#pragma unroll
      for (int q = 0; q < 8; q++) {
        w[q] = (uint32_t)(v[4 * q] & 0xff) | ((uint32_t)(v[4 * q + 1] & 0xff) << 8) |
               ((uint32_t)(v[4 * q + 2] & 0xff) << 16) | ((uint32_t)(v[4 * q + 3] & 0xff) << 24);
      }
      out[0] = make_uint4(w[0], w[1], w[2], w[3]);
      out[1] = make_uint4(w[4], w[5], w[6], w[7]);
    } else if (kDstBytes == 2) {
#pragma unroll
      for (int q = 0; q < 4; q++) {
        uint32_t w[4];
#pragma unroll
        for (int t = 0; t < 4; t++) {
          w[t] = (uint32_t)(v[8 * q + 2 * t] & 0xffff) | ((uint32_t)(v[8 * q + 2 * t + 1] & 0xffff) << 16);
        }
        out[q] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; q++) {
        out[q] = make_uint4((uint32_t)v[4 * q], (uint32_t)v[4 * q + 1], (uint32_t)v[4 * q + 2], (uint32_t)v[4 * q + 3]);
      }
    }
    return;
  }
  for (int q = 0; q < 32; q++) {
    if (n0 + q < a.size_n) store_int(a.dst, a.ep.dst_dtype, m, n0 + q, v[q]);
  }
}

// kDstBytes: 1 (int8/uint8), 2 (int16), 4 (int32: raw accumulators, no multiplier, no clamp).
// kX86: the two-step rounding of ruy's x86 kernels instead of the reference rounding.
template <int kDstBytes, bool kX86>
__global__ void __launch_bounds__(kThreads, 1)
tc_i8_kernel(const __grid_constant__ CUtensorMap map_m, const __grid_constant__ CUtensorMap map_n,
             const KernelArgs args) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t acc_full_bar[2];
  __shared__ __align__(8) uint64_t acc_empty_bar[2];
  __shared__ __align__(16) NTerms n_terms[2][kMaxBlockN];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int warp = threadIdx.x / 32;
  const int lane = threadIdx.x % 32;
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&acc_full_bar[b], 1);
      mbar_init(&acc_empty_bar[b], kEpilogueWarps);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const int num_tiles = args.tiles_m * args.tiles_n;
  const int k_blocks = (args.depth + kBlockKBytes - 1) / kBlockKBytes;
  volatile int* abortp = &abort_flag;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      const uint32_t stage_tx = (uint32_t)(kABytes + args.block_n * kBlockKBytes);
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int tm = tile / args.tiles_n;
        const int tn = tile % args.tiles_n;
        for (int kb = 0; kb < k_blocks; kb++, it++) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abortp)) {
            if (!*abortp) atomicCAS(args.status, 0, kTimeoutProducer);
            *abortp = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * kStageBytes;
          uint8_t* sb = sa + kABytes;
          mbar_expect_tx(&full_bar[s], stage_tx);
          tma_load_2d(sa, &map_m, kb * kBlockKBytes, tm * kBlockM, &full_bar[s]);
          tma_load_2d(sb, &map_n, kb * kBlockKBytes, tn * args.block_n, &full_bar[s]);
        }
      }
      if (!ok && it > 0) {
        // give copies that are still in flight a bounded chance to land before the CTA exits
        const uint32_t last = it - 1;
        for (uint32_t i = 0; i < kSpinLimit / 64; i++) {
          if (mbar_try_wait(&full_bar[last % kStages], (last / kStages) & 1)) break;
          __nanosleep(100);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t tcount = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tcount++) {
        const int buf = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&acc_empty_bar[buf], aph ^ 1, abortp)) {
          if (!*abortp) atomicCAS(args.status, 0, kTimeoutMma);
          *abortp = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(buf * kMaxBlockN);
        for (int kb = 0; kb < k_blocks; kb++, it++) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!mbar_wait(&full_bar[s], ph, abortp)) {
            if (!*abortp) atomicCAS(args.status, 0, kTimeoutMma);
            *abortp = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * kStageBytes);
          const uint32_t sb = sa + kABytes;
          const int rem = args.depth - kb * kBlockKBytes;
          const int ksteps = rem >= kBlockKBytes ? 4 : (rem + 31) / 32;
          for (int k = 0; k < ksteps; k++) {
            const uint64_t da = make_smem_desc(sa + k * 32);
            const uint64_t db = make_smem_desc(sb + k * 32);
            mma_i8(tmem_d, da, db, args.idesc, (kb | k) != 0);
          }
          mma_commit(&empty_bar[s]);   // frees the stage once these MMAs have read it
        }
        if (ok) mma_commit(&acc_full_bar[buf]);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    const Epilogue& ep = args.ep;
    const int ew = warp - 2;
    const int lane_group = warp % 4;       // the TMEM lane quarter this warp may read
    const int chunk_parity = ew / 4;       // the two warps of a lane quarter alternate 32-column chunks
    const int etid = threadIdx.x - 64;
    const bool ch_n = ep.channel_on_n != 0;
    const int32_t zz = ep.zp_m * ep.zp_n * ep.depth;
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, tcount++) {
      const int tm = tile / args.tiles_n;
      const int tn = tile % args.tiles_n;
      const int buf = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      // stage the per-n terms of this tile (overlaps the tile's main loop)
      NTerms* nt = n_terms[buf];
      for (int i = etid; i < args.block_n; i += 32 * kEpilogueWarps) {
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
        nt[i] = t;
      }
      // per-m terms of this thread's row
      const int m = tm * kBlockM + lane_group * 32 + lane;
      const bool m_ok = m < args.size_m;
      int32_t add_m = 0, mul_m = ep.mfp, exp_m = ep.mexp;
      if (m_ok) {
        if (ep.zp_n) add_m -= ep.zp_n * ep.sums_m[m];
        if (!ch_n) {
          if (ep.bias) add_m += ((const int32_t*)ep.bias)[m];
          if (ep.mfp_pc) mul_m = ep.mfp_pc[m];
          if (ep.mexp_pc) exp_m = ep.mexp_pc[m];
        }
      }
      if (!mbar_wait(&acc_full_bar[buf], aph, abortp)) {
        if (!*abortp) atomicCAS(args.status, 0, kTimeoutEpilogue);
        *abortp = 1;
        ok = false;
      }
      // One named-barrier reduction over all epilogue threads: it publishes the staged terms and
      // makes the continue/abort decision collective, so no warp is ever left waiting for another
      // that has already left the loop.
      ok = epilogue_all(ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + (uint32_t)(buf * kMaxBlockN);
      for (int c = chunk_parity * 32; c < args.block_n; c += 64) {
        const int n0 = tn * args.block_n + c;
        if (n0 >= args.size_n) break;   // uniform across the warp
        uint32_t r[32];
        tmem_ld_32(taddr + c, r);
        tmem_ld_wait();
        if (m_ok) {
          int32_t v[32];
#pragma unroll
          for (int q = 0; q < 32; q++) {
            const NTerms t = nt[c + q];
            int32_t x = (int32_t)(r[q] + (uint32_t)t.add + (uint32_t)add_m);
            if (kDstBytes != 4) {
              const int32_t mul = ch_n ? t.mul : mul_m;
              const int e = ch_n ? t.exp : exp_m;
              x = kX86 ? requant_x86(x, mul, e) : requant_reference(x, mul, e);
              x = (int32_t)((uint32_t)x + (uint32_t)ep.dst_zp);
              x = max(min(x, ep.clamp_max), ep.clamp_min);
            } else {
              x = (int32_t)((uint32_t)x + (uint32_t)ep.dst_zp);
            }
            v[q] = x;
          }
          store_run32<kDstBytes>(args, m, n0, v);
        }
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

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = (EncodeTiledFn)p;
    }
  }
  return fn;
}

// 2-D map over a width x depth byte matrix: dim0 = depth (contiguous), dim1 = width.
bool make_map(CUtensorMap* map, const SideView& s, int depth, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)depth, (cuuint64_t)s.width};
  cuuint64_t strides[1] = {(cuuint64_t)s.stride_w};
  cuuint32_t box[2] = {(cuuint32_t)kBlockKBytes, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(s.data), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool is_8bit(uint8_t dtype) { return dtype == RUYB200_I8 || dtype == RUYB200_U8; }

template <int kDstBytes, bool kX86>
cudaError_t launch_variant(const CUtensorMap& map_m, const CUtensorMap& map_n, const KernelArgs& a, int grid,
                           cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(tc_i8_kernel<kDstBytes, kX86>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kSmemBytes);
    if (e != cudaSuccess) return e;
    attr_set = true;
  }
  tc_i8_kernel<kDstBytes, kX86><<<grid, kThreads, kSmemBytes, stream>>>(map_m, map_n, a);
  return cudaGetLastError();
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
  KernelArgs a;
  a.dst = L.dst;
  a.ep = L.ep;
  a.size_m = L.m_side.width;
  a.size_n = L.n_side.width;
  a.depth = L.depth;
  int bn = (a.size_n + 15) / 16 * 16;
  if (bn > kMaxBlockN) bn = kMaxBlockN;
  a.block_n = bn;
  a.tiles_m = (a.size_m + kBlockM - 1) / kBlockM;
  a.tiles_n = (a.size_n + bn - 1) / bn;
  const uint32_t fmt_m = L.m_side.dtype == RUYB200_I8 ? 1u : 0u;
  const uint32_t fmt_n = L.n_side.dtype == RUYB200_I8 ? 1u : 0u;
  // instruction descriptor: int32 accumulate, operand signedness, both operands depth-major,
  // N/8 at bit 17, M/16 at bit 24
  a.idesc = (2u << 4) | (fmt_m << 7) | (fmt_n << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kBlockM >> 4) << 24);
  a.status = L.status;
  CUtensorMap map_m, map_n;
  if (!make_map(&map_m, L.m_side, L.depth, kBlockM) || !make_map(&map_n, L.n_side, L.depth, bn)) {
    return cudaErrorInvalidValue;
  }
  const long long tiles = (long long)a.tiles_m * a.tiles_n;
  const int grid = (int)(tiles < L.sm_count ? tiles : L.sm_count);
  const bool x86 = L.ep.rounding_x86 != 0;
  switch (L.ep.dst_dtype) {
    case RUYB200_I8:
    case RUYB200_U8:
      return x86 ? launch_variant<1, true>(map_m, map_n, a, grid, stream)
                 : launch_variant<1, false>(map_m, map_n, a, grid, stream);
    case RUYB200_I16:
      return x86 ? launch_variant<2, true>(map_m, map_n, a, grid, stream)
                 : launch_variant<2, false>(map_m, map_n, a, grid, stream);
    default:
      return launch_variant<4, false>(map_m, map_n, a, grid, stream);
  }
}

}  // namespace ruyb200
