// fp32 matmul on the tensor core: ruy's KernelFloat* (ruy/kernel_avx512.cc:872-1236, ruy/kernel_x86.h:598-805)
// for shapes large enough to fill tiles, at fp32 accuracy.
//
// The tensor core multiplies TF32 (11 significant bits).  Each operand is therefore split once, by a small pre-pass,
// into hi = tf32(x) and lo = tf32(x - hi); both halves are exact TF32 numbers, every product of two halves is exact
// in fp32, and  a*b ~= lo_a*hi_b + hi_a*lo_b + hi_a*hi_b  drops only the lo*lo term (relative 2^-22).  The pre-pass
// also brings any storage order into depth-contiguous rows padded to 32 floats (ruy's packing, ruy/pack.h:105-151).
//
// What limits accuracy is then the accumulation: the tensor core adds into its fp32 accumulator with truncation, and
// a chain over the whole depth would drift past the 1e-5 this library promises.  So the chain is kept short: every
// 128-byte stage (32 floats of depth, 12 MMAs) starts a fresh accumulator in tensor memory, and the epilogue warps
// fold the finished stage into register sums with a compensated (Kahan) add while the next stage is being multiplied
// into the other accumulator buffer.  The register sums play the role of the running total in ruy's kernel; bias and
// clamp (ruy/kernel_x86.h:700-760) are applied when the tile is complete.
//
//   warp 0     : TMA producer (hi and lo tiles of both operands per stage; no cluster multicast)
//   warp 1     : issues tcgen05.mma kind::tf32, M=128, N<=128, K=8; ping-pongs between two accumulator buffers per stage
//   warps 2-9  : fold stages into registers; each warp owns one lane quarter and every other 32-column chunk
//
// All mbarrier waits are bounded, as in the 8-bit kernel: a wait that gives up writes a code to *status, raises a
// CTA-wide abort flag, every role leaves its loops, tensor memory is released and the kernel returns.
#include <cuda.h>

#include <cstring>
#include <mutex>

#include "common.cuh"

namespace ruyb200 {

namespace {

constexpr int kBlockM = 128;
constexpr int kMaxBlockN = 128;
constexpr int kStageFloats = 32;                       // 128 bytes of depth
constexpr int kTileBytes = 128 * 128;                  // one half (hi or lo) of one operand: 128 rows x 128 bytes
constexpr int kStageBytes = 4 * kTileBytes;            // a_hi, a_lo, b_hi, b_lo
constexpr int kStages = 3;
constexpr int kSmemBytes = kStages * kStageBytes + 1024;
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kTmemCols = 256;                         // two accumulator buffers of 128 columns
constexpr uint32_t kSpinLimit = 4u << 20;
constexpr int kMaxDevices = 64;

struct F32Args {
  DstView dst;
  Epilogue ep;
  int size_m, size_n;
  int k_blocks;      // stages per tile
  int block_n;       // multiple of 16, <= 128
  int tiles_m, tiles_n;
  uint32_t idesc;
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
// Bounded wait of one thread.
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
// Bounded wait of a converged warp: every lane probes, no sleep (the shortest wake-up).
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
// Shared-memory matrix descriptor of a depth-contiguous tile of 128-byte rows with the 128-byte swizzle: 8-row groups
// 1024 bytes apart, descriptor version 1 at bit 46, swizzle mode 2 at bits 61..63.
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr) { return ((smem_addr & 0x3FFFF) >> 4) | (1u << 16); }

// The four K=8 MMAs that cover one 128-byte stage of one product (descriptors advance by 32 bytes = +2).
__device__ __forceinline__ void mma_tf32_x4(uint32_t tmem_d, uint32_t lo_a, uint32_t lo_b, uint32_t idesc, uint32_t first_accumulates) {
  asm volatile(
      "{\n\t.reg .pred p, t;\n\t.reg .b64 da, db;\n\t.reg .b32 la, lb;\n\t"
      "setp.ne.u32 p, %4, 0;\n\t"
      "setp.eq.u32 t, 0, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\tmov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %3, p;\n\t"
      "add.u32 la, %1, 2;\n\tadd.u32 lb, %2, 2;\n\tmov.b64 da, {la, %5};\n\tmov.b64 db, {lb, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %3, t;\n\t"
      "add.u32 la, %1, 4;\n\tadd.u32 lb, %2, 4;\n\tmov.b64 da, {la, %5};\n\tmov.b64 db, {lb, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %3, t;\n\t"
      "add.u32 la, %1, 6;\n\tadd.u32 lb, %2, 6;\n\tmov.b64 da, {la, %5};\n\tmov.b64 db, {lb, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], da, db, %3, t;\n\t}"
      ::"r"(tmem_d), "r"(lo_a), "r"(lo_b), "r"(idesc), "r"(first_accumulates), "r"(kDescHi)
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
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// AND-reduction of `ok` over the epilogue threads (named barrier 1).
__device__ __forceinline__ bool epilogue_all(bool ok) {
  uint32_t res;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(res)
      : "r"((uint32_t)ok), "r"(32 * kEpilogueWarps)
      : "memory");
  return res != 0;
}

__global__ void __launch_bounds__(kThreads, 1)
tc_f32_kernel(const __grid_constant__ CUtensorMap map_a_hi, const __grid_constant__ CUtensorMap map_a_lo,
              const __grid_constant__ CUtensorMap map_b_hi, const __grid_constant__ CUtensorMap map_b_lo, const F32Args args) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kStages];
  __shared__ __align__(8) uint64_t empty_bar[kStages];
  __shared__ __align__(8) uint64_t acc_full_bar[2];
  __shared__ __align__(8) uint64_t acc_empty_bar[2];
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
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  volatile int* abortp = &abort_flag;
  const int num_tiles = args.tiles_m * args.tiles_n;
  const int k_blocks = args.k_blocks;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t s = 0, ph = 0, issued = 0;
      const uint32_t stage_tx = (uint32_t)(2 * (kBlockM + args.block_n) * 128);
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int row_m = (tile / args.tiles_n) * kBlockM;
        const int row_n = (tile % args.tiles_n) * args.block_n;
        for (int kb = 0; kb < k_blocks; kb++) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abortp)) {
            if (!*abortp) atomicCAS(args.status, 0, 1);
            *abortp = 1;
            ok = false;
            break;
          }
          uint8_t* st = smem + s * kStageBytes;
          mbar_expect_tx(&full_bar[s], stage_tx);
          tma_load_2d(st, &map_a_hi, kb * kStageFloats, row_m, &full_bar[s]);
          tma_load_2d(st + kTileBytes, &map_a_lo, kb * kStageFloats, row_m, &full_bar[s]);
          tma_load_2d(st + 2 * kTileBytes, &map_b_hi, kb * kStageFloats, row_n, &full_bar[s]);
          tma_load_2d(st + 3 * kTileBytes, &map_b_lo, kb * kStageFloats, row_n, &full_bar[s]);
          issued++;
          if (++s == kStages) { s = 0; ph ^= 1; }
        }
      }
      if (!ok && issued > 0) {
        // give copies that are still in flight a bounded chance to land before the CTA exits
        const uint32_t last = issued - 1;
        for (uint32_t i = 0; i < kSpinLimit / 64; i++) {
          if (mbar_try_wait(&full_bar[last % kStages], (last / kStages) & 1)) break;
          __nanosleep(100);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one accumulator buffer per stage, alternating ----------------
    uint32_t s = 0, ph = 0, stage_count = 0;
    bool ok = true;
    const uint32_t lo0 = desc_lo(smem_u32(smem));
    const uint32_t stage_step = (uint32_t)kStageBytes >> 4, tile_step = (uint32_t)kTileBytes >> 4;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      for (int kb = 0; kb < k_blocks; kb++, stage_count++) {
        const uint32_t b = stage_count & 1, aph = (stage_count >> 1) & 1;
        if (!mbar_wait(&acc_empty_bar[b], aph ^ 1, abortp) || !mbar_wait(&full_bar[s], ph, abortp)) {
          if (!*abortp) atomicCAS(args.status, 0, 2);
          *abortp = 1;
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_hi = lo0 + s * stage_step, a_lo = a_hi + tile_step, b_hi = a_hi + 2 * tile_step, b_lo = a_hi + 3 * tile_step;
        const uint32_t tmem_d = tmem_base + b * (uint32_t)kMaxBlockN;
        if (elect_one()) {
          // the two small products first, then the large one
          mma_tf32_x4(tmem_d, a_lo, b_hi, args.idesc, 0);
          mma_tf32_x4(tmem_d, a_hi, b_lo, args.idesc, 1);
          mma_tf32_x4(tmem_d, a_hi, b_hi, args.idesc, 1);
          mma_commit(&empty_bar[s]);
          mma_commit(&acc_full_bar[b]);
        }
        __syncwarp();
        if (++s == kStages) { s = 0; ph ^= 1; }
      }
    }
  } else {
    // ---------------- epilogue warps: fold stages into register sums, finish tiles ----------------
    const Epilogue& ep = args.ep;
    const int ew = warp - 2;
    const int lane_group = warp % 4;     // the TMEM lane quarter this warp may read
    const int half = ew / 4;             // this warp takes the 32-column chunks of this parity
    const bool ch_n = ep.channel_on_n != 0;
    const float cmin = __int_as_float(ep.clamp_min), cmax = __int_as_float(ep.clamp_max);
    uint32_t stage_count = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      const int tm = tile / args.tiles_n, tn = tile % args.tiles_n;
      const int n_tile0 = tn * args.block_n;
      const int n_end = min(args.size_n, n_tile0 + args.block_n);   // a 32-column chunk may reach past the tile's columns
      float sum[2][32], comp[2][32];
#pragma unroll
      for (int c = 0; c < 2; c++)
#pragma unroll
        for (int j = 0; j < 32; j++) sum[c][j] = comp[c][j] = 0.f;
      for (int kb = 0; kb < k_blocks && ok; kb++, stage_count++) {
        const uint32_t b = stage_count & 1, aph = (stage_count >> 1) & 1;
        if (!mbar_wait_warp(&acc_full_bar[b], aph, abortp)) {
          if (lane == 0) {
            if (!*abortp) atomicCAS(args.status, 0, 3);
            *abortp = 1;
          }
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(lane_group * 32) << 16) + b * (uint32_t)kMaxBlockN;
#pragma unroll
        for (int c = 0; c < 2; c++) {
          const int col = (2 * c + half) * 32;
          if (col < args.block_n) {     // uniform across the warp
            uint32_t r[32];
            tmem_ld_32(taddr + col, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; j++) {
              const float y = __uint_as_float(r[j]) - comp[c][j];
              const float t = sum[c][j] + y;
              comp[c][j] = (t - sum[c][j]) - y;
              sum[c][j] = t;
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty_bar[b]);
      }
      // the continue/abort decision is collective, so that no warp waits for one that has left
      ok = epilogue_all(ok);
      if (!ok) break;
      const int m = tm * kBlockM + lane_group * 32 + lane;
      if (m < args.size_m) {
        const float bias_m = (!ch_n && ep.bias) ? ((const float*)ep.bias)[m] : 0.f;
#pragma unroll
        for (int c = 0; c < 2; c++) {
          const int col = (2 * c + half) * 32;
          const int n0 = n_tile0 + col;
          if (col >= args.block_n || n0 >= n_end) continue;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; j++) {
            float x = sum[c][j] + bias_m;
            if (ch_n && ep.bias && n0 + j < n_end) x += ((const float*)ep.bias)[n0 + j];
            v[j] = fmaxf(fminf(x, cmax), cmin);
          }
          float* out = (float*)args.dst.data + (int64_t)m * args.dst.stride_m + n0;
          if (n0 + 32 <= n_end && (((uintptr_t)out) & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 8; q++) __stcs(reinterpret_cast<float4*>(out) + q, make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
          } else {
#pragma unroll
            for (int j = 0; j < 32; j++) if (n0 + j < n_end) out[j] = v[j];
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

__device__ __forceinline__ float to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return __uint_as_float(r);
}

// The pre-pass: out_hi / out_lo [width][kpad] (depth-contiguous, zero padded to a multiple of 32 floats) from a side
// in any storage order.  A 32 x 32 tile goes through shared memory so that reads and writes are both coalesced.
__global__ void __launch_bounds__(256) split_tf32_kernel(SideView s, int depth, int kpad, float* __restrict__ out_hi,
                                                         float* __restrict__ out_lo) {
  __shared__ float tile[32][33];
  const int tx = threadIdx.x % 32, ty = threadIdx.x / 32;
  const int w0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  const float* src = (const float*)s.data;
  for (int r = 0; r < 4; r++) {
    int w, k;
    if (s.stride_k == 1) { k = tx; w = ty + 8 * r; } else { w = tx; k = ty + 8 * r; }
    float v = 0.f;
    if (w0 + w < s.width && k0 + k < depth) v = src[(int64_t)(w0 + w) * s.stride_w + (int64_t)(k0 + k) * s.stride_k];
    tile[w][k] = v;
  }
  __syncthreads();
  for (int r = 0; r < 4; r++) {
    const int w = ty + 8 * r, k = tx;
    if (w0 + w < s.width) {
      const float v = tile[w][k];
      const float hi = to_tf32(v);
      const float lo = to_tf32(v - hi);
      const int64_t o = (int64_t)(w0 + w) * kpad + k0 + k;
      out_hi[o] = hi;
      out_lo[o] = lo;
    }
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

// 2-D map over a [width][kpad] float matrix: dim0 = depth (contiguous), dim1 = width; boxes of 32 floats x box_rows.
bool make_map(CUtensorMap* map, const float* base, int kpad, int width, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)kpad, (cuuint64_t)width};
  cuuint64_t strides[1] = {(cuuint64_t)kpad * 4};
  cuuint32_t box[2] = {(cuuint32_t)kStageFloats, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

size_t tc_f32_scratch_bytes(int width, int depth) {
  const size_t kpad = (size_t)(depth + kStageFloats - 1) / kStageFloats * kStageFloats;
  return 2 * (((size_t)width * kpad * 4 + 255) & ~size_t(255));
}

cudaError_t launch_tc_f32(const SideView& m_side, const SideView& n_side, const DstView& dst, const Epilogue& ep, void* scratch_m,
                          void* scratch_n, int sm_count, int* status, cudaStream_t stream) {
  if (dst.size_m <= 0 || dst.size_n <= 0) return cudaSuccess;
  const int depth = ep.depth;
  const int kpad = (depth + kStageFloats - 1) / kStageFloats * kStageFloats;
  auto half_bytes = [&](int width) { return ((size_t)width * kpad * 4 + 255) & ~size_t(255); };
  float* m_hi = (float*)scratch_m;
  float* m_lo = (float*)((char*)scratch_m + half_bytes(m_side.width));
  float* n_hi = (float*)scratch_n;
  float* n_lo = (float*)((char*)scratch_n + half_bytes(n_side.width));
  const SideView* sides[2] = {&m_side, &n_side};
  float* his[2] = {m_hi, n_hi};
  float* los[2] = {m_lo, n_lo};
  for (int i = 0; i < 2; i++) {
    dim3 grid((sides[i]->width + 31) / 32, kpad / 32);
    if (grid.y > 65535) return cudaErrorInvalidConfiguration;
    split_tf32_kernel<<<grid, 256, 0, stream>>>(*sides[i], depth, kpad, his[i], los[i]);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
  }
  F32Args a;
  a.dst = dst;
  a.ep = ep;
  a.size_m = m_side.width;
  a.size_n = n_side.width;
  a.k_blocks = kpad / kStageFloats;
  // n tiles of equal width, a multiple of 16, at most 128 columns; narrower when that puts more SMs to work
  const int tiles_m = (a.size_m + kBlockM - 1) / kBlockM;
  int n_tiles = (a.size_n + kMaxBlockN - 1) / kMaxBlockN;
  while ((long long)tiles_m * n_tiles * 2 <= sm_count && (a.size_n + 2 * n_tiles - 1) / (2 * n_tiles) >= 32) n_tiles *= 2;
  a.block_n = ((a.size_n + n_tiles - 1) / n_tiles + 15) / 16 * 16;
  a.tiles_m = tiles_m;
  a.tiles_n = (a.size_n + a.block_n - 1) / a.block_n;
  // instruction descriptor: fp32 accumulate (1 at bit 4), TF32 operands (2 at bits 7 and 10), both depth-major,
  // N / 8 at bit 17, M / 16 at bit 24
  a.idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(a.block_n >> 3) << 17) | ((uint32_t)(kBlockM >> 4) << 24);
  a.status = status;
  CUtensorMap map_a_hi, map_a_lo, map_b_hi, map_b_lo;
  if (!make_map(&map_a_hi, m_hi, kpad, a.size_m, kBlockM) || !make_map(&map_a_lo, m_lo, kpad, a.size_m, kBlockM) ||
      !make_map(&map_b_hi, n_hi, kpad, a.size_n, a.block_n) || !make_map(&map_b_lo, n_lo, kpad, a.size_n, a.block_n)) {
    return cudaErrorInvalidValue;
  }
  {
    // the opt-in to more than 48 KB of dynamic shared memory is per device
    static std::mutex mu;
    static bool attr_set[kMaxDevices] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(mu);
    if (dev < 0 || dev >= kMaxDevices || !attr_set[dev]) {
      cudaError_t e = cudaFuncSetAttribute(tc_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
      if (e != cudaSuccess) return e;
      if (dev >= 0 && dev < kMaxDevices) attr_set[dev] = true;
    }
  }
  const long long tiles = (long long)a.tiles_m * a.tiles_n;
  const int grid = (int)(tiles < sm_count ? tiles : sm_count);
  tc_f32_kernel<<<grid, kThreads, kSmemBytes, stream>>>(map_a_hi, map_a_lo, map_b_hi, map_b_lo, a);
  return cudaGetLastError();
}

}  // namespace ruyb200
