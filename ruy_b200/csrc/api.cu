// Host side of libruy_b200.so: the C ABI of include/ruy_b200.h.
//
// This file plays the role of ruy's front end and middle end for the device:
//   validate          ruy/validate.h:40-83
//   canonicalize      CreateTrMulParams: Mul -> TrMul view, row-major dst => operand swap
//                     (ruy/create_trmul_params.h:465-480)
//   prepare operands  PreparePackedMatrices + PrepackedCache (ruy/prepare_packed_matrices.cc:38-95,
//                     ruy/prepacked_cache.cc:79-127), with the cache resident in HBM
//   dispatch          TrMul (ruy/trmul.cc:309-422): pick the kernel and launch it
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <tuple>
#include <vector>

#include "common.cuh"
#include <nvtx3/nvToolsExt.h>

#include "batch_i8.h"
#include "plan.h"

using namespace ruyb200;

namespace {

thread_local std::string g_last_error;

int fail(int status, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return status;
}

#define CUDA_TRY(expr)                                                                   \
  do {                                                                                   \
    cudaError_t e__ = (expr);                                                            \
    if (e__ != cudaSuccess)                                                              \
      return fail(e__ == cudaErrorMemoryAllocation ? RUYB200_ERR_OOM : RUYB200_ERR_CUDA, \
                  "%s: %s", #expr, cudaGetErrorString(e__));                             \
  } while (0)

size_t dtype_size(int dtype) {
  switch (dtype) {
    case RUYB200_I8:
    case RUYB200_U8:
      return 1;
    case RUYB200_I16:
      return 2;
    case RUYB200_F64:
      return 8;
    default:
      return 4;
  }
}

bool dtype_range(int dtype, int64_t* lo, int64_t* hi) {
  switch (dtype) {
    case RUYB200_I8: *lo = -128; *hi = 127; return true;
    case RUYB200_U8: *lo = 0; *hi = 255; return true;
    case RUYB200_I16: *lo = -32768; *hi = 32767; return true;
    case RUYB200_I32: *lo = INT32_MIN; *hi = INT32_MAX; return true;
    default: return false;
  }
}

constexpr uint32_t kCompiledPaths = RUYB200_PATH_STANDARD_CPP | RUYB200_PATH_AVX | RUYB200_PATH_AVX2_FMA |
                                    RUYB200_PATH_AVX512;
constexpr uint32_t kX86Paths = RUYB200_PATH_AVX | RUYB200_PATH_AVX2_FMA | RUYB200_PATH_AVX512;
// Width of the "kernel cell" used by the caching heuristics (ruy/prepare_packed_matrices.cc:51-61):
// here the row count of one tensor-core tile.
constexpr int kKernelWidth = 128;

uint32_t most_significant_bit(uint32_t v) {
  uint32_t r = 0;
  while (v) {
    r = v & (~v + 1);
    v &= v - 1;
  }
  return r;
}

// Device scratch that converges to a single block, reset at the start of every mul
// (the role of ruy::Allocator, ruy/allocator.h:59-96).  All use is ordered on one stream.
struct Arena {
  struct Block {
    char* p;
    size_t cap;
  };
  std::vector<Block> blocks;
  size_t cur = 0;
  size_t off = 0;

  void* alloc(size_t bytes) {
    bytes = (bytes + 255) & ~size_t(255);
    if (bytes == 0) bytes = 256;
    while (cur < blocks.size()) {
      if (off + bytes <= blocks[cur].cap) {
        void* r = blocks[cur].p + off;
        off += bytes;
        return r;
      }
      cur++;
      off = 0;
    }
    size_t cap = std::max<size_t>(bytes, size_t(1) << 20);
    if (!blocks.empty()) cap = std::max(cap, blocks.back().cap * 2);
    char* p = nullptr;
    if (cudaMalloc(&p, cap) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;
    }
    blocks.push_back({p, cap});
    cur = blocks.size() - 1;
    off = bytes;
    return p;
  }
  // Must only be called when no enqueued work can still touch the blocks being merged.
  void reset(bool may_merge) {
    if (may_merge && blocks.size() > 1) {
      size_t total = 0;
      for (auto& b : blocks) {
        total += b.cap;
        cudaFree(b.p);
      }
      blocks.clear();
      char* p = nullptr;
      if (cudaMalloc(&p, total) == cudaSuccess) {
        blocks.push_back({p, total});
      } else {
        cudaGetLastError();
      }
    }
    cur = 0;
    off = 0;
  }
  void release() {
    for (auto& b : blocks) cudaFree(b.p);
    blocks.clear();
    cur = off = 0;
  }
};

struct CacheEntry {
  void* packed = nullptr;
  int32_t* sums = nullptr;
  int packed_depth = 0;
  size_t bytes = 0;
  uint64_t stamp = 0;
  int pins = 0;   // plans that hold pointers into this entry; pinned entries are never evicted or cleared
  int slab = -1;  // which CacheSlab the entry was carved from
};

// Cache entries are carved out of large device blocks instead of one cudaMalloc each (a plan over thousands of
// small cached weights would otherwise pay thousands of allocations).  A block is a bump allocator with a
// count of live entries; it is returned to the driver when its last entry dies (the block being filled is
// rewound instead).  Entries of a quarter block or more get a block of their own.
struct CacheSlab {
  char* base = nullptr;
  size_t cap = 0;
  size_t used = 0;
  int live = 0;
};
constexpr size_t kCacheSlabBytes = size_t(32) << 20;

}  // namespace

constexpr int kMaxChunks = 16;
constexpr size_t kBounceBytes = size_t(1) << 20;   // pinned staging for per-channel vectors (3 x 16384 channels and more), small host operands and destinations

struct ruyb200_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  int sm_count = 148;
  int max_num_threads = 1;
  uint32_t enabled_paths = 0;  // 0 = not set explicitly
  uint32_t last_used_path = 0;
  int advisory = RUYB200_ADVISORY_NONE;
  Arena arena;
  std::map<CacheKey, CacheEntry> cache;
  // Tensor maps for the copy-engine stores of mirrored destinations, in device memory, by (destination and mirror
  // addresses, shape, stride): a step loop passes the same few buffers again and again.  RUYB200_NO_STORE_MAPS=1
  // keeps the mirrored epilogue on store instructions.
  std::map<std::vector<uint64_t>, void*> store_maps;
  bool no_store_maps = false;
  std::vector<CacheSlab> cache_slabs;
  int cache_open_slab = -1;   // the block new small entries are carved from
  size_t cache_bytes = 0;
  size_t cache_budget = size_t(8) << 30;
  uint64_t cache_clock = 0;
  int* d_status = nullptr;
  int* h_status = nullptr;  // pinned
  unsigned long long peer_wait_ns = 2000000000ull;   // limit of ruyb200_peer_wait / _exchange
  uint64_t counters[6] = {0, 0, 0, 0, 0, 0};
  int force_kernel = 0;  // RUYB200_KERNEL_* or 0
  bool no_pair = false;  // RUYB200_NO_PAIR=1: keep the tensor-core kernel on one CTA per tile
  // RUYB200_TILE=[pair|single][:columns] overrides the tile-shape choice of the tensor-core kernel (tests, measurements)
  int force_pair = -1;
  int force_block_n = 0;
  bool no_shallow = false;   // RUYB200_NO_SHALLOW=1: keep shallow-depth muls on the general tensor-core kernel
  int tc_f32_max_depth = 1 << 30;   // RUYB200_TC_F32_MAX_DEPTH: deepest fp32 mul that goes to the tensor-core kernel (measurements)
  // synchronous muls with large host operands are cut into chunks that move on these two streams while the
  // kernel of another chunk runs on `stream` (created on first use)
  cudaStream_t copy_in = nullptr;
  cudaStream_t copy_out = nullptr;
  cudaEvent_t chunk_in[kMaxChunks] = {};
  cudaEvent_t chunk_done[kMaxChunks] = {};
  char* bounce = nullptr;   // pinned staging for small host vectors (bias, multipliers), operands and destinations, kBounceBytes
  size_t bounce_off = 0;
  char* d_bounce = nullptr;       // device mirror of `bounce`: what is staged for upload travels in one copy per launch
  size_t bounce_h2d_end = 0;      // end of the staged uploads in `bounce`
  size_t bounce_flushed = 0;      // what of them has been sent
  cudaEvent_t chunk_out[kMaxChunks] = {};   // only with RUYB200_TRACE: when each chunk's destination rows have left
  cudaEvent_t chunk_start = nullptr;
  bool no_chunks = false;   // RUYB200_NO_CHUNKS=1: one copy in, one kernel, one copy out
  int chunk_target = 4;     // RUYB200_CHUNKS=n: how many chunks a large host-operand mul is cut into (2..16)
  bool trace = false;       // RUYB200_TRACE=1: one line per mul on stderr with the decisions taken (cf. ruy/trace.h)
};

namespace {

struct DeviceGuard {
  int prev = -1;
  explicit DeviceGuard(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
  }
  ~DeviceGuard() {
    int cur = -1;
    cudaGetDevice(&cur);
    if (prev >= 0 && cur != prev) cudaSetDevice(prev);
  }
};

bool is_device_pointer(const void* p) {
  if (!p) return false;
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
    cudaGetLastError();
    return false;
  }
  return attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
}

uint32_t effective_paths(const ruyb200_ctx* ctx) {
  // ruy/ctx.cc:150-173: an explicit setting (which always keeps kStandardCpp, ruy/ctx.cc:67-76)
  // wins over RUY_PATHS (hex, taken verbatim), which wins over detection.  There is no CPU to
  // detect here, so "detection" reports every path.
  if (ctx->enabled_paths) return ctx->enabled_paths | RUYB200_PATH_STANDARD_CPP;
  const char* env = getenv("RUY_PATHS");
  if (env && *env) {
    const uint32_t v = (uint32_t)strtoul(env, nullptr, 16) & 0xFF;
    if (v) return v;
  }
  return kCompiledPaths | 0xE;
}

bool paths_explicit(const ruyb200_ctx* ctx) {
  if (ctx->enabled_paths) return true;
  const char* env = getenv("RUY_PATHS");
  return env && *env && strtoul(env, nullptr, 16) != 0;
}

int validate_desc(const ruyb200_mul_desc* d) {
  if (!d) return fail(RUYB200_ERR_INVALID, "null descriptor");
  const ruyb200_matrix* ms[3] = {&d->lhs, &d->rhs, &d->dst};
  const char* names[3] = {"lhs", "rhs", "dst"};
  for (int i = 0; i < 3; i++) {
    const ruyb200_matrix* m = ms[i];
    if (m->dtype > RUYB200_F64) return fail(RUYB200_ERR_UNSUPPORTED, "%s: unknown dtype %d", names[i], m->dtype);
    if (m->order > 1) return fail(RUYB200_ERR_INVALID, "%s: bad order", names[i]);
    if (m->rows < 0 || m->cols < 0) return fail(RUYB200_ERR_INVALID, "%s: negative dimension", names[i]);
    const int inner = m->order == RUYB200_COL_MAJOR ? m->rows : m->cols;
    if (m->stride < inner) return fail(RUYB200_ERR_INVALID, "%s: stride %d < %d", names[i], m->stride, inner);
    if (m->rows > 0 && m->cols > 0 && !m->data) return fail(RUYB200_ERR_INVALID, "%s: null data", names[i]);
    if (m->cache_policy > RUYB200_ALWAYS_CACHE) return fail(RUYB200_ERR_INVALID, "%s: bad cache policy", names[i]);
    if (m->dtype == RUYB200_F32 || m->dtype == RUYB200_F64) {
      if (m->zero_point) return fail(RUYB200_ERR_INVALID, "%s: float zero_point must be 0", names[i]);
    } else {
      int64_t lo, hi;
      dtype_range(m->dtype, &lo, &hi);
      if (m->zero_point < lo || m->zero_point > hi)
        return fail(RUYB200_ERR_INVALID, "%s: zero_point outside the scalar type's range", names[i]);
    }
  }
  if (d->lhs.cols != d->rhs.rows || d->lhs.rows != d->dst.rows || d->rhs.cols != d->dst.cols)
    return fail(RUYB200_ERR_INVALID, "shape mismatch: lhs %dx%d rhs %dx%d dst %dx%d", d->lhs.rows, d->lhs.cols,
                d->rhs.rows, d->rhs.cols, d->dst.rows, d->dst.cols);
  const ruyb200_mul_params& p = d->params;
  if (p.channel_dimension > 1) return fail(RUYB200_ERR_INVALID, "bad channel_dimension");
  if (p.rounding_mode > RUYB200_ROUNDING_X86) return fail(RUYB200_ERR_INVALID, "bad rounding_mode");
  const int L = d->lhs.dtype, R = d->rhs.dtype, D = d->dst.dtype;
  if (p.accum_dtype == RUYB200_F32) {
    if (L != RUYB200_F32 || R != RUYB200_F32 || D != RUYB200_F32)
      return fail(RUYB200_ERR_UNSUPPORTED, "float accumulation needs float operands and destination");
    return RUYB200_OK;
  }
  if (p.accum_dtype == RUYB200_F64) {
    // ruy's mixed floating-point cases, (f64, f32, f64, f32) and (f32, f64, f64, f64) in ruy/BUILD:1195-1207, and
    // every other mix of float and double operands with a double accumulator
    const auto fp = [](int t) { return t == RUYB200_F32 || t == RUYB200_F64; };
    if (!fp(L) || !fp(R) || !fp(D))
      return fail(RUYB200_ERR_UNSUPPORTED, "double accumulation needs float or double operands and destination");
    return RUYB200_OK;
  }
  if (p.accum_dtype != RUYB200_I32) return fail(RUYB200_ERR_UNSUPPORTED, "accumulator must be int32, float or double");
  const auto wide = [](int t) { return t == RUYB200_F32 || t == RUYB200_F64; };
  if (wide(L) || wide(R) || wide(D)) return fail(RUYB200_ERR_UNSUPPORTED, "unsupported integer type combination");
  if (L == RUYB200_F32 || R == RUYB200_F32 || D == RUYB200_F32 || L == RUYB200_I32 || R == RUYB200_I32)
    return fail(RUYB200_ERR_UNSUPPORTED, "unsupported integer type combination");
  const bool has16 = L == RUYB200_I16 || R == RUYB200_I16;
  if (has16) {
    if (L == RUYB200_I16 && R == RUYB200_I16) return fail(RUYB200_ERR_UNSUPPORTED, "int16 x int16 is not supported");
    // ruy/validate.h:47-57
    if (d->lhs.zero_point || d->rhs.zero_point || d->dst.zero_point)
      return fail(RUYB200_ERR_INVALID, "16-bit inputs require all zero points to be 0");
  }
  if (!(L == RUYB200_U8 && R == RUYB200_U8)) {
    // ruy/validate.h:59-65
    int64_t llo, lhi, rlo, rhi;
    dtype_range(L, &llo, &lhi);
    dtype_range(R, &rlo, &rhi);
    if (d->lhs.zero_point == llo && d->rhs.zero_point == rlo)
      return fail(RUYB200_ERR_INVALID, "lhs and rhs zero points are both the lowest value of their types");
  }
  if (D != RUYB200_I32) {
    const bool pc = p.multiplier_fixedpoint_perchannel || p.multiplier_exponent_perchannel;
    if (pc && !(p.multiplier_fixedpoint_perchannel && p.multiplier_exponent_perchannel))
      return fail(RUYB200_ERR_INVALID, "per-channel multiplier needs both the fixedpoint and the exponent buffer");
    if (!pc) {
      // ruy/apply_multiplier.cc:45-51
      if (p.multiplier_fixedpoint < 0) return fail(RUYB200_ERR_INVALID, "multiplier_fixedpoint < 0");
      if (p.multiplier_exponent < -31 || p.multiplier_exponent > 30)
        return fail(RUYB200_ERR_INVALID, "multiplier_exponent outside [-31, 30]");
    }
    int64_t lo, hi;
    dtype_range(D, &lo, &hi);
    if (p.clamp_min.i < lo || p.clamp_max.i > hi)
      return fail(RUYB200_ERR_INVALID, "clamp outside the destination type's range");
  }
  return RUYB200_OK;
}

// TrMul view of a matrix: side 0 = LHS (width = rows, depth = cols), side 1 = RHS.
SideView side_view(const ruyb200_matrix& m, int side, const void* data) {
  SideView s;
  s.data = data;
  s.dtype = m.dtype;
  s.zero_point = m.zero_point;
  const bool row_major = m.order == RUYB200_ROW_MAJOR;
  if (side == 0) {
    s.width = m.rows;
    s.stride_w = row_major ? m.stride : 1;
    s.stride_k = row_major ? 1 : m.stride;
  } else {
    s.width = m.cols;
    s.stride_w = row_major ? 1 : m.stride;
    s.stride_k = row_major ? m.stride : 1;
  }
  return s;
}

size_t storage_span_bytes(const ruyb200_matrix& m) {
  const int inner = m.order == RUYB200_COL_MAJOR ? m.rows : m.cols;
  const int outer = m.order == RUYB200_COL_MAJOR ? m.cols : m.rows;
  if (inner <= 0 || outer <= 0) return 0;
  return ((size_t)(outer - 1) * (size_t)m.stride + (size_t)inner) * dtype_size(m.dtype);
}

// Device memory for one cache entry (`bytes` is a multiple of 256).  Returns nullptr when the device is out of memory.
void* cache_alloc(ruyb200_ctx* ctx, size_t bytes, int* slab_out) {
  auto new_slab = [&](size_t cap) -> int {
    char* p = nullptr;
    if (cudaMalloc(&p, cap) != cudaSuccess) {
      cudaGetLastError();
      return -1;
    }
    for (size_t i = 0; i < ctx->cache_slabs.size(); i++) {
      if (!ctx->cache_slabs[i].base) {
        ctx->cache_slabs[i] = CacheSlab{p, cap, 0, 0};
        return (int)i;
      }
    }
    ctx->cache_slabs.push_back(CacheSlab{p, cap, 0, 0});
    return (int)ctx->cache_slabs.size() - 1;
  };
  int idx;
  if (bytes >= kCacheSlabBytes / 4) {
    idx = new_slab(bytes);
    if (idx < 0) return nullptr;
  } else {
    idx = ctx->cache_open_slab;
    if (idx < 0 || ctx->cache_slabs[idx].used + bytes > ctx->cache_slabs[idx].cap) {
      // the block being left keeps its entries; if it has none it can go at once
      if (idx >= 0 && ctx->cache_slabs[idx].live == 0) {
        cudaFree(ctx->cache_slabs[idx].base);
        ctx->cache_slabs[idx] = CacheSlab();
      }
      idx = new_slab(kCacheSlabBytes);
      if (idx < 0) {
        ctx->cache_open_slab = -1;
        return nullptr;
      }
      ctx->cache_open_slab = idx;
    }
  }
  CacheSlab& sl = ctx->cache_slabs[idx];
  void* p = sl.base + sl.used;
  sl.used += bytes;
  sl.live++;
  *slab_out = idx;
  return p;
}

void cache_free(ruyb200_ctx* ctx, const CacheEntry& e) {
  if (e.slab < 0 || e.slab >= (int)ctx->cache_slabs.size()) return;
  CacheSlab& sl = ctx->cache_slabs[e.slab];
  if (--sl.live > 0) return;
  if (e.slab == ctx->cache_open_slab) {
    sl.used = 0;   // keep filling the same block from its start
  } else {
    cudaFree(sl.base);
    sl = CacheSlab();
  }
}

// Evicts the least recently used unpinned entry; false if there is none.
bool cache_evict_one(ruyb200_ctx* ctx) {
  auto oldest = ctx->cache.end();
  for (auto it = ctx->cache.begin(); it != ctx->cache.end(); ++it) {
    if (it->second.pins > 0) continue;
    if (oldest == ctx->cache.end() || it->second.stamp < oldest->second.stamp) oldest = it;
  }
  if (oldest == ctx->cache.end()) return false;
  ctx->cache_bytes -= oldest->second.bytes;
  cache_free(ctx, oldest->second);
  ctx->cache.erase(oldest);
  return true;
}

// ruy/prepare_packed_matrices.cc:38-66.
bool should_cache(const ruyb200_matrix& m, int other_width) {
  switch (m.cache_policy) {
    case RUYB200_ALWAYS_CACHE: return true;
    case RUYB200_CACHE_IF_LARGE_SPEEDUP: return other_width <= kKernelWidth;
    case RUYB200_CACHE_IF_SIGNIFICANT_SPEEDUP: return other_width <= 4 * kKernelWidth;
    default: return false;
  }
}

int packed_depth_for(int depth, int dtype) {
  const int per16 = 16 / (int)dtype_size(dtype);
  return std::max(per16, (depth + per16 - 1) / per16 * per16);
}

// Row length of the packed form this library makes for its own kernels (cache entries, per-call packing).  8-bit rows
// of 256 bytes or more are padded to whole 128-byte lines: the tensor-core kernel's copy engine fetches 128-byte box
// rows, and rows that start 16 bytes into a line make every one of them straddle two lines (measured 4096 x 4100 x
// 4096, rows of 4112 bytes: 68 us against 53 us for depth 4096).
int tc_packed_depth(int depth, int dtype) {
  if (dtype_size(dtype) == 1 && depth >= 256) return (depth + 127) / 128 * 128;
  return packed_depth_for(depth, dtype);
}

// A fully resolved mul: device pointers only, canonical (n = destination-contiguous) view.
struct Resolved {
  SideView m_side, n_side;
  DstView dst;
  Epilogue ep;
  int depth;
};

// `bytes` of the context's pinned staging buffer, or null when it is full (or could not be had).  Copies between
// pageable host memory and the device hold the calling thread (measured: 100 to 300 us per synchronous mul with a 4 KB
// operand and a 4 KB destination); small operands and destinations go through this buffer instead, with a host memcpy on
// the pageable side.  Host pointers only occur in synchronous muls, so the buffer is free again when the next call starts.
char* bounce_take(ruyb200_ctx* ctx, size_t bytes) {
  const size_t padded = (bytes + 63) & ~size_t(63);
  if (!ctx->bounce && cudaHostAlloc(&ctx->bounce, kBounceBytes, cudaHostAllocDefault) != cudaSuccess) {
    cudaGetLastError();
    ctx->bounce = nullptr;
  }
  if (!ctx->bounce || ctx->bounce_off + padded > kBounceBytes) return nullptr;
  char* p = ctx->bounce + ctx->bounce_off;
  ctx->bounce_off += padded;
  return p;
}

// Stages `bytes` of host data for upload: copies them into the pinned buffer and returns where they will be on the
// device once bounce_flush has run (null: no room, the caller copies by itself).  All that is staged between two
// flushes travels in ONE copy: a small synchronous mul with a host operand and three per-channel vectors issues one
// upload instead of four.
void* bounce_stage(ruyb200_ctx* ctx, const void* src, size_t bytes) {
  if (!ctx->d_bounce) {
    if (cudaMalloc(&ctx->d_bounce, kBounceBytes) != cudaSuccess) {
      cudaGetLastError();
      ctx->d_bounce = nullptr;
      return nullptr;
    }
  }
  char* pinned = bounce_take(ctx, bytes);
  if (!pinned) return nullptr;
  memcpy(pinned, src, bytes);
  ctx->bounce_h2d_end = ctx->bounce_off;
  return ctx->d_bounce + (pinned - ctx->bounce);
}

// Sends what has been staged since the last flush; called before every launch that may read staged data.
cudaError_t bounce_flush(ruyb200_ctx* ctx) {
  if (ctx->bounce_h2d_end <= ctx->bounce_flushed) return cudaSuccess;
  const size_t from = ctx->bounce_flushed;
  ctx->bounce_flushed = ctx->bounce_h2d_end;
  return cudaMemcpyAsync(ctx->d_bounce + from, ctx->bounce + from, ctx->bounce_h2d_end - from, cudaMemcpyHostToDevice, ctx->stream);
}

// One operand: finds or builds its device-resident form.
//   cached   -> packed copy + sums from the prepacked cache (built on a miss)
//   host     -> staged into the arena
//   device   -> used in place
// `need_sums`: the other side has a non-zero zero point (integer case).
// `want_packed`: the tensor-core kernel will run and this operand is not in its layout.
// `sums_if_packed`: sums the caller can do without (the tensor-core kernel can make its m-side sums itself, at the
// price of one-CTA tiles) but takes when a packing pass runs anyway and yields them for free.
int prepare_side(ruyb200_ctx* ctx, const ruyb200_matrix& m, int side, int depth, bool cache_it, bool need_sums,
                 bool tc_path, SideView* out, const int32_t** sums_out, bool sums_if_packed = false) {
  *sums_out = nullptr;
  const bool integer = m.dtype != RUYB200_F32 && m.dtype != RUYB200_F64;
  SideView src = side_view(m, side, m.data);
  const size_t esz = dtype_size(m.dtype);
  const bool on_device = is_device_pointer(m.data);
  if (src.width == 0 || depth == 0) {
    *out = src;
    if (need_sums && src.width > 0) {
      int32_t* z = (int32_t*)ctx->arena.alloc(sizeof(int32_t) * src.width);
      if (!z) return fail(RUYB200_ERR_OOM, "arena allocation failed");
      CUDA_TRY(cudaMemsetAsync(z, 0, sizeof(int32_t) * src.width, ctx->stream));
      *sums_out = z;
    }
    return RUYB200_OK;
  }

  auto stage_to_device = [&](SideView* v) -> int {
    const size_t span = storage_span_bytes(m);
    ctx->counters[3] += span;
    if (span <= kBounceBytes / 4) {
      if (void* staged = bounce_stage(ctx, m.data, span)) {
        v->data = staged;
        return RUYB200_OK;
      }
    }
    void* dptr = ctx->arena.alloc(span);
    if (!dptr) return fail(RUYB200_ERR_OOM, "arena allocation of %zu bytes failed", span);
    CUDA_TRY(cudaMemcpyAsync(dptr, m.data, span, cudaMemcpyHostToDevice, ctx->stream));
    v->data = dptr;
    return RUYB200_OK;
  };

  if (cache_it) {
    CacheKey key(m.data, src.width, depth, src.stride_w, src.stride_k, m.zero_point, (int)m.dtype, side);
    auto it = ctx->cache.find(key);
    if (it == ctx->cache.end()) {
      ctx->counters[2]++;
      const int pd = tc_packed_depth(depth, m.dtype);
      const size_t data_bytes = ((size_t)src.width * pd * esz + 255) & ~size_t(255);
      const size_t sums_bytes = integer ? (((size_t)src.width * 4 + 255) & ~size_t(255)) : 0;
      const size_t total = data_bytes + sums_bytes;
      // ruy/prepacked_cache.cc:104-127: make room first, oldest entries go first
      while (!ctx->cache.empty() && ctx->cache_bytes + total > ctx->cache_budget) {
        if (!cache_evict_one(ctx)) break;
      }
      CacheEntry e;
      void* buf = cache_alloc(ctx, total, &e.slab);
      if (!buf) return fail(RUYB200_ERR_OOM, "prepacked cache: allocation of %zu bytes failed", total);
      SideView staged = src;
      if (!on_device) {
        int rc = stage_to_device(&staged);
        if (rc) {
          cache_free(ctx, e);
          return rc;
        }
      }
      e.packed = buf;
      e.sums = integer ? (int32_t*)((char*)buf + data_bytes) : nullptr;
      e.packed_depth = pd;
      e.bytes = total;
      cudaError_t ce = bounce_flush(ctx);
      if (ce == cudaSuccess) ce = launch_pack(staged, depth, pd, e.packed, e.sums, ctx->stream);
      ctx->counters[0]++;
      if (ce != cudaSuccess) {
        cache_free(ctx, e);
        return fail(RUYB200_ERR_CUDA, "pack launch: %s", cudaGetErrorString(ce));
      }
      ctx->cache_bytes += total;
      it = ctx->cache.emplace(key, e).first;
    } else {
      ctx->counters[1]++;
    }
    it->second.stamp = ++ctx->cache_clock;
    out->data = it->second.packed;
    out->dtype = m.dtype;
    out->zero_point = m.zero_point;
    out->width = src.width;
    out->stride_w = it->second.packed_depth;
    out->stride_k = 1;
    *sums_out = it->second.sums;
    return RUYB200_OK;
  }

  SideView v = src;
  if (!on_device) {
    int rc = stage_to_device(&v);
    if (rc) return rc;
  }
  const bool layout_ok = v.stride_k == 1 && ((uintptr_t)v.data % 16 == 0) && ((v.stride_w * (int64_t)esz) % 16 == 0);
  if (tc_path && !layout_ok) {
    // PackImpl: re-tile into the depth-contiguous padded layout, sums on the way
    const int pd = tc_packed_depth(depth, m.dtype);
    void* packed = ctx->arena.alloc((size_t)v.width * pd * esz);
    const bool with_sums = (need_sums || sums_if_packed) && integer;
    int32_t* sums = with_sums ? (int32_t*)ctx->arena.alloc(sizeof(int32_t) * v.width) : nullptr;
    if (!packed || (with_sums && !sums)) return fail(RUYB200_ERR_OOM, "arena allocation failed");
    cudaError_t ce = bounce_flush(ctx);
    if (ce == cudaSuccess) ce = launch_pack(v, depth, pd, packed, sums, ctx->stream);
    ctx->counters[0]++;
    if (ce != cudaSuccess) return fail(RUYB200_ERR_CUDA, "pack launch: %s", cudaGetErrorString(ce));
    v.data = packed;
    v.stride_w = pd;
    v.stride_k = 1;
    *sums_out = sums;
  } else if (need_sums) {
    int32_t* sums = (int32_t*)ctx->arena.alloc(sizeof(int32_t) * v.width);
    if (!sums) return fail(RUYB200_ERR_OOM, "arena allocation failed");
    cudaError_t ce = bounce_flush(ctx);
    if (ce == cudaSuccess) ce = launch_sums(v, depth, sums, ctx->stream);
    ctx->counters[0]++;
    if (ce != cudaSuccess) return fail(RUYB200_ERR_CUDA, "sums launch: %s", cudaGetErrorString(ce));
    *sums_out = sums;
  }
  *out = v;
  return RUYB200_OK;
}

// Copies a small host vector (bias / multipliers) into the arena unless it already lives on the device.
// Such vectors are usually pageable memory, from which a copy holds the calling thread for some 10 us; they go through
// a pinned buffer of the context instead (host pointers only occur in synchronous muls, so the buffer is free again
// when the next call starts).
int stage_vector(ruyb200_ctx* ctx, const void* p, size_t count, const void** out, size_t elem = 4) {
  *out = p;
  if (!p || count == 0 || is_device_pointer(p)) return RUYB200_OK;
  const size_t bytes = count * elem;
  ctx->counters[3] += bytes;
  if (void* staged = bounce_stage(ctx, p, bytes)) {
    *out = staged;
    return RUYB200_OK;
  }
  void* d = ctx->arena.alloc(bytes);
  if (!d) return fail(RUYB200_ERR_OOM, "arena allocation failed");
  CUDA_TRY(cudaMemcpyAsync(d, p, bytes, cudaMemcpyHostToDevice, ctx->stream));
  *out = d;
  return RUYB200_OK;
}

int choose_kernel(const ruyb200_ctx* ctx, const ruyb200_mul_desc& d) {
  if (ctx->force_kernel == RUYB200_KERNEL_GENERIC) return ctx->force_kernel;
  if (d.params.accum_dtype == RUYB200_F32) return RUYB200_KERNEL_SGEMM;
  if (d.params.accum_dtype == RUYB200_F64) return RUYB200_KERNEL_GENERIC;
  const bool both8 = dtype_size(d.lhs.dtype) == 1 && dtype_size(d.rhs.dtype) == 1;
  if (both8 && d.lhs.cols > 0) return RUYB200_KERNEL_TC_I8;
  return RUYB200_KERNEL_GENERIC;
}

// The chunked path of a synchronous tensor-core mul whose m-side operand and/or destination live on the host
// (m_host / dst_host are null for the one that is already on the device).
// `L` describes the whole mul with device addresses (the m-side buffer is still empty); chunk c covers m
// indices [c * step, ...): its operand rows are copied in on `copy_in`, its kernel runs on the context's
// stream once they have arrived, and its destination rows leave on `copy_out` once the kernel is done.
int run_chunks(ruyb200_ctx* ctx, const ruyb200_mul_desc& d, const TcI8Launch& L, const char* m_host, char* dst_host,
               size_t dst_esz) {
  if (!ctx->copy_in) {
    CUDA_TRY(cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
    CUDA_TRY(cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
    // with the decision log on, the events keep time so that the log can show each chunk's way through the pipeline
    const unsigned flags = ctx->trace ? cudaEventDefault : cudaEventDisableTiming;
    CUDA_TRY(cudaEventCreateWithFlags(&ctx->chunk_start, flags));
    for (int i = 0; i < kMaxChunks; i++) {
      CUDA_TRY(cudaEventCreateWithFlags(&ctx->chunk_in[i], flags));
      CUDA_TRY(cudaEventCreateWithFlags(&ctx->chunk_done[i], flags));
      if (ctx->trace) CUDA_TRY(cudaEventCreateWithFlags(&ctx->chunk_out[i], flags));
    }
  }
  const int width = L.m_side.width;
  const int64_t stride_w = L.m_side.stride_w;            // bytes: the operand is 8-bit
  // chunks of a multiple of 256 m indices (whole two-CTA tiles), at least 1 MiB each.  Few chunks leave the first copy
  // in and the last copy out exposed; many chunks pay a cross-stream hand-off each.  Measured on config 3 (33.6 MB each
  // way): 4 chunks 1.02 ms, 8 1.06, 12 1.10, 16 1.19.
  const size_t dst_pitch = (size_t)d.dst.stride * dst_esz;
  const int64_t moved_per_m = (m_host ? stride_w : 0) + (dst_host ? (int64_t)dst_pitch : 0);   // bytes over PCIe per m index
  const int target = ctx->chunk_target;
  int step = ((width + target - 1) / target + 255) / 256 * 256;
  while ((int64_t)step * moved_per_m < (1 << 20) && step < width) step *= 2;
  int chunks = (width + step - 1) / step;
  if (chunks > kMaxChunks) {
    step = ((width + kMaxChunks - 1) / kMaxChunks + 255) / 256 * 256;
    chunks = (width + step - 1) / step;
  }
  const size_t dst_row_bytes = (size_t)L.dst.size_n * dst_esz;
  // the copy streams start after whatever the context's stream has queued (operand staging, packing)
  CUDA_TRY(cudaEventRecord(ctx->chunk_start, ctx->stream));
  CUDA_TRY(cudaStreamWaitEvent(ctx->copy_in, ctx->chunk_start, 0));
  CUDA_TRY(cudaStreamWaitEvent(ctx->copy_out, ctx->chunk_start, 0));
  for (int c = 0; c < chunks; c++) {
    const int w0 = c * step;
    const int w = std::min(step, width - w0);
    const size_t off = (size_t)w0 * (size_t)stride_w;
    const size_t span = (size_t)(w - 1) * (size_t)stride_w + (size_t)L.depth;
    if (m_host) {
      CUDA_TRY(cudaMemcpyAsync((char*)L.m_side.data + off, m_host + off, span, cudaMemcpyHostToDevice, ctx->copy_in));
      ctx->counters[3] += span;
      CUDA_TRY(cudaEventRecord(ctx->chunk_in[c], ctx->copy_in));
      CUDA_TRY(cudaStreamWaitEvent(ctx->stream, ctx->chunk_in[c], 0));
    }
    TcI8Launch part = L;
    part.m_side.data = (const char*)L.m_side.data + off;
    part.m_side.width = w;
    part.dst.data = (char*)L.dst.data + (size_t)w0 * dst_pitch;
    part.dst.size_m = w;
    if (part.ep.sums_m) part.ep.sums_m += w0;
    // per-channel buffers indexed along m move with the chunk
    if (!part.ep.channel_on_n) {
      if (part.ep.bias) part.ep.bias = (const char*)part.ep.bias + (size_t)w0 * 4;
      if (part.ep.mfp_pc) part.ep.mfp_pc += w0;
      if (part.ep.mexp_pc) part.ep.mexp_pc += w0;
    }
    cudaError_t ce = launch_tc_i8(part, ctx->stream);
    ctx->counters[0]++;
    if (ce != cudaSuccess) return fail(RUYB200_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(ce));
    if (dst_host) {
      CUDA_TRY(cudaEventRecord(ctx->chunk_done[c], ctx->stream));
      CUDA_TRY(cudaStreamWaitEvent(ctx->copy_out, ctx->chunk_done[c], 0));
      if (dst_row_bytes == dst_pitch) {   // a dense destination leaves as one linear copy
        CUDA_TRY(cudaMemcpyAsync(dst_host + (size_t)w0 * dst_pitch, part.dst.data, dst_pitch * (size_t)w, cudaMemcpyDeviceToHost,
                                 ctx->copy_out));
      } else {
        CUDA_TRY(cudaMemcpy2DAsync(dst_host + (size_t)w0 * dst_pitch, dst_pitch, part.dst.data, dst_pitch, dst_row_bytes, w,
                                   cudaMemcpyDeviceToHost, ctx->copy_out));
      }
      ctx->counters[4] += dst_row_bytes * (size_t)w;
      if (ctx->trace) CUDA_TRY(cudaEventRecord(ctx->chunk_out[c], ctx->copy_out));
    }
  }
  if (dst_host) CUDA_TRY(cudaStreamSynchronize(ctx->copy_out));
  if (ctx->trace && m_host && dst_host) {
    CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    fprintf(stderr, "ruy_b200: %d chunks of %d m indices; microseconds after the first copy could start (operand in, kernel done, destination out):", chunks, step);
    for (int c = 0; c < chunks; c++) {
      float a = 0, b = 0, o = 0;
      cudaEventElapsedTime(&a, ctx->chunk_start, ctx->chunk_in[c]);
      cudaEventElapsedTime(&b, ctx->chunk_start, ctx->chunk_done[c]);
      cudaEventElapsedTime(&o, ctx->chunk_start, ctx->chunk_out[c]);
      fprintf(stderr, " [%.0f %.0f %.0f]", a * 1e3, b * 1e3, o * 1e3);
    }
    fprintf(stderr, "\n");
  }
  return RUYB200_OK;
}

// The device array of tensor maps (destination first, then the mirrors) that lets the copy engine write a mirrored
// 8-bit destination; made on first use of a set of buffers (one synchronous 1 KB copy), null when a base or the stride
// is not 16-byte aligned.
const void* mirrored_store_maps(ruyb200_ctx* ctx, const DstView& dst, void* const* mirrors, int n_mirrors) {
  std::vector<uint64_t> key;
  key.push_back((uint64_t)(uintptr_t)dst.data);
  for (int i = 0; i < n_mirrors; i++) key.push_back((uint64_t)(uintptr_t)mirrors[i]);
  key.push_back((uint64_t)dst.size_m);
  key.push_back((uint64_t)dst.size_n);
  key.push_back((uint64_t)dst.stride_m);
  auto it = ctx->store_maps.find(key);
  if (it != ctx->store_maps.end()) return it->second;
  alignas(64) unsigned char host[8 * kStoreMapBytes];
  for (int i = 0; i <= n_mirrors; i++) {
    void* base = i == 0 ? dst.data : mirrors[i - 1];
    if (!make_i8_store_map(host + i * kStoreMapBytes, base, dst.size_n, dst.size_m, dst.stride_m)) return nullptr;
  }
  if (ctx->store_maps.size() >= 64) {   // a caller that keeps changing buffers: start over rather than grow
    cudaStreamSynchronize(ctx->stream);
    for (auto& kv : ctx->store_maps) cudaFree(kv.second);
    ctx->store_maps.clear();
  }
  void* dev = nullptr;
  if (cudaMalloc(&dev, 8 * kStoreMapBytes) != cudaSuccess) {
    cudaGetLastError();
    return nullptr;
  }
  if (cudaMemcpy(dev, host, (size_t)(n_mirrors + 1) * kStoreMapBytes, cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(dev);
    return nullptr;
  }
  ctx->store_maps.emplace(std::move(key), dev);
  return dev;
}

// The flag exchange a mirrored mul can carry out at its end.
struct Exchange {
  uint32_t* const* remote = nullptr;
  const uint32_t* local = nullptr;
  int n = 0;
  uint32_t value = 0;
  void* multicast = nullptr;   // the destination's address in a multicast mapping over all ranks' copies, or null
};

int run_mul(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc, bool synchronous, void* const* mirrors = nullptr,
            int n_mirrors = 0, const Exchange* xchg = nullptr) {
  int rc = validate_desc(desc);
  if (rc) return rc;
  const ruyb200_mul_desc& d = *desc;
  DeviceGuard guard(ctx->device);
  ctx->advisory = RUYB200_ADVISORY_NONE;  // ruy/frontend.h:90
  const uint32_t paths = effective_paths(ctx);
  ctx->last_used_path = most_significant_bit(paths & kCompiledPaths);
  if (d.dst.rows == 0 || d.dst.cols == 0) return RUYB200_OK;

  const bool dst_on_device = is_device_pointer(d.dst.data);
  if (!synchronous) {
    const void* ptrs[6] = {d.lhs.data, d.rhs.data, d.dst.data, d.params.bias, d.params.multiplier_fixedpoint_perchannel,
                           d.params.multiplier_exponent_perchannel};
    for (const void* p : ptrs) {
      if (p && !is_device_pointer(p)) return fail(RUYB200_ERR_INVALID, "ruyb200_mul_async needs device pointers");
    }
  }
  ctx->arena.reset(synchronous);
  ctx->bounce_off = ctx->bounce_h2d_end = ctx->bounce_flushed = 0;

  const int depth = d.lhs.cols;
  // double accumulation (ruy's mixed float/double cases) runs on the CUDA-core kernel only, straight from the
  // operands as stored: no packing, no cache entry
  const bool is_f64 = d.params.accum_dtype == RUYB200_F64;
  const bool is_float = d.params.accum_dtype == RUYB200_F32 || is_f64;
  int kernel = choose_kernel(ctx, d);
  if (kernel == RUYB200_KERNEL_TC_I8 && (is_float || dtype_size(d.lhs.dtype) != 1 || dtype_size(d.rhs.dtype) != 1 ||
                                         depth == 0)) {
    kernel = RUYB200_KERNEL_GENERIC;
  }
  if (kernel == RUYB200_KERNEL_SGEMM && !is_float) kernel = RUYB200_KERNEL_GENERIC;
  // Narrow muls (at most kGemvMaxNarrow destination rows or columns) are a single pass over the wide operand
  // (ruy's single-column kernels, ruy/kernel_avx512.cc:628-870,1238-1320).  Both operands must be
  // depth-contiguous where the kernel will read them: as stored, or in their packed form when they are cached.
  const int narrow_rows = std::min(d.dst.rows, d.dst.cols);
  // 9 to kGemvMmaMaxNarrow narrow rows take that kernel only in its MMA form: 8-bit operands whose rows start on
  // 16-byte boundaries (as stored, or packed, which always do)
  const auto rows_aligned = [&](const ruyb200_matrix& m, int side, int other_width) {
    if (should_cache(m, other_width)) return true;
    const SideView v = side_view(m, side, m.data);
    return v.stride_k == 1 && (((uintptr_t)m.data | (uintptr_t)v.stride_w) & 15) == 0;
  };
  const bool mma_form = !is_float && kernel == RUYB200_KERNEL_TC_I8 &&
                        gemv_mma_shape(narrow_rows, std::max(d.dst.rows, d.dst.cols), depth) &&
                        rows_aligned(d.lhs, 0, d.rhs.cols) && rows_aligned(d.rhs, 1, d.lhs.rows);
  if ((kernel == RUYB200_KERNEL_TC_I8 || kernel == RUYB200_KERNEL_SGEMM) && !ctx->force_kernel && n_mirrors == 0 && !xchg && depth > 0 &&
      (narrow_rows <= kGemvMaxNarrow || mma_form)) {
    const bool lhs_ok = side_view(d.lhs, 0, d.lhs.data).stride_k == 1 || should_cache(d.lhs, d.rhs.cols);
    const bool rhs_ok = side_view(d.rhs, 1, d.rhs.data).stride_k == 1 || should_cache(d.rhs, d.lhs.rows);
    // one warp per wide row: a wide side of fewer than 128 rows leaves most SMs idle, and with a very deep 8-bit depth
    // and more than one narrow row the tensor-core kernel is faster (64 x 16384 x 4: 47 us against 68 us)
    const int wide_rows = std::max(d.dst.rows, d.dst.cols);
    const bool few_deep_rows = !is_float && wide_rows >= 32 && wide_rows < 128 && depth >= 8192 &&
                               std::min(d.dst.rows, d.dst.cols) > 1;
    if (lhs_ok && rhs_ok && !few_deep_rows) kernel = RUYB200_KERNEL_GEMV;
  }
  // fp32 muls that fill tensor-core tiles go to the 3 x TF32 kernel; small ones stay on the FFMA kernel, whose single
  // launch costs less than the split pre-pass.  Depth does not decide: both kernels add 32-deep chains into a compensated
  // total, their error grows alike with the square root of the depth, and measured against double precision the
  // tensor-core kernel is the closer one at every depth (1024 x 4096 x 1024: 8.0e-6 against 1.02e-5 of max(|ref|, 1);
  // depth 16384: 1.65e-5 against 1.84e-5) while being five to ten times faster.
  if (kernel == RUYB200_KERNEL_SGEMM && ctx->force_kernel != RUYB200_KERNEL_SGEMM && std::min(d.dst.rows, d.dst.cols) >= 64 &&
      depth >= 32 && depth <= ctx->tc_f32_max_depth && (double)d.dst.rows * d.dst.cols * depth >= (double)(1 << 21)) {
    kernel = RUYB200_KERNEL_TC_F32;
  }
  const bool tc = kernel == RUYB200_KERNEL_TC_I8;
  if ((n_mirrors > 0 || xchg) && (!tc || !dst_on_device || n_mirrors > 7)) {
    return fail(RUYB200_ERR_UNSUPPORTED, "mirrored destinations need 8-bit operands, a device destination and at most 7 mirrors");
  }

  // ruy/create_trmul_params.h:294-319: ruy re-allocates per-channel buffers that are shorter
  // than the padded width and says so; here nothing is read past the logical size, the
  // advisory is kept for callers that watch it.
  const bool channel_row = d.params.channel_dimension == RUYB200_CHANNEL_ROW;
  const int nch = channel_row ? d.dst.rows : d.dst.cols;
  if (!is_float && (d.params.bias || d.params.multiplier_fixedpoint_perchannel)) {
    const int rounding = 1 << d.params.perchannel_buffers_capacity_rounding_log2;
    const int capacity = (nch + rounding - 1) / rounding * rounding;
    const int padded = (nch + 15) / 16 * 16;
    if (capacity < padded) ctx->advisory = RUYB200_ADVISORY_REALLOCATED_PERCHANNEL_BUFFER;
  }

  // operands
  SideView lhs_v, rhs_v;
  const int32_t *lhs_sums = nullptr, *rhs_sums = nullptr;
  // the generic kernel subtracts zero points while loading and the narrow kernel sums while it streams: neither needs sums
  const bool generic = kernel == RUYB200_KERNEL_GENERIC || kernel == RUYB200_KERNEL_GEMV;
  const bool need_lhs_sums = !is_float && !generic && d.rhs.zero_point != 0;
  const bool need_rhs_sums = !is_float && !generic && d.lhs.zero_point != 0;
  // The tensor-core kernel can produce the sums of its m-side operand (the RHS for a column-major destination,
  // the LHS otherwise) itself, so no separate pass over that operand is requested for it.
  const bool m_is_rhs = d.dst.order == RUYB200_COL_MAJOR;
  // Host-resident m-side operand and destination of a large synchronous mul: instead of copy-in, kernel,
  // copy-out one after the other, the m dimension is cut into chunks whose copies (both directions, on two
  // copy streams) overlap each other and the kernels of other chunks.  The m-side operand then goes to the
  // device chunk by chunk, below, not through prepare_side.
  const ruyb200_matrix& m_mat = m_is_rhs ? d.rhs : d.lhs;
  const SideView m_host = side_view(m_mat, m_is_rhs ? 1 : 0, m_mat.data);
  const size_t m_span = storage_span_bytes(m_mat);
  const bool m_on_host = !is_device_pointer(m_mat.data);
  const size_t dst_span = (size_t)(m_is_rhs ? d.dst.cols : d.dst.rows) * (size_t)d.dst.stride * dtype_size(d.dst.dtype);
  const bool streamed = synchronous && tc && n_mirrors == 0 && !ctx->no_chunks && (m_on_host || !dst_on_device) &&
                        !should_cache(m_mat, m_is_rhs ? d.lhs.rows : d.rhs.cols) && m_host.stride_k == 1 &&
                        (m_host.stride_w & 15) == 0 && ((uintptr_t)m_mat.data & 15) == 0 && m_host.width >= 2048 &&
                        (m_on_host ? m_span : 0) + (dst_on_device ? 0 : dst_span) >= (size_t(4) << 20);
  const bool m_streamed = streamed && m_on_host;   // the m-side operand itself travels in chunks
  void* m_dev = nullptr;
  if (m_streamed) {
    m_dev = ctx->arena.alloc(m_span);
    if (!m_dev) return fail(RUYB200_ERR_OOM, "arena allocation of %zu bytes failed", m_span);
  }
  if (m_streamed && !m_is_rhs) {
    lhs_v = side_view(d.lhs, 0, m_dev);
  } else {
    rc = prepare_side(ctx, d.lhs, 0, depth, !is_f64 && should_cache(d.lhs, d.rhs.cols), need_lhs_sums && !(tc && !m_is_rhs), tc, &lhs_v,
                      &lhs_sums, need_lhs_sums);
    if (rc) return rc;
  }
  if (m_streamed && m_is_rhs) {
    rhs_v = side_view(d.rhs, 1, m_dev);
  } else {
    rc = prepare_side(ctx, d.rhs, 1, depth, !is_f64 && should_cache(d.rhs, d.lhs.rows), need_rhs_sums && !(tc && m_is_rhs), tc, &rhs_v,
                      &rhs_sums, need_rhs_sums);
    if (rc) return rc;
  }

  Epilogue ep;
  memset(&ep, 0, sizeof(ep));
  const void* p;
  rc = stage_vector(ctx, d.params.bias, nch, &p, is_f64 ? 8 : 4);
  if (rc) return rc;
  ep.bias = p;
  if (!is_float && d.dst.dtype != RUYB200_I32) {
    rc = stage_vector(ctx, d.params.multiplier_fixedpoint_perchannel, nch, &p);
    if (rc) return rc;
    ep.mfp_pc = (const int32_t*)p;
    rc = stage_vector(ctx, d.params.multiplier_exponent_perchannel, nch, &p);
    if (rc) return rc;
    ep.mexp_pc = (const int32_t*)p;
    ep.mfp = d.params.multiplier_fixedpoint;
    ep.mexp = d.params.multiplier_exponent;
  }
  ep.clamp_min = d.params.clamp_min.i;
  ep.clamp_max = d.params.clamp_max.i;
  ep.dst_zp = d.dst.zero_point;
  ep.depth = depth;
  ep.dst_dtype = d.dst.dtype;
  ep.is_float = is_float;
  int rounding = d.params.rounding_mode;
  if (rounding == RUYB200_ROUNDING_FROM_PATH) {
    rounding = (paths_explicit(ctx) && (ctx->last_used_path & kX86Paths)) ? RUYB200_ROUNDING_X86
                                                                            : RUYB200_ROUNDING_REFERENCE;
  }
  // ruy's x86 back end has 8-bit and int8 x int16 kernels only (ruy/kernel_x86.h:34-233); with an
  // int16 LHS (after the row-major-dst operand swap) it falls back to the standard C++ kernel and
  // therefore to the reference rounding.
  const int canonical_lhs_dtype = d.dst.order == RUYB200_COL_MAJOR ? d.lhs.dtype : d.rhs.dtype;
  if (canonical_lhs_dtype == RUYB200_I16) rounding = RUYB200_ROUNDING_REFERENCE;
  ep.rounding_x86 = rounding == RUYB200_ROUNDING_X86;

  // destination: n is its contiguous dimension.  Col-major dst: n = row (LHS side);
  // row-major dst: n = col (RHS side) -- ruy's operand swap (ruy/create_trmul_params.h:474-479).
  const size_t dst_esz = dtype_size(d.dst.dtype);
  const bool dst_col_major = d.dst.order == RUYB200_COL_MAJOR;
  const int dst_inner = dst_col_major ? d.dst.rows : d.dst.cols;
  const int dst_outer = dst_col_major ? d.dst.cols : d.dst.rows;
  void* dst_dev = d.dst.data;
  if (!dst_on_device) {
    dst_dev = ctx->arena.alloc((size_t)dst_outer * d.dst.stride * dst_esz);
    if (!dst_dev) return fail(RUYB200_ERR_OOM, "arena allocation failed");
  }
  Resolved r;
  r.depth = depth;
  r.dst.data = dst_dev;
  r.dst.stride_m = d.dst.stride;
  r.dst.size_m = dst_outer;
  r.dst.size_n = dst_inner;
  if (dst_col_major) {
    r.n_side = lhs_v;
    r.m_side = rhs_v;
    ep.sums_n = lhs_sums;
    ep.sums_m = rhs_sums;
    ep.channel_on_n = channel_row;
  } else {
    r.n_side = rhs_v;
    r.m_side = lhs_v;
    ep.sums_n = rhs_sums;
    ep.sums_m = lhs_sums;
    ep.channel_on_n = !channel_row;
  }
  ep.zp_m = r.m_side.zero_point;
  ep.zp_n = r.n_side.zero_point;
  r.ep = ep;

  // every small host operand and vector staged above goes up in one copy, ahead of the kernel that reads them
  cudaError_t ce = bounce_flush(ctx);
  if (ce != cudaSuccess) return fail(RUYB200_ERR_CUDA, "upload of staged host data: %s", cudaGetErrorString(ce));
  if (tc) {
    if (!tc_i8_eligible(r.m_side, r.n_side)) return fail(RUYB200_ERR_CUDA, "internal: operands not packed for the tensor-core kernel");
    TcI8Launch L;
    L.m_side = r.m_side;
    L.n_side = r.n_side;
    L.dst = r.dst;
    L.ep = r.ep;
    L.depth = depth;
    L.sm_count = ctx->sm_count;
    L.status = ctx->d_status;
    L.allow_pair = !ctx->no_pair;
    L.allow_shallow = !ctx->no_shallow;
    L.force_pair = ctx->force_pair;
    L.force_block_n = ctx->force_block_n;
    L.fuse_sums_m = true;
    L.n_mirrors = n_mirrors;
    L.multicast = xchg ? xchg->multicast : nullptr;
    for (int i = 0; i < 7; i++) L.mirrors[i] = i < n_mirrors ? mirrors[i] : nullptr;
    if (n_mirrors > 0 && !L.multicast && !ctx->no_store_maps && dtype_size(d.dst.dtype) == 1) {
      L.store_maps = mirrored_store_maps(ctx, r.dst, mirrors, n_mirrors);   // null: the epilogue uses store instructions
    }
    if (xchg && xchg->n > 0) {
      L.xchg_remote = xchg->remote;
      L.xchg_local = xchg->local;
      L.n_xchg = xchg->n;
      L.xchg_value = xchg->value;
      L.xchg_counter = (unsigned int*)(ctx->d_status + 1);
      L.xchg_limit_ns = ctx->peer_wait_ns;
    }
    TcI8Info info = {};
    if (ctx->trace) L.info = &info;
    struct TraceAtExit {   // prints after the launch has filled `info`
      ruyb200_ctx* ctx; const ruyb200_mul_desc& d; const TcI8Info& info; bool x86, streamed; int mirrors;
      ~TraceAtExit() {
        if (!ctx->trace) return;
        if (info.shallow) {
          fprintf(stderr, "ruy_b200: mul %dx%dx%d kernel=tc_i8 (shallow depth: %d activation rows per 128-byte line, %d tiles of %d rows x %d, "
                  "row sums from shared memory), rounding=%s\n", d.lhs.rows, d.lhs.cols, d.rhs.cols, info.shallow, info.tiles, 128 * info.shallow,
                  info.block_n, x86 ? "x86" : "reference");
          return;
        }
        fprintf(stderr, "ruy_b200: mul %dx%dx%d kernel=tc_i8 tiles=%d of %s x %d (estimated %.0f cycles), %d-byte tile rows, m-side sums %s, rounding=%s%s, mirrors=%d\n",
                d.lhs.rows, d.lhs.cols, d.rhs.cols, info.tiles, info.pair ? "256 (two CTAs)" : "128", info.block_n, info.est_cycles, info.row_pitch,
                info.fused_sums ? "from the tensor core" : "not fused", x86 ? "x86" : "reference",
                streamed ? ", host operands in chunks" : "", mirrors);
      }
    } trace_at_exit{ctx, d, info, ep.rounding_x86 != 0, streamed, n_mirrors};
    if (streamed) {
      rc = run_chunks(ctx, d, L, m_streamed ? (const char*)m_mat.data : nullptr, dst_on_device ? nullptr : (char*)d.dst.data, dst_esz);
      if (rc) return rc;
      ctx->counters[5] = kernel;
      return ruyb200_ctx_sync(ctx);
    }
    ce = launch_tc_i8(L, ctx->stream);
  } else if (kernel == RUYB200_KERNEL_TC_F32) {
    void* sm_ = ctx->arena.alloc(tc_f32_scratch_bytes(r.m_side.width, depth));
    void* sn_ = ctx->arena.alloc(tc_f32_scratch_bytes(r.n_side.width, depth));
    if (!sm_ || !sn_) return fail(RUYB200_ERR_OOM, "arena allocation failed");
    ce = launch_tc_f32(r.m_side, r.n_side, r.dst, r.ep, sm_, sn_, ctx->sm_count, ctx->d_status, ctx->stream);
    ctx->counters[0] += 2;   // the two split launches
    if (ctx->trace) fprintf(stderr, "ruy_b200: mul %dx%dx%d kernel=tc_f32 (tcgen05 kind::tf32, hi/lo split, three products, 32-deep accumulation chains)\n",
                            d.lhs.rows, d.lhs.cols, d.rhs.cols);
  } else if (kernel == RUYB200_KERNEL_GEMV && gemv_eligible(r.m_side, r.n_side, depth, is_float)) {
    ce = launch_gemv(r.m_side, r.n_side, r.dst, r.ep, ctx->stream);
    if (ctx->trace) fprintf(stderr, "ruy_b200: mul %dx%dx%d kernel=gemv (one pass over the wide operand, %s)\n", d.lhs.rows, d.lhs.cols, d.rhs.cols,
                            is_float ? "fp32 FFMA, compensated" : "dp4a or register-level MMAs, sums on the way");
  } else if (is_f64) {
    kernel = RUYB200_KERNEL_GENERIC;
    ce = launch_generic_f64(r.m_side, r.n_side, r.dst, r.ep, d.params.clamp_min.d, d.params.clamp_max.d, ctx->stream);
    if (ctx->trace) fprintf(stderr, "ruy_b200: mul %dx%dx%d kernel=generic (CUDA cores, double accumulation)\n", d.lhs.rows, d.lhs.cols, d.rhs.cols);
  } else if (is_float && kernel != RUYB200_KERNEL_GENERIC) {
    kernel = RUYB200_KERNEL_SGEMM;
    ce = launch_sgemm(r.m_side, r.n_side, r.dst, r.ep, ctx->stream);
    if (ctx->trace) fprintf(stderr, "ruy_b200: mul %dx%dx%d kernel=sgemm (fp32 FFMA, compensated)\n", d.lhs.rows, d.lhs.cols, d.rhs.cols);
  } else {
    kernel = RUYB200_KERNEL_GENERIC;
    ce = launch_generic(r.m_side, r.n_side, r.dst, r.ep, ctx->stream);
    if (ctx->trace) fprintf(stderr, "ruy_b200: mul %dx%dx%d kernel=generic (CUDA cores, any type/layout)\n", d.lhs.rows, d.lhs.cols, d.rhs.cols);
  }
  ctx->counters[0]++;
  ctx->counters[5] = kernel;
  if (ce != cudaSuccess) return fail(RUYB200_ERR_CUDA, "kernel launch: %s", cudaGetErrorString(ce));

  if (!dst_on_device) {
    const size_t row_bytes = (size_t)dst_inner * dst_esz, pitch = (size_t)d.dst.stride * dst_esz;
    ctx->counters[4] += row_bytes * dst_outer;
    char* pinned = synchronous && row_bytes * dst_outer <= kBounceBytes / 2 ? bounce_take(ctx, row_bytes * dst_outer) : nullptr;
    if (pinned) {
      // a small destination: to the pinned buffer (rows packed tightly), then by memcpy to where the caller wants it
      CUDA_TRY(cudaMemcpy2DAsync(pinned, row_bytes, dst_dev, pitch, row_bytes, dst_outer, cudaMemcpyDeviceToHost, ctx->stream));
      const int rc_sync = ruyb200_ctx_sync(ctx);
      if (rc_sync) return rc_sync;
      for (int i = 0; i < dst_outer; i++) memcpy((char*)d.dst.data + (size_t)i * pitch, pinned + (size_t)i * row_bytes, row_bytes);
      return RUYB200_OK;
    }
    CUDA_TRY(cudaMemcpy2DAsync(d.dst.data, pitch, dst_dev, pitch, row_bytes, dst_outer, cudaMemcpyDeviceToHost, ctx->stream));
  }
  if (synchronous) return ruyb200_ctx_sync(ctx);
  return RUYB200_OK;
}


// ---- prepacked-cache persistence ---------------------------------------------------------------
//
// ruy packs a cached operand once per process and has no on-disk format (ruy/prepacked_cache.cc:79-127).  Here an
// entry can be taken out of the device cache as a self-describing blob and put back later (another process,
// another run), so that weights are packed once per model.  Blob = 64-byte header, packed data, sums.

struct BlobHeader {
  char magic[8];           // "RUYB2PCK"
  uint32_t abi_version;    // RUYB200_ABI_VERSION of the writer
  uint32_t format;         // RUYB200_CACHE_FORMAT_ROWS16: [width][packed_depth] depth-contiguous rows + int32 sums[width]
  uint8_t dtype, side, has_sums, reserved;
  int32_t width, depth, packed_depth, zero_point;
  uint64_t data_bytes, sums_bytes;
  uint64_t checksum;       // FNV-1a of the header up to here and of the payload
};
static_assert(sizeof(BlobHeader) == 64, "blob header is 64 bytes");
const char kBlobMagic[8] = {'R', 'U', 'Y', 'B', '2', 'P', 'C', 'K'};

uint64_t fnv1a(const void* p, size_t n, uint64_t h) {
  const unsigned char* b = (const unsigned char*)p;
  for (size_t i = 0; i < n; i++) {
    h ^= b[i];
    h *= 1099511628211ull;
  }
  return h;
}

uint64_t blob_checksum(const BlobHeader& h, const void* payload, size_t payload_bytes) {
  uint64_t c = fnv1a(&h, offsetof(BlobHeader, checksum), 14695981039346656037ull);
  return fnv1a(payload, payload_bytes, c);
}

// Checks everything that can be checked without a device.
int parse_blob(const void* blob, size_t n, BlobHeader* out) {
  if (!blob || n < sizeof(BlobHeader)) return fail(RUYB200_ERR_INVALID, "cache blob: shorter than its header");
  BlobHeader h;
  memcpy(&h, blob, sizeof(h));
  if (memcmp(h.magic, kBlobMagic, 8) != 0) return fail(RUYB200_ERR_INVALID, "cache blob: bad magic");
  if (h.abi_version != RUYB200_ABI_VERSION)
    return fail(RUYB200_ERR_INVALID, "cache blob: written by ABI version %u, this library is version %d", h.abi_version, RUYB200_ABI_VERSION);
  if (h.format != RUYB200_CACHE_FORMAT_ROWS16) return fail(RUYB200_ERR_INVALID, "cache blob: unknown tile format %u", h.format);
  if (h.dtype > RUYB200_F32 || h.dtype == RUYB200_I32 || h.side > 1 || h.width <= 0 || h.depth <= 0)
    return fail(RUYB200_ERR_INVALID, "cache blob: bad field");
  if (h.packed_depth != packed_depth_for(h.depth, h.dtype) && h.packed_depth != tc_packed_depth(h.depth, h.dtype)) return fail(RUYB200_ERR_INVALID, "cache blob: packed depth does not match this library's layout");
  const uint64_t want_data = (uint64_t)h.width * h.packed_depth * dtype_size(h.dtype);
  const uint64_t want_sums = h.has_sums ? (uint64_t)h.width * 4 : 0;
  if ((h.has_sums != 0) != (h.dtype != RUYB200_F32) || h.data_bytes != want_data || h.sums_bytes != want_sums ||
      n != sizeof(BlobHeader) + want_data + want_sums)
    return fail(RUYB200_ERR_INVALID, "cache blob: sizes do not add up");
  if (blob_checksum(h, (const char*)blob + sizeof(BlobHeader), n - sizeof(BlobHeader)) != h.checksum)
    return fail(RUYB200_ERR_INVALID, "cache blob: checksum mismatch");
  *out = h;
  return RUYB200_OK;
}

}  // namespace

// ---- exported C ABI ------------------------------------------------------------------------

extern "C" {

int ruyb200_abi_version(void) { return RUYB200_ABI_VERSION; }

int ruyb200_device_count(void) {
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) {
    cudaGetLastError();
    return fail(RUYB200_ERR_NO_DEVICE, "no CUDA device or driver");
  }
  return n;
}

const char* ruyb200_last_error(void) { return g_last_error.c_str(); }

int ruyb200_ctx_create_on_stream(int device, void* cuda_stream, ruyb200_ctx** out) {
  if (!out) return fail(RUYB200_ERR_INVALID, "null out pointer");
  *out = nullptr;
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    cudaGetLastError();
    return fail(RUYB200_ERR_NO_DEVICE, "no CUDA device available (this library has no CPU path)");
  }
  if (device < 0) CUDA_TRY(cudaGetDevice(&device));
  if (device >= count) return fail(RUYB200_ERR_INVALID, "device %d out of range (%d devices)", device, count);
  cudaDeviceProp prop;
  CUDA_TRY(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10) {
    return fail(RUYB200_ERR_NO_DEVICE, "device %d is sm_%d%d; this library is built for sm_100a only", device,
                prop.major, prop.minor);
  }
  DeviceGuard guard(device);
  ruyb200_ctx* ctx = new ruyb200_ctx;
  ctx->device = device;
  ctx->sm_count = prop.multiProcessorCount;
  if (cuda_stream) {
    ctx->stream = (cudaStream_t)cuda_stream;
  } else {
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
      delete ctx;
      return fail(RUYB200_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    ctx->own_stream = true;
  }
  // word 0: status of bounded waits; word 1: finished-CTA counter of launches that end with a flag exchange
  if (cudaMalloc(&ctx->d_status, 4 * sizeof(int)) != cudaSuccess || cudaMemset(ctx->d_status, 0, 4 * sizeof(int)) != cudaSuccess ||
      cudaMallocHost(&ctx->h_status, sizeof(int)) != cudaSuccess) {
    cudaGetLastError();
    ruyb200_ctx_destroy(ctx);
    return fail(RUYB200_ERR_CUDA, "context allocation failed");
  }
  *ctx->h_status = 0;
  const char* fk = getenv("RUYB200_FORCE_KERNEL");
  if (fk && !strcmp(fk, "generic")) ctx->force_kernel = RUYB200_KERNEL_GENERIC;
  if (fk && !strcmp(fk, "tc_i8")) ctx->force_kernel = RUYB200_KERNEL_TC_I8;
  if (fk && !strcmp(fk, "sgemm")) ctx->force_kernel = RUYB200_KERNEL_SGEMM;   // keeps fp32 muls on the FFMA kernel   // keeps narrow 8-bit muls on the tensor-core kernel
  const char* np = getenv("RUYB200_NO_PAIR");
  ctx->no_pair = np && *np && *np != '0';
  const char* tile = getenv("RUYB200_TILE");
  if (tile && *tile) {
    if (!strncmp(tile, "pair", 4)) ctx->force_pair = 1;
    if (!strncmp(tile, "single", 6)) ctx->force_pair = 0;
    const char* colon = strchr(tile, ':');
    if (colon && atoi(colon + 1) > 0) ctx->force_block_n = atoi(colon + 1);
  }
  const char* fd = getenv("RUYB200_TC_F32_MAX_DEPTH");
  if (fd && atoi(fd) >= 32) ctx->tc_f32_max_depth = atoi(fd);
  const char* ns = getenv("RUYB200_NO_SHALLOW");
  ctx->no_shallow = ns && *ns && *ns != '0';
  const char* nc = getenv("RUYB200_NO_CHUNKS");
  ctx->no_chunks = nc && *nc && *nc != '0';
  const char* nsm = getenv("RUYB200_NO_STORE_MAPS");
  ctx->no_store_maps = nsm && *nsm && *nsm != '0';
  const char* ck = getenv("RUYB200_CHUNKS");
  if (ck && atoi(ck) >= 2 && atoi(ck) <= kMaxChunks) ctx->chunk_target = atoi(ck);
  const char* tr = getenv("RUYB200_TRACE");
  ctx->trace = tr && *tr && *tr != '0';
  *out = ctx;
  return RUYB200_OK;
}

int ruyb200_ctx_create(int device, ruyb200_ctx** out) { return ruyb200_ctx_create_on_stream(device, nullptr, out); }

int ruyb200_ctx_destroy(ruyb200_ctx* ctx) {
  if (!ctx) return RUYB200_OK;
  DeviceGuard guard(ctx->device);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  ctx->cache.clear();
  for (CacheSlab& sl : ctx->cache_slabs) {
    if (sl.base) cudaFree(sl.base);
  }
  ctx->cache_slabs.clear();
  ctx->arena.release();
  if (ctx->bounce) cudaFreeHost(ctx->bounce);
  if (ctx->d_bounce) cudaFree(ctx->d_bounce);
  for (auto& kv : ctx->store_maps) cudaFree(kv.second);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->h_status) cudaFreeHost(ctx->h_status);
  if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
  if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
  for (int i = 0; i < kMaxChunks; i++) {
    if (ctx->chunk_in[i]) cudaEventDestroy(ctx->chunk_in[i]);
    if (ctx->chunk_done[i]) cudaEventDestroy(ctx->chunk_done[i]);
    if (ctx->chunk_out[i]) cudaEventDestroy(ctx->chunk_out[i]);
  }
  if (ctx->chunk_start) cudaEventDestroy(ctx->chunk_start);
  if (ctx->own_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
  cudaGetLastError();
  delete ctx;
  return RUYB200_OK;
}

int ruyb200_ctx_set_max_num_threads(ruyb200_ctx* ctx, int value) {
  if (!ctx || value < 1) return fail(RUYB200_ERR_INVALID, "max_num_threads must be >= 1");
  ctx->max_num_threads = value;
  return RUYB200_OK;
}

int ruyb200_ctx_get_max_num_threads(const ruyb200_ctx* ctx) { return ctx ? ctx->max_num_threads : 0; }

int ruyb200_ctx_set_runtime_enabled_paths(ruyb200_ctx* ctx, uint32_t path_mask) {
  if (!ctx) return fail(RUYB200_ERR_INVALID, "null context");
  ctx->enabled_paths = path_mask & 0xFF;
  return RUYB200_OK;
}

uint32_t ruyb200_ctx_get_runtime_enabled_paths(ruyb200_ctx* ctx) { return ctx ? effective_paths(ctx) : 0; }

uint32_t ruyb200_ctx_last_used_path(const ruyb200_ctx* ctx) { return ctx ? ctx->last_used_path : 0; }

int ruyb200_ctx_performance_advisory(const ruyb200_ctx* ctx, int advisory) {
  return ctx && advisory != RUYB200_ADVISORY_NONE && (ctx->advisory & advisory) ? 1 : 0;
}

int ruyb200_ctx_clear_prepacked_cache(ruyb200_ctx* ctx) {
  if (!ctx) return fail(RUYB200_ERR_INVALID, "null context");
  DeviceGuard guard(ctx->device);
  if (ctx->stream) cudaStreamSynchronize(ctx->stream);
  for (auto it = ctx->cache.begin(); it != ctx->cache.end();) {
    if (it->second.pins > 0) {   // a live plan still reads this entry
      ++it;
      continue;
    }
    ctx->cache_bytes -= it->second.bytes;
    cache_free(ctx, it->second);
    it = ctx->cache.erase(it);
  }
  return RUYB200_OK;
}

int ruyb200_ctx_set_prepacked_cache_budget(ruyb200_ctx* ctx, size_t bytes) {
  if (!ctx) return fail(RUYB200_ERR_INVALID, "null context");
  ctx->cache_budget = bytes;
  return RUYB200_OK;
}

size_t ruyb200_ctx_prepacked_cache_bytes(const ruyb200_ctx* ctx) { return ctx ? ctx->cache_bytes : 0; }

int ruyb200_ctx_prepacked_cache_entries(const ruyb200_ctx* ctx) { return ctx ? (int)ctx->cache.size() : 0; }

int ruyb200_ctx_counters(const ruyb200_ctx* ctx, uint64_t out[6]) {
  if (!ctx || !out) return fail(RUYB200_ERR_INVALID, "null argument");
  for (int i = 0; i < 6; i++) out[i] = ctx->counters[i];
  return RUYB200_OK;
}

void* ruyb200_ctx_stream(const ruyb200_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int ruyb200_ctx_sync(ruyb200_ctx* ctx) {
  if (!ctx) return fail(RUYB200_ERR_INVALID, "null context");
  DeviceGuard guard(ctx->device);
  CUDA_TRY(cudaMemcpyAsync(ctx->h_status, ctx->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream));
  CUDA_TRY(cudaStreamSynchronize(ctx->stream));
  if (*ctx->h_status != 0) {
    const int code = *ctx->h_status;
    *ctx->h_status = 0;
    cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream);
    cudaStreamSynchronize(ctx->stream);
    return fail(RUYB200_ERR_TIMEOUT, "a bounded device-side wait gave up (role code %d); results are invalid", code);
  }
  return RUYB200_OK;
}

int ruyb200_validate(const ruyb200_mul_desc* desc) { return validate_desc(desc); }

int ruyb200_mul(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc) {
  if (!ctx) return fail(RUYB200_ERR_INVALID, "null context");
  // the labels ruy's own profiler uses (ruy/frontend.h:86-89), as NVTX ranges
  nvtxRangePushA("Mul");
  if (desc) {
    char label[64];
    snprintf(label, sizeof(label), "matmul shape: %dx%dx%d", desc->lhs.rows, desc->lhs.cols, desc->rhs.cols);
    nvtxRangePushA(label);
  }
  const int rc = run_mul(ctx, desc, true);
  if (desc) nvtxRangePop();
  nvtxRangePop();
  return rc;
}

int ruyb200_mul_async(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc) {
  if (!ctx) return fail(RUYB200_ERR_INVALID, "null context");
  return run_mul(ctx, desc, false);
}

int ruyb200_mul_async_mirrored(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc, void* const* mirror_dst, int n_mirrors) {
  if (!ctx) return fail(RUYB200_ERR_INVALID, "null context");
  if (n_mirrors < 0 || (n_mirrors > 0 && !mirror_dst)) return fail(RUYB200_ERR_INVALID, "bad mirror list");
  return run_mul(ctx, desc, false, mirror_dst, n_mirrors);
}

int ruyb200_mul_async_mirrored_exchange(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc, void* const* mirror_dst, int n_mirrors,
                                        uint32_t* const* remote_flags_device_array, const uint32_t* local_flags, int n_flags,
                                        uint32_t value) {
  if (!ctx) return fail(RUYB200_ERR_INVALID, "null context");
  if (n_mirrors < 0 || (n_mirrors > 0 && !mirror_dst)) return fail(RUYB200_ERR_INVALID, "bad mirror list");
  if (!remote_flags_device_array || !local_flags || n_flags < 1 || n_flags > 32) return fail(RUYB200_ERR_INVALID, "bad flag arguments");
  Exchange x;
  x.remote = remote_flags_device_array;
  x.local = local_flags;
  x.n = n_flags;
  x.value = value;
  return run_mul(ctx, desc, false, mirror_dst, n_mirrors, &x);
}

int ruyb200_mul_async_multicast_exchange(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc, void* multicast_dst,
                                         uint32_t* const* remote_flags_device_array, const uint32_t* local_flags, int n_flags,
                                         uint32_t value) {
  if (!ctx) return fail(RUYB200_ERR_INVALID, "null context");
  if (!multicast_dst) return fail(RUYB200_ERR_INVALID, "null multicast address");
  if (!remote_flags_device_array || !local_flags || n_flags < 1 || n_flags > 32) return fail(RUYB200_ERR_INVALID, "bad flag arguments");
  if (desc && desc->dst.dtype != RUYB200_I8 && desc->dst.dtype != RUYB200_U8)
    return fail(RUYB200_ERR_UNSUPPORTED, "a multicast destination must be 8-bit");
  if (desc) {
    const int inner = desc->dst.order == RUYB200_COL_MAJOR ? desc->dst.rows : desc->dst.cols;
    if ((((uintptr_t)desc->dst.data | (uintptr_t)multicast_dst) & 15) != 0 || (desc->dst.stride & 15) != 0 || (inner & 15) != 0)
      return fail(RUYB200_ERR_UNSUPPORTED, "a multicast destination needs a 16-byte aligned base and stride and a contiguous dimension that is a multiple of 16");
  }
  Exchange x;
  x.remote = remote_flags_device_array;
  x.local = local_flags;
  x.n = n_flags;
  x.value = value;
  x.multicast = multicast_dst;
  return run_mul(ctx, desc, false, nullptr, 0, &x);
}

int ruyb200_pack(ruyb200_ctx* ctx, const ruyb200_matrix* src, int side, void* packed, size_t packed_capacity,
                 int32_t* sums, int32_t* packed_depth) {
  if (!ctx || !src || !packed || side < 0 || side > 1) return fail(RUYB200_ERR_INVALID, "bad argument");
  if (src->dtype > RUYB200_F32 || src->dtype == RUYB200_I32) return fail(RUYB200_ERR_UNSUPPORTED, "bad dtype");
  DeviceGuard guard(ctx->device);
  const int depth = side == 0 ? src->cols : src->rows;
  const int pd = packed_depth_for(depth, src->dtype);
  if (packed_depth) *packed_depth = pd;
  SideView v = side_view(*src, side, src->data);
  if ((size_t)v.width * pd * dtype_size(src->dtype) > packed_capacity)
    return fail(RUYB200_ERR_INVALID, "packed buffer too small");
  ctx->arena.reset(false);
  if (!is_device_pointer(src->data)) {
    const size_t span = storage_span_bytes(*src);
    void* dptr = ctx->arena.alloc(span);
    if (!dptr) return fail(RUYB200_ERR_OOM, "arena allocation failed");
    CUDA_TRY(cudaMemcpyAsync(dptr, src->data, span, cudaMemcpyHostToDevice, ctx->stream));
    v.data = dptr;
  }
  cudaError_t ce = launch_pack(v, depth, pd, packed, src->dtype == RUYB200_F32 ? nullptr : sums, ctx->stream);
  ctx->counters[0]++;
  if (ce != cudaSuccess) return fail(RUYB200_ERR_CUDA, "pack launch: %s", cudaGetErrorString(ce));
  return ruyb200_ctx_sync(ctx);
}

int ruyb200_ctx_set_peer_wait_ms(ruyb200_ctx* ctx, uint32_t ms) {
  if (!ctx || ms == 0) return fail(RUYB200_ERR_INVALID, "bad argument");
  ctx->peer_wait_ns = (unsigned long long)ms * 1000000ull;
  return RUYB200_OK;
}

int ruyb200_cache_blob_info(const void* blob, size_t n, ruyb200_cache_blob* out) {
  BlobHeader h;
  int rc = parse_blob(blob, n, &h);
  if (rc) return rc;
  if (out) {
    out->abi_version = h.abi_version;
    out->format = h.format;
    out->dtype = h.dtype;
    out->side = h.side;
    out->has_sums = h.has_sums;
    out->reserved = 0;
    out->width = h.width;
    out->depth = h.depth;
    out->packed_depth = h.packed_depth;
    out->zero_point = h.zero_point;
    out->data_bytes = h.data_bytes;
    out->sums_bytes = h.sums_bytes;
  }
  return RUYB200_OK;
}

int ruyb200_cache_export(ruyb200_ctx* ctx, const ruyb200_matrix* src, int side, void* blob, size_t* n) {
  if (!ctx || !src || !n || side < 0 || side > 1) return fail(RUYB200_ERR_INVALID, "bad argument");
  const int depth = side == 0 ? src->cols : src->rows;
  SideView v = side_view(*src, side, src->data);
  CacheKey key(src->data, v.width, depth, v.stride_w, v.stride_k, src->zero_point, (int)src->dtype, side);
  auto it = ctx->cache.find(key);
  if (it == ctx->cache.end()) return fail(RUYB200_ERR_INVALID, "ruyb200_cache_export: this matrix is not in the prepacked cache");
  const CacheEntry& e = it->second;
  BlobHeader h;
  memset(&h, 0, sizeof(h));
  memcpy(h.magic, kBlobMagic, 8);
  h.abi_version = RUYB200_ABI_VERSION;
  h.format = RUYB200_CACHE_FORMAT_ROWS16;
  h.dtype = src->dtype;
  h.side = (uint8_t)side;
  h.has_sums = e.sums != nullptr;
  h.width = v.width;
  h.depth = depth;
  h.packed_depth = e.packed_depth;
  h.zero_point = src->zero_point;
  h.data_bytes = (uint64_t)v.width * e.packed_depth * dtype_size(src->dtype);
  h.sums_bytes = e.sums ? (uint64_t)v.width * 4 : 0;
  const size_t need = sizeof(BlobHeader) + h.data_bytes + h.sums_bytes;
  if (!blob) {   // size query
    *n = need;
    return RUYB200_OK;
  }
  if (*n < need) {
    *n = need;
    return fail(RUYB200_ERR_INVALID, "ruyb200_cache_export: the buffer is too small (%zu bytes needed)", need);
  }
  DeviceGuard guard(ctx->device);
  char* payload = (char*)blob + sizeof(BlobHeader);
  CUDA_TRY(cudaStreamSynchronize(ctx->stream));   // the entry may still be being packed
  CUDA_TRY(cudaMemcpy(payload, e.packed, h.data_bytes, cudaMemcpyDeviceToHost));
  if (e.sums) CUDA_TRY(cudaMemcpy(payload + h.data_bytes, e.sums, h.sums_bytes, cudaMemcpyDeviceToHost));
  h.checksum = blob_checksum(h, payload, h.data_bytes + h.sums_bytes);
  memcpy(blob, &h, sizeof(h));
  *n = need;
  return RUYB200_OK;
}

int ruyb200_cache_import(ruyb200_ctx* ctx, const ruyb200_matrix* src, int side, const void* blob, size_t n) {
  if (!ctx || !src || side < 0 || side > 1) return fail(RUYB200_ERR_INVALID, "bad argument");
  BlobHeader h;
  int rc = parse_blob(blob, n, &h);
  if (rc) return rc;
  const int depth = side == 0 ? src->cols : src->rows;
  SideView v = side_view(*src, side, src->data);
  if (h.side != side || h.dtype != src->dtype || h.width != v.width || h.depth != depth || h.zero_point != src->zero_point)
    return fail(RUYB200_ERR_INVALID, "ruyb200_cache_import: the blob describes another matrix (side %d, dtype %d, %d x %d, zero point %d)",
                h.side, h.dtype, h.width, h.depth, h.zero_point);
  CacheKey key(src->data, v.width, depth, v.stride_w, v.stride_k, src->zero_point, (int)src->dtype, side);
  if (ctx->cache.count(key)) return RUYB200_OK;   // already resident
  DeviceGuard guard(ctx->device);
  const size_t data_bytes = ((size_t)h.data_bytes + 255) & ~size_t(255);
  const size_t sums_bytes = h.has_sums ? (((size_t)h.sums_bytes + 255) & ~size_t(255)) : 0;
  const size_t total = data_bytes + sums_bytes;
  while (!ctx->cache.empty() && ctx->cache_bytes + total > ctx->cache_budget) {
    if (!cache_evict_one(ctx)) break;
  }
  CacheEntry e;
  void* buf = cache_alloc(ctx, total, &e.slab);
  if (!buf) return fail(RUYB200_ERR_OOM, "prepacked cache: allocation of %zu bytes failed", total);
  e.packed = buf;
  e.sums = h.has_sums ? (int32_t*)((char*)buf + data_bytes) : nullptr;
  e.packed_depth = h.packed_depth;
  e.bytes = total;
  e.stamp = ++ctx->cache_clock;
  const char* payload = (const char*)blob + sizeof(BlobHeader);
  cudaError_t ce = cudaMemcpyAsync(e.packed, payload, h.data_bytes, cudaMemcpyHostToDevice, ctx->stream);
  if (ce == cudaSuccess && e.sums) ce = cudaMemcpyAsync(e.sums, payload + h.data_bytes, h.sums_bytes, cudaMemcpyHostToDevice, ctx->stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(ctx->stream);   // the caller may free the blob on return
  if (ce != cudaSuccess) {
    cache_free(ctx, e);
    return fail(RUYB200_ERR_CUDA, "ruyb200_cache_import: %s", cudaGetErrorString(ce));
  }
  ctx->counters[3] += h.data_bytes + h.sums_bytes;
  ctx->cache_bytes += total;
  ctx->cache.emplace(key, e);
  return RUYB200_OK;
}

}  // extern "C"

// ---- plan support (used by plan.cu) -----------------------------------------------------------
namespace ruyb200 {

cudaStream_t ctx_stream(ruyb200_ctx* ctx) { return ctx->stream; }
int ctx_device(ruyb200_ctx* ctx) { return ctx->device; }
int ctx_sm_count(ruyb200_ctx* ctx) { return ctx->sm_count; }
int* ctx_status_word(ruyb200_ctx* ctx) { return ctx->d_status; }
void ctx_count_launch(ruyb200_ctx* ctx, int kernel) {
  ctx->counters[0]++;
  ctx->counters[5] = kernel;
}
int ctx_fail(int status, const char* msg) { return fail(status, "%s", msg); }
int ctx_validate(const ruyb200_mul_desc* d) { return validate_desc(d); }
bool ptr_on_device(const void* p) { return is_device_pointer(p); }
int ctx_rounding_is_x86(ruyb200_ctx* ctx, int rounding_mode) {
  if (rounding_mode == RUYB200_ROUNDING_X86) return 1;
  if (rounding_mode == RUYB200_ROUNDING_REFERENCE) return 0;
  const uint32_t paths = effective_paths(ctx);
  ctx->last_used_path = most_significant_bit(paths & kCompiledPaths);
  return paths_explicit(ctx) && (ctx->last_used_path & kX86Paths) ? 1 : 0;
}
int ctx_run_mul_async(ruyb200_ctx* ctx, const ruyb200_mul_desc* d) { return run_mul(ctx, d, false); }

// Resolves one (already validated, device-resident) mul for a plan.  Operands whose cache policy asks for
// it are taken from the prepacked cache (packed now on a miss) and pinned there; `pinned` receives the
// entries to unpin when the plan dies.  *fits tells whether the mul can be an item of the batched kernel.
int ctx_plan_item(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc, BatchItem* out, bool* fits,
                  std::vector<CacheKey>* pinned) {
  const ruyb200_mul_desc& d = *desc;
  *fits = false;
  memset(out, 0, sizeof(*out));
  if (d.params.accum_dtype != RUYB200_I32 || d.dst.rows == 0 || d.dst.cols == 0 || d.lhs.cols == 0) return RUYB200_OK;
  DeviceGuard guard(ctx->device);
  const int depth = d.lhs.cols;
  SideView views[2];
  const int32_t* cached_sums[2] = {nullptr, nullptr};
  const ruyb200_matrix* mats[2] = {&d.lhs, &d.rhs};
  for (int side = 0; side < 2; side++) {
    const ruyb200_matrix& m = *mats[side];
    const int other_width = side == 0 ? d.rhs.cols : d.lhs.rows;
    if (should_cache(m, other_width) && dtype_size(m.dtype) == 1) {
      const int32_t* sums = nullptr;
      ctx->arena.reset(false);
      int rc = prepare_side(ctx, m, side, depth, true, false, true, &views[side], &sums);
      if (rc) return rc;
      cached_sums[side] = sums;
      SideView src = side_view(m, side, m.data);
      CacheKey key(m.data, src.width, depth, src.stride_w, src.stride_k, m.zero_point, (int)m.dtype, side);
      auto it = ctx->cache.find(key);
      if (it != ctx->cache.end()) {
        it->second.pins++;
        pinned->push_back(key);
      }
    } else {
      views[side] = side_view(m, side, m.data);
    }
  }
  const bool dst_col_major = d.dst.order == RUYB200_COL_MAJOR;
  const SideView& ms = dst_col_major ? views[0] : views[1];   // the destination's contiguous dimension
  const SideView& ns = dst_col_major ? views[1] : views[0];
  if (!batch_i8_fits(ms, ns, depth)) return RUYB200_OK;
  const bool channel_row = d.params.channel_dimension == RUYB200_CHANNEL_ROW;
  out->m_ptr = (const uint8_t*)ms.data;
  out->n_ptr = (const uint8_t*)ns.data;
  out->dst = (uint8_t*)d.dst.data;
  out->bias = (const int32_t*)d.params.bias;
  if (d.dst.dtype != RUYB200_I32) {
    out->mfp_pc = d.params.multiplier_fixedpoint_perchannel;
    out->mexp_pc = d.params.multiplier_exponent_perchannel;
    out->mfp = d.params.multiplier_fixedpoint;
    out->mexp = d.params.multiplier_exponent;
  }
  out->size_m = ms.width;
  out->size_n = ns.width;
  out->depth = depth;
  out->stride_m = (int32_t)ms.stride_w;
  out->stride_n = (int32_t)ns.stride_w;
  out->dst_stride = d.dst.stride;
  out->zp_m = ms.zero_point;
  out->zp_n = ns.zero_point;
  out->dst_zp = d.dst.zero_point;
  out->clamp_min = d.params.clamp_min.i;
  out->clamp_max = d.params.clamp_max.i;
  uint32_t flags = 0;
  const bool channel_on_m = dst_col_major ? channel_row : !channel_row;
  if (!channel_on_m) flags |= kItemChannelOnN;
  if (ms.dtype == RUYB200_I8) flags |= kItemMSigned;
  if (ns.dtype == RUYB200_I8) flags |= kItemNSigned;
  if (ctx_rounding_is_x86(ctx, d.params.rounding_mode)) flags |= kItemX86;
  flags |= (uint32_t)d.dst.dtype << kItemDstShift;
  // the cache's sums stay valid as long as the entry is pinned by the plan
  out->sums_m = ns.zero_point != 0 ? cached_sums[dst_col_major ? 0 : 1] : nullptr;
  auto tma_ok = [](const SideView& v) { return (((uintptr_t)v.data | (uintptr_t)v.stride_w) & 15) == 0; };
  if (tma_ok(ms)) flags |= kItemMTma;
  if (tma_ok(ns)) flags |= kItemNTma;
  const int nch = channel_on_m ? ms.width : ns.width;
  bool vec_bulk = (nch & 3) == 0 && (ms.width & 3) == 0;
  const void* vec_ptrs[4] = {out->bias, out->mfp_pc, out->mexp_pc, out->sums_m};
  for (const void* p : vec_ptrs) vec_bulk = vec_bulk && ((uintptr_t)p & 15) == 0;
  if (vec_bulk) flags |= kItemVecBulk;
  out->flags = flags;
  *fits = true;
  return RUYB200_OK;
}

// Releases exactly the entries a plan pinned (the full key: the same source pointer may be cached more than once,
// e.g. as LHS of one mul and RHS of another, or with two zero points).
void ctx_unpin(ruyb200_ctx* ctx, const std::vector<CacheKey>& pinned) {
  for (const CacheKey& key : pinned) {
    auto it = ctx->cache.find(key);
    if (it != ctx->cache.end() && it->second.pins > 0) it->second.pins--;
  }
}

unsigned long long ctx_peer_wait_ns(ruyb200_ctx* ctx) { return ctx->peer_wait_ns; }

}  // namespace ruyb200
