/* ruy_b200.h -- C ABI of libruy_b200.so, the B200 (sm_100a) implementation of
 * ruy's matrix-multiplication hot path.
 *
 * ruy (google/ruy) has no FFI layer: its boundary is the C++ template
 * ruy::Mul(lhs, rhs, mul_params, context, &dst) (ruy/ruy.h:37-50,98-104), which
 * type-erases its arguments into ruy::TrMulParams (ruy/trmul_params.h:61-90)
 * and hands them to MulFrontEndFromTrMulParams (ruy/frontend.cc:25-35).  This
 * header is that type-erased boundary restated as plain C: every entry point
 * takes POD structs, raw pointers and sizes.  The ruy-compatible C++ headers
 * shipped beside this file (include/ruy/ruy.h ...) and the Python mirror
 * (ruy_b200/api.py) are thin shims that flatten their arguments into
 * ruyb200_mul_desc and call these functions.
 *
 * All functions return RUYB200_OK (0) or a negative ruyb200_status.  Nothing
 * here ever computes on the CPU: if no sm_100-class device is usable the calls
 * fail with RUYB200_ERR_NO_DEVICE.
 */
#ifndef RUY_B200_H_
#define RUY_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RUYB200_ABI_VERSION 2

#if defined(__GNUC__)
#define RUYB200_API __attribute__((visibility("default")))
#else
#define RUYB200_API
#endif

typedef enum ruyb200_status {
  RUYB200_OK = 0,
  RUYB200_ERR_INVALID = -1,      /* descriptor failed validation; nothing was launched */
  RUYB200_ERR_UNSUPPORTED = -2,  /* type combination outside ruy's type space */
  RUYB200_ERR_NO_DEVICE = -3,    /* no usable CUDA device / driver */
  RUYB200_ERR_CUDA = -4,         /* a CUDA runtime call failed; see ruyb200_last_error */
  RUYB200_ERR_TIMEOUT = -5,      /* a bounded device-side wait gave up (kernel returned cleanly) */
  RUYB200_ERR_OOM = -6
} ruyb200_status;

/* Scalar types of ruy's supported (Lhs,Rhs,Accum,Dst) quadruples (ruy/BUILD:1195-1207). */
typedef enum ruyb200_dtype {
  RUYB200_I8 = 0,
  RUYB200_U8 = 1,
  RUYB200_I16 = 2,
  RUYB200_I32 = 3,
  RUYB200_F32 = 4,
  RUYB200_F64 = 5   /* only in ruy's mixed float cases: (f64, f32, f64, f32) and (f32, f64, f64, f64) */
} ruyb200_dtype;

/* ruy::Order (ruy/matrix.h:30). */
enum { RUYB200_COL_MAJOR = 0, RUYB200_ROW_MAJOR = 1 };
/* ruy::CachePolicy (ruy/matrix.h:117-122). */
enum {
  RUYB200_NEVER_CACHE = 0,
  RUYB200_CACHE_IF_LARGE_SPEEDUP = 1,
  RUYB200_CACHE_IF_SIGNIFICANT_SPEEDUP = 2,
  RUYB200_ALWAYS_CACHE = 3
};
/* ruy::ChannelDimension (ruy/mul_params.h:30-38). */
enum { RUYB200_CHANNEL_ROW = 0, RUYB200_CHANNEL_COL = 1 };
/* ruy::Path bit values on x86 (ruy/path.h:55-90). */
enum {
  RUYB200_PATH_NONE = 0,
  RUYB200_PATH_STANDARD_CPP = 0x1,
  RUYB200_PATH_INTERNAL_VARIANT1 = 0x2,
  RUYB200_PATH_INTERNAL_VARIANT2 = 0x4,
  RUYB200_PATH_INTERNAL_VARIANT3 = 0x8,
  RUYB200_PATH_AVX = 0x10,
  RUYB200_PATH_AVX2_FMA = 0x20,
  RUYB200_PATH_AVX512 = 0x40
};
/* Requantization contract.  REFERENCE = ruy::detail::MultiplyByQuantizedMultiplier
 * (ruy/apply_multiplier.cc:48-65), used by ReferenceMul, Path::kStandardCpp and the
 * ARM kernels.  X86 = the two-step rounding of ruy's AVX/AVX2/AVX-512 kernels
 * (ruy/kernel_avx512.cc:340-465).  FROM_PATH picks X86 when the most significant
 * enabled path of the context is one of kAvx/kAvx2Fma/kAvx512 and REFERENCE otherwise. */
enum { RUYB200_ROUNDING_FROM_PATH = 0, RUYB200_ROUNDING_REFERENCE = 1, RUYB200_ROUNDING_X86 = 2 };
/* ruy::PerformanceAdvisory (ruy/performance_advisory.h:21-24). */
enum { RUYB200_ADVISORY_NONE = 0, RUYB200_ADVISORY_REALLOCATED_PERCHANNEL_BUFFER = 1 };

/* Which device kernel served the last ruyb200_mul (diagnostic; ruy has no counterpart). */
enum {
  RUYB200_KERNEL_NONE = 0,
  RUYB200_KERNEL_GENERIC = 1,   /* CUDA-core kernel, any type / layout / stride */
  RUYB200_KERNEL_TC_I8 = 2,     /* tcgen05 kind::i8, TMA-staged, fused epilogue */
  RUYB200_KERNEL_SGEMM = 3,     /* fp32 FFMA tiled kernel (small shapes) */
  RUYB200_KERNEL_GEMV = 4,      /* narrow muls (at most 8 destination rows or columns): one pass over the wide operand */
  RUYB200_KERNEL_BATCH_I8 = 5,  /* persistent many-small-muls kernel (plans) */
  RUYB200_KERNEL_TC_F32 = 6     /* fp32 on tcgen05 kind::tf32: hi/lo split operands, three products, short accumulation chains */
};

/* A non-owning matrix view: ruy::Matrix<T> / ruy::Mat<T> (ruy/matrix.h:132-165,
 * ruy/mat.h:207-242) with the scalar type erased.  `data` may be a host pointer
 * (pageable or pinned) or a device pointer; the library classifies it. */
typedef struct ruyb200_matrix {
  void* data;
  int32_t rows;
  int32_t cols;
  int32_t stride;        /* elements between adjacent columns (col-major) or rows (row-major) */
  int32_t zero_point;    /* must be 0 for F32 (ruy/validate.h:33-38) */
  uint8_t order;         /* RUYB200_COL_MAJOR / RUYB200_ROW_MAJOR */
  uint8_t dtype;         /* ruyb200_dtype */
  uint8_t cache_policy;  /* RUYB200_*_CACHE */
  uint8_t reserved;
} ruyb200_matrix;

/* ruy::MulParams<Accum,Dst> (ruy/mul_params.h:102-223) with types erased.
 * accum_dtype is RUYB200_I32, RUYB200_F32 or RUYB200_F64.  For the float case bias points to
 * floats and clamp_* hold floats in .f; with a double accumulator (an operand or the destination is
 * RUYB200_F64) bias points to doubles and clamp_* hold doubles in .d; multipliers are ignored.
 * Per-channel pointers, when non-NULL, take precedence over the scalar pair
 * (ruy/apply_multiplier.h:66-79).  Per-channel buffers hold one entry per dst
 * row (CHANNEL_ROW) or column (CHANNEL_COL); the library never reads past that
 * count, so the capacity rounding only matters for the advisory flag. */
typedef union ruyb200_scalar {
  int32_t i;
  float f;
  double d;
} ruyb200_scalar;

typedef struct ruyb200_mul_params {
  const void* bias;
  const int32_t* multiplier_fixedpoint_perchannel;
  const int32_t* multiplier_exponent_perchannel;
  int32_t multiplier_fixedpoint;
  int32_t multiplier_exponent;
  ruyb200_scalar clamp_min;
  ruyb200_scalar clamp_max;
  uint8_t channel_dimension;
  uint8_t perchannel_buffers_capacity_rounding_log2;
  uint8_t accum_dtype;
  uint8_t rounding_mode;  /* RUYB200_ROUNDING_* */
} ruyb200_mul_params;

typedef struct ruyb200_mul_desc {
  ruyb200_matrix lhs;
  ruyb200_matrix rhs;
  ruyb200_matrix dst;
  ruyb200_mul_params params;
} ruyb200_mul_desc;

typedef struct ruyb200_ctx ruyb200_ctx;
typedef struct ruyb200_plan ruyb200_plan;

/* ---- library ---------------------------------------------------------- */

/* ABI version of the loaded library (== RUYB200_ABI_VERSION it was built with). */
RUYB200_API int ruyb200_abi_version(void);
/* Number of usable CUDA devices, or a negative status. */
RUYB200_API int ruyb200_device_count(void);
/* Message of the last failure on the calling thread ("" if none). */
RUYB200_API const char* ruyb200_last_error(void);

/* ---- context: ruy::Context (ruy/context.h:38-112) ---------------------- */

/* Replaces ruy::Context::Context().  device < 0 means the current CUDA device.
 * The context owns one CUDA stream, a device scratch arena and the device-side
 * prepacked cache.  Like ruy's, a context is not thread-safe: one per calling
 * thread (ruy/ruy.h:84-87). */
RUYB200_API int ruyb200_ctx_create(int device, ruyb200_ctx** out);
/* Same, but all work is enqueued on `cuda_stream` (a cudaStream_t) owned by the caller. */
RUYB200_API int ruyb200_ctx_create_on_stream(int device, void* cuda_stream, ruyb200_ctx** out);
RUYB200_API int ruyb200_ctx_destroy(ruyb200_ctx* ctx);

/* ruy::Context::{max_num_threads,set_max_num_threads}: kept for API parity; the
 * value is stored and returned but does not change how the device is used. */
RUYB200_API int ruyb200_ctx_set_max_num_threads(ruyb200_ctx* ctx, int value);
RUYB200_API int ruyb200_ctx_get_max_num_threads(const ruyb200_ctx* ctx);
/* ruy::Context::{set,get}_runtime_enabled_paths (ruy/context.h:96-99). A mask of 0
 * restores the default (all of kDefaultPaths, or RUY_PATHS from the environment, ruy/ctx.cc:150-173). */
RUYB200_API int ruyb200_ctx_set_runtime_enabled_paths(ruyb200_ctx* ctx, uint32_t path_mask);
RUYB200_API uint32_t ruyb200_ctx_get_runtime_enabled_paths(ruyb200_ctx* ctx);
/* ruy::Context::last_used_path: most significant bit of compiled & enabled (ruy/ctx.cc:175-178). */
RUYB200_API uint32_t ruyb200_ctx_last_used_path(const ruyb200_ctx* ctx);
/* ruy::Context::performance_advisory (ruy/context.h:79). */
RUYB200_API int ruyb200_ctx_performance_advisory(const ruyb200_ctx* ctx, int advisory);
/* ruy::Context::ClearPrepackedCache (ruy/context.h:85). */
RUYB200_API int ruyb200_ctx_clear_prepacked_cache(ruyb200_ctx* ctx);
/* PrepackedCache budget (ruy/prepacked_cache.h:45, default 256 MiB there; here the
 * default is 8 GiB of HBM).  Entries are evicted least-recently-used first. */
RUYB200_API int ruyb200_ctx_set_prepacked_cache_budget(ruyb200_ctx* ctx, size_t bytes);
/* Introspection of the prepacked cache (ruy::PrepackedCache::{TotalSize,MatrixCount} as
 * used by ruy/prepacked_cache_test.cc). */
RUYB200_API size_t ruyb200_ctx_prepacked_cache_bytes(const ruyb200_ctx* ctx);
RUYB200_API int ruyb200_ctx_prepacked_cache_entries(const ruyb200_ctx* ctx);
/* Counters: [0] kernel launches, [1] cache hits, [2] cache misses, [3] H2D bytes staged,
 * [4] D2H bytes staged, [5] id of the kernel that served the last mul (RUYB200_KERNEL_*). */
RUYB200_API int ruyb200_ctx_counters(const ruyb200_ctx* ctx, uint64_t out[6]);
/* The cudaStream_t the context enqueues on. */
RUYB200_API void* ruyb200_ctx_stream(const ruyb200_ctx* ctx);
/* Blocks until everything enqueued by this context has finished; reports device-side
 * status words (RUYB200_ERR_TIMEOUT) raised by bounded waits. */
RUYB200_API int ruyb200_ctx_sync(ruyb200_ctx* ctx);

/* ---- the operation ----------------------------------------------------- */

/* Replaces ruy::Mul / MulFrontEnd (ruy/ruy.h:37-50, ruy/frontend.h:82-95).
 * Synchronous, like ruy: dst is valid when the call returns.  Host operands are
 * staged to the device and the result copied back; device operands are used in place. */
RUYB200_API int ruyb200_mul(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc);
/* Stream-ordered variant for device-resident operands: validates, enqueues on the
 * context's stream and returns without synchronizing.  All pointers in `desc`
 * (matrices and per-channel buffers) must be device pointers.  Additive: ruy has no
 * asynchronous entry point. */
RUYB200_API int ruyb200_mul_async(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc);
/* Host-side validation only (ruy/validate.h:40-83 plus pointer / stride / shape checks). */
RUYB200_API int ruyb200_validate(const ruyb200_mul_desc* desc);

/* An 8-bit mul for callers that must not allocate device memory at call time (a runtime whose own
 * pool owns the whole device, a service under a fixed memory budget, a latency-critical loop that
 * cannot take the synchronisation an allocation implies).  It has no counterpart in the reference:
 * ruy::Mul always goes through a ruy::Context and its allocator.  No context is needed; the only
 * memory used besides the operands and the destination is a 128.25 KiB static device array inside
 * the library (zero-point sums and a status word), so: at most 16384 destination rows and 16384
 * destination columns (larger shapes are refused with RUYB200_ERR_INVALID); int8/uint8 operands that
 * are depth-contiguous (row-major LHS, column-major RHS) with 16-byte aligned base addresses and
 * strides; all pointers in `desc` device pointers.  No cudaMalloc, cudaFree or other allocating
 * call is made.  The work is enqueued on `cuda_stream` (a cudaStream_t, NULL for the default
 * stream) of the current device and the call returns after that stream has finished: it always
 * synchronises that stream (it reads back the status word of the kernel's bounded waits), so it
 * serves callers that may not allocate, not callers that may not block.  The first call on each
 * device does one-time set-up under a lock: it looks up the array's device address
 * (cudaGetSymbolAddress) and, like the first use of any kernel variant of this library, raises
 * that kernel's dynamic shared-memory limit (cudaFuncSetAttribute) and asks how many two-CTA
 * clusters fit the device (cudaOccupancyMaxActiveClusters); make that first call before starting
 * any stream capture.  Every call shares the one array: two calls whose GPU work overlaps
 * (different streams or threads) race on it and must be serialised by the caller.
 * rounding_mode RUYB200_ROUNDING_FROM_PATH means the reference rounding here. */
RUYB200_API int ruyb200_mul_noalloc(const ruyb200_mul_desc* desc, void* cuda_stream);

/* ---- plans: many independent muls in one launch ------------------------ */

/* Additive surface (ruy::Mul is one-matmul-per-call).  A plan plays the role that
 * TrMul's BlockMap + atomic block queue (ruy/trmul.cc:78-119, ruy/block_map.cc:339-471)
 * play inside one mul, across many: the descriptors are validated once, LHS operands
 * with a caching policy are prepacked into the context's device cache, the work list is
 * sorted and uploaded, and every ruyb200_plan_run replays it with a single persistent
 * launch.  All operand pointers must be device pointers that stay valid for the life of
 * the plan. */
RUYB200_API int ruyb200_plan_create(ruyb200_ctx* ctx, const ruyb200_mul_desc* descs, int n, ruyb200_plan** out);
/* Enqueue the whole plan on the context's stream (no synchronization). */
RUYB200_API int ruyb200_plan_run(ruyb200_plan* plan);
RUYB200_API int ruyb200_plan_destroy(ruyb200_plan* plan);
/* Algorithmic bytes (operands read once + dst written once + per-channel params) and
 * 2*rows*cols*depth operations summed over the plan's muls. */
RUYB200_API int ruyb200_plan_stats(const ruyb200_plan* plan, uint64_t* bytes, uint64_t* ops);

/* ---- multi-GPU: destination mirrored into peers' memory ------------------------- */

/* Additive (ruy has no multi-device notion).  For the column-sharded large mul each rank (one process per GPU)
 * computes its column block and must end up with the whole destination.  Instead of a collective after the
 * kernel, ruyb200_mul_async_mirrored makes the kernel's epilogue store every destination element both at
 * desc->dst.data and at the corresponding address of each mirror (mirror_dst[i] is the address, in a peer GPU's
 * buffer mapped into this process, that corresponds to desc->dst.data), so the gather overlaps the math.
 * 8-bit operands served by the tensor-core kernel only; n_mirrors <= 7.  The peer buffers come from
 * ruyb200_peer_alloc (plain cudaMalloc, zeroed), are exported with ruyb200_peer_export (a 64-byte
 * cudaIpcMemHandle_t to be sent to the other processes by any means) and mapped with ruyb200_peer_open.
 * ruyb200_peer_signal raises, after all earlier work of the context's stream, the flag words remote_flags[i]
 * (addresses in peers' memory; the array itself lives in device memory) to `value`; ruyb200_peer_wait makes the
 * stream wait until local_flags[0..n) have all reached `value`, giving up after the context's wait limit (2 s unless
 * changed) with RUYB200_ERR_TIMEOUT at the next ruyb200_ctx_sync.  ruyb200_peer_exchange does both in one launch (signal, then wait).  Only stores
 * ever cross NVLink; no load reads a peer's memory. */
RUYB200_API int ruyb200_mul_async_mirrored(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc, void* const* mirror_dst,
                                           int n_mirrors);
/* The same mul with the step's flag exchange folded into the launch: the CTA that finishes last does what
 * ruyb200_peer_exchange does (raise remote_flags[i] to `value`, then wait, within the context's wait limit, until
 * local_flags[0..n_flags) have reached it), which saves a launch per step.
 * Reuse rule for mirrored destinations: the exchange tells a rank that every peer's tiles of this step have landed
 * in its buffer; it does not tell a rank that its peers are done READING their copies.  A rank that mirrors step s+1
 * into the same buffers may therefore overwrite data a slower peer is still consuming.  Alternate between two sets
 * of buffers (step parity): a rank can only reach step s+2 after every peer has signalled step s+1, and a peer
 * signals step s+1 after, in its stream, everything that read step s. */
RUYB200_API int ruyb200_mul_async_mirrored_exchange(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc, void* const* mirror_dst,
                                                    int n_mirrors, uint32_t* const* remote_flags_device_array,
                                                    const uint32_t* local_flags, int n_flags, uint32_t value);
/* The same step with the gather done by NVSwitch: `multicast_dst` is the address that corresponds to desc->dst.data in
 * an NVLink multicast mapping bound to every rank's copy of the destination (this rank's included; created by the
 * caller, e.g. with cuMulticastCreate / cuMulticastBindMem or a library that wraps them).  Every 16-byte piece of the
 * destination is stored there once (multimem.st) and the switch writes it into all copies, so a rank sends its shard
 * over NVLink once instead of once per peer.  8-bit destinations only; base addresses and stride multiples of 16 bytes,
 * contiguous dimension a multiple of 16 elements (RUYB200_ERR_UNSUPPORTED otherwise).  The flag arguments and the
 * two-buffer reuse rule are those of ruyb200_mul_async_mirrored_exchange.  Unbind and free the multicast mapping only
 * after every rank has passed a barrier that follows its last use. */
RUYB200_API int ruyb200_mul_async_multicast_exchange(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc, void* multicast_dst,
                                                     uint32_t* const* remote_flags_device_array, const uint32_t* local_flags,
                                                     int n_flags, uint32_t value);
RUYB200_API int ruyb200_peer_alloc(size_t bytes, void** out);
RUYB200_API int ruyb200_peer_free(void* ptr);
RUYB200_API int ruyb200_peer_export(void* ptr, unsigned char handle[64]);
RUYB200_API int ruyb200_peer_open(const unsigned char handle[64], void** out);
RUYB200_API int ruyb200_peer_close(void* ptr);
RUYB200_API int ruyb200_peer_signal(ruyb200_ctx* ctx, uint32_t* const* remote_flags_device_array, int n, uint32_t value);
RUYB200_API int ruyb200_peer_wait(ruyb200_ctx* ctx, const uint32_t* local_flags, int n, uint32_t value);
RUYB200_API int ruyb200_peer_exchange(ruyb200_ctx* ctx, uint32_t* const* remote_flags_device_array, const uint32_t* local_flags,
                                      int n, uint32_t value);
/* How long ruyb200_peer_wait / ruyb200_peer_exchange of this context wait before they give up (default 2000 ms).
 * A wait that runs out returns by itself; the next ruyb200_ctx_sync reports RUYB200_ERR_TIMEOUT and the context
 * stays usable. */
RUYB200_API int ruyb200_ctx_set_peer_wait_ms(ruyb200_ctx* ctx, uint32_t ms);

/* ---- prepacked-cache persistence --------------------------------------------------------------- */

/* Additive.  ruy's PrepackedCache lives and dies with its process: an entry is identified by (source pointer,
 * packed layout, zero point) (ruy/prepacked_cache.h:68-80) and holds the packed data plus the sums
 * (ruy/prepacked_cache.cc:29-45,79-127); there is no serialised form.  These calls take an entry of the device
 * cache out as a self-describing, versioned blob and put one back, so that weights are packed once per model
 * rather than once per process.  Blob layout (little endian): a 64-byte header -- bytes 0-7 "RUYB2PCK", 8-11 ABI
 * version, 12-15 tile-format id, 16 dtype, 17 side, 18 has_sums, 19 zero, 20-23 width, 24-27 depth, 28-31 packed
 * depth, 32-35 zero point, 36-39 zero, 40-47 data bytes, 48-55 sums bytes, 56-63 FNV-1a (64 bit) of header bytes
 * 0-55 followed by the payload -- then the packed data, then the int32 sums.
 * `src` + `side` (0 = LHS, 1 = RHS) name the entry exactly as a later ruyb200_mul will look it up; import never
 * reads src->data, it only uses the pointer as the key.  After a successful import the next mul with that
 * operand is a cache hit and launches no packing kernel. */
#define RUYB200_CACHE_FORMAT_ROWS16 1u   /* [width][packed_depth] depth-contiguous rows, int32 sums[width]; packed_depth is
                                          * the depth rounded up to 16 bytes, or, for 8-bit rows of 256 bytes or more, to
                                          * 128 bytes (what this library writes; both are accepted) */
typedef struct ruyb200_cache_blob {
  uint32_t abi_version;
  uint32_t format;
  uint8_t dtype, side, has_sums, reserved;
  int32_t width, depth, packed_depth, zero_point;
  uint64_t data_bytes, sums_bytes;
} ruyb200_cache_blob;
/* Validates a blob on the host (magic, version, tile format, sizes, checksum) and describes it; needs no device.
 * RUYB200_ERR_INVALID for anything this library version cannot use. */
RUYB200_API int ruyb200_cache_blob_info(const void* blob, size_t n, ruyb200_cache_blob* out);
/* Copies the cached form of `src` out of the context's cache.  With blob == NULL only *n (bytes needed) is
 * returned; otherwise *n is the capacity on entry and the size written on return.  RUYB200_ERR_INVALID when
 * the matrix is not cached or the buffer is too small. */
RUYB200_API int ruyb200_cache_export(ruyb200_ctx* ctx, const ruyb200_matrix* src, int side, void* blob, size_t* n);
/* Installs a blob as the cache entry of `src`.  The blob must describe a matrix of the same side, type, shape
 * and zero point and come from the same ABI version and tile format; anything else is RUYB200_ERR_INVALID and
 * leaves the cache unchanged.  The cache budget applies (older unpinned entries are evicted to make room). */
RUYB200_API int ruyb200_cache_import(ruyb200_ctx* ctx, const ruyb200_matrix* src, int side, const void* blob, size_t n);

/* ---- packing: PackImpl / RunPack (ruy/pack.h:105-151) -------------------- */

/* Packs a device- or host-resident integer matrix into the device layout the tensor-core
 * kernel consumes (depth-contiguous, depth padded to 16 bytes) and computes the per-row /
 * per-column sums used for the zero-point terms.  side: 0 = LHS, 1 = RHS.  Exposed for
 * tests and benchmarks; ruyb200_mul calls it internally.  `packed` (device, capacity
 * packed_capacity bytes) and `sums` (device int32[width]) are caller-provided. */
RUYB200_API int ruyb200_pack(ruyb200_ctx* ctx, const ruyb200_matrix* src, int side, void* packed,
                 size_t packed_capacity, int32_t* sums, int32_t* packed_depth);

#ifdef __cplusplus
}
#endif

#endif /* RUY_B200_H_ */
