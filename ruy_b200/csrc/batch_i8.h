// Work-item descriptor of the persistent many-small-muls kernel (batch_i8.cu).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace ruyb200 {

enum : uint32_t {
  kItemChannelOnN = 1u << 0,   // per-channel buffers are indexed by n (else by m)
  kItemMSigned = 1u << 1,      // m-side operand is int8 (else uint8)
  kItemNSigned = 1u << 2,
  kItemX86 = 1u << 3,          // x86 two-step rounding
  kItemDstShift = 4,           // 3 bits: ruyb200_dtype of the destination
  kItemMTma = 1u << 8,         // the m-side operand is fetched by one tensor-map copy (16-byte aligned base and row stride)
  kItemNTma = 1u << 9,         // the same for the n-side operand
  kItemVecBulk = 1u << 10      // every per-channel vector is 16-byte aligned with a length that is a multiple of 4
};

// One small mul, fully resolved to device pointers.  "m" is the destination's contiguous dimension
// (it sits on the tensor-memory lanes), "n" the other one; element (m, n) is stored at
// dst[n * dst_stride + m].  Both operands are depth-contiguous with rows stride_* bytes apart.
struct alignas(16) BatchItem {
  const uint8_t* m_ptr;
  const uint8_t* n_ptr;
  uint8_t* dst;
  const int32_t* bias;
  const int32_t* mfp_pc;
  const int32_t* mexp_pc;
  const int32_t* sums_m;   // per-m sums over depth of the m-side operand when the prepacked cache holds them, else null
  int32_t size_m;
  int32_t size_n;
  int32_t depth;
  int32_t stride_m;
  int32_t stride_n;
  int32_t dst_stride;
  int32_t zp_m;
  int32_t zp_n;
  int32_t dst_zp;
  int32_t clamp_min;
  int32_t clamp_max;
  int32_t mfp;
  int32_t mexp;
  uint32_t flags;
  int32_t m_off;       // first tile row (TMEM lane) used by this item: 0, 32, 64 or 96; spreads small items over the lane quarters
  // Tensor-memory columns of this item's accumulator, assigned by the plan in schedule order: bits 0-2 first
  // 64-column unit, bit 3 set if it takes two units (more than 64 destination columns along n), bits 4 / 5 the
  // parity of the first / second unit's use count (which phase of the unit's barriers this item sees).
  uint32_t acc;
  int32_t reserved[2];
};
static_assert(sizeof(BatchItem) == 128, "BatchItem is copied as eight 16-byte pieces");

// True when a mul can be a work item: 8-bit depth-contiguous operands, all three dimensions <= 128,
// 8-byte aligned rows.
bool batch_i8_fits(const SideView& m_side, const SideView& n_side, int depth);

// `items` is a device array already in schedule order: CTA b of `grid` handles items[b], items[b + grid], ...
// `maps` holds two tensor maps per item in the same order (m side, n side); an entry is only read when the
// item's kItemMTma / kItemNTma flag is set.
cudaError_t launch_batch_i8(const BatchItem* items, const CUtensorMap* maps, int num_items, int grid, int* status,
                            cudaStream_t stream);

// Tensor map over a width x depth byte matrix (depth contiguous, rows stride_w bytes apart) whose copies land
// as rows of 128 bytes with the 128-byte swizzle, zero-filled past depth and width: `box_rows` rows per copy.
bool make_i8_tile_map(CUtensorMap* map, const void* base, int depth, int width, int64_t stride_w, int box_rows);

// Accumulator units (64 tensor-memory columns each) per SM and what an item takes.
constexpr int kBatchAccUnits = 8;
inline int batch_acc_units(int size_n) { return size_n > 64 ? 2 : 1; }

// Rows copied for an item's sides (also the byte count the copy reports: 128 bytes per row).
inline int batch_box_rows_m(int size_m) { return (size_m + 7) & ~7; }
inline int batch_box_rows_n(int size_n) { return (size_n + 15) & ~15; }

}  // namespace ruyb200
