// Plans: many independent muls submitted once and replayed (see ruyb200_plan_create).
//
// The muls whose three dimensions fit one tensor-core tile become work items of the persistent batched
// kernel (batch_i8.cu): one launch per replay, whatever their number.  The others are replayed through
// the ordinary single-mul dispatch.
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "batch_i8.h"
#include "common.cuh"
#include "plan.h"

using namespace ruyb200;

struct ruyb200_plan {
  ruyb200_ctx* ctx = nullptr;
  std::vector<ruyb200_mul_desc> single;     // muls replayed one launch at a time
  std::vector<CacheKey> pinned;             // prepacked-cache entries this plan reads
  BatchItem* d_items = nullptr;   // in schedule order
  CUtensorMap* d_maps = nullptr;  // two per item (m side, n side), same order
  int num_items = 0;
  int grid = 0;
  uint64_t bytes = 0;
  uint64_t ops = 0;
};

namespace {

size_t esize(int dtype) { return dtype == RUYB200_I8 || dtype == RUYB200_U8 ? 1 : (dtype == RUYB200_I16 ? 2 : 4); }

void free_plan(ruyb200_plan* plan) {
  if (!plan) return;
  ScopedDevice on_device(ctx_device(plan->ctx));
  if (plan->d_items) cudaFree(plan->d_items);
  if (plan->d_maps) cudaFree(plan->d_maps);
  ctx_unpin(plan->ctx, plan->pinned);
  delete plan;
}

}  // namespace

extern "C" {

int ruyb200_plan_create(ruyb200_ctx* ctx, const ruyb200_mul_desc* descs, int n, ruyb200_plan** out) {
  if (!ctx || !out || n < 0 || (n > 0 && !descs)) return ctx_fail(RUYB200_ERR_INVALID, "bad argument");
  *out = nullptr;
  ScopedDevice on_device(ctx_device(ctx));
  ruyb200_plan* plan = new ruyb200_plan;
  plan->ctx = ctx;
  std::vector<BatchItem> items;
  std::vector<long long> cost;
  for (int i = 0; i < n; i++) {
    const ruyb200_mul_desc& d = descs[i];
    int rc = ctx_validate(&d);
    if (rc) {
      free_plan(plan);
      return rc;
    }
    const void* ptrs[6] = {d.lhs.data, d.rhs.data, d.dst.data, d.params.bias, d.params.multiplier_fixedpoint_perchannel,
                           d.params.multiplier_exponent_perchannel};
    for (const void* p : ptrs) {
      if (p && !ptr_on_device(p)) {
        free_plan(plan);
        return ctx_fail(RUYB200_ERR_INVALID, "plans need device pointers");
      }
    }
    const uint64_t r = d.lhs.rows, k = d.lhs.cols, c = d.rhs.cols;
    plan->ops += 2 * r * k * c;
    plan->bytes += r * k * esize(d.lhs.dtype) + k * c * esize(d.rhs.dtype) + r * c * esize(d.dst.dtype);
    const uint64_t nch = d.params.channel_dimension == RUYB200_CHANNEL_ROW ? r : c;
    if (d.params.bias) plan->bytes += 4 * nch;
    if (d.params.multiplier_fixedpoint_perchannel) plan->bytes += 8 * nch;
    BatchItem item;
    bool fits = false;
    rc = ctx_plan_item(ctx, &d, &item, &fits, &plan->pinned);
    if (rc) {
      free_plan(plan);
      return rc;
    }
    if (fits) {
      items.push_back(item);
      // estimated cycles of an item on its SM: a fixed hand-off cost, the epilogue's columns (its rows sit on
      // parallel lanes, so they count little) and the bytes to fetch; coefficients fitted on the 16..128 mix
      const int quarters = (item.size_m + 31) / 32;
      const long long est = 1000 + 40ll * item.size_n + 4ll * item.size_n * quarters +
                            ((long long)(item.size_m + item.size_n) * item.depth) / 64;
      cost.push_back(est);
    } else {
      plan->single.push_back(d);
    }
  }
  plan->num_items = (int)items.size();
  if (plan->num_items > 0) {
    std::vector<int32_t> order(items.size());
    for (size_t i = 0; i < order.size(); i++) order[i] = (int32_t)i;
    std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return cost[a] > cost[b]; });
    // CTA b takes positions b, b + grid, ...: reverse every other round so heavy and light items pair up
    const int grid = std::min<int>(plan->num_items, ctx_sm_count(ctx));
    plan->grid = grid;
    for (size_t start = grid; start + 1 < order.size(); start += 2 * (size_t)grid) {
      const size_t end = std::min(order.size(), start + grid);
      std::reverse(order.begin() + start, order.begin() + end);
    }
    // Items that use at most 32 (64) tensor-memory lanes are rotated over the four (two) lane ranges, so
    // that the epilogue work spreads evenly over the SM's four schedulers.
    std::vector<BatchItem> scheduled(items.size());
    std::vector<int> rot32(grid, 0), rot64(grid, 0);
    // Accumulator units are handed out per CTA in the order the CTA will meet its items; the parity of a unit's use
    // count tells the kernel which phase of that unit's barriers the item waits for.  A parity wait is only sound
    // when the successive users of a unit are waited for by the same warp, in order; the kernel's two MMA warps
    // take the even and the odd items of a CTA independently of each other, so each of them gets its own half
    // of the units (a ring of four): a unit never passes from one warp's items to the other's.
    constexpr int kHalf = kBatchAccUnits / 2;
    struct AccRing { int next = 0; int uses[kHalf] = {}; };
    std::vector<AccRing> rings(2 * (size_t)grid);
    for (size_t pos = 0; pos < order.size(); pos++) {
      BatchItem it = items[order[pos]];
      const int cta = (int)(pos % grid);
      if (it.size_m <= 32) {
        it.m_off = 32 * (rot32[cta]++ & 3);
      } else if (it.size_m <= 64) {
        it.m_off = 64 * (rot64[cta]++ & 1);
      } else {
        it.m_off = 0;
      }
      const int stream_of_item = (int)((pos / grid) & 1);   // which MMA warp will issue it
      AccRing& ring = rings[2 * (size_t)cta + stream_of_item];
      const int units = batch_acc_units(it.size_n);
      if (units == 2 && ring.next == kHalf - 1) ring.next = 0;   // two units never wrap around
      const int u = ring.next;
      const int base = stream_of_item * kHalf;
      uint32_t acc = (uint32_t)(base + u) | ((uint32_t)(ring.uses[u]++ & 1) << 4);
      if (units == 2) acc |= (1u << 3) | ((uint32_t)(ring.uses[u + 1]++ & 1) << 5);
      ring.next = (u + units) % kHalf;
      it.acc = acc;
      scheduled[pos] = it;
    }
    // Operands with 16-byte aligned rows are fetched by one tensor-map copy each: encode the maps now.
    std::vector<CUtensorMap> maps(2 * scheduled.size());
    memset(maps.data(), 0, maps.size() * sizeof(CUtensorMap));
    for (size_t pos = 0; pos < scheduled.size(); pos++) {
      BatchItem& it = scheduled[pos];
      if ((it.flags & kItemMTma) &&
          !make_i8_tile_map(&maps[2 * pos], it.m_ptr, it.depth, it.size_m, it.stride_m, batch_box_rows_m(it.size_m))) {
        it.flags &= ~kItemMTma;
      }
      if ((it.flags & kItemNTma) &&
          !make_i8_tile_map(&maps[2 * pos + 1], it.n_ptr, it.depth, it.size_n, it.stride_n, batch_box_rows_n(it.size_n))) {
        it.flags &= ~kItemNTma;
      }
    }
    if (cudaMalloc(&plan->d_items, scheduled.size() * sizeof(BatchItem)) != cudaSuccess ||
        cudaMalloc(&plan->d_maps, maps.size() * sizeof(CUtensorMap)) != cudaSuccess) {
      cudaGetLastError();
      free_plan(plan);
      return ctx_fail(RUYB200_ERR_OOM, "plan allocation failed");
    }
    cudaMemcpy(plan->d_items, scheduled.data(), scheduled.size() * sizeof(BatchItem), cudaMemcpyHostToDevice);
    cudaMemcpy(plan->d_maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice);
  }
  // packing launched for cache misses has finished before the plan is used
  int rc = ruyb200_ctx_sync(ctx);
  if (rc) {
    free_plan(plan);
    return rc;
  }
  *out = plan;
  return RUYB200_OK;
}

int ruyb200_plan_run(ruyb200_plan* plan) {
  if (!plan) return ctx_fail(RUYB200_ERR_INVALID, "null plan");
  ScopedDevice on_device(ctx_device(plan->ctx));
  if (plan->num_items > 0) {
    cudaError_t ce = launch_batch_i8(plan->d_items, plan->d_maps, plan->num_items, plan->grid, ctx_status_word(plan->ctx),
                                     ctx_stream(plan->ctx));
    ctx_count_launch(plan->ctx, RUYB200_KERNEL_BATCH_I8);
    if (ce != cudaSuccess) return ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(ce));
  }
  for (const ruyb200_mul_desc& d : plan->single) {
    int rc = ctx_run_mul_async(plan->ctx, &d);
    if (rc) return rc;
  }
  return RUYB200_OK;
}

int ruyb200_plan_destroy(ruyb200_plan* plan) {
  free_plan(plan);
  return RUYB200_OK;
}

int ruyb200_plan_stats(const ruyb200_plan* plan, uint64_t* bytes, uint64_t* ops) {
  if (!plan) return ctx_fail(RUYB200_ERR_INVALID, "null plan");
  if (bytes) *bytes = plan->bytes;
  if (ops) *ops = plan->ops;
  return RUYB200_OK;
}

}  // extern "C"
