// Internal glue between the context (api.cu) and plans (plan.cu).
#pragma once

#include <cuda_runtime.h>

#include <tuple>
#include <vector>

#include "../../include/ruy_b200.h"
#include "batch_i8.h"

namespace ruyb200 {

// Makes `dev` the current device for the scope of a call and restores the caller's device afterwards.
struct ScopedDevice {
  int prev = -1;
  explicit ScopedDevice(int dev) {
    cudaGetDevice(&prev);
    if (prev != dev) cudaSetDevice(dev);
  }
  ~ScopedDevice() {
    int cur = -1;
    cudaGetDevice(&cur);
    if (prev >= 0 && cur != prev) cudaSetDevice(prev);
  }
};

// Key of the prepacked cache: the source pointer, the layout of the TrMul view (width, depth, both strides) and
// the zero point (ruy/prepacked_cache.h:68-80), plus the element type and the side.
typedef std::tuple<const void*, int, int, int64_t, int64_t, int, int, int> CacheKey;

cudaStream_t ctx_stream(ruyb200_ctx* ctx);
int ctx_device(ruyb200_ctx* ctx);
int ctx_sm_count(ruyb200_ctx* ctx);
int* ctx_status_word(ruyb200_ctx* ctx);
void ctx_count_launch(ruyb200_ctx* ctx, int kernel);
int ctx_fail(int status, const char* msg);
int ctx_validate(const ruyb200_mul_desc* d);
bool ptr_on_device(const void* p);
int ctx_rounding_is_x86(ruyb200_ctx* ctx, int rounding_mode);
int ctx_run_mul_async(ruyb200_ctx* ctx, const ruyb200_mul_desc* d);
int ctx_plan_item(ruyb200_ctx* ctx, const ruyb200_mul_desc* desc, BatchItem* out, bool* fits,
                  std::vector<CacheKey>* pinned);
void ctx_unpin(ruyb200_ctx* ctx, const std::vector<CacheKey>& pinned);
unsigned long long ctx_peer_wait_ns(ruyb200_ctx* ctx);

}  // namespace ruyb200
