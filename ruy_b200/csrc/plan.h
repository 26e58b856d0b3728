// Internal glue between the context (api.cu) and plans (plan.cu).
#pragma once

#include <cuda_runtime.h>

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
                  std::vector<const void*>* pinned_sources);
void ctx_unpin(ruyb200_ctx* ctx, const std::vector<const void*>& sources);

}  // namespace ruyb200
