// Multi-GPU support for the column-sharded large mul: instead of gathering destination shards with a collective
// after the kernel, a rank's epilogue stores every destination tile into its own buffer and into the same place of
// every peer's buffer (plain stores through NVLink to IPC-mapped memory), so the gather overlaps the math tile by
// tile.  This file holds the plumbing around that: allocations that can be shared between processes, handle
// export/import, and the flag exchange that tells a rank that all peers' tiles have landed.
//
// No load ever reads peer memory here, and nothing uses cluster multicast.
#include <cuda_runtime.h>

#include "common.cuh"
#include "plan.h"

using namespace ruyb200;

namespace {


// One thread per peer: everything this GPU wrote before (the previous kernels of the stream) is made visible
// system-wide, then the peer's flag word is raised to `value`.
__global__ void signal_kernel(uint32_t* const* remote_flags, int n, uint32_t value) {
  const int i = threadIdx.x;
  if (i < n && remote_flags[i]) {
    __threadfence_system();   // one system-scope fence, then a relaxed store: a release store would fence again
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(remote_flags[i]), "r"(value) : "memory");
  }
}

// One thread per peer spins, with a time limit, until that peer's flag in local memory reaches `value`.
__global__ void wait_kernel(const uint32_t* local_flags, int n, uint32_t value, int* status, unsigned long long limit_ns) {
  const int i = threadIdx.x;
  if (i >= n) return;
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local_flags + i) : "memory");
    if ((int32_t)(v - value) >= 0) {
      __threadfence_system();   // acquire side, once: relaxed polls are cheap, acquire loads are not
      return;
    }
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > limit_ns) {
      atomicCAS(status, 0, 9);   // a peer never signalled: report, do not hang
      return;
    }
    __nanosleep(200);
  }
}

// Both in one launch: thread i raises this rank's flag in peer i's memory, then waits (bounded) for peer i's flag
// in local memory.  The peers run on other GPUs, so nothing here waits for another launch of the same GPU.
__global__ void exchange_kernel(uint32_t* const* remote_flags, const uint32_t* local_flags, int n, uint32_t value, int* status,
                                unsigned long long limit_ns) {
  const int i = threadIdx.x;
  if (i >= n) return;
  if (remote_flags[i]) {
    __threadfence_system();
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(remote_flags[i]), "r"(value) : "memory");
  }
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (unsigned it = 0;; it++) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(local_flags + i) : "memory");
    if ((int32_t)(v - value) >= 0) {
      __threadfence_system();
      return;
    }
    if ((it & 15) == 15) {
      unsigned long long t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t - t0 > limit_ns) {
        atomicCAS(status, 0, 9);   // a peer never signalled: report, do not hang
        return;
      }
    }
  }
}

}  // namespace

extern "C" {

int ruyb200_peer_alloc(size_t bytes, void** out) {
  if (!out || bytes == 0) return ctx_fail(RUYB200_ERR_INVALID, "bad argument");
  void* p = nullptr;
  if (cudaMalloc(&p, bytes) != cudaSuccess) {
    cudaGetLastError();
    return ctx_fail(RUYB200_ERR_OOM, "cudaMalloc failed");
  }
  if (cudaMemset(p, 0, bytes) != cudaSuccess) {
    cudaFree(p);
    return ctx_fail(RUYB200_ERR_CUDA, "cudaMemset failed");
  }
  *out = p;
  return RUYB200_OK;
}

int ruyb200_peer_free(void* ptr) {
  if (ptr && cudaFree(ptr) != cudaSuccess) return ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
  return RUYB200_OK;
}

int ruyb200_peer_export(void* ptr, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  if (!ptr || !handle || cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) {
    cudaGetLastError();
    return ctx_fail(RUYB200_ERR_CUDA, "cudaIpcGetMemHandle failed");
  }
  memcpy(handle, &h, 64);
  return RUYB200_OK;
}

int ruyb200_peer_open(const unsigned char handle[64], void** out) {
  if (!handle || !out) return ctx_fail(RUYB200_ERR_INVALID, "bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(e));
  }
  *out = p;
  return RUYB200_OK;
}

int ruyb200_peer_close(void* ptr) {
  if (ptr && cudaIpcCloseMemHandle(ptr) != cudaSuccess) return ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
  return RUYB200_OK;
}

int ruyb200_peer_signal(ruyb200_ctx* ctx, uint32_t* const* remote_flags_device_array, int n, uint32_t value) {
  if (!ctx || !remote_flags_device_array || n < 1 || n > 32) return ctx_fail(RUYB200_ERR_INVALID, "bad argument");
  ScopedDevice on_device(ctx_device(ctx));
  signal_kernel<<<1, 32, 0, ctx_stream(ctx)>>>(remote_flags_device_array, n, value);
  ctx_count_launch(ctx, RUYB200_KERNEL_NONE);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? RUYB200_OK : ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(e));
}

int ruyb200_peer_wait(ruyb200_ctx* ctx, const uint32_t* local_flags, int n, uint32_t value) {
  if (!ctx || !local_flags || n < 1 || n > 32) return ctx_fail(RUYB200_ERR_INVALID, "bad argument");
  ScopedDevice on_device(ctx_device(ctx));
  wait_kernel<<<1, 32, 0, ctx_stream(ctx)>>>(local_flags, n, value, ctx_status_word(ctx), ctx_peer_wait_ns(ctx));
  ctx_count_launch(ctx, RUYB200_KERNEL_NONE);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? RUYB200_OK : ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(e));
}

int ruyb200_peer_exchange(ruyb200_ctx* ctx, uint32_t* const* remote_flags_device_array, const uint32_t* local_flags, int n,
                          uint32_t value) {
  if (!ctx || !remote_flags_device_array || !local_flags || n < 1 || n > 32) return ctx_fail(RUYB200_ERR_INVALID, "bad argument");
  ScopedDevice on_device(ctx_device(ctx));
  exchange_kernel<<<1, 32, 0, ctx_stream(ctx)>>>(remote_flags_device_array, local_flags, n, value, ctx_status_word(ctx),
                                                ctx_peer_wait_ns(ctx));
  ctx_count_launch(ctx, RUYB200_KERNEL_NONE);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? RUYB200_OK : ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(e));
}

}  // extern "C"
