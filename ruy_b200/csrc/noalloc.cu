// ruyb200_mul_noalloc: the 8-bit tensor-core mul for callers that must not allocate.
//
// Some users of this library cannot call cudaMalloc (or anything that allocates) at the point where
// they multiply: an inference runtime that handed the whole device to its own memory pool at start-up,
// a service running under a fixed memory budget that must not fail with out-of-memory in the middle
// of a request, or a latency-critical loop that cannot afford the device-wide synchronisation an
// allocation or a free implies.  ruyb200_mul needs a context, and a context owns a growing scratch
// arena, a prepacked cache and a status word, all of them allocated on demand.  This entry point
// needs none of that: the only global memory it touches besides the caller's operands and
// destination is the fixed array below, which is part of the library image (every device that loads
// the library holds it until the process exits).
//
// The scratch holds what the tensor-core kernel needs beyond its inputs and outputs: the depth-wise
// sums of both operands (the zero-point correction terms, ruy/pack.h:117-129) and the status word of
// the kernel's bounded waits.  Capacity: 16384 destination rows and 16384 destination columns.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "common.cuh"
#include "plan.h"

using namespace ruyb200;

namespace {

constexpr int kMaxWidth = 16384;                        // max destination rows, and max destination columns
constexpr size_t kStatusBytes = 256;
constexpr size_t kScratchBytes = kStatusBytes + 2 * sizeof(int32_t) * kMaxWidth;   // 128.25 KiB

// File-scope device scratch.  In host code this name is only a handle for the runtime: it is NOT a
// device address and must never be passed to a kernel.  The address is obtained once per device with
// cudaGetSymbolAddress (below) and that pointer is what the kernels receive.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
struct DeviceSetup {
  bool ready = false;
  unsigned char* scratch = nullptr;   // device address of g_noalloc_scratch on this device
  int sm_count = 0;
};
DeviceSetup g_setup[kMaxDevices];
std::mutex g_setup_mutex;   // two threads may make their first call on a device at the same time

// Runs once per device, with that device current.
int setup_device(int device, DeviceSetup** out) {
  if (device < 0 || device >= kMaxDevices) return ctx_fail(RUYB200_ERR_INVALID, "device index out of range");
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  DeviceSetup& s = g_setup[device];
  if (!s.ready) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
      cudaGetLastError();
      return ctx_fail(RUYB200_ERR_CUDA, "cudaGetSymbolAddress failed for the static scratch");
    }
    int sms = 0, major = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) {
      cudaGetLastError();
      return ctx_fail(RUYB200_ERR_CUDA, "cudaDeviceGetAttribute failed");
    }
    if (major != 10) return ctx_fail(RUYB200_ERR_NO_DEVICE, "this library is built for sm_100a only");
    s.scratch = static_cast<unsigned char*>(ptr);
    s.sm_count = sms;
    s.ready = true;
  }
  *out = &s;
  return RUYB200_OK;
}

SideView make_side(const ruyb200_matrix& m, int side) {
  SideView v;
  v.data = m.data;
  v.dtype = m.dtype;
  v.zero_point = m.zero_point;
  const bool row_major = m.order == RUYB200_ROW_MAJOR;
  if (side == 0) {
    v.width = m.rows;
    v.stride_w = row_major ? m.stride : 1;
    v.stride_k = row_major ? 1 : m.stride;
  } else {
    v.width = m.cols;
    v.stride_w = row_major ? 1 : m.stride;
    v.stride_k = row_major ? m.stride : 1;
  }
  return v;
}

}  // namespace

extern "C" int ruyb200_mul_noalloc(const ruyb200_mul_desc* desc, void* cuda_stream) {
  int rc = ctx_validate(desc);
  if (rc) return rc;
  const ruyb200_mul_desc& d = *desc;
  if (d.params.accum_dtype != RUYB200_I32 || (d.lhs.dtype != RUYB200_I8 && d.lhs.dtype != RUYB200_U8) ||
      (d.rhs.dtype != RUYB200_I8 && d.rhs.dtype != RUYB200_U8)) {
    return ctx_fail(RUYB200_ERR_UNSUPPORTED, "ruyb200_mul_noalloc: 8-bit operands with int32 accumulation only");
  }
  if (d.dst.rows > kMaxWidth || d.dst.cols > kMaxWidth) {
    return ctx_fail(RUYB200_ERR_INVALID,
                    "ruyb200_mul_noalloc: destination exceeds the static scratch (at most 16384 rows and 16384 columns)");
  }
  if (d.dst.rows == 0 || d.dst.cols == 0) return RUYB200_OK;
  if (d.lhs.cols == 0) return ctx_fail(RUYB200_ERR_UNSUPPORTED, "ruyb200_mul_noalloc: depth must be at least 1");
  const void* ptrs[6] = {d.lhs.data, d.rhs.data, d.dst.data, d.params.bias, d.params.multiplier_fixedpoint_perchannel,
                         d.params.multiplier_exponent_perchannel};
  for (const void* p : ptrs) {
    if (p && !ptr_on_device(p)) return ctx_fail(RUYB200_ERR_INVALID, "ruyb200_mul_noalloc needs device pointers");
  }
  SideView lhs = make_side(d.lhs, 0), rhs = make_side(d.rhs, 1);
  if (!tc_i8_eligible(lhs, rhs)) {
    return ctx_fail(RUYB200_ERR_UNSUPPORTED,
                    "ruyb200_mul_noalloc: operands must be depth-contiguous (row-major LHS, column-major RHS) with "
                    "16-byte aligned base addresses and strides; repacking would need scratch this entry point does not have");
  }
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    return ctx_fail(RUYB200_ERR_NO_DEVICE, "no current CUDA device");
  }
  DeviceSetup* setup = nullptr;
  rc = setup_device(device, &setup);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  int* status = reinterpret_cast<int*>(setup->scratch);
  int32_t* lhs_sums = reinterpret_cast<int32_t*>(setup->scratch + kStatusBytes);
  int32_t* rhs_sums = lhs_sums + kMaxWidth;
  const int depth = d.lhs.cols;

  // The array keeps whatever the previous call left in it.  The status word must start at zero; the sums
  // are rewritten in full (for the widths of this call) before the kernel reads them.
  if (cudaMemsetAsync(status, 0, sizeof(int), stream) != cudaSuccess) {
    return ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
  }
  const bool need_lhs_sums = d.rhs.zero_point != 0;
  const bool need_rhs_sums = d.lhs.zero_point != 0;
  cudaError_t ce = cudaSuccess;
  if (need_lhs_sums) ce = launch_sums(lhs, depth, lhs_sums, stream);
  if (ce == cudaSuccess && need_rhs_sums) ce = launch_sums(rhs, depth, rhs_sums, stream);
  if (ce != cudaSuccess) return ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(ce));

  TcI8Launch L;
  Epilogue ep;
  memset(&ep, 0, sizeof(ep));
  ep.bias = d.params.bias;
  if (d.dst.dtype != RUYB200_I32) {
    ep.mfp_pc = d.params.multiplier_fixedpoint_perchannel;
    ep.mexp_pc = d.params.multiplier_exponent_perchannel;
    ep.mfp = d.params.multiplier_fixedpoint;
    ep.mexp = d.params.multiplier_exponent;
  }
  ep.clamp_min = d.params.clamp_min.i;
  ep.clamp_max = d.params.clamp_max.i;
  ep.dst_zp = d.dst.zero_point;
  ep.depth = depth;
  ep.dst_dtype = d.dst.dtype;
  ep.is_float = 0;
  // There is no context here, hence no path selection: the reference rounding unless the x86 one is asked for.
  ep.rounding_x86 = d.params.rounding_mode == RUYB200_ROUNDING_X86;
  const bool channel_row = d.params.channel_dimension == RUYB200_CHANNEL_ROW;
  const bool dst_col_major = d.dst.order == RUYB200_COL_MAJOR;
  L.dst.data = d.dst.data;
  L.dst.stride_m = d.dst.stride;
  L.dst.size_m = dst_col_major ? d.dst.cols : d.dst.rows;
  L.dst.size_n = dst_col_major ? d.dst.rows : d.dst.cols;
  if (dst_col_major) {
    L.n_side = lhs;
    L.m_side = rhs;
    ep.sums_n = need_lhs_sums ? lhs_sums : nullptr;
    ep.sums_m = need_rhs_sums ? rhs_sums : nullptr;
    ep.channel_on_n = channel_row;
  } else {
    L.n_side = rhs;
    L.m_side = lhs;
    ep.sums_n = need_rhs_sums ? rhs_sums : nullptr;
    ep.sums_m = need_lhs_sums ? lhs_sums : nullptr;
    ep.channel_on_n = !channel_row;
  }
  ep.zp_m = L.m_side.zero_point;
  ep.zp_n = L.n_side.zero_point;
  L.ep = ep;
  L.depth = depth;
  L.sm_count = setup->sm_count;
  L.status = status;
  L.allow_pair = true;
  L.fuse_sums_m = false;
  L.n_mirrors = 0;
  ce = launch_tc_i8(L, stream);
  if (ce != cudaSuccess) return ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(ce));

  int host_status = 0;
  if (cudaMemcpyAsync(&host_status, status, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess) {
    return ctx_fail(RUYB200_ERR_CUDA, cudaGetErrorString(cudaGetLastError()));
  }
  if (host_status != 0) return ctx_fail(RUYB200_ERR_TIMEOUT, "a bounded device-side wait gave up; results are invalid");
  return RUYB200_OK;
}
