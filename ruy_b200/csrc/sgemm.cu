// fp32 matmul on the CUDA cores: ruy's KernelFloat* (ruy/kernel_avx512.cc:872-1236,
// ruy/kernel_x86.h:598-912) with the bias + clamp epilogue fused.  Products are accumulated with
// FFMA in fp32 over chunks of 32 depth steps, and the chunk sums are folded into the running total
// with a compensated (Kahan) addition.  A plain fp32 chain over depth 1024 drifts by a few 1e-5 from
// a double-precision reference once the partial sums reach ~10; the two-level sum stays below 1e-5
// of max(|ref|, 1) up to a depth of about 4096 on uniform [-1, 1] data (measured 1.0e-5 there, 1.8e-5 at 16384: the
// 32-deep chains' own rounding adds up with the square root of the depth), and a single-pass TF32 tensor-core product
// would be at 1e-3.
#include "common.cuh"

namespace ruyb200 {

namespace {

constexpr int kBK = 16;

// Block tile BM x BN, 256 threads as 16 (n) x 16 (m), each thread TM x TN outputs strided by 16
// so that shared-memory reads are conflict-free and destination stores are coalesced along n.
template <int BM, int BN>
__global__ void __launch_bounds__(256) sgemm_kernel(SideView ms, SideView ns, DstView dst, Epilogue ep) {
  constexpr int TM = BM / 16;
  constexpr int TN = BN / 16;
  __shared__ __align__(16) float As[2][kBK][BM + 4];
  __shared__ __align__(16) float Bs[2][kBK][BN + 4];
  const int tid = threadIdx.x;
  const int tn = tid % 16;
  const int tm = tid / 16;
  const int m0 = blockIdx.y * BM;
  const int n0 = blockIdx.x * BN;
  const float* A = (const float*)ms.data;
  const float* B = (const float*)ns.data;
  const int depth = ep.depth;

  float acc[TM][TN], comp[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) acc[i][j] = comp[i][j] = 0.f;

  constexpr int A_PER = BM * kBK / 256;
  constexpr int B_PER = BN * kBK / 256;
  float ra[A_PER], rb[B_PER];

  auto fetch = [&](int k0) {
#pragma unroll
    for (int i = 0; i < A_PER; i++) {
      const int e = tid + i * 256;
      int w, k;
      if (ms.stride_k == 1) { k = e % kBK; w = e / kBK; } else { w = e % BM; k = e / BM; }
      float v = 0.f;
      if (m0 + w < ms.width && k0 + k < depth) v = A[(int64_t)(m0 + w) * ms.stride_w + (int64_t)(k0 + k) * ms.stride_k];
      ra[i] = v;
    }
#pragma unroll
    for (int i = 0; i < B_PER; i++) {
      const int e = tid + i * 256;
      int w, k;
      if (ns.stride_k == 1) { k = e % kBK; w = e / kBK; } else { w = e % BN; k = e / BN; }
      float v = 0.f;
      if (n0 + w < ns.width && k0 + k < depth) v = B[(int64_t)(n0 + w) * ns.stride_w + (int64_t)(k0 + k) * ns.stride_k];
      rb[i] = v;
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int i = 0; i < A_PER; i++) {
      const int e = tid + i * 256;
      int w, k;
      if (ms.stride_k == 1) { k = e % kBK; w = e / kBK; } else { w = e % BM; k = e / BM; }
      As[buf][k][w] = ra[i];
    }
#pragma unroll
    for (int i = 0; i < B_PER; i++) {
      const int e = tid + i * 256;
      int w, k;
      if (ns.stride_k == 1) { k = e % kBK; w = e / kBK; } else { w = e % BN; k = e / BN; }
      Bs[buf][k][w] = rb[i];
    }
  };

  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  // Thread (tm, tn) owns m in {tm*4..tm*4+3} + 64*g and n in {tn*4..tn*4+3} + 64*h when the tile is at least 64 wide
  // (operands then come out of shared memory four at a time and the destination is written 16 bytes at a time);
  // the 32 x 32 tile keeps the strided assignment.
  constexpr bool kVec = (BM % 64 == 0) && (BN % 64 == 0);
  float part[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; i++)
#pragma unroll
    for (int j = 0; j < TN; j++) part[i][j] = 0.f;
  int chunk = 0;
  for (int k0 = 0; k0 < depth; k0 += kBK, chunk++) {
    const bool more = k0 + kBK < depth;
    if (more) fetch(k0 + kBK);
#pragma unroll
    for (int k = 0; k < kBK; k++) {
      float a[TM], b[TN];
      if (kVec) {
#pragma unroll
        for (int g = 0; g < TM / 4; g++) {
          const float4 v = *reinterpret_cast<const float4*>(&As[buf][k][g * 64 + tm * 4]);
          a[4 * g] = v.x; a[4 * g + 1] = v.y; a[4 * g + 2] = v.z; a[4 * g + 3] = v.w;
        }
#pragma unroll
        for (int h = 0; h < TN / 4; h++) {
          const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][k][h * 64 + tn * 4]);
          b[4 * h] = v.x; b[4 * h + 1] = v.y; b[4 * h + 2] = v.z; b[4 * h + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < TM; i++) a[i] = As[buf][k][tm + 16 * i];
#pragma unroll
        for (int j = 0; j < TN; j++) b[j] = Bs[buf][k][tn + 16 * j];
      }
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) part[i][j] = fmaf(a[i], b[j], part[i][j]);
    }
    // compensated fold of the partial sum (32 depth steps, or what is left) into the running total
    if ((chunk & 1) || !more) {
#pragma unroll
      for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) {
          const float y = part[i][j] - comp[i][j];
          const float t = acc[i][j] + y;
          comp[i][j] = (t - acc[i][j]) - y;
          acc[i][j] = t;
          part[i][j] = 0.f;
        }
    }
    if (more) {
      stash(buf ^ 1);
      __syncthreads();
      buf ^= 1;
    }
  }
  if (kVec) {
    const bool vec_ok = (((uintptr_t)dst.data | (uintptr_t)(dst.stride_m * 4)) & 15) == 0;
#pragma unroll
    for (int i = 0; i < TM; i++) {
      const int m = m0 + (i / 4) * 64 + tm * 4 + (i % 4);
      if (m >= dst.size_m) continue;
#pragma unroll
      for (int h = 0; h < TN / 4; h++) {
        const int n = n0 + h * 64 + tn * 4;
        float* out = (float*)dst.data + (int64_t)m * dst.stride_m + n;
        float v[4];
#pragma unroll
        for (int t = 0; t < 4; t++) v[t] = (n + t < dst.size_n) ? finish_float(acc[i][4 * h + t], m, n + t, ep) : 0.f;
        if (vec_ok && n + 3 < dst.size_n) {
          *reinterpret_cast<float4*>(out) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
          for (int t = 0; t < 4; t++) if (n + t < dst.size_n) out[t] = v[t];
        }
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < TM; i++) {
      const int m = m0 + tm + 16 * i;
      if (m >= dst.size_m) continue;
#pragma unroll
      for (int j = 0; j < TN; j++) {
        const int n = n0 + tn + 16 * j;
        if (n < dst.size_n) ((float*)dst.data)[(int64_t)m * dst.stride_m + n] = finish_float(acc[i][j], m, n, ep);
      }
    }
  }
}

// Few outputs and a long depth (e.g. 17 x 301 x 9): one warp per destination element, lanes striding over depth,
// so the depth loop is 32 times shorter than in the tiled kernel, where a single CTA would walk it alone.
__global__ void __launch_bounds__(256) sgemm_dot_kernel(SideView ms, SideView ns, DstView dst, Epilogue ep) {
  const int lane = threadIdx.x % 32;
  const long long out = (long long)blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32;
  if (out >= (long long)dst.size_m * dst.size_n) return;
  const int m = (int)(out / dst.size_n);
  const int n = (int)(out % dst.size_n);
  const float* a = (const float*)ms.data + (int64_t)m * ms.stride_w;
  const float* b = (const float*)ns.data + (int64_t)n * ns.stride_w;
  float sum = 0.f, comp = 0.f;
  for (int k = lane; k < ep.depth; k += 32) {
    const float y = a[(int64_t)k * ms.stride_k] * b[(int64_t)k * ns.stride_k] - comp;   // product rounded once, as FFMA into 0 would
    const float t = sum + y;
    comp = (t - sum) - y;
    sum = t;
  }
  // pairwise tree over the lanes, each step compensated with the partner's correction term
  for (int d = 16; d > 0; d >>= 1) {
    const float other = __shfl_xor_sync(0xffffffffu, sum, d);
    const float other_c = __shfl_xor_sync(0xffffffffu, comp, d);
    const float y = other - (comp + other_c);
    const float t = sum + y;
    comp = (t - sum) - y;
    sum = t;
  }
  if (lane == 0) ((float*)dst.data)[(int64_t)m * dst.stride_m + n] = finish_float(sum, m, n, ep);
}

}  // namespace

cudaError_t launch_sgemm(const SideView& m_side, const SideView& n_side, const DstView& dst,
                         const Epilogue& ep, cudaStream_t stream) {
  if (dst.size_m <= 0 || dst.size_n <= 0) return cudaSuccess;
  const long long outputs = (long long)dst.size_m * dst.size_n;
  if (outputs <= 1024 && ep.depth >= 128) {
    sgemm_dot_kernel<<<(unsigned)((outputs + 7) / 8), 256, 0, stream>>>(m_side, n_side, dst, ep);
    return cudaGetLastError();
  }
  const long long big_tiles = (long long)((dst.size_m + 127) / 128) * ((dst.size_n + 63) / 64);
  if (big_tiles >= 64) {
    dim3 grid((dst.size_n + 63) / 64, (dst.size_m + 127) / 128);
    if (grid.y > 65535) return cudaErrorInvalidConfiguration;
    sgemm_kernel<128, 64><<<grid, 256, 0, stream>>>(m_side, n_side, dst, ep);
  } else if ((long long)((dst.size_m + 63) / 64) * ((dst.size_n + 63) / 64) >= 32) {
    dim3 grid((dst.size_n + 63) / 64, (dst.size_m + 63) / 64);
    sgemm_kernel<64, 64><<<grid, 256, 0, stream>>>(m_side, n_side, dst, ep);
  } else {
    dim3 grid((dst.size_n + 31) / 32, (dst.size_m + 31) / 32);
    if (grid.y > 65535) return cudaErrorInvalidConfiguration;
    sgemm_kernel<32, 32><<<grid, 256, 0, stream>>>(m_side, n_side, dst, ep);
  }
  return cudaGetLastError();
}

}  // namespace ruyb200
