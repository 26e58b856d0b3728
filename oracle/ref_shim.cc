// ref_shim.cc -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// A C-ABI wrapper around the UNMODIFIED reference (google/ruy), compiled from the
// reference's own sources where they lie (see oracle/Makefile) into
// oracle/_ref/libruy_ref.so.  It takes the same POD descriptor as the product
// library (include/ruy_b200.h), rebuilds ruy::Matrix / ruy::MulParams from it and
// calls ruy::Mul or ruy::ReferenceMul.  Used to pin the C restatement in
// oracle/ruy_oracle.c, to generate tests/golden/, and as the timed CPU baseline.
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "ruy/context.h"
#include "ruy/matrix.h"
#include "ruy/mul_params.h"
#include "ruy/path.h"
#include "ruy/reference_mul.h"
#include "ruy/ruy.h"

#include "../include/ruy_b200.h"

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {

template <typename T>
ruy::Matrix<T> ToMatrix(const ruyb200_matrix& m, bool is_dst) {
  ruy::Matrix<T> out;
  out.mutable_layout()->set_rows(m.rows);
  out.mutable_layout()->set_cols(m.cols);
  out.mutable_layout()->set_stride(m.stride);
  out.mutable_layout()->set_order(m.order == RUYB200_ROW_MAJOR ? ruy::Order::kRowMajor
                                                               : ruy::Order::kColMajor);
  if (is_dst) {
    out.set_data(static_cast<T*>(m.data));
  } else {
    out.set_data(static_cast<const T*>(m.data));
  }
  out.set_zero_point(static_cast<T>(m.zero_point));
  out.set_cache_policy(static_cast<ruy::CachePolicy>(m.cache_policy));
  return out;
}

template <typename Accum, typename Dst>
struct FillParams {
  static void Run(const ruyb200_mul_params& p, ruy::MulParams<Accum, Dst>* out) {
    // Quantized, narrowing destination.
    out->set_bias(static_cast<const Accum*>(p.bias));
    if (p.multiplier_fixedpoint_perchannel || p.multiplier_exponent_perchannel) {
      out->set_multiplier_fixedpoint_perchannel(p.multiplier_fixedpoint_perchannel);
      out->set_multiplier_exponent_perchannel(p.multiplier_exponent_perchannel);
    } else {
      out->set_multiplier_fixedpoint(p.multiplier_fixedpoint);
      out->set_multiplier_exponent(p.multiplier_exponent);
    }
    out->set_clamp_min(static_cast<Dst>(p.clamp_min.i));
    out->set_clamp_max(static_cast<Dst>(p.clamp_max.i));
  }
};
template <>
struct FillParams<std::int32_t, std::int32_t> {
  static void Run(const ruyb200_mul_params& p, ruy::MulParams<std::int32_t, std::int32_t>* out) {
    out->set_bias(static_cast<const std::int32_t*>(p.bias));
  }
};
template <>
struct FillParams<float, float> {
  static void Run(const ruyb200_mul_params& p, ruy::MulParams<float, float>* out) {
    out->set_bias(static_cast<const float*>(p.bias));
    out->set_clamp_min(p.clamp_min.f);
    out->set_clamp_max(p.clamp_max.f);
  }
};

// ruy's mixed floating-point cases (ruy/BUILD:1195-1207): double accumulator and bias, bounds in .d
template <typename Dst>
struct FillParams<double, Dst> {
  static void Run(const ruyb200_mul_params& p, ruy::MulParams<double, Dst>* out) {
    out->set_bias(static_cast<const double*>(p.bias));
    out->set_clamp_min(static_cast<Dst>(p.clamp_min.d));
    out->set_clamp_max(static_cast<Dst>(p.clamp_max.d));
  }
};

template <typename L, typename R, typename Accum, typename Dst>
int Run(ruy::Context* ctx, const ruyb200_mul_desc& d, bool reference_mul) {
  ruy::Matrix<L> lhs = ToMatrix<L>(d.lhs, false);
  ruy::Matrix<R> rhs = ToMatrix<R>(d.rhs, false);
  ruy::Matrix<Dst> dst = ToMatrix<Dst>(d.dst, true);
  ruy::MulParams<Accum, Dst> params;
  FillParams<Accum, Dst>::Run(d.params, &params);
  params.set_channel_dimension(d.params.channel_dimension == RUYB200_CHANNEL_COL
                                   ? ruy::ChannelDimension::kCol
                                   : ruy::ChannelDimension::kRow);
  params.set_perchannel_buffers_capacity_rounding(
      1 << d.params.perchannel_buffers_capacity_rounding_log2);
  if (reference_mul) {
    ruy::ReferenceMul(lhs, rhs, params, &dst);
  } else {
    ruy::Mul(lhs, rhs, params, ctx, &dst);
  }
  return 0;
}

int Dispatch(ruy::Context* ctx, const ruyb200_mul_desc& d, bool reference_mul) {
  const int l = d.lhs.dtype, r = d.rhs.dtype, o = d.dst.dtype;
  using i8 = std::int8_t;
  using u8 = std::uint8_t;
  using i16 = std::int16_t;
  using i32 = std::int32_t;
#define CASE(LT, RT, DT, L, R, A, D) \
  if (l == LT && r == RT && o == DT) return Run<L, R, A, D>(ctx, d, reference_mul);
  CASE(RUYB200_F32, RUYB200_F32, RUYB200_F32, float, float, float, float)
  CASE(RUYB200_F64, RUYB200_F32, RUYB200_F32, double, float, double, float)
  CASE(RUYB200_F32, RUYB200_F64, RUYB200_F64, float, double, double, double)
  CASE(RUYB200_I8, RUYB200_I8, RUYB200_I8, i8, i8, i32, i8)
  CASE(RUYB200_I8, RUYB200_I8, RUYB200_U8, i8, i8, i32, u8)
  CASE(RUYB200_I8, RUYB200_I8, RUYB200_I16, i8, i8, i32, i16)
  CASE(RUYB200_I8, RUYB200_I8, RUYB200_I32, i8, i8, i32, i32)
  CASE(RUYB200_U8, RUYB200_U8, RUYB200_U8, u8, u8, i32, u8)
  CASE(RUYB200_U8, RUYB200_U8, RUYB200_I8, u8, u8, i32, i8)
  CASE(RUYB200_U8, RUYB200_U8, RUYB200_I16, u8, u8, i32, i16)
  CASE(RUYB200_U8, RUYB200_U8, RUYB200_I32, u8, u8, i32, i32)
  CASE(RUYB200_I8, RUYB200_U8, RUYB200_I8, i8, u8, i32, i8)
  CASE(RUYB200_I8, RUYB200_U8, RUYB200_I32, i8, u8, i32, i32)
  CASE(RUYB200_U8, RUYB200_I8, RUYB200_I8, u8, i8, i32, i8)
  CASE(RUYB200_I8, RUYB200_I16, RUYB200_I16, i8, i16, i32, i16)
  CASE(RUYB200_I16, RUYB200_I8, RUYB200_I16, i16, i8, i32, i16)
#undef CASE
  return RUYB200_ERR_UNSUPPORTED;
}

}  // namespace

REF_API void* ruy_ref_ctx_create(int path_mask, int max_threads) {
  auto* ctx = new ruy::Context;
  if (path_mask) ctx->set_runtime_enabled_paths(static_cast<ruy::Path>(path_mask));
  ctx->set_max_num_threads(max_threads > 0 ? max_threads : 1);
  return ctx;
}

REF_API void ruy_ref_ctx_destroy(void* ctx) { delete static_cast<ruy::Context*>(ctx); }

REF_API int ruy_ref_last_used_path(void* ctx) {
  return static_cast<int>(static_cast<ruy::Context*>(ctx)->last_used_path());
}

REF_API void ruy_ref_clear_cache(void* ctx) {
  static_cast<ruy::Context*>(ctx)->ClearPrepackedCache();
}

// ruy::Mul through the context's enabled path.
REF_API int ruy_ref_mul(void* ctx, const ruyb200_mul_desc* d) {
  return Dispatch(static_cast<ruy::Context*>(ctx), *d, false);
}

// ruy::ReferenceMul (the triple loop).
REF_API int ruy_ref_reference_mul(const ruyb200_mul_desc* d) { return Dispatch(nullptr, *d, true); }

// ruy::detail::MultiplyByQuantizedMultiplier, for the known-answer tests.
REF_API std::int32_t ruy_ref_multiply_by_quantized_multiplier(std::int32_t x, std::int32_t m, int e) {
  return ruy::detail::MultiplyByQuantizedMultiplier(x, m, e);
}

// Timed loop over one mul: returns the best seconds-per-call over `windows` windows of at
// least `min_secs` each (the protocol of ruy/test.h:2082-2136).
REF_API double ruy_ref_time_mul(void* ctx, const ruyb200_mul_desc* d, int windows, double min_secs) {
  using clock = std::chrono::steady_clock;
  Dispatch(static_cast<ruy::Context*>(ctx), *d, false);  // warm-up (also fills the cache)
  double best = 1e30;
  for (int w = 0; w < windows; w++) {
    int iters = 0;
    const auto t0 = clock::now();
    double elapsed = 0;
    do {
      Dispatch(static_cast<ruy::Context*>(ctx), *d, false);
      iters++;
      elapsed = std::chrono::duration<double>(clock::now() - t0).count();
    } while (elapsed < min_secs);
    if (elapsed / iters < best) best = elapsed / iters;
  }
  return best;
}

// Many independent muls on `threads` host threads, one ruy::Context per thread over
// disjoint contiguous ranges (ruy's threading contract, ruy/ruy.h:84-87).  Runs the whole
// list `passes` times after one untimed pass (which fills each context's prepacked cache)
// and returns the seconds of the fastest pass.
REF_API double ruy_ref_time_batch(const ruyb200_mul_desc* descs, int n, int threads, int path_mask,
                                  int passes) {
  using clock = std::chrono::steady_clock;
  if (threads < 1) threads = 1;
  std::vector<ruy::Context*> ctxs(threads);
  for (auto& c : ctxs) {
    c = new ruy::Context;
    if (path_mask) c->set_runtime_enabled_paths(static_cast<ruy::Path>(path_mask));
    c->set_max_num_threads(1);
  }
  auto run_pass = [&]() {
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; t++) {
      pool.emplace_back([&, t]() {
        const int begin = static_cast<int>(static_cast<long long>(n) * t / threads);
        const int end = static_cast<int>(static_cast<long long>(n) * (t + 1) / threads);
        for (int i = begin; i < end; i++) Dispatch(ctxs[t], descs[i], false);
      });
    }
    for (auto& th : pool) th.join();
  };
  run_pass();
  double best = 1e30;
  for (int p = 0; p < passes; p++) {
    const auto t0 = clock::now();
    run_pass();
    const double s = std::chrono::duration<double>(clock::now() - t0).count();
    if (s < best) best = s;
  }
  for (auto* c : ctxs) delete c;
  return best;
}
