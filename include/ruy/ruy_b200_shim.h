// Header-only C++ front end with ruy's public names and signatures, implemented over the C ABI of
// libruy_b200.so (include/ruy_b200.h).  Code written against ruy's own headers --
//   ruy::Matrix / Layout / MakeSimpleLayout / Order / CachePolicy   (ruy/matrix.h:30-172)
//   ruy::MulParams / ChannelDimension                                (ruy/mul_params.h:30-223)
//   ruy::Context                                                     (ruy/context.h:38-112)
//   ruy::Path, kDefaultPaths, kAllPaths                              (ruy/path.h:55-196)
//   ruy::Mul                                                         (ruy/ruy.h:37-50,98-104)
// -- compiles unchanged against these and runs on the GPU.  Every Mul goes to the device; nothing is
// computed on the CPU.  Like ruy, Mul returns void and treats misuse as fatal: a non-zero status from
// the library prints its message and aborts (ruy/check_macros.h:102-110).
#ifndef RUY_B200_SHIM_H_
#define RUY_B200_SHIM_H_

#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <limits>
#include <type_traits>

#include "../ruy_b200.h"

namespace ruy {

enum class Order : std::uint8_t { kColMajor, kRowMajor };

class Layout final {
 public:
  int rows() const { return rows_; }
  int cols() const { return cols_; }
  int stride() const { return stride_; }
  Order order() const { return order_; }
  void set_rows(int v) { rows_ = v; }
  void set_cols(int v) { cols_ = v; }
  void set_stride(int v) { stride_ = v; }
  void set_order(Order v) { order_ = v; }

 private:
  int rows_ = 0, cols_ = 0, stride_ = 0;
  Order order_ = Order::kColMajor;
};

inline void MakeSimpleLayout(int rows, int cols, Order order, Layout* layout) {
  layout->set_rows(rows);
  layout->set_cols(cols);
  layout->set_order(order);
  layout->set_stride(order == Order::kColMajor ? rows : cols);
}

enum class CachePolicy : std::uint8_t { kNeverCache, kCacheIfLargeSpeedup, kCacheIfSignificantSpeedup, kAlwaysCache };

// A non-owning view; use Matrix<T> for inputs and outputs alike (never Matrix<const T>).
template <typename Scalar>
class Matrix final {
  static_assert(!std::is_const<Scalar>::value, "use Matrix<T>, not Matrix<const T>");

 public:
  Scalar* data() { return const_cast<Scalar*>(data_); }
  const Scalar* data() const { return data_; }
  void set_data(Scalar* p) { data_ = p; }
  void set_data(const Scalar* p) { data_ = p; }
  void set_data(std::nullptr_t) { data_ = nullptr; }
  const Layout& layout() const { return layout_; }
  Layout* mutable_layout() { return &layout_; }
  Scalar zero_point() const { return zero_point_; }
  void set_zero_point(Scalar v) { zero_point_ = v; }
  CachePolicy cache_policy() const { return cache_policy_; }
  void set_cache_policy(CachePolicy v) { cache_policy_ = v; }

 private:
  const Scalar* data_ = nullptr;
  Layout layout_;
  Scalar zero_point_ = 0;
  CachePolicy cache_policy_ = CachePolicy::kNeverCache;
};

enum class ChannelDimension : std::int8_t { kRow, kCol };

namespace b200_detail {
// Default clamp bounds: the destination type's range, or +-infinity for floating point.
template <typename T, bool kFloat = std::is_floating_point<T>::value>
struct Bounds {
  static T lo() { return std::numeric_limits<T>::lowest(); }
  static T hi() { return std::numeric_limits<T>::max(); }
};
template <typename T>
struct Bounds<T, true> {
  static T lo() { return -std::numeric_limits<T>::infinity(); }
  static T hi() { return std::numeric_limits<T>::infinity(); }
};
template <typename T> struct TypeCode;
template <> struct TypeCode<std::int8_t> { static constexpr std::uint8_t value = RUYB200_I8; };
template <> struct TypeCode<std::uint8_t> { static constexpr std::uint8_t value = RUYB200_U8; };
template <> struct TypeCode<std::int16_t> { static constexpr std::uint8_t value = RUYB200_I16; };
template <> struct TypeCode<std::int32_t> { static constexpr std::uint8_t value = RUYB200_I32; };
template <> struct TypeCode<float> { static constexpr std::uint8_t value = RUYB200_F32; };
template <> struct TypeCode<double> { static constexpr std::uint8_t value = RUYB200_F64; };
}  // namespace b200_detail

// Same accessors and defaults as ruy's: no bias, multiplier 0 with exponent 0 (so a quantized Mul whose
// multiplier was never set yields clamp(dst zero point)), full-range clamp, channel dimension kRow.
// Setting a scalar multiplier leaves per-channel mode and vice versa, as in ruy.
template <typename tAccumScalar, typename tDstScalar>
class MulParams final {
 public:
  using AccumScalar = tAccumScalar;
  using DstScalar = tDstScalar;
  static constexpr bool kQuantized = std::is_same<AccumScalar, std::int32_t>::value && !std::is_same<DstScalar, std::int32_t>::value;

  const AccumScalar* bias() const { return bias_; }
  void set_bias(const AccumScalar* p) { bias_ = p; }
  AccumScalar multiplier_fixedpoint() const { return perchannel_ ? 0 : mfp_; }
  void set_multiplier_fixedpoint(AccumScalar v) { perchannel_ = false; mfp_pc_ = nullptr; mexp_pc_ = nullptr; mfp_ = v; }
  int multiplier_exponent() const { return perchannel_ ? 0 : mexp_; }
  void set_multiplier_exponent(int v) { perchannel_ = false; mfp_pc_ = nullptr; mexp_pc_ = nullptr; mexp_ = v; }
  const AccumScalar* multiplier_fixedpoint_perchannel() const { return perchannel_ ? mfp_pc_ : nullptr; }
  void set_multiplier_fixedpoint_perchannel(const AccumScalar* p) { enter_perchannel(); mfp_pc_ = p; }
  const int* multiplier_exponent_perchannel() const { return perchannel_ ? mexp_pc_ : nullptr; }
  void set_multiplier_exponent_perchannel(const int* p) { enter_perchannel(); mexp_pc_ = p; }
  DstScalar clamp_min() const { return clamp_min_; }
  void set_clamp_min(DstScalar v) { clamp_min_ = v; }
  DstScalar clamp_max() const { return clamp_max_; }
  void set_clamp_max(DstScalar v) { clamp_max_ = v; }
  ChannelDimension channel_dimension() const { return channel_dimension_; }
  void set_channel_dimension(ChannelDimension v) { channel_dimension_ = v; }
  int perchannel_buffers_capacity_rounding() const { return 1 << capacity_rounding_log2_; }
  void set_perchannel_buffers_capacity_rounding(int v) {
    int log2 = 0;
    while ((1 << log2) < v) log2++;
    capacity_rounding_log2_ = static_cast<std::int8_t>(log2);
  }

 private:
  void enter_perchannel() {
    if (!perchannel_) { perchannel_ = true; mfp_ = 0; mexp_ = 0; }
  }
  const AccumScalar* bias_ = nullptr;
  const AccumScalar* mfp_pc_ = nullptr;
  const int* mexp_pc_ = nullptr;
  AccumScalar mfp_ = 0;
  int mexp_ = 0;
  DstScalar clamp_min_ = b200_detail::Bounds<DstScalar>::lo();
  DstScalar clamp_max_ = b200_detail::Bounds<DstScalar>::hi();
  ChannelDimension channel_dimension_ = ChannelDimension::kRow;
  bool perchannel_ = false;
  std::int8_t capacity_rounding_log2_ = 0;
};

enum class Path : std::uint8_t {
  kNone = 0,
  kStandardCpp = 0x1,
  kInternalStandardCppVariant1 = 0x2,
  kInternalStandardCppVariant2 = 0x4,
  kInternalStandardCppVariant3 = 0x8,
  kAvx = 0x10,
  kAvx2Fma = 0x20,
  kAvx512 = 0x40,
};
inline constexpr Path operator|(Path p, Path q) { return static_cast<Path>(static_cast<unsigned>(p) | static_cast<unsigned>(q)); }
inline constexpr Path operator&(Path p, Path q) { return static_cast<Path>(static_cast<unsigned>(p) & static_cast<unsigned>(q)); }
inline constexpr Path operator^(Path p, Path q) { return static_cast<Path>(static_cast<unsigned>(p) ^ static_cast<unsigned>(q)); }
inline constexpr Path operator~(Path p) { return static_cast<Path>(~static_cast<unsigned>(p) & 0xFFu); }
inline constexpr bool Disjoint(Path p, Path q) { return (p & q) == Path::kNone; }
constexpr Path kNonArchPaths = Path::kStandardCpp;
constexpr Path kDefaultArchPaths = Path::kAvx | Path::kAvx2Fma | Path::kAvx512;
constexpr Path kDefaultPaths = Path::kStandardCpp | kDefaultArchPaths;
constexpr Path kAllPaths = kDefaultPaths;

enum class PerformanceAdvisory { kNone = 0, kReallocatedPerChannelBuffer = 0x1 };
enum class Tuning { kAuto, kGeneric, kA55ish, kX1 };
enum class NumThreadsStrategy : std::uint8_t { kDefault, kForceMaxNumThreads };

namespace b200_detail {
inline void Check(int status, const char* what) {
  if (status != RUYB200_OK) {
    std::fprintf(stderr, "ruy (B200): %s failed with status %d: %s\n", what, status, ruyb200_last_error());
    std::abort();
  }
}
}  // namespace b200_detail

// One per calling thread, as with ruy.  The device context is created on first use.
class Context final {
 public:
  Context() = default;
  ~Context() {
    if (handle_) ruyb200_ctx_destroy(handle_);
  }
  Context(const Context&) = delete;
  Context& operator=(const Context&) = delete;

  Path last_used_path() const { return static_cast<Path>(ruyb200_ctx_last_used_path(handle())); }
  Tuning explicit_tuning() const { return tuning_; }
  void set_explicit_tuning(Tuning v) { tuning_ = v; }   // CPU-only notion: stored, not used
  int max_num_threads() const { return ruyb200_ctx_get_max_num_threads(handle()); }
  void set_max_num_threads(int v) { b200_detail::Check(ruyb200_ctx_set_max_num_threads(handle(), v), "set_max_num_threads"); }
  NumThreadsStrategy num_threads_strategy() const { return strategy_; }
  void set_num_threads_strategy(NumThreadsStrategy v) { strategy_ = v; }
  bool performance_advisory(PerformanceAdvisory a) const {
    return ruyb200_ctx_performance_advisory(handle(), static_cast<int>(a)) != 0;
  }
  void ClearPrepackedCache() { b200_detail::Check(ruyb200_ctx_clear_prepacked_cache(handle()), "ClearPrepackedCache"); }
  void set_runtime_enabled_paths(Path paths) {
    b200_detail::Check(ruyb200_ctx_set_runtime_enabled_paths(handle(), static_cast<std::uint32_t>(paths)), "set_runtime_enabled_paths");
  }
  Path get_runtime_enabled_paths() { return static_cast<Path>(ruyb200_ctx_get_runtime_enabled_paths(handle())); }

  // Not part of ruy: the underlying C-ABI context (for ruyb200_mul_async, plans, counters).
  ruyb200_ctx* b200() const { return handle(); }

 private:
  ruyb200_ctx* handle() const {
    if (!handle_) b200_detail::Check(ruyb200_ctx_create(-1, &handle_), "ruyb200_ctx_create");
    return handle_;
  }
  mutable ruyb200_ctx* handle_ = nullptr;
  Tuning tuning_ = Tuning::kAuto;
  NumThreadsStrategy strategy_ = NumThreadsStrategy::kDefault;
};

namespace b200_detail {
template <typename T>
ruyb200_matrix Flatten(const Matrix<T>& m) {
  ruyb200_matrix out{};
  out.data = const_cast<T*>(m.data());
  out.rows = m.layout().rows();
  out.cols = m.layout().cols();
  out.stride = m.layout().stride();
  out.zero_point = static_cast<std::int32_t>(m.zero_point());
  out.order = m.layout().order() == Order::kRowMajor ? RUYB200_ROW_MAJOR : RUYB200_COL_MAJOR;
  out.dtype = TypeCode<T>::value;
  out.cache_policy = static_cast<std::uint8_t>(m.cache_policy());
  return out;
}
template <typename Accum, typename Dst>
void FlattenClamp(const MulParams<Accum, Dst>& p, ruyb200_mul_params* out, std::true_type /*float*/) {
  if (std::is_same<Accum, double>::value) {   // the mixed float/double cases carry their bounds as doubles
    out->clamp_min.d = static_cast<double>(p.clamp_min());
    out->clamp_max.d = static_cast<double>(p.clamp_max());
  } else {
    out->clamp_min.f = static_cast<float>(p.clamp_min());
    out->clamp_max.f = static_cast<float>(p.clamp_max());
  }
}
template <typename Accum, typename Dst>
void FlattenClamp(const MulParams<Accum, Dst>& p, ruyb200_mul_params* out, std::false_type) {
  out->clamp_min.i = static_cast<std::int32_t>(p.clamp_min());
  out->clamp_max.i = static_cast<std::int32_t>(p.clamp_max());
}
}  // namespace b200_detail

// ruy::Mul with an explicit set of compiled paths (ruy/ruy.h:37-50).  The path set only selects the
// rounding contract (see RUYB200_ROUNDING_FROM_PATH); execution is always on the GPU.
template <Path CompiledPaths, typename LhsScalar, typename RhsScalar, typename AccumScalar, typename DstScalar>
void Mul(const Matrix<LhsScalar>& lhs, const Matrix<RhsScalar>& rhs, const MulParams<AccumScalar, DstScalar>& mul_params,
         Context* context, Matrix<DstScalar>* dst) {
  static_assert(CompiledPaths != Path::kNone, "at least one path must be compiled");
  ruyb200_mul_desc d{};
  d.lhs = b200_detail::Flatten(lhs);
  d.rhs = b200_detail::Flatten(rhs);
  d.dst = b200_detail::Flatten(*dst);
  d.params.bias = mul_params.bias();
  d.params.multiplier_fixedpoint_perchannel = reinterpret_cast<const std::int32_t*>(mul_params.multiplier_fixedpoint_perchannel());
  d.params.multiplier_exponent_perchannel = reinterpret_cast<const std::int32_t*>(mul_params.multiplier_exponent_perchannel());
  d.params.multiplier_fixedpoint = static_cast<std::int32_t>(mul_params.multiplier_fixedpoint());
  d.params.multiplier_exponent = mul_params.multiplier_exponent();
  b200_detail::FlattenClamp(mul_params, &d.params, std::is_floating_point<AccumScalar>());
  d.params.channel_dimension = mul_params.channel_dimension() == ChannelDimension::kCol ? RUYB200_CHANNEL_COL : RUYB200_CHANNEL_ROW;
  int log2 = 0;
  while ((1 << log2) < mul_params.perchannel_buffers_capacity_rounding()) log2++;
  d.params.perchannel_buffers_capacity_rounding_log2 = static_cast<std::uint8_t>(log2);
  d.params.accum_dtype = b200_detail::TypeCode<AccumScalar>::value;
  d.params.rounding_mode = RUYB200_ROUNDING_FROM_PATH;
  b200_detail::Check(ruyb200_mul(context->b200(), &d), "ruy::Mul");
}

// ruy::Mul with the default paths (ruy/ruy.h:98-104).
template <typename LhsScalar, typename RhsScalar, typename AccumScalar, typename DstScalar>
void Mul(const Matrix<LhsScalar>& lhs, const Matrix<RhsScalar>& rhs, const MulParams<AccumScalar, DstScalar>& mul_params,
         Context* context, Matrix<DstScalar>* dst) {
  Mul<kDefaultPaths>(lhs, rhs, mul_params, context, dst);
}

}  // namespace ruy

#endif  // RUY_B200_SHIM_H_
