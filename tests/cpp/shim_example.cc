// The usage patterns of the reference's example program (example/example.cc:21-182), written against the
// drop-in headers: float, float with bias and clamp, double x float, asymmetric uint8, per-channel int8, raw int32
// accumulators, int8 x int16.  Prints each destination as one line of integers/floats so that the Python
// test can compare them with the oracle.  Also exercises the Context methods.
#include <cstdint>
#include <cstdio>

#include "ruy/ruy.h"

template <typename T>
void Print(const char* name, const T* d, int n) {
  std::printf("%s", name);
  for (int i = 0; i < n; i++) std::printf(" %g", static_cast<double>(d[i]));
  std::printf("\n");
}

int main() {
  ruy::Context context;
  {
    const float lhs_data[] = {1, 2, 3, 4}, rhs_data[] = {1, 2, 3, 4};
    float dst_data[4];
    ruy::Matrix<float> lhs, rhs, dst;
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kRowMajor, lhs.mutable_layout());
    lhs.set_data(lhs_data);
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, rhs.mutable_layout());
    rhs.set_data(rhs_data);
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, dst.mutable_layout());
    dst.set_data(dst_data);
    ruy::MulParams<float, float> mul_params;
    ruy::Mul(lhs, rhs, mul_params, &context, &dst);
    Print("float", dst_data, 4);
    const float bias_data[] = {1, 0};
    mul_params.set_bias(bias_data);
    mul_params.set_clamp_min(0);
    mul_params.set_clamp_max(15);
    ruy::Mul(lhs, rhs, mul_params, &context, &dst);
    Print("float_bias_clamp", dst_data, 4);
  }
  {
    // one of ruy's mixed floating-point cases: double LHS, float RHS, double accumulator and bias, float destination
    const double lhs_data[] = {1.5, 2, 3, 4};
    const float rhs_data[] = {1, 2, 3, 4.25f};
    const double bias_data[] = {0.5, -1};
    float dst_data[4];
    ruy::Matrix<double> lhs;
    ruy::Matrix<float> rhs, dst;
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kRowMajor, lhs.mutable_layout());
    lhs.set_data(lhs_data);
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, rhs.mutable_layout());
    rhs.set_data(rhs_data);
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, dst.mutable_layout());
    dst.set_data(dst_data);
    ruy::MulParams<double, float> mul_params;
    mul_params.set_bias(bias_data);
    mul_params.set_clamp_max(20);
    ruy::Mul(lhs, rhs, mul_params, &context, &dst);
    Print("double_lhs_float_rhs", dst_data, 4);
  }
  {
    const std::uint8_t lhs_data[] = {124, 125, 126, 127}, rhs_data[] = {129, 130, 131, 132};
    std::uint8_t dst_data[4];
    ruy::Matrix<std::uint8_t> lhs, rhs, dst;
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kRowMajor, lhs.mutable_layout());
    lhs.set_data(lhs_data);
    lhs.set_zero_point(125);
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, rhs.mutable_layout());
    rhs.set_data(rhs_data);
    rhs.set_zero_point(132);
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, dst.mutable_layout());
    dst.set_data(dst_data);
    dst.set_zero_point(129);
    ruy::MulParams<std::int32_t, std::uint8_t> mul_params;
    mul_params.set_multiplier_fixedpoint(1 << 30);
    mul_params.set_multiplier_exponent(0);
    ruy::Mul(lhs, rhs, mul_params, &context, &dst);
    Print("uint8_asymmetric", dst_data, 4);
  }
  {
    const std::int8_t lhs_data[] = {1, 2, 3, 4}, rhs_data[] = {1, 2, 3, 4};
    const std::int32_t multiplier_data[] = {3 << 28, 5 << 28};
    const int exponent_data[] = {1, -2};
    std::int8_t dst_data[4];
    ruy::Matrix<std::int8_t> lhs, rhs, dst;
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kRowMajor, lhs.mutable_layout());
    lhs.set_data(lhs_data);
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, rhs.mutable_layout());
    rhs.set_data(rhs_data);
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, dst.mutable_layout());
    dst.set_data(dst_data);
    ruy::MulParams<std::int32_t, std::int8_t> mul_params;
    mul_params.set_multiplier_fixedpoint_perchannel(multiplier_data);
    mul_params.set_multiplier_exponent_perchannel(exponent_data);
    ruy::Mul(lhs, rhs, mul_params, &context, &dst);
    Print("int8_perchannel", dst_data, 4);

    std::int32_t raw[4];
    ruy::Matrix<std::int32_t> dst32;
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, dst32.mutable_layout());
    dst32.set_data(raw);
    ruy::MulParams<std::int32_t, std::int32_t> raw_params;
    ruy::Mul(lhs, rhs, raw_params, &context, &dst32);
    Print("int8_raw_accumulators", raw, 4);

    const std::int16_t rhs16_data[] = {1000, 2000, 3000, 4000};
    std::int16_t dst16_data[4];
    ruy::Matrix<std::int16_t> rhs16, dst16;
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, rhs16.mutable_layout());
    rhs16.set_data(rhs16_data);
    ruy::MakeSimpleLayout(2, 2, ruy::Order::kColMajor, dst16.mutable_layout());
    dst16.set_data(dst16_data);
    ruy::MulParams<std::int32_t, std::int16_t> params16;
    params16.set_multiplier_fixedpoint_perchannel(multiplier_data);
    params16.set_multiplier_exponent_perchannel(exponent_data);
    ruy::Mul(lhs, rhs16, params16, &context, &dst16);
    Print("int8_times_int16", dst16_data, 4);
  }
  // context surface
  std::printf("last_used_path %d\n", static_cast<int>(context.last_used_path()));
  context.set_runtime_enabled_paths(ruy::Path::kStandardCpp);
  std::printf("enabled_paths %d\n", static_cast<int>(context.get_runtime_enabled_paths()));
  context.set_max_num_threads(4);
  std::printf("max_num_threads %d\n", context.max_num_threads());
  context.ClearPrepackedCache();
  std::printf("advisory %d\n", context.performance_advisory(ruy::PerformanceAdvisory::kReallocatedPerChannelBuffer) ? 1 : 0);
  return 0;
}
