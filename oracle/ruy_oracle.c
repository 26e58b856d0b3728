/* ruy_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C, single-threaded restatement of the arithmetic of ruy's matrix
 * multiplication, used only as the checker in tests, in the smoke test and as
 * the "port" CPU baseline of the benchmark.  Nothing in the shipped library
 * links, loads or calls this file.
 *
 * Parity status: PINNED.  The restatement is checked (tests/test_oracle.py)
 * against (1) the known-answer cases of ruy/apply_multiplier_test.cc:39-124 and
 * ruy/test_overflow_dst_zero_point.cc:46-125, parsed from the reference test
 * sources when they are present, (2) golden vectors under tests/golden/ that
 * were produced by running the compiled reference itself (ruy::ReferenceMul,
 * ruy::Mul on Path::kStandardCpp and on Path::kAvx512), and (3) the compiled
 * reference directly whenever oracle/_ref/libruy_ref.so exists.
 *
 * What each function follows:
 *   oracle_requant_reference  ruy/apply_multiplier.cc:48-65
 *   oracle_requant_x86        ruy/kernel_avx512.cc:340-465 (same results as
 *                             ruy/kernel_avx2_fma.cc:370-517)
 *   ruy_oracle_mul            ruy/reference_mul.h:29-52 with ApplyMultiplier
 *                             dispatch of ruy/apply_multiplier.h:55-88
 *   ruy_oracle_validate       ruy/validate.h:33-75
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#include "../include/ruy_b200.h"

#if defined(__GNUC__)
#define ORACLE_API __attribute__((visibility("default")))
#else
#define ORACLE_API
#endif

/* (int64(x)*m + 2^(30-e)) >> (31-e), arithmetic shift, result truncated to int32. */
ORACLE_API int32_t oracle_requant_reference(int32_t x, int32_t m, int e) {
  const int total_shift = 31 - e;
  const int64_t round = (int64_t)1 << (total_shift - 1);
  int64_t r = (int64_t)x * (int64_t)m + round;
  r >>= total_shift;
  return (int32_t)r;
}

/* Two-step rounding of the x86 kernels: left shift in int32 (wrapping), rounding
 * doubling high multiply, then a rounding right shift with an overflow guard. */
ORACLE_API int32_t oracle_requant_x86(int32_t x, int32_t m, int e) {
  const int ls = e > 0 ? e : 0;
  const int rs = e < 0 ? -e : 0;
  const int32_t a = (int32_t)((uint32_t)x << ls);
  const int32_t t = (int32_t)(((int64_t)a * (int64_t)m + ((int64_t)1 << 30)) >> 31);
  const int32_t nudge = rs > 0 ? (int32_t)((uint32_t)1 << (rs - 1)) : 0;
  if (t > INT32_MAX - nudge) {
    return (int32_t)((uint32_t)1 << (31 - rs));
  }
  return (t + nudge) >> rs;
}

static size_t elem_size(int dtype) {
  switch (dtype) {
    case RUYB200_I8:
    case RUYB200_U8:
      return 1;
    case RUYB200_I16:
      return 2;
    default:
      return 4;
  }
}

static size_t offset_of(const ruyb200_matrix* m, int r, int c) {
  return m->order == RUYB200_COL_MAJOR ? (size_t)c * (size_t)m->stride + (size_t)r
                                       : (size_t)r * (size_t)m->stride + (size_t)c;
}

static int32_t load_int(const ruyb200_matrix* m, int r, int c) {
  const char* p = (const char*)m->data + offset_of(m, r, c) * elem_size(m->dtype);
  switch (m->dtype) {
    case RUYB200_I8:
      return *(const int8_t*)p;
    case RUYB200_U8:
      return *(const uint8_t*)p;
    case RUYB200_I16:
      return *(const int16_t*)p;
    default:
      return *(const int32_t*)p;
  }
}

static int dtype_lowest(int dtype) {
  switch (dtype) {
    case RUYB200_I8:
      return -128;
    case RUYB200_U8:
      return 0;
    case RUYB200_I16:
      return -32768;
    default:
      return INT32_MIN;
  }
}

static int is_fp(int dtype) { return dtype == RUYB200_F32 || dtype == RUYB200_F64; }
static double load_fp(const ruyb200_matrix* m, int64_t off) {
  return m->dtype == RUYB200_F64 ? ((const double*)m->data)[off] : (double)((const float*)m->data)[off];
}

/* Returns 0 when ruy would accept the arguments (its checks are debug asserts). */
ORACLE_API int ruy_oracle_validate(const ruyb200_mul_desc* d) {
  const ruyb200_matrix* l = &d->lhs;
  const ruyb200_matrix* r = &d->rhs;
  const ruyb200_matrix* o = &d->dst;
  if (l->cols != r->rows || l->rows != o->rows || r->cols != o->cols) return -1;
  const int is_float = d->params.accum_dtype == RUYB200_F32;
  if (is_float) {
    if (l->dtype != RUYB200_F32 || r->dtype != RUYB200_F32 || o->dtype != RUYB200_F32) return -2;
    if (l->zero_point || r->zero_point || o->zero_point) return -1;
    return 0;
  }
  if (d->params.accum_dtype == RUYB200_F64) {
    /* ruy's mixed floating-point cases: (f64, f32, f64, f32) and (f32, f64, f64, f64), ruy/BUILD:1195-1207 */
    if (!is_fp(l->dtype) || !is_fp(r->dtype) || !is_fp(o->dtype)) return -2;
    if (l->zero_point || r->zero_point || o->zero_point) return -1;
    return 0;
  }
  if (is_fp(l->dtype) || is_fp(r->dtype) || is_fp(o->dtype)) return -2;
  if (l->dtype == RUYB200_I16 || r->dtype == RUYB200_I16) {
    if (l->zero_point || r->zero_point || o->zero_point) return -1;
  }
  if (!(l->dtype == RUYB200_U8 && r->dtype == RUYB200_U8)) {
    if (l->zero_point == dtype_lowest(l->dtype) && r->zero_point == dtype_lowest(r->dtype)) return -1;
  }
  return 0;
}

/* rounding: RUYB200_ROUNDING_REFERENCE or RUYB200_ROUNDING_X86.
 * wide_float: accumulate float muls in double and round once at the end (the
 * yardstick for the relative-error check) instead of float like ReferenceMul<float>. */
ORACLE_API int ruy_oracle_mul(const ruyb200_mul_desc* d, int rounding, int wide_float) {
  const ruyb200_matrix* L = &d->lhs;
  const ruyb200_matrix* R = &d->rhs;
  const ruyb200_matrix* D = &d->dst;
  const ruyb200_mul_params* P = &d->params;
  const int rc = ruy_oracle_validate(d);
  if (rc) return rc;
  const int rows = L->rows, depth = L->cols, cols = R->cols;
  const int chan_row = P->channel_dimension == RUYB200_CHANNEL_ROW;

  if (P->accum_dtype == RUYB200_F32) {
    const float* bias = (const float*)P->bias;
    for (int i = 0; i < rows; i++) {
      for (int j = 0; j < cols; j++) {
        const int ch = chan_row ? i : j;
        float out;
        if (wide_float) {
          double acc = 0;
          for (int k = 0; k < depth; k++) {
            acc += (double)((const float*)L->data)[offset_of(L, i, k)] *
                   (double)((const float*)R->data)[offset_of(R, k, j)];
          }
          if (bias) acc += (double)bias[ch];
          acc = acc < (double)P->clamp_max.f ? acc : (double)P->clamp_max.f;
          acc = acc > (double)P->clamp_min.f ? acc : (double)P->clamp_min.f;
          out = (float)acc;
        } else {
          float acc = 0;
          for (int k = 0; k < depth; k++) {
            acc += ((const float*)L->data)[offset_of(L, i, k)] *
                   ((const float*)R->data)[offset_of(R, k, j)];
          }
          if (bias) acc += bias[ch];
          acc = acc < P->clamp_max.f ? acc : P->clamp_max.f;
          acc = acc > P->clamp_min.f ? acc : P->clamp_min.f;
          out = acc;
        }
        ((float*)D->data)[offset_of(D, i, j)] = out;
      }
    }
    return 0;
  }

  if (P->accum_dtype == RUYB200_F64) {
    /* the standard C++ kernel with AccumScalar = double (ruy/kernel.h:211-237): operands widened to double,
     * summed in depth order, double bias, bounds applied in double, then the cast to the destination type */
    const double* bias64 = (const double*)P->bias;
    for (int i = 0; i < rows; i++) {
      for (int j = 0; j < cols; j++) {
        double acc = 0;
        for (int k = 0; k < depth; k++) acc += load_fp(L, offset_of(L, i, k)) * load_fp(R, offset_of(R, k, j));
        if (bias64) acc += bias64[chan_row ? i : j];
        acc = acc < P->clamp_max.d ? acc : P->clamp_max.d;
        acc = acc > P->clamp_min.d ? acc : P->clamp_min.d;
        if (D->dtype == RUYB200_F64) ((double*)D->data)[offset_of(D, i, j)] = acc;
        else ((float*)D->data)[offset_of(D, i, j)] = (float)acc;
      }
    }
    return 0;
  }

  const int32_t* bias = (const int32_t*)P->bias;
  for (int i = 0; i < rows; i++) {
    for (int j = 0; j < cols; j++) {
      uint32_t uacc = 0; /* int32 accumulation with defined wrap-around */
      for (int k = 0; k < depth; k++) {
        const int32_t lv = load_int(L, i, k) - L->zero_point;
        const int32_t rv = load_int(R, k, j) - R->zero_point;
        uacc += (uint32_t)(lv * rv);
      }
      const int ch = chan_row ? i : j;
      if (bias) uacc += (uint32_t)bias[ch];
      int32_t acc = (int32_t)uacc;
      if (D->dtype != RUYB200_I32) {
        int32_t m = P->multiplier_fixedpoint;
        int e = P->multiplier_exponent;
        if (P->multiplier_fixedpoint_perchannel) m = P->multiplier_fixedpoint_perchannel[ch];
        if (P->multiplier_exponent_perchannel) e = P->multiplier_exponent_perchannel[ch];
        acc = rounding == RUYB200_ROUNDING_X86 ? oracle_requant_x86(acc, m, e)
                                               : oracle_requant_reference(acc, m, e);
      }
      acc = (int32_t)((uint32_t)acc + (uint32_t)D->zero_point);
      if (D->dtype != RUYB200_I32) {
        acc = acc < P->clamp_max.i ? acc : P->clamp_max.i;
        acc = acc > P->clamp_min.i ? acc : P->clamp_min.i;
      }
      char* p = (char*)D->data + offset_of(D, i, j) * elem_size(D->dtype);
      switch (D->dtype) {
        case RUYB200_I8:
          *(int8_t*)p = (int8_t)acc;
          break;
        case RUYB200_U8:
          *(uint8_t*)p = (uint8_t)acc;
          break;
        case RUYB200_I16:
          *(int16_t*)p = (int16_t)acc;
          break;
        default:
          *(int32_t*)p = acc;
          break;
      }
    }
  }
  return 0;
}

/* Column sums of the TrMul view (ruy/pack.h:117-129 without padding): for side 0 (LHS)
 * sums[i] = sum_k lhs[i,k]; for side 1 (RHS) sums[j] = sum_k rhs[k,j]. */
ORACLE_API int ruy_oracle_sums(const ruyb200_matrix* m, int side, int32_t* sums) {
  const int width = side == 0 ? m->rows : m->cols;
  const int depth = side == 0 ? m->cols : m->rows;
  for (int w = 0; w < width; w++) {
    uint32_t s = 0;
    for (int k = 0; k < depth; k++) {
      s += (uint32_t)(side == 0 ? load_int(m, w, k) : load_int(m, k, w));
    }
    sums[w] = (int32_t)s;
  }
  return 0;
}
