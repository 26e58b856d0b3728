// Plans: many independent muls submitted once and replayed (see ruyb200_plan_create).
#include <vector>

#include "common.cuh"
#include "plan.h"

using namespace ruyb200;

struct ruyb200_plan {
  ruyb200_ctx* ctx = nullptr;
  std::vector<ruyb200_mul_desc> descs;
  uint64_t bytes = 0;
  uint64_t ops = 0;
};

namespace {

size_t esize(int dtype) { return dtype == RUYB200_I8 || dtype == RUYB200_U8 ? 1 : (dtype == RUYB200_I16 ? 2 : 4); }

}  // namespace

extern "C" {

int ruyb200_plan_create(ruyb200_ctx* ctx, const ruyb200_mul_desc* descs, int n, ruyb200_plan** out) {
  if (!ctx || !out || n < 0 || (n > 0 && !descs)) return ctx_fail(RUYB200_ERR_INVALID, "bad argument");
  *out = nullptr;
  ruyb200_plan* plan = new ruyb200_plan;
  plan->ctx = ctx;
  plan->descs.assign(descs, descs + n);
  for (int i = 0; i < n; i++) {
    const ruyb200_mul_desc& d = descs[i];
    int rc = ctx_validate(&d);
    if (rc) {
      delete plan;
      return rc;
    }
    const void* ptrs[6] = {d.lhs.data, d.rhs.data, d.dst.data, d.params.bias, d.params.multiplier_fixedpoint_perchannel,
                           d.params.multiplier_exponent_perchannel};
    for (const void* p : ptrs) {
      if (p && !ptr_on_device(p)) {
        delete plan;
        return ctx_fail(RUYB200_ERR_INVALID, "plans need device pointers");
      }
    }
    const uint64_t r = d.lhs.rows, k = d.lhs.cols, c = d.rhs.cols;
    plan->ops += 2 * r * k * c;
    plan->bytes += r * k * esize(d.lhs.dtype) + k * c * esize(d.rhs.dtype) + r * c * esize(d.dst.dtype);
    const uint64_t nch = d.params.channel_dimension == RUYB200_CHANNEL_ROW ? r : c;
    if (d.params.bias) plan->bytes += 4 * nch;
    if (d.params.multiplier_fixedpoint_perchannel) plan->bytes += 8 * nch;
  }
  *out = plan;
  return RUYB200_OK;
}

int ruyb200_plan_run(ruyb200_plan* plan) {
  if (!plan) return ctx_fail(RUYB200_ERR_INVALID, "null plan");
  for (const ruyb200_mul_desc& d : plan->descs) {
    int rc = ctx_run_mul_async(plan->ctx, &d);
    if (rc) return rc;
  }
  return RUYB200_OK;
}

int ruyb200_plan_destroy(ruyb200_plan* plan) {
  delete plan;
  return RUYB200_OK;
}

int ruyb200_plan_stats(const ruyb200_plan* plan, uint64_t* bytes, uint64_t* ops) {
  if (!plan) return ctx_fail(RUYB200_ERR_INVALID, "null plan");
  if (bytes) *bytes = plan->bytes;
  if (ops) *ops = plan->ops;
  return RUYB200_OK;
}

}  // extern "C"
