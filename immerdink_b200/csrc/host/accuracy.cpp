// Error estimates of one configuration from operand statistics (never from data): the closed
// form documented with imd_err_estimate in the reference header (include/immerdink/
// immerdink_host.h:841-865; implementation src/host/accuracy.cpp:120-176):
//   E = 2 delta (nu_a + nu_b) s / d + 4 delta^2 k s^2 / d^2,  s = sqrt(1 + k 2^-60),
//   RN: delta = 1/2, d = T - kappa / 2;  TRUNC: delta = 1, d = T;  nu = min(l1 ratio, sqrt k).
// Every returned double is inflated by (1 + 2^-40) so that it is >= the exact real bound.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <limits>
#include <new>

#include "immerdink/immerdink_host.h"
#include "plan.hpp"

namespace {

constexpr double kUnit = 0x1p-53;
constexpr double kSlack = 1.0 + 0x1p-40;
constexpr double kTinyAbs = 0x1p-1071;  // gradual underflow of the final rounding and the few before it
constexpr double kInf = std::numeric_limits<double>::infinity();

struct Stats {
  int metric = IMD_ERR_NORMWISE, basis = IMD_ERR_BASIS_BOUND;
  double target = 0, cond = 1, norm_product = 1, l1a = 0, l1b = 0, fail_prob = 0;
};

bool finite_at_least(double v, double lo) { return std::isfinite(v) && v >= lo; }

bool read_request(const imd_err_request_t* r, Stats* s) {
  *s = Stats{};
  if (r == nullptr) return true;
  if (r->struct_size < sizeof(imd_err_request_t) || r->reserved != 0) return false;
  if (r->metric < IMD_ERR_NORMWISE || r->metric > IMD_ERR_ABSOLUTE) return false;
  if (!finite_at_least(r->target, 0)) return false;
  if (r->metric == IMD_ERR_ELEMENTWISE && !finite_at_least(r->cond, 1)) return false;
  if (r->metric == IMD_ERR_ABSOLUTE && !(std::isfinite(r->norm_product) && r->norm_product > 0))
    return false;
  if (!(r->l1_ratio_a == 0 || finite_at_least(r->l1_ratio_a, 1))) return false;
  if (!(r->l1_ratio_b == 0 || finite_at_least(r->l1_ratio_b, 1))) return false;
  if (r->basis != IMD_ERR_BASIS_BOUND && r->basis != IMD_ERR_BASIS_TYPICAL) return false;
  if (!(r->fail_prob == 0 || (r->fail_prob > 0 && r->fail_prob < 1))) return false;
  s->metric = r->metric, s->basis = r->basis, s->target = r->target, s->cond = r->cond;
  s->norm_product = r->norm_product, s->l1a = r->l1_ratio_a, s->l1b = r->l1_ratio_b;
  s->fail_prob = r->fail_prob;
  return true;
}

double metric_scale(const Stats& s) {
  return s.metric == IMD_ERR_ELEMENTWISE ? s.cond : s.metric == IMD_ERR_ABSOLUTE ? s.norm_product : 1.0;
}

// Coefficient E of ||a|| ||b|| -> bound in the metric; the final rounding adds E u + u.
double in_metric(const Stats& s, double E) {
  if (s.metric == IMD_ERR_ELEMENTWISE) {
    const double er = E * s.cond;
    return er + er * kUnit + kUnit;
  }
  const double n = E + E * kUnit + kUnit;
  return s.metric == IMD_ERR_ABSOLUTE ? n * s.norm_product : n;
}

double threshold_T(int N) {
  const imd::PlanConstants c = imd::plan_constants(N);
  double t = 0;
  for (int w = imd::kBigLimbs - 1; w >= 0; --w) t = t * 4294967296.0 + c.T.w[w];
  return t;
}

struct Estimate {
  double bound = 0, typical = 0, unit_bound = 0, unit_typical = 0;
  int status = IMD_ERR_UNCHECKED;
};

Estimate estimate(int N, int rounding, int dispatch, int64_t k, int64_t outputs, const Stats& s) {
  Estimate o;
  if (dispatch == IMD_DISPATCH_NOOP || dispatch == IMD_DISPATCH_SCALE || k <= 0) {
    // nothing is multiplied
  } else if (dispatch == IMD_DISPATCH_DIRECT) {
    const double ku = static_cast<double>(k) * kUnit;
    if (ku >= 0.5) {
      o.unit_bound = o.bound = kInf;
    } else {
      const double gk = ku / (1 - ku);
      o.unit_bound = gk * kSlack;
      o.bound = gk * metric_scale(s) * kSlack;
      if (s.metric == IMD_ERR_ABSOLUTE) o.bound += (static_cast<double>(k) + 16) * 0x1p-1074;
    }
    o.unit_typical = o.unit_bound, o.typical = o.bound;
  } else {
    const bool rn = rounding == IMD_RN;
    const uint64_t kappa = imd::ceil_sqrt_u64(static_cast<uint64_t>(k));
    if (rn && imd::kappa_at_least_T(kappa, N)) {
      o.unit_bound = o.bound = o.unit_typical = o.typical = kInf;
    } else {
      const double kd = static_cast<double>(k), T = threshold_T(N);
      const double delta = rn ? 0.5 : 1.0;
      const double d = rn ? T - 0.5 * static_cast<double>(kappa) : T;
      const double s2 = 1 + kd * 0x1p-60, sq = std::sqrt(s2), rk = std::sqrt(kd);
      const double na = s.l1a == 0 ? rk : std::min(s.l1a, rk);
      const double nb = s.l1b == 0 ? rk : std::min(s.l1b, rk);
      const double quad = 4 * delta * delta * kd * s2 / (d * d);
      const double E = 2 * delta * (na + nb) * sq / d + quad;
      o.unit_bound = E * kSlack;
      o.bound = in_metric(s, E) * kSlack;
      if (s.metric == IMD_ERR_ABSOLUTE) o.bound += kTinyAbs;
      if (rn) {
        const double M = static_cast<double>(std::max<int64_t>(outputs, 1));
        const double p = s.fail_prob > 0 ? s.fail_prob : 0x1p-40;
        const double h = sq / d * std::sqrt(8 * std::log(2 * M / p)) + quad;
        o.unit_typical = std::min(o.unit_bound, h);
        o.typical = std::min(o.bound, in_metric(s, o.unit_typical) +
                                          (s.metric == IMD_ERR_ABSOLUTE ? kTinyAbs : 0.0));
      } else {
        o.unit_typical = o.unit_bound, o.typical = o.bound;
      }
    }
  }
  if (s.target > 0) {
    const double v = s.basis == IMD_ERR_BASIS_TYPICAL ? o.typical : o.bound;
    o.status = v <= s.target ? IMD_ERR_MET : IMD_ERR_MISSED;
  }
  return o;
}

void write_out(imd_err_t* r, int N, int rounding, int dispatch, int64_t k, int64_t outputs,
               const Estimate& e) {
  r->num_moduli = N, r->rounding = rounding, r->dispatch = dispatch, r->k = k, r->outputs = outputs;
  r->bound = e.bound, r->typical = e.typical, r->unit_bound = e.unit_bound;
  r->unit_typical = e.unit_typical, r->err_status = e.status;
}

}  // namespace

extern "C" {

imd_status_t imd_err_estimate(int32_t num_moduli, int32_t rounding, int32_t dispatch, int64_t k,
                              int64_t outputs, const imd_err_request_t* request, imd_err_t* out) {
  if (out == nullptr || out->struct_size < sizeof(imd_err_t)) return IMD_STATUS_INVALID_VALUE;
  Stats s;
  if (num_moduli < imd::kMinModuli || num_moduli > imd::kMaxModuli ||
      (rounding != IMD_RN && rounding != IMD_TRUNC) || dispatch < IMD_DISPATCH_NOOP ||
      dispatch > IMD_DISPATCH_SCALE || k < 0 || outputs < 0 || !read_request(request, &s))
    return IMD_STATUS_INVALID_VALUE;
  imd_err_t r;
  std::memset(&r, 0, sizeof r);
  r.struct_size = out->struct_size;
  write_out(&r, num_moduli, rounding, dispatch, k, outputs,
            estimate(num_moduli, rounding, dispatch, k, outputs, s));
  r.status = IMD_STATUS_SUCCESS;
  std::memcpy(out, &r, std::min<size_t>(out->struct_size, sizeof r));
  return IMD_STATUS_SUCCESS;
}

imd_status_t imd_err_min_moduli(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                                const imd_options_t* options, int32_t n_lo, int32_t n_hi,
                                const imd_err_request_t* request, imd_err_t* out) {
  if (out == nullptr || out->struct_size < sizeof(imd_err_t) || options == nullptr ||
      request == nullptr)
    return IMD_STATUS_INVALID_VALUE;
  Stats s;
  if (!read_request(request, &s) || !(s.target > 0)) return IMD_STATUS_INVALID_VALUE;
  const int lo = n_lo == 0 ? imd::kMinModuli : n_lo, hi = n_hi == 0 ? imd::kMaxModuli : n_hi;
  if (lo < imd::kMinModuli || hi > imd::kMaxModuli || lo > hi) return IMD_STATUS_INVALID_VALUE;
  imd_err_t r;
  std::memset(&r, 0, sizeof r);
  r.struct_size = out->struct_size;
  int32_t st = IMD_STATUS_INVALID_VALUE;
  try {
    const imd_options_t& o = *options;
    if ((o.rounding != IMD_RN && o.rounding != IMD_TRUNC) ||
        (o.mode != IMD_EMULATE && o.mode != IMD_DIRECT) || A == nullptr || B == nullptr ||
        C == nullptr) {
      st = IMD_STATUS_INVALID_VALUE;
    } else {
      imd::GemmView v;
      st = imd::lower(*A, *B, *C, &v);
      if (st == IMD_STATUS_SUCCESS && o.mode == IMD_EMULATE && !v.empty_output() && v.k >= 2 &&
          (v.m > INT32_MAX || v.n > INT32_MAX - 15))
        st = IMD_STATUS_INVALID_VALUE;
      if (st == IMD_STATUS_SUCCESS) {
        const int dispatch = v.empty_output()                      ? IMD_DISPATCH_NOOP
                             : v.k == 0                            ? IMD_DISPATCH_SCALE
                             : (o.mode == IMD_DIRECT || v.k == 1)  ? IMD_DISPATCH_DIRECT
                                                                   : IMD_DISPATCH_EMULATE;
        const int64_t outputs = v.b * v.m * v.n;
        for (int N = lo; N <= hi; ++N) {
          const Estimate e = estimate(N, o.rounding, dispatch, v.k, outputs, s);
          if (e.status == IMD_ERR_MET || N == hi) {
            write_out(&r, N, o.rounding, dispatch, v.k, outputs, e);
            if (e.status == IMD_ERR_MET) {
              st = IMD_STATUS_SUCCESS;
            } else {
              r.num_moduli = 0;
              st = IMD_STATUS_NOT_SUPPORTED;
            }
            break;
          }
        }
      }
    }
  } catch (const std::bad_alloc&) {
    st = IMD_STATUS_ALLOC_FAILED;
  } catch (...) {
    st = IMD_STATUS_INVALID_VALUE;
  }
  if (st != IMD_STATUS_SUCCESS && st != IMD_STATUS_NOT_SUPPORTED) {
    std::memset(&r, 0, sizeof r);
    r.struct_size = out->struct_size;
  } else if (st == IMD_STATUS_NOT_SUPPORTED && r.err_status != IMD_ERR_MISSED) {
    // the lowering's own NOT_SUPPORTED: out zeroed, err_status UNCHECKED
    std::memset(&r, 0, sizeof r);
    r.struct_size = out->struct_size;
  }
  r.status = st;
  std::memcpy(out, &r, std::min<size_t>(out->struct_size, sizeof r));
  return static_cast<imd_status_t>(st);
}

}  // extern "C"
