// Performance model of this engine behind the reference's imd_perf_* interface (struct layouts,
// enum values, argument checks and ranking order: include/immerdink/immerdink_host.h:409-839 and
// src/host/perf.cpp:1499-1875 of the reference). The phases, their features and the shipped
// calibration describe THIS engine's kernels on a B200; see the header for the phase table.
// CUDA-free: everything is computed from the plan analysis.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <limits>
#include <string>
#include <vector>

#include "immerdink/immerdink_host.h"
#include "pack.hpp"
#include "perf_text.hpp"
#include "plan.hpp"

namespace imd {
namespace {

constexpr int kP = IMD_PERF_MAX_PARAMS;
constexpr int kGemmByteSlot = 4;
// A tile's epilogue (tensor memory -> residues mod p -> u8 stores) takes as long as the main loop
// over about this many K bytes; shorter main loops do not hide it.
constexpr int64_t kGemmEpilogueK = 1536;

// Struct sizes of the interface versions (fields are only ever appended).
constexpr uint32_t kRequestV1 = offsetof(imd_perf_request_t, regime);
constexpr uint32_t kRequestV7 = offsetof(imd_perf_request_t, accuracy);
constexpr uint32_t kRequestV8 = sizeof(imd_perf_request_t);
constexpr uint32_t kPerfV1 = offsetof(imd_perf_t, regime);
constexpr uint32_t kRankV1 = offsetof(imd_perf_rank_request_t, regime);
constexpr uint32_t kRankV7 = offsetof(imd_perf_rank_request_t, accuracy);
constexpr uint32_t kRankV8 = sizeof(imd_perf_rank_request_t);
constexpr uint32_t kCandidateV1 = offsetof(imd_perf_candidate_t, time_lo_s);
static_assert(sizeof(imd_perf_phase_t) == 96 && kPerfV1 == 1648 && sizeof(imd_perf_t) == 1976,
              "imd_perf_t layout");
static_assert(sizeof(imd_perf_calib_t) == 3744 && offsetof(imd_perf_calib_t, kernel) == 1232,
              "imd_perf_calib_t layout");
static_assert(kRequestV1 == 24 && kRequestV7 == 40 && kRequestV8 == 48, "imd_perf_request_t");
static_assert(kRankV1 == 64 && kRankV7 == 88 && kRankV8 == 96, "imd_perf_rank_request_t");
static_assert(kCandidateV1 == 128 && sizeof(imd_perf_candidate_t) == 192, "imd_perf_candidate_t");

template <class F>
imd_status_t guarded(F&& f) {
  try {
    return f();
  } catch (const std::bad_alloc&) {
    return IMD_STATUS_ALLOC_FAILED;
  } catch (...) {
    return IMD_STATUS_INVALID_VALUE;
  }
}

double d(int64_t v) { return static_cast<double>(v); }
int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- phases ---------------------------------------------------------------------------------
struct Phase {
  int32_t phase = 0, cls = 0;
  int64_t launches = 0;
  double bytes = 0, ops = 0;
  int peak = 0;  // bound: 0 DRAM only, 1 int8 ops, 2 FP64 flops
  double x[kP] = {0, 0, 0, 0, 0, 0};
};
struct Phases {
  std::vector<Phase> list;
  int64_t launches = 0;
  Phase& add(int32_t phase, int32_t cls, int64_t launches_) {
    Phase p;
    p.phase = phase, p.cls = cls, p.launches = launches_;
    launches += launches_;
    list.push_back(p);
    return list.back();
  }
};

// The GEMM launches of a plan as the kernels run them (gemm_tcgen05.cu): CTA pairs on 256 x 256
// tiles when m > 128, else one CTA per 128 x 256 tile; persistent over planes x tiles; K in blocks
// of 128; tile rows walked in bands sized to 32 MB of A (B is re-read once per band).
// Features: x[0] "round" = tile rounds whose main loop is too short to hide the epilogue, x[1]
// "mac1" = MACs of the busiest SM over the other rounds (tile padding included), x[4] "byte" =
// modelled DRAM bytes. The launches themselves are in the call class.
void gemm_features(const ExecPlan& e, int sms, Phase* p) {
  const bool pair = e.m > 128;
  const int64_t tile_m = pair ? 256 : 128, tile_n = 256;
  const int64_t units = std::max<int64_t>(pair ? sms / 2 : sms, 1);
  const int64_t tiles_m = ceil_div(e.m, tile_m), tiles_n = ceil_div(e.n_hat, tile_n);
  double macs = 0, dram = 0, short_rounds = 0;
  int64_t launches = 0;
  for (int g0 = 0; g0 < e.N; g0 += e.g) {
    const int64_t mods = std::min<int64_t>(e.g, e.N - g0);
    for (int64_t c = 0; c < e.k_chunks; ++c) {
      const int64_t k0 = c * kChunk, klen = std::min<int64_t>(kChunk, e.k_hat - k0);
      const int64_t k_blocks = ceil_div(klen, 128);
      const int64_t planes = mods * e.b;
      const int64_t rounds = ceil_div(planes * tiles_m * tiles_n, units);
      if (k_blocks * 128 >= kGemmEpilogueK) macs += d(rounds) * 128.0 * d(tile_n) * d(k_blocks * 128);
      else short_rounds += d(rounds);
      int64_t band = (int64_t{32} << 20) / std::max<int64_t>(tile_m * klen, 1);
      band = std::min(std::max<int64_t>(band, 4), tiles_m);
      const int64_t bands = ceil_div(tiles_m, std::max<int64_t>(band, 1));
      dram += d(planes) * (d(e.m) * d(klen) + d(e.n_hat) * d(klen) * d(bands) +
                           d(e.m) * d(e.n_hat) * (c > 0 ? 2.0 : 1.0));
      ++launches;
    }
  }
  p->launches = launches;
  p->x[0] = short_rounds;
  p->x[1] = macs;
  p->x[kGemmByteSlot] = dram;
  p->ops = 2.0 * d(e.N) * d(e.b) * d(e.m) * d(e.n) * d(e.k);
  p->bytes = d(e.N) * d(e.b) * ((d(e.m) + d(e.n_hat)) * d(e.k_hat) + d(e.m) * d(e.n_hat));
  p->peak = 1;
}

void contract_phases(const Analysis& an, const ExecPlan& e, int32_t flags, int sms, Phases* P) {
  if (e.path == Path::kNoop) return;
  const double outputs = d(e.b) * d(e.m) * d(e.n);
  const double c_bytes = 8.0 * outputs * ((flags & IMD_PERF_BETA_NONZERO) ? 2.0 : 1.0);
  if (!e.vec_resident) {
    Phase& p = P->add(IMD_PERF_PHASE_K0, IMD_PERF_CLASS_K0, 1);
    p.bytes = 8.0 * d(an.view.vec_entries());
    p.x[0] = 1, p.x[1] = p.bytes;
  }
  const bool scale_only = (flags & IMD_PERF_ALPHA_ZERO) || e.k == 0;
  if (scale_only) {
    Phase& p = P->add(IMD_PERF_PHASE_BETA, IMD_PERF_CLASS_BETA, 1);
    p.bytes = c_bytes;
    p.x[0] = 1, p.x[1] = p.bytes;
  } else if (!e.emulated()) {
    Phase& p = P->add(IMD_PERF_PHASE_DIRECT, IMD_PERF_CLASS_DIRECT, 1);
    p.bytes = 8.0 * d(e.b) * d(e.k) * (d(e.m) + d(e.n)) + c_bytes;
    p.ops = 2.0 * outputs * d(e.k);
    p.peak = 2;
    p.x[0] = 1, p.x[1] = p.bytes, p.x[2] = p.ops;
  } else if (e.small()) {
    // one fused launch: every 32 x 32 tile quantises its 64 rows of kh entries for N moduli,
    // multiplies them and runs the CRT of its outputs
    Phase& p = P->add(IMD_PERF_PHASE_KF, IMD_PERF_CLASS_KF, 1);
    const double tiles = d(ceil_div(e.m, 32)) * d(ceil_div(e.n, 32)) * d(e.b);
    const double kh = d(ceil_div(e.k, 32) * 32);
    p.bytes = 8.0 * d(e.b) * d(e.k) * (d(e.m) + d(e.n)) + c_bytes;
    p.ops = 2.0 * d(e.N) * outputs * d(e.k);
    p.x[0] = 1, p.x[1] = p.bytes, p.x[2] = tiles * 64.0 * kh * d(e.N), p.x[3] = tiles * 1024.0 * d(e.N);
    // what one SM does one tile after the other (a tile is not shared between SMs)
    p.x[5] = d(ceil_div(static_cast<int64_t>(tiles), std::max(sms, 1))) * 64.0 * kh * d(e.N);
  } else {
    const int64_t groups = ceil_div(e.N, e.g);
    const int64_t rows[2] = {e.m, e.n}, rows_pad[2] = {e.m, e.n_hat};
    const int32_t scale_phase[2] = {IMD_PERF_PHASE_KL_A, IMD_PERF_PHASE_KL_B};
    const int32_t res_phase[2] = {IMD_PERF_PHASE_PACK_A, IMD_PERF_PHASE_PACK_B};
    for (int x = 0; x < 2; ++x) {
      if ((e.packed >> x) & 1) continue;
      // only an operand that is contiguous along its rows has a scale launch of its own; the
      // others get their shifts inside the first quantise launch (the phase stays, empty)
      const bool own = e.rows_fast[x];
      Phase& p = P->add(scale_phase[x], IMD_PERF_CLASS_KL, own ? 1 : 0);
      const double elems = own ? d(e.b) * d(rows[x]) * d(e.k) : 0.0;
      p.bytes = 8.0 * elems;
      p.x[0] = own ? 1 : 0, p.x[1] = p.bytes, p.x[2] = elems;
    }
    for (int x = 0; x < 2; ++x) {
      if ((e.packed >> x) & 1) continue;
      Phase& p = P->add(res_phase[x], IMD_PERF_CLASS_PACK, groups);
      const double elems = d(e.b) * d(rows[x]) * d(e.k);
      p.bytes = 8.0 * elems * d(groups) + d(e.N) * d(e.b) * d(rows_pad[x]) * d(e.k_hat);
      p.x[0] = d(groups), p.x[1] = p.bytes, p.x[2] = elems * d(e.N), p.x[4] = elems * d(groups);
      p.x[3] = e.rows_fast[x] ? 0.0 : elems;  // the scan of the fused first launch (shift of the rows)
    }
    gemm_features(e, sms, &P->add(IMD_PERF_PHASE_K4, IMD_PERF_CLASS_K4_128x256, 0));
    P->launches += P->list.back().launches;
    Phase& p = P->add(IMD_PERF_PHASE_K5, IMD_PERF_CLASS_K5, 1);
    p.bytes = d(e.N) * d(e.b) * d(e.m) * d(e.n_hat) + c_bytes;
    p.x[0] = 1, p.x[1] = p.bytes, p.x[2] = outputs * d(e.N);
  }
  Phase& call = P->add(IMD_PERF_PHASE_CALL, IMD_PERF_CLASS_CALL, 0);
  call.x[0] = 1, call.x[1] = d(P->launches);
}

void pack_phases(const PackLowered& pl, Phases* P) {
  if (pl.layout.total == 0) return;
  const double elems = d(pl.b) * d(pl.r) * d(pl.k);
  Phase& prep = P->add(IMD_PERF_PHASE_PACK_PREP, IMD_PERF_CLASS_K0, 2);
  prep.bytes = 8.0 * (d(pl.r) + d(pl.k) + d(pl.b));
  prep.x[0] = 2, prep.x[1] = prep.bytes;
  ExecPlan e;
  pack_exec(pl, &e);
  const bool own = e.rows_fast[0];  // as in contract_phases
  Phase& sc = P->add(IMD_PERF_PHASE_PACK_KL, IMD_PERF_CLASS_KL, own ? 1 : 0);
  sc.bytes = own ? 8.0 * elems : 0.0;
  sc.x[0] = own ? 1 : 0, sc.x[1] = sc.bytes, sc.x[2] = own ? elems : 0.0;
  Phase& rs = P->add(IMD_PERF_PHASE_PACK_A, IMD_PERF_CLASS_PACK, 1);
  rs.bytes = 8.0 * elems + static_cast<double>(pl.layout.bytes[kPackRes]);
  rs.x[0] = 1, rs.x[1] = rs.bytes, rs.x[2] = elems * d(pl.N), rs.x[4] = elems;
  rs.x[3] = own ? 0.0 : elems;
  Phase& call = P->add(IMD_PERF_PHASE_CALL, IMD_PERF_CLASS_CALL, 0);
  call.x[0] = 1, call.x[1] = d(P->launches);
}

double phase_seconds(const imd_perf_calib_t& cal, const Phase& p) {
  const double* th = &cal.param[p.cls * kP];
  double t = 0;
  const bool gemm = p.cls >= IMD_PERF_CLASS_K4_128x256 && p.cls <= IMD_PERF_CLASS_K4_64x64;
  for (int j = 0; j < kP; ++j)
    if (!(gemm && j == kGemmByteSlot)) t += th[j] * p.x[j];
  if (gemm) t = std::max(t, th[kGemmByteSlot] * p.x[kGemmByteSlot]);
  return t * 1e-9;
}

// ---- requests -------------------------------------------------------------------------------
struct Req {
  int32_t flags = 0, regime = IMD_PERF_REGIME_DEFAULT, cache = IMD_PERF_CACHE_COLD;
  double clock = 0;
  const imd_err_request_t* accuracy = nullptr;
};

bool eps_valid(double f) { return f < 0 || (f >= 0 && f <= 1); }
bool v7_valid(int32_t regime, int32_t cache, double clock) {
  return regime >= IMD_PERF_REGIME_DEFAULT && regime <= IMD_PERF_REGIME_SUSTAINED &&
         cache >= IMD_PERF_CACHE_COLD && cache <= IMD_PERF_CACHE_CLEAN && std::isfinite(clock) &&
         clock >= 0;
}
// An accuracy request is valid iff imd_err_estimate accepts it.
bool accuracy_valid(const imd_err_request_t* a) {
  if (a == nullptr) return true;
  imd_err_t probe;
  std::memset(&probe, 0, sizeof probe);
  probe.struct_size = sizeof probe;
  return imd_err_estimate(14, IMD_RN, IMD_DISPATCH_EMULATE, 2, 1, a, &probe) == IMD_STATUS_SUCCESS;
}
bool request_valid(const imd_perf_request_t* req, Req* q) {
  *q = Req{};
  if (req == nullptr) return true;
  if (req->struct_size < kRequestV1) return false;
  if ((req->flags & ~(IMD_PERF_BETA_NONZERO | IMD_PERF_ALPHA_ZERO)) != 0) return false;
  if (req->k4_config < -1 || req->k4_config >= IMD_K4_CONFIG_COUNT) return false;
  if (!eps_valid(req->eps_fraction)) return false;
  q->flags = req->flags;
  if (req->struct_size >= kRequestV7) {
    if (!v7_valid(req->regime, req->cache, req->clock_mhz)) return false;
    q->regime = req->regime, q->cache = req->cache, q->clock = req->clock_mhz;
  }
  if (req->struct_size >= kRequestV8) {
    if (!accuracy_valid(req->accuracy)) return false;
    q->accuracy = req->accuracy;
  }
  return true;
}

int band_of(double t) {
  return t < 100e-6 ? IMD_PERF_BAND_SMALL : t < 1e-3 ? IMD_PERF_BAND_MID : IMD_PERF_BAND_LARGE;
}

void fill(const imd_perf_calib_t& cal, const Phases& P, const Req& q, imd_perf_t* r) {
  const int n = static_cast<int>(std::min<size_t>(P.list.size(), IMD_PERF_MAX_PHASES));
  r->num_phases = n;
  r->k4_config = IMD_K4_128x256;
  r->sm_count = cal.sm_count;
  r->kernel_launches = P.launches;
  double t = 0, bound = 0;
  for (int i = 0; i < n; ++i) {
    const Phase& p = P.list[static_cast<size_t>(i)];
    imd_perf_phase_t& o = r->phase[i];
    o.phase = p.phase, o.cls = p.cls, o.launches = p.launches;
    o.time_s = phase_seconds(cal, p);
    o.bytes = p.bytes, o.ops = p.ops;
    const double peak = p.peak == 1 ? cal.peak_int8_ops_per_s
                        : p.peak == 2 ? cal.peak_fp64_flops_per_s : 0.0;
    o.bound_s = std::max(cal.peak_dram_bytes_per_s > 0 ? p.bytes / cal.peak_dram_bytes_per_s : 0.0,
                         peak > 0 ? p.ops / peak : 0.0);
    for (int j = 0; j < kP; ++j) o.x[j] = p.x[j];
    const bool call = p.cls == IMD_PERF_CLASS_CALL;
    r->phase_lo_s[i] = call ? o.time_s : o.time_s * cal.band_class[p.cls][0];
    r->phase_hi_s[i] = call ? o.time_s : o.time_s * cal.band_class[p.cls][1];
    t += o.time_s;
    bound += o.bound_s;
  }
  r->time_s = t, r->bound_s = bound;
  r->tflops_eq = t > 0 ? r->flops_eq / t * 1e-12 : 0;
  const double* bc = cal.band_call[band_of(t)];
  r->time_lo_s = t * bc[0], r->time_hi_s = t * bc[1];
  r->regime = IMD_PERF_REGIME_BURST;  // no power model: SUSTAINED = BURST
  r->cache = q.cache;
  r->clock_mhz = cal.clock_eff_mhz;
  r->power_w = 0, r->warm_bytes = 0;
}

imd_status_t analyze_packing(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                             const imd_options_t* options, const imd_packing_t* packing,
                             Analysis* an) {
  if (const imd_status_t st = analyze(A, B, C, options, an); st != IMD_STATUS_SUCCESS) return st;
  if (packing == nullptr || (packing->A == nullptr && packing->B == nullptr))
    return IMD_STATUS_SUCCESS;
  const imd_pack_desc_t* pd[2] = {packing->A, packing->B};
  PackLowered pl[2];
  PackSource ps[2];
  const PackSource* src[2] = {nullptr, nullptr};
  for (int x = 0; x < 2; ++x) {
    if (pd[x] == nullptr) continue;
    if (const imd_status_t st = pack_lower(*pd[x], &pl[x]); st != IMD_STATUS_SUCCESS) return st;
    ps[x] = PackSource{pd[x]->tensor->rank, pd[x]->tensor->label, &pl[x]};
    src[x] = &ps[x];
  }
  return match_packs(A, B, src, an);
}

imd_status_t predict_contract(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                              const imd_options_t* options, const imd_packing_t* packing,
                              const Req& q, const imd_perf_calib_t& cal, imd_perf_t* r) {
  Analysis an;
  if (const imd_status_t st = analyze_packing(A, B, C, options, packing, &an);
      st != IMD_STATUS_SUCCESS)
    return st;
  ExecPlan e;
  if (const imd_status_t st = make_plan(an, &e); st != IMD_STATUS_SUCCESS) return st;
  Phases P;
  contract_phases(an, e, q.flags, cal.sm_count, &P);
  r->dispatch = e.path == Path::kNoop ? IMD_DISPATCH_NOOP
                : e.k == 0            ? IMD_DISPATCH_SCALE
                : e.emulated()        ? IMD_DISPATCH_EMULATE
                                      : IMD_DISPATCH_DIRECT;
  r->workspace_bytes = an.layout.total;
  r->plan_device_bytes = e.vec_resident ? e.device_bytes : 0;
  r->flops_eq = 2.0 * d(e.b) * d(e.m) * d(e.n) * d(e.k);
  fill(cal, P, q, r);
  imd_err_t err;
  std::memset(&err, 0, sizeof err);
  err.struct_size = sizeof err;
  const int64_t outputs = e.b * e.m * e.n;
  if (imd_err_estimate(e.N, options->rounding, r->dispatch, e.k, outputs, q.accuracy, &err) ==
      IMD_STATUS_SUCCESS) {
    r->err_bound = err.bound, r->err_typical = err.typical, r->err_status = err.err_status;
  } else {
    r->err_bound = r->err_typical = std::numeric_limits<double>::infinity();
    r->err_status = IMD_ERR_UNCHECKED;
  }
  r->err_metric = q.accuracy != nullptr ? q.accuracy->metric : IMD_ERR_NORMWISE;
  return IMD_STATUS_SUCCESS;
}

imd_status_t predict_pack(const imd_pack_desc_t& desc, const Req& q, const imd_perf_calib_t& cal,
                          imd_perf_t* r) {
  PackLowered pl;
  if (const imd_status_t st = pack_lower(desc, &pl); st != IMD_STATUS_SUCCESS) return st;
  Phases P;
  pack_phases(pl, &P);
  r->dispatch = IMD_DISPATCH_EMULATE;
  r->pack_bytes = pl.layout.total;
  r->pack_ws_bytes = pl.ws_bytes;
  fill(cal, P, q, r);
  return IMD_STATUS_SUCCESS;
}

imd_status_t finish(imd_perf_t& r, imd_perf_t* out) {
  if (r.status != IMD_STATUS_SUCCESS) {
    const uint32_t size = r.struct_size;
    const int32_t st = r.status;
    std::memset(&r, 0, sizeof r);
    r.struct_size = size, r.status = st;
  }
  std::memcpy(out, &r, std::min<size_t>(out->struct_size, sizeof r));
  return static_cast<imd_status_t>(r.status);
}

bool add_u64(uint64_t a, uint64_t b, uint64_t* out) {
  if (a > UINT64_MAX - b) return false;
  *out = a + b;
  return true;
}

}  // namespace
}  // namespace imd

// ---- C ABI ------------------------------------------------------------------------------------
namespace {

using imd::CalibError;

constexpr uint32_t kCalibV1 = offsetof(imd_perf_calib_t, kernel);
constexpr uint32_t kErrorMin = 16;

// NULL: the shipped calibration. Else a copy of the caller's struct_size bytes over zeros (an
// older, shorter struct keeps the appended fields 0), which must be a valid format-2 calibration.
imd_status_t resolve(const imd_perf_calib_t* in, imd_perf_calib_t* scratch,
                     const imd_perf_calib_t** out) {
  if (in == nullptr) {
    *out = imd::perf_calib_shipped(nullptr);
    return *out != nullptr ? IMD_STATUS_SUCCESS : IMD_STATUS_INVALID_VALUE;
  }
  if (in->struct_size < kCalibV1) return IMD_STATUS_INVALID_VALUE;
  std::memset(scratch, 0, sizeof *scratch);
  std::memcpy(scratch, in, std::min<size_t>(in->struct_size, sizeof *scratch));
  if (in->struct_size <= kCalibV1) {  // no occupancy, bands or tie ratio in that layout
    for (auto& k : scratch->kernel) k = imd_perf_kernel_t{1, 0, 0, 256};
    for (auto& b : scratch->band_call) b[0] = b[1] = 1;
    for (auto& b : scratch->band_class) b[0] = b[1] = 1;
    scratch->tie_ratio = 1;
  }
  if (!imd::perf_calib_valid(*scratch)) return IMD_STATUS_INVALID_VALUE;
  *out = scratch;
  return IMD_STATUS_SUCCESS;
}

void store_error(imd_perf_calib_error_t* err, const CalibError& e) {
  if (err == nullptr) return;
  imd_perf_calib_error_t r;
  std::memset(&r, 0, sizeof r);
  r.struct_size = err->struct_size;
  r.line = e.line, r.reason = e.reason;
  std::snprintf(r.key, sizeof r.key, "%s", e.key.c_str());
  std::snprintf(r.message, sizeof r.message, "%s", e.message.c_str());
  std::memcpy(err, &r, std::min<size_t>(err->struct_size, sizeof r));
}

bool out_ok(const imd_perf_calib_t* out, const imd_perf_calib_error_t* err) {
  return out != nullptr && out->struct_size >= kCalibV1 && (err == nullptr || err->struct_size >= kErrorMin);
}

void store_calib(const imd_perf_calib_t& c, imd_perf_calib_t* out) {
  const uint32_t size = out->struct_size;
  std::memcpy(out, &c, std::min<size_t>(size, sizeof c));
  out->struct_size = size;
}

imd_status_t parse_into(std::string_view text, imd_perf_calib_t* out, imd_perf_calib_error_t* err) {
  CalibError e;
  imd_perf_calib_t c;
  const imd_status_t st = imd::perf_calib_parse(text, &c, &e);
  if (st == IMD_STATUS_SUCCESS) store_calib(c, out);
  store_error(err, e);
  return st;
}

imd_status_t argument_error(imd_perf_calib_error_t* err) {
  if (err != nullptr && err->struct_size >= kErrorMin) {
    CalibError e;
    e.reason = IMD_PERF_CALIB_ERR_ARGUMENT;
    e.message = "NULL or undersized argument";
    store_error(err, e);
  }
  return IMD_STATUS_INVALID_VALUE;
}

}  // namespace

extern "C" {

const char* imd_perf_kernel_name(int32_t kernel) { return imd::perf_kernel_name(kernel); }
const char* imd_perf_class_name(int32_t cls) { return imd::perf_class_name(cls); }
const char* imd_perf_param_name(int32_t cls, int32_t j) { return imd::perf_param_name(cls, j); }
const char* imd_perf_phase_name(int32_t phase) { return imd::perf_phase_name(phase); }
const char* imd_perf_calib_error_name(int32_t reason) { return imd::perf_calib_error_name(reason); }

imd_status_t imd_perf_calib_default_ex(imd_perf_calib_t* out, imd_perf_calib_error_t* err) {
  if (!out_ok(out, err)) return argument_error(err);
  return imd::guarded([&]() -> imd_status_t {
    CalibError e;
    const imd_perf_calib_t* c = imd::perf_calib_shipped(&e);
    if (c != nullptr) store_calib(*c, out);
    store_error(err, e);
    return c != nullptr ? IMD_STATUS_SUCCESS : IMD_STATUS_INVALID_VALUE;
  });
}
imd_status_t imd_perf_calib_default(imd_perf_calib_t* out) {
  return imd_perf_calib_default_ex(out, nullptr);
}

imd_status_t imd_perf_calib_parse_ex(const char* text, size_t length, imd_perf_calib_t* out,
                                     imd_perf_calib_error_t* err) {
  if (text == nullptr || !out_ok(out, err)) return argument_error(err);
  return imd::guarded([&] { return parse_into(std::string_view(text, length), out, err); });
}
imd_status_t imd_perf_calib_parse(const char* text, size_t length, imd_perf_calib_t* out,
                                  int32_t* error_line) {
  imd_perf_calib_error_t e;
  std::memset(&e, 0, sizeof e);
  e.struct_size = sizeof e;
  const imd_status_t st = imd_perf_calib_parse_ex(text, length, out, &e);
  if (error_line != nullptr) *error_line = e.line;
  return st;
}

imd_status_t imd_perf_calib_load_ex(const char* path, imd_perf_calib_t* out,
                                    imd_perf_calib_error_t* err) {
  if (path == nullptr || !out_ok(out, err)) return argument_error(err);
  return imd::guarded([&]() -> imd_status_t {
    std::string text;
    bool ok = false;
    if (std::FILE* f = std::fopen(path, "rb")) {
      char buf[4096];
      size_t n;
      ok = true;
      while ((n = std::fread(buf, 1, sizeof buf, f)) > 0) {
        text.append(buf, n);
        if (text.size() >= (size_t{1} << 20)) {
          ok = false;
          break;
        }
      }
      ok = ok && std::ferror(f) == 0;
      std::fclose(f);
    }
    if (!ok) {
      CalibError e;
      e.reason = IMD_PERF_CALIB_ERR_FILE;
      e.message = "cannot open or read the file, or it is 1 MiB or more";
      store_error(err, e);
      return IMD_STATUS_INVALID_VALUE;
    }
    return parse_into(text, out, err);
  });
}
imd_status_t imd_perf_calib_load(const char* path, imd_perf_calib_t* out, int32_t* error_line) {
  imd_perf_calib_error_t e;
  std::memset(&e, 0, sizeof e);
  e.struct_size = sizeof e;
  const imd_status_t st = imd_perf_calib_load_ex(path, out, &e);
  if (error_line != nullptr) *error_line = e.line;
  return st;
}

imd_status_t imd_perf_calib_format(const imd_perf_calib_t* calib, char* buf, size_t capacity,
                                   size_t* length) {
  if (length == nullptr || (buf == nullptr && capacity > 0)) return IMD_STATUS_INVALID_VALUE;
  return imd::guarded([&]() -> imd_status_t {
    imd_perf_calib_t scratch;
    const imd_perf_calib_t* c = nullptr;
    if (const imd_status_t st = resolve(calib, &scratch, &c); st != IMD_STATUS_SUCCESS) return st;
    const std::string s = imd::perf_calib_format(*c);
    *length = s.size();
    if (capacity <= s.size()) return IMD_STATUS_INSUFFICIENT_WORKSPACE;
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return IMD_STATUS_SUCCESS;
  });
}

imd_status_t imd_perf_predict(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                              const imd_options_t* options, const imd_packing_t* packing,
                              const imd_perf_request_t* request, const imd_perf_calib_t* calib,
                              imd_perf_t* out) {
  if (out == nullptr || out->struct_size < imd::kPerfV1) return IMD_STATUS_INVALID_VALUE;
  imd::Req q;
  if (!imd::request_valid(request, &q)) return IMD_STATUS_INVALID_VALUE;
  imd_perf_t r;
  std::memset(&r, 0, sizeof r);
  r.struct_size = out->struct_size;
  r.status = imd::guarded([&]() -> imd_status_t {
    imd_perf_calib_t scratch;
    const imd_perf_calib_t* cal = nullptr;
    if (const imd_status_t st = resolve(calib, &scratch, &cal); st != IMD_STATUS_SUCCESS) return st;
    return imd::predict_contract(A, B, C, options, packing, q, *cal, &r);
  });
  return imd::finish(r, out);
}

imd_status_t imd_perf_predict_pack(const imd_pack_desc_t* desc, const imd_perf_request_t* request,
                                   const imd_perf_calib_t* calib, imd_perf_t* out) {
  if (desc == nullptr || out == nullptr || out->struct_size < imd::kPerfV1)
    return IMD_STATUS_INVALID_VALUE;
  imd::Req q;
  if (!imd::request_valid(request, &q)) return IMD_STATUS_INVALID_VALUE;
  q.flags = 0;
  imd_perf_t r;
  std::memset(&r, 0, sizeof r);
  r.struct_size = out->struct_size;
  r.status = imd::guarded([&]() -> imd_status_t {
    imd_perf_calib_t scratch;
    const imd_perf_calib_t* cal = nullptr;
    if (const imd_status_t st = resolve(calib, &scratch, &cal); st != IMD_STATUS_SUCCESS) return st;
    return imd::predict_pack(*desc, q, *cal, &r);
  });
  return imd::finish(r, out);
}

imd_status_t imd_perf_rank(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                           const imd_options_t* base, const imd_perf_rank_request_t* req,
                           const imd_perf_calib_t* calib, imd_perf_candidate_t* out,
                           int32_t capacity, int32_t* num_candidates) {
  using namespace imd;
  if (A == nullptr || B == nullptr || C == nullptr || base == nullptr || req == nullptr ||
      num_candidates == nullptr || req->struct_size < kRankV1 || capacity < 0 ||
      (capacity > 0 && (out == nullptr || req->candidate_size < kCandidateV1)))
    return IMD_STATUS_INVALID_VALUE;
  if (req->num_moduli_count < 1 || req->num_moduli == nullptr || req->residue_group_count < 0 ||
      (req->residue_group_count > 0 && req->residue_groups == nullptr) || req->reuse < 1 ||
      (req->vec_modes & ~(IMD_PERF_VEC_GENERATE | IMD_PERF_VEC_RESIDENT)) != 0 ||
      (req->pack_modes &
       ~(IMD_PERF_PACK_NONE | IMD_PERF_PACK_A | IMD_PERF_PACK_B | IMD_PERF_PACK_AB)) != 0 ||
      (req->flags & ~IMD_PERF_BETA_NONZERO) != 0 || !eps_valid(req->eps_fraction))
    return IMD_STATUS_INVALID_VALUE;
  Req q;
  q.flags = req->flags;
  int32_t order = IMD_PERF_ORDER_TIME;
  if (req->struct_size >= kRankV7) {
    if (!v7_valid(req->regime, req->cache, req->clock_mhz) ||
        (req->order != IMD_PERF_ORDER_TIME && req->order != IMD_PERF_ORDER_TIES_BY_FOOTPRINT))
      return IMD_STATUS_INVALID_VALUE;
    q.regime = req->regime, q.cache = req->cache, q.clock = req->clock_mhz;
    order = req->order;
  }
  if (req->struct_size >= kRankV8) {
    if (!accuracy_valid(req->accuracy)) return IMD_STATUS_INVALID_VALUE;
    q.accuracy = req->accuracy;
  }
  for (int32_t i = 0; i < req->num_moduli_count; ++i)
    if (req->num_moduli[i] < 2 || req->num_moduli[i] > kMaxModuli) return IMD_STATUS_INVALID_VALUE;
  for (int32_t i = 0; i < req->residue_group_count; ++i)
    if (req->residue_groups[i] < 1) return IMD_STATUS_INVALID_VALUE;
  return guarded([&]() -> imd_status_t {
    imd_perf_calib_t scratch;
    const imd_perf_calib_t* cal = nullptr;
    if (const imd_status_t st = resolve(calib, &scratch, &cal); st != IMD_STATUS_SUCCESS) return st;
    const int32_t vec_mask = req->vec_modes != 0 ? req->vec_modes : IMD_PERF_VEC_GENERATE;
    const int32_t pack_mask = req->pack_modes != 0 ? req->pack_modes : IMD_PERF_PACK_NONE;
    struct Entry {
      imd_perf_candidate_t c;
      int64_t seq;
    };
    std::vector<Entry> all;
    const int32_t pack_bits[4] = {IMD_PERF_PACK_NONE, IMD_PERF_PACK_A, IMD_PERF_PACK_B, IMD_PERF_PACK_AB};
    for (int32_t ni = 0; ni < req->num_moduli_count; ++ni) {
      const int32_t N = req->num_moduli[ni];
      std::vector<int32_t> gs;
      if (req->residue_group_count == 0) {
        for (int32_t g = 1; g <= N; ++g) gs.push_back(g);
      } else {
        for (int32_t i = 0; i < req->residue_group_count; ++i)
          if (req->residue_groups[i] <= N) gs.push_back(req->residue_groups[i]);
      }
      for (const int32_t g : gs)
        for (int32_t vec = IMD_VEC_GENERATE; vec <= IMD_VEC_RESIDENT; ++vec) {
          if (!(vec_mask & (vec == IMD_VEC_GENERATE ? IMD_PERF_VEC_GENERATE : IMD_PERF_VEC_RESIDENT)))
            continue;
          for (int32_t packed = 0; packed < 4; ++packed) {
            if (!(pack_mask & pack_bits[packed])) continue;
            imd_options_t o = *base;
            o.num_moduli = N, o.residue_group = g, o.vec_mode = vec;
            Entry en;
            std::memset(&en, 0, sizeof en);
            en.seq = static_cast<int64_t>(all.size());
            imd_perf_candidate_t& c = en.c;
            c.num_moduli = N, c.residue_group = g, c.vec_mode = vec, c.packed = packed;
            imd_pack_desc_t desc[2];
            std::vector<int32_t> labels[2];
            imd_status_t st = IMD_STATUS_SUCCESS;
            for (int x = 0; x < 2 && st == IMD_STATUS_SUCCESS; ++x) {
              if (!(packed & (1 << x))) continue;
              const imd_tensor_t* X = x == 0 ? A : B;
              labels[x].assign(static_cast<size_t>(std::max(X->rank, 1)), 0);
              std::memset(&desc[x], 0, sizeof desc[x]);
              desc[x].struct_size = sizeof desc[x];
              st = imd_pack_desc_for(A, B, C, &o, x, &desc[x], labels[x].data(),
                                     static_cast<int32_t>(labels[x].size()));
            }
            const imd_packing_t packing = {(packed & 1) ? &desc[0] : nullptr,
                                           (packed & 2) ? &desc[1] : nullptr};
            imd_perf_t pr;
            std::memset(&pr, 0, sizeof pr);
            if (st == IMD_STATUS_SUCCESS)
              st = predict_contract(A, B, C, &o, packed ? &packing : nullptr, q, *cal, &pr);
            double pack_s = 0, pack_lo = 0, pack_hi = 0;
            uint64_t pack_bytes = 0, pack_ws = 0;
            for (int x = 0; x < 2 && st == IMD_STATUS_SUCCESS; ++x) {
              if (!(packed & (1 << x))) continue;
              imd_perf_t pp;
              std::memset(&pp, 0, sizeof pp);
              st = predict_pack(desc[x], q, *cal, &pp);
              pack_s += pp.time_s, pack_lo += pp.time_lo_s, pack_hi += pp.time_hi_s;
              pack_bytes += pp.pack_bytes, pack_ws += pp.pack_ws_bytes;
            }
            c.status = st;
            if (st == IMD_STATUS_SUCCESS) {
              c.k4_config = pr.k4_config, c.dispatch = pr.dispatch;
              c.contract_s = pr.time_s, c.pack_s = pack_s;
              c.time_s = pr.time_s + pack_s / req->reuse;
              c.tflops_eq = c.time_s > 0 ? pr.flops_eq / c.time_s * 1e-12 : 0;
              c.workspace_bytes = pr.workspace_bytes, c.plan_device_bytes = pr.plan_device_bytes;
              c.pack_bytes = pack_bytes, c.pack_ws_bytes = pack_ws;
              uint64_t total = 0;
              const bool fits = add_u64(c.workspace_bytes, c.plan_device_bytes, &total) &&
                                add_u64(total, pack_bytes, &total) && add_u64(total, pack_ws, &total);
              c.total_bytes = fits ? total : UINT64_MAX;
              if (req->budget_bytes != 0 && c.total_bytes > req->budget_bytes)
                c.infeasible |= IMD_PERF_INFEASIBLE_BUDGET;
              c.kernel_launches = pr.kernel_launches;
              c.time_lo_s = pr.time_lo_s + pack_lo / req->reuse;
              c.time_hi_s = pr.time_hi_s + pack_hi / req->reuse;
              c.clock_mhz = pr.clock_mhz, c.power_w = pr.power_w;
              c.err_bound = pr.err_bound, c.err_typical = pr.err_typical, c.err_status = pr.err_status;
              if (pr.err_status == IMD_ERR_MISSED) c.infeasible |= IMD_PERF_INFEASIBLE_ACCURACY;
            } else {
              c.infeasible = IMD_PERF_INFEASIBLE_STATUS;
              c.err_bound = c.err_typical = std::numeric_limits<double>::infinity();
            }
            c.feasible = c.infeasible == 0 ? 1 : 0;
            all.push_back(en);
          }
        }
    }
    // feasible by time, then infeasible SUCCESS ones by time, then the rest as enumerated
    const auto tier = [](const imd_perf_candidate_t& c) {
      return c.status != IMD_STATUS_SUCCESS ? 2 : c.feasible ? 0 : 1;
    };
    const auto by_config = [](const imd_perf_candidate_t& x, const imd_perf_candidate_t& y) {
      if (x.num_moduli != y.num_moduli) return x.num_moduli < y.num_moduli;
      if (x.residue_group != y.residue_group) return x.residue_group < y.residue_group;
      if (x.vec_mode != y.vec_mode) return x.vec_mode < y.vec_mode;
      return x.packed < y.packed;
    };
    std::stable_sort(all.begin(), all.end(), [&](const Entry& x, const Entry& y) {
      const int tx = tier(x.c), ty = tier(y.c);
      if (tx != ty) return tx < ty;
      if (tx == 2) return x.seq < y.seq;
      if (x.c.time_s != y.c.time_s) return x.c.time_s < y.c.time_s;
      if (x.c.total_bytes != y.c.total_bytes) return x.c.total_bytes < y.c.total_bytes;
      return by_config(x.c, y.c);
    });
    for (size_t i = 0; i < all.size(); ++i) all[i].c.raw_rank = static_cast<int32_t>(i);
    if (!all.empty() && tier(all[0].c) == 0) {
      const double limit = all[0].c.time_s * cal->tie_ratio;
      for (Entry& en : all) en.c.tie = tier(en.c) == 0 && en.c.time_s <= limit ? 1 : 0;
      if (order == IMD_PERF_ORDER_TIES_BY_FOOTPRINT)
        std::stable_sort(all.begin(), all.end(), [&](const Entry& x, const Entry& y) {
          if (x.c.tie != y.c.tie) return x.c.tie > y.c.tie;
          if (!x.c.tie) return x.c.raw_rank < y.c.raw_rank;
          if (x.c.total_bytes != y.c.total_bytes) return x.c.total_bytes < y.c.total_bytes;
          if (x.c.time_s != y.c.time_s) return x.c.time_s < y.c.time_s;
          return by_config(x.c, y.c);
        });
    }
    if (all.size() > static_cast<size_t>(INT32_MAX)) return IMD_STATUS_INVALID_VALUE;
    auto* dst = reinterpret_cast<unsigned char*>(out);
    for (size_t i = 0; i < std::min(all.size(), static_cast<size_t>(capacity)); ++i)
      std::memcpy(dst + i * req->candidate_size, &all[i].c,
                  std::min<size_t>(req->candidate_size, sizeof(imd_perf_candidate_t)));
    *num_candidates = static_cast<int32_t>(all.size());
    return IMD_STATUS_SUCCESS;
  });
}

}  // extern "C"
