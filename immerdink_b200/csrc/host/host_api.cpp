// C ABI of libimmerdink_host.so: pure host queries over plan.hpp. Nothing here touches CUDA.
// No exception leaves a function: allocation failures map to ALLOC_FAILED.
#include <algorithm>
#include <cstring>
#include <new>

#include <vector>

#include "immerdink/immerdink_host.h"
#include "pack.hpp"
#include "plan.hpp"

namespace {

using imd::Analysis;
using imd::ExecPlan;

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

// Plan analysis with optional pack descriptors: the plan's own legality first, then each
// descriptor's status (as imd_pack_layout), then the plan-side match.
imd_status_t analyze_with(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                          const imd_options_t* options, const imd_packing_t* packing, Analysis* an) {
  if (const imd_status_t st = imd::analyze(A, B, C, options, an); st != IMD_STATUS_SUCCESS) return st;
  if (packing == nullptr || (packing->A == nullptr && packing->B == nullptr)) return IMD_STATUS_SUCCESS;
  const imd_pack_desc_t* d[2] = {packing->A, packing->B};
  imd::PackLowered pl[2];
  imd::PackSource ps[2];
  const imd::PackSource* src[2] = {nullptr, nullptr};
  for (int x = 0; x < 2; ++x) {
    if (d[x] == nullptr) continue;
    if (const imd_status_t st = imd::pack_lower(*d[x], &pl[x]); st != IMD_STATUS_SUCCESS) return st;
    ps[x] = imd::PackSource{d[x]->tensor->rank, d[x]->tensor->label, &pl[x]};
    src[x] = &ps[x];
  }
  return imd::match_packs(A, B, src, an);
}

static_assert(sizeof(imd_tensor_t) == 32 && sizeof(imd_options_t) == 24, "ABI struct sizes");
static_assert(sizeof(imd_region_t) == 16 && sizeof(imd_lowering_t) == 192, "ABI struct sizes");
static_assert(offsetof(imd_lowering_t, fused) == 136 && offsetof(imd_lowering_t, sm_count) == 152 &&
                  offsetof(imd_lowering_t, fused_large) == 168 &&
                  offsetof(imd_lowering_t, packed) == 176 && offsetof(imd_lowering_t, k_align) == 184,
              "imd_lowering_t version boundaries");
static_assert(sizeof(imd_pack_desc_t) == 72 && sizeof(imd_pack_layout_t) == 136 &&
                  sizeof(imd_packing_t) == 16,
              "ABI struct sizes");
static_assert(sizeof(imd_err_request_t) == 64 && sizeof(imd_err_t) == 72, "ABI struct sizes");

imd_status_t lowering_impl(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                           const imd_options_t* options, const imd_packing_t* packing,
                           imd_lowering_t* out) {
  if (out == nullptr || out->struct_size < 136) return IMD_STATUS_INVALID_VALUE;
  imd_lowering_t r;
  std::memset(&r, 0, sizeof r);
  r.struct_size = out->struct_size;
  const int32_t sms_in = out->struct_size >= 168 ? out->sm_count : 0;
  if (sms_in < 0) return IMD_STATUS_INVALID_VALUE;
  r.status = guarded([&]() -> imd_status_t {
    Analysis an;
    const imd_status_t ast = analyze_with(A, B, C, options, packing, &an);
    if (ast != IMD_STATUS_SUCCESS && ast != IMD_STATUS_PACK_MISMATCH) return ast;
    r.packed = an.packed.caller;
    r.pack_mismatch = an.packed.mismatch;
    ExecPlan e;
    imd_status_t plan_st = imd::make_plan(an, &e);
    if (ast != IMD_STATUS_SUCCESS) plan_st = ast;  // a mismatch still reports the view
    r.lowered = 1;
    r.num_moduli = e.N;
    r.residue_group = e.g;
    r.swapped = e.swapped ? 1 : 0;
    r.m = e.m, r.n = e.n, r.k = e.k, r.b = e.b;
    r.n_hat = e.n_hat, r.k_hat = e.k_hat;
    r.k_align = e.k_align;
    r.kappa = e.k >= 1 ? imd::ceil_sqrt_u64(static_cast<uint64_t>(e.k)) : 0;
    r.workspace_bytes = an.layout.total;
    r.dispatch = e.path == imd::Path::kNoop ? IMD_DISPATCH_NOOP
                 : e.k == 0                 ? IMD_DISPATCH_SCALE
                 : e.emulated()             ? IMD_DISPATCH_EMULATE
                                            : IMD_DISPATCH_DIRECT;
    if (e.path != imd::Path::kNoop) r.vec_entries = an.view.vec_entries();
    if (r.dispatch == IMD_DISPATCH_EMULATE) {
      r.num_groups = (e.N + e.g - 1) / e.g;
      r.k_chunks = imd::plan_k_chunks(e);
      r.gemm_launches = imd::plan_gemm_launches(e);
    }
    e.vec_resident = an.options.vec_mode == IMD_VEC_RESIDENT && e.path != imd::Path::kNoop;
    r.kernel_launches = imd::plan_kernel_launches(e);
    r.fused = e.small() ? 1 : 0;
    r.sm_count = sms_in > 0 ? sms_in : imd::kDefaultSms;
    r.k4_config = IMD_K4_128x256;
    if (plan_st != IMD_STATUS_SUCCESS) return plan_st;
    r.plan_device_bytes = e.device_bytes;
    r.plan_host_bytes = imd::plan_host_bytes(*A, *B, *C, an, e);
    return IMD_STATUS_SUCCESS;
  });
  std::memcpy(out, &r, std::min<size_t>(out->struct_size, sizeof r));
  return static_cast<imd_status_t>(r.status);
}

imd_status_t layout_impl(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                         const imd_options_t* options, const imd_packing_t* packing,
                         imd_region_t* regions, int32_t capacity, int32_t* num_regions,
                         size_t* total) {
  if (capacity < 0 || (capacity > 0 && regions == nullptr)) return IMD_STATUS_INVALID_VALUE;
  return guarded([&]() -> imd_status_t {
    Analysis an;
    if (const imd_status_t st = analyze_with(A, B, C, options, packing, &an); st != IMD_STATUS_SUCCESS)
      return st;
    const int32_t n = std::min<int32_t>(capacity, IMD_REGION_COUNT);
    for (int32_t r = 0; r < n; ++r) regions[r] = {an.layout.offset[r], an.layout.bytes[r]};
    if (num_regions != nullptr) *num_regions = IMD_REGION_COUNT;
    if (total != nullptr) *total = static_cast<size_t>(an.layout.total);
    return IMD_STATUS_SUCCESS;
  });
}

}  // namespace

extern "C" {

uint32_t imd_host_api_version(void) { return IMD_HOST_API_VERSION; }

imd_status_t imd_workspace_size(const imd_tensor_t* A, const imd_tensor_t* B,
                                const imd_tensor_t* C, const imd_options_t* options,
                                size_t* bytes) {
  if (bytes == nullptr) return IMD_STATUS_INVALID_VALUE;
  return guarded([&]() -> imd_status_t {
    Analysis an;
    if (const imd_status_t st = imd::analyze(A, B, C, options, &an); st != IMD_STATUS_SUCCESS)
      return st;
    *bytes = static_cast<size_t>(an.layout.total);
    return IMD_STATUS_SUCCESS;
  });
}

imd_status_t imd_workspace_layout(const imd_tensor_t* A, const imd_tensor_t* B,
                                  const imd_tensor_t* C, const imd_options_t* options,
                                  imd_region_t* regions, int32_t capacity, int32_t* num_regions,
                                  size_t* total) {
  return layout_impl(A, B, C, options, nullptr, regions, capacity, num_regions, total);
}

const char* imd_region_name(int32_t region) {
  static const char* const names[IMD_REGION_COUNT] = {"sA", "sB", "fA", "fB", "vec", "RA", "RB", "W"};
  return region >= 0 && region < IMD_REGION_COUNT ? names[region] : nullptr;
}

imd_status_t imd_plan_bytes(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                            const imd_options_t* options, size_t* device_bytes,
                            size_t* host_bytes) {
  return guarded([&]() -> imd_status_t {
    Analysis an;
    if (const imd_status_t st = imd::analyze(A, B, C, options, &an); st != IMD_STATUS_SUCCESS)
      return st;
    ExecPlan e;
    if (const imd_status_t st = imd::make_plan(an, &e); st != IMD_STATUS_SUCCESS) return st;
    if (device_bytes != nullptr) *device_bytes = static_cast<size_t>(e.device_bytes);
    if (host_bytes != nullptr)
      *host_bytes = static_cast<size_t>(imd::plan_host_bytes(*A, *B, *C, an, e));
    return IMD_STATUS_SUCCESS;
  });
}

imd_status_t imd_lowering(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                          const imd_options_t* options, imd_lowering_t* out) {
  return lowering_impl(A, B, C, options, nullptr, out);
}

const char* imd_status_string(imd_status_t status) {
  switch (status) {
    case IMD_STATUS_SUCCESS: return "IMD_STATUS_SUCCESS";
    case IMD_STATUS_INVALID_VALUE: return "IMD_STATUS_INVALID_VALUE";
    case IMD_STATUS_NOT_SUPPORTED: return "IMD_STATUS_NOT_SUPPORTED";
    case IMD_STATUS_ALIASING: return "IMD_STATUS_ALIASING";
    case IMD_STATUS_INSUFFICIENT_WORKSPACE: return "IMD_STATUS_INSUFFICIENT_WORKSPACE";
    case IMD_STATUS_MISALIGNED: return "IMD_STATUS_MISALIGNED";
    case IMD_STATUS_CUDA_ERROR: return "IMD_STATUS_CUDA_ERROR";
    case IMD_STATUS_ALLOC_FAILED: return "IMD_STATUS_ALLOC_FAILED";
    case IMD_STATUS_PACK_MISMATCH: return "IMD_STATUS_PACK_MISMATCH";
  }
  return "IMD_STATUS_UNKNOWN";
}

/* ---- packed operands --------------------------------------------------------------------------- */
imd_status_t imd_pack_layout(const imd_pack_desc_t* desc, imd_pack_layout_t* out) {
  if (desc == nullptr || out == nullptr || out->struct_size < 136) return IMD_STATUS_INVALID_VALUE;
  imd_pack_layout_t r;
  std::memset(&r, 0, sizeof r);
  r.struct_size = out->struct_size;
  r.status = guarded([&]() -> imd_status_t {
    imd::PackLowered pl;
    const imd_status_t st = imd::pack_lower(*desc, &pl);
    if (!pl.sized) return st;  // INVALID_VALUE: only struct_size and status
    r.format = static_cast<int32_t>(pl.format);
    r.num_moduli = pl.N, r.rounding = pl.rounding;
    r.b = pl.b, r.r = pl.r, r.k = pl.k, r.k_hat = pl.k_hat;
    r.kappa = pl.kappa;
    r.sig = {pl.layout.offset[imd::kPackSig], pl.layout.bytes[imd::kPackSig]};
    r.flag = {pl.layout.offset[imd::kPackFlag], pl.layout.bytes[imd::kPackFlag]};
    r.res = {pl.layout.offset[imd::kPackRes], pl.layout.bytes[imd::kPackRes]};
    r.pack_bytes = pl.layout.total;
    r.pack_ws_bytes = pl.ws_bytes;
    r.key_digest = st == IMD_STATUS_SUCCESS ? imd::key_digest(pl.key) : 0;
    return st;
  });
  std::memcpy(out, &r, std::min<size_t>(out->struct_size, sizeof r));
  return static_cast<imd_status_t>(r.status);
}

imd_status_t imd_pack_desc_for(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                               const imd_options_t* options, int32_t operand, imd_pack_desc_t* out,
                               int32_t* labels, int32_t capacity) {
  if ((operand != 0 && operand != 1) || out == nullptr || out->struct_size < sizeof(imd_pack_desc_t) ||
      capacity < 0 || (capacity > 0 && labels == nullptr))
    return IMD_STATUS_INVALID_VALUE;
  return guarded([&]() -> imd_status_t {
    Analysis an;
    if (const imd_status_t st = imd::analyze(A, B, C, options, &an); st != IMD_STATUS_SUCCESS) return st;
    const imd::GemmView& v = an.view;
    const imd_tensor_t& X = operand == 0 ? *A : *B;
    const imd_tensor_t& P = operand == 0 ? *B : *A;
    const int role = ((operand == 0) != v.swapped) ? 0 : 1;
    const int cls[3] = {imd::kClsK, imd::kClsL, role == 0 ? imd::kClsI : imd::kClsJ};
    const auto in = [](const imd_tensor_t& t, int32_t lab) {
      for (int32_t p = 0; p < t.rank; ++p)
        if (t.label[p] == lab) return true;
      return false;
    };
    std::vector<int32_t> lists[3];
    for (int cl = 0; cl < 3; ++cl)
      for (const int32_t lab : v.order[cls[cl]])
        if (in(X, lab)) lists[cl].push_back(lab);
    for (int32_t p = 0; p < X.rank; ++p) {  // extent-1 labels of X, by membership
      const int32_t lab = X.label[p];
      bool listed = false;
      for (const auto& l : lists) listed = listed || std::find(l.begin(), l.end(), lab) != l.end();
      if (!listed) lists[!in(*C, lab) ? 0 : in(P, lab) ? 1 : 2].push_back(lab);
    }
    if (lists[0].size() + lists[1].size() + lists[2].size() > static_cast<size_t>(capacity))
      return IMD_STATUS_INVALID_VALUE;
    int32_t* w = labels;
    const int32_t* starts[3];
    for (int cl = 0; cl < 3; ++cl) {
      starts[cl] = w;
      for (const int32_t lab : lists[cl]) *w++ = lab;
    }
    const uint32_t size = out->struct_size;
    std::memset(out, 0, sizeof(imd_pack_desc_t));
    out->struct_size = size;
    out->num_moduli = an.options.num_moduli;
    out->rounding = an.options.rounding;
    out->order = IMD_PACK_ORDER_GIVEN;
    out->tensor = &X;
    out->num_contracted = static_cast<int32_t>(lists[0].size());
    out->contracted = lists[0].empty() ? nullptr : starts[0];
    out->num_batch = static_cast<int32_t>(lists[1].size());
    out->batch = lists[1].empty() ? nullptr : starts[1];
    out->num_rows = static_cast<int32_t>(lists[2].size());
    out->rows = lists[2].empty() ? nullptr : starts[2];
    return IMD_STATUS_SUCCESS;
  });
}

imd_status_t imd_workspace_size_packed(const imd_tensor_t* A, const imd_tensor_t* B,
                                       const imd_tensor_t* C, const imd_options_t* options,
                                       const imd_packing_t* packing, size_t* bytes) {
  if (bytes == nullptr) return IMD_STATUS_INVALID_VALUE;
  return guarded([&]() -> imd_status_t {
    Analysis an;
    if (const imd_status_t st = analyze_with(A, B, C, options, packing, &an); st != IMD_STATUS_SUCCESS)
      return st;
    *bytes = static_cast<size_t>(an.layout.total);
    return IMD_STATUS_SUCCESS;
  });
}
imd_status_t imd_workspace_layout_packed(const imd_tensor_t* A, const imd_tensor_t* B,
                                         const imd_tensor_t* C, const imd_options_t* options,
                                         const imd_packing_t* packing, imd_region_t* regions,
                                         int32_t capacity, int32_t* num_regions, size_t* total) {
  return layout_impl(A, B, C, options, packing, regions, capacity, num_regions, total);
}
imd_status_t imd_lowering_packed(const imd_tensor_t* A, const imd_tensor_t* B,
                                 const imd_tensor_t* C, const imd_options_t* options,
                                 const imd_packing_t* packing, imd_lowering_t* out) {
  return lowering_impl(A, B, C, options, packing, out);
}

}  // extern "C"
