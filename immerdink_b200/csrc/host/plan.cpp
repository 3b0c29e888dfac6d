#include "plan.hpp"

namespace imd {
namespace {

bool options_valid(const imd_options_t& o) {
  return o.num_moduli >= kMinModuli && o.num_moduli <= kMaxModuli && o.residue_group >= 0 &&
         o.residue_group <= o.num_moduli && (o.rounding == IMD_RN || o.rounding == IMD_TRUNC) &&
         (o.mode == IMD_EMULATE || o.mode == IMD_DIRECT) &&
         (o.vec_mode == IMD_VEC_GENERATE || o.vec_mode == IMD_VEC_RESIDENT) &&
         (o.k4_tune == IMD_K4_TUNE_OFF || o.k4_tune == IMD_K4_TUNE_ON);
}

using u128 = unsigned __int128;

// Product of nonnegative factors in uint64; false on overflow.
bool product(std::initializer_list<uint64_t> xs, uint64_t* out) {
  u128 r = 1;
  for (uint64_t x : xs) {
    r *= x;
    if (r >> 64) return false;
  }
  *out = static_cast<uint64_t>(r);
  return true;
}

uint64_t round_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

}  // namespace

bool workspace_regions(const GemmView& v, const imd_options_t& o, int k_align, int packed_roles,
                       Layout* L) {
  *L = Layout{};
  if (v.empty_output()) return true;
  const uint64_t m = v.m, n = v.n, k = v.k, b = v.b;
  const uint64_t k_hat = round_up(k, static_cast<uint64_t>(k_align));
  const uint64_t n_hat = round_up(n, 16);
  uint64_t vec = 0;
  {
    u128 e = static_cast<u128>(2) * m + static_cast<u128>(2) * n + static_cast<u128>(2) * k +
             static_cast<u128>(3) * b;
    e *= 8;
    if (e >> 64) return false;
    vec = static_cast<uint64_t>(e);
  }
  uint64_t bytes[IMD_REGION_COUNT] = {};
  if (o.mode == IMD_DIRECT || k <= 1) {
    bytes[IMD_REGION_VEC] = vec;
  } else {
    const uint64_t g = o.residue_group, N = o.num_moduli;
    bool ok = product({2, b, m}, &bytes[IMD_REGION_SA]) && product({2, b, n}, &bytes[IMD_REGION_SB]) &&
              product({b, m}, &bytes[IMD_REGION_FA]) && product({b, n}, &bytes[IMD_REGION_FB]) &&
              product({g, b, m, k_hat}, &bytes[IMD_REGION_RA]) &&
              product({g, b, n_hat, k_hat}, &bytes[IMD_REGION_RB]) &&
              product({N, b, m, n_hat}, &bytes[IMD_REGION_W]);
    if (!ok) return false;
    bytes[IMD_REGION_VEC] = vec;
  }
  if (o.vec_mode == IMD_VEC_RESIDENT) bytes[IMD_REGION_VEC] = 0;  // plan memory instead
  if (packed_roles & 1) bytes[IMD_REGION_SA] = bytes[IMD_REGION_FA] = bytes[IMD_REGION_RA] = 0;
  if (packed_roles & 2) bytes[IMD_REGION_SB] = bytes[IMD_REGION_FB] = bytes[IMD_REGION_RB] = 0;
  uint64_t off = 0;
  for (int r = 0; r < IMD_REGION_COUNT; ++r) {
    if (bytes[r] == 0) continue;
    L->offset[r] = off;
    L->bytes[r] = bytes[r];
    const u128 next = static_cast<u128>(off) + round_up(bytes[r], kRegionAlign);
    if (bytes[r] > UINT64_MAX - (kRegionAlign - 1) || (next >> 64)) return false;
    off = static_cast<uint64_t>(next);
  }
  L->total = off;
  return true;
}

namespace {

// An operand is gathered along its rows when its fastest row (or batch) mode is faster than its
// fastest K mode; otherwise along K.
bool rows_are_fast(const GemmView& v, int X) {
  auto mg = [](int64_t s) { return s < 0 ? 0 - static_cast<uint64_t>(s) : static_cast<uint64_t>(s); };
  uint64_t best = UINT64_MAX;
  for (int g : {X == kTenA ? kClsI : kClsJ, kClsL})
    for (const Mode& md : v.modes[g]) {
      const uint64_t s = mg(md.stride[X]);
      if (s != 0 && s < best) best = s;
    }
  const uint64_t ks = v.modes[kClsK].empty() ? 0 : mg(v.modes[kClsK].front().stride[X]);
  return best != UINT64_MAX && (ks == 0 || best < ks);
}

}  // namespace

imd_status_t analyze(const imd_tensor_t* A, const imd_tensor_t* B, const imd_tensor_t* C,
                     const imd_options_t* options, Analysis* out) {
  if (A == nullptr || B == nullptr || C == nullptr || options == nullptr)
    return IMD_STATUS_INVALID_VALUE;
  if (!options_valid(*options)) return IMD_STATUS_INVALID_VALUE;
  out->options = *options;
  if (out->options.residue_group == 0) out->options.residue_group = out->options.num_moduli;
  if (const imd_status_t st = lower(*A, *B, *C, &out->view); st != IMD_STATUS_SUCCESS) return st;
  const GemmView& v = out->view;
  // int32 tile coordinates of the GEMM: only when the emulated GEMM runs.
  if (out->options.mode == IMD_EMULATE && !v.empty_output() && v.k >= 2 &&
      (v.m > INT32_MAX || v.n > INT32_MAX - 15))
    return IMD_STATUS_INVALID_VALUE;
  out->k_align = v.k > 96 ? 64 : 16;
  if (!workspace_regions(v, out->options, out->k_align, 0, &out->layout)) return IMD_STATUS_INVALID_VALUE;
  if (out->layout.total > SIZE_MAX) return IMD_STATUS_INVALID_VALUE;
  return IMD_STATUS_SUCCESS;
}

imd_status_t make_plan(const Analysis& an, ExecPlan* out) {
  const GemmView& v = an.view;
  ExecPlan e;
  e.swapped = v.swapped;
  e.m = v.m, e.n = v.n, e.k = v.k, e.b = v.b;
  e.n_hat = (v.n + 15) / 16 * 16;
  e.N = an.options.num_moduli;
  e.g = an.options.residue_group;
  e.trunc = an.options.rounding == IMD_TRUNC;
  e.layout = an.layout;
  e.path = v.empty_output() ? Path::kNoop
           : (an.options.mode == IMD_DIRECT || v.k == 1) ? Path::kDirect
                                                          : Path::kGemm;
  e.k_align = e.emulated() ? an.k_align : 16;
  e.packed = an.packed.role;
  for (int x = 0; x < 2; ++x)
    if (e.packed & (1 << x)) {
      for (int r = 0; r < 3; ++r) e.pack_off[x][r] = an.packed.layout[x].offset[r];
      e.pack_bytes[x] = an.packed.layout[x].total;
    }
  e.k_hat = (v.k + e.k_align - 1) / e.k_align * e.k_align;
  const bool rn = !e.trunc;
  *out = e;
  if (e.emulated() && rn && kappa_at_least_T(ceil_sqrt_u64(static_cast<uint64_t>(v.k)), e.N))
    return IMD_STATUS_NOT_SUPPORTED;
  if (e.emulated()) {
    e.rhs = shift_rhs(e.N, rn, static_cast<uint64_t>(v.k));
    e.lhs_shift = rn ? 2 : 0;
    e.fast = shift_fast(e.rhs, static_cast<uint64_t>(v.k));
    e.rows_fast[0] = rows_are_fast(v, kTenA);
    e.rows_fast[1] = rows_are_fast(v, kTenB);
    e.k_chunks = plan_k_chunks(e);
  }
  if (e.path != Path::kNoop) {
    auto mg = [](int64_t s) { return s < 0 ? 0 - static_cast<uint64_t>(s) : static_cast<uint64_t>(s); };
    const auto& Lm = v.modes[kClsL];
    const auto& Jm = v.modes[kClsJ];
    e.c_batch_fast = !Lm.empty() && (Jm.empty() || mg(Lm.front().stride[kTenC]) < mg(Jm.front().stride[kTenC]));
    e.vec_count = v.vec_entries();
    int at = 0;
    for (int g = 0; g < 4; ++g) {
      e.modes.first[g] = at;
      e.modes.count[g] = static_cast<int32_t>(v.modes[g].size());
      for (const Mode& md : v.modes[g]) {
        if (at >= kMaxVecModes) return IMD_STATUS_INVALID_VALUE;
        e.modes.extent[at] = md.extent;
        for (int x = 0; x < 3; ++x) e.modes.stride[at][x] = md.stride[x];
        ++at;
      }
    }
    if (an.options.vec_mode == IMD_VEC_RESIDENT) {
      e.vec_resident = true;
      e.device_bytes = static_cast<uint64_t>(e.vec_count) * 8;
    }
  }
  *out = e;
  return IMD_STATUS_SUCCESS;
}

int64_t plan_k_chunks(const ExecPlan& e) {
  if (!e.emulated()) return 0;
  return (e.k_hat + kChunk - 1) / kChunk;
}

int64_t plan_gemm_launches(const ExecPlan& e) {
  if (!e.emulated()) return 0;
  const int64_t groups = (e.N + e.g - 1) / e.g;
  return groups * plan_k_chunks(e);
}

int64_t plan_kernel_launches(const ExecPlan& e) {
  if (e.path == Path::kNoop) return 0;
  const int64_t vec = e.vec_resident ? 0 : 1;
  if (!e.emulated()) return vec + 1;  // native FP64 kernel, or C <- beta C
  if (e.small()) return vec + 1;      // everything in one fused launch
  const int64_t groups = (e.N + e.g - 1) / e.g;
  // vectors; per group one quantise launch per operand and the GEMM launches; one CRT launch.
  // an in-line operand that is contiguous along its rows needs its own scale launch; the others
  // get their shifts from the first quantise launch
  int64_t inline_ops = 0, scale_launches = 0;
  for (int x = 0; x < 2; ++x)
    if (!(e.packed & (1 << x))) {
      ++inline_ops;
      if (e.rows_fast[x]) ++scale_launches;
    }
  return vec + scale_launches + inline_ops * groups + plan_gemm_launches(e) + 1;
}

uint64_t plan_host_bytes(const imd_tensor_t& A, const imd_tensor_t& B, const imd_tensor_t& C,
                         const Analysis& an, const ExecPlan&) {
  uint64_t bytes = sizeof(imd_plan_st);
  const uint64_t modes = static_cast<uint64_t>(A.rank) + B.rank + C.rank;
  bytes += (8 + 8 + 4) * modes;
  bytes += sizeof(Label) * an.view.labels.size();
  for (int g = 0; g < 4; ++g)
    bytes += 4 * an.view.order[g].size() + sizeof(Mode) * an.view.modes[g].size();
  bytes += 8 * (an.packed.key[0].size() + an.packed.key[1].size());
  return bytes;
}

}  // namespace imd
