#include "pack.hpp"

#include <algorithm>
#include <array>

namespace imd {
namespace {

using u128 = unsigned __int128;
using i128 = __int128;

uint64_t mag(int64_t s) { return s < 0 ? 0 - static_cast<uint64_t>(s) : static_cast<uint64_t>(s); }
bool align_up(uint64_t x, uint64_t a, uint64_t* out) {
  if (x > UINT64_MAX - (a - 1)) return false;
  *out = (x + a - 1) / a * a;
  return true;
}

struct XLabel {  // one distinct label of X; a repeated label is a diagonal (strides summed)
  int32_t id = 0;
  int64_t extent = 0, stride = 0;
  int first = 0;
  int cls = -1;
};

XLabel* find(std::vector<XLabel>& v, int32_t id) {
  for (XLabel& l : v)
    if (l.id == id) return &l;
  return nullptr;
}

void fuse_append(std::vector<PackMode>& f, int64_t extent, int64_t stride) {
  if (!f.empty() && static_cast<i128>(f.back().stride) * f.back().extent == stride)
    f.back().extent *= extent;
  else
    f.push_back({extent, stride});
}

std::vector<int64_t> make_key(int64_t format, int N, int32_t rounding, int64_t b, int64_t r,
                              int64_t k, const std::vector<PackMode>& L,
                              const std::vector<PackMode>& R, const std::vector<PackMode>& K) {
  std::vector<int64_t> w = {format, N, rounding == IMD_TRUNC ? 1 : 0, b, r, k};
  for (const std::vector<PackMode>* f : {&L, &R, &K}) {
    w.push_back(static_cast<int64_t>(f->size()));
    for (const PackMode& m : *f) {
      w.push_back(m.extent);
      w.push_back(m.stride);
    }
  }
  return w;
}

// First differing part of two keys, as an IMD_PACK_MISMATCH_* reason; the format word is judged last.
int32_t key_difference(const std::vector<int64_t>& slot, const std::vector<int64_t>& pack) {
  if (slot == pack) return IMD_PACK_MISMATCH_NONE;
  std::vector<int32_t> kind = {IMD_PACK_MISMATCH_FORMAT,  IMD_PACK_MISMATCH_MODULI,
                               IMD_PACK_MISMATCH_ROUNDING, IMD_PACK_MISMATCH_EXTENTS,
                               IMD_PACK_MISMATCH_EXTENTS,  IMD_PACK_MISMATCH_EXTENTS};
  for (size_t p = 6; p < slot.size();) {
    const int64_t cnt = slot[p];
    kind.push_back(IMD_PACK_MISMATCH_EXTENTS);
    for (int64_t t = 0; t < cnt; ++t) {
      kind.push_back(IMD_PACK_MISMATCH_EXTENTS);
      kind.push_back(IMD_PACK_MISMATCH_STRIDES);
    }
    p += 1 + 2 * static_cast<size_t>(cnt);
  }
  const size_t n = std::min({slot.size(), pack.size(), kind.size()});
  for (size_t i = 1; i < n; ++i)
    if (slot[i] != pack[i]) return kind[i];
  if (slot.size() != pack.size()) return IMD_PACK_MISMATCH_EXTENTS;
  return IMD_PACK_MISMATCH_FORMAT;
}

int k_align_of(int64_t k) { return k > 96 ? 64 : 16; }

}  // namespace

bool pack_regions(int64_t b, int64_t r, int64_t k, int N, int32_t k_align, PackRegions* out) {
  *out = PackRegions{};
  if (k_align != 16 && k_align != 64) return false;
  if (b == 0 || r == 0 || k == 0) return true;
  const u128 kh = (static_cast<u128>(k) + k_align - 1) / k_align * k_align;
  const u128 rh = (static_cast<u128>(r) + 15) / 16 * 16;
  const u128 br = static_cast<u128>(b) * r;
  const u128 res = br * kh * N + (rh - r) * kh;
  if ((br >> 62) || (res >> 64)) return false;
  const uint64_t bytes[3] = {static_cast<uint64_t>(2 * br), static_cast<uint64_t>(br),
                             static_cast<uint64_t>(res)};
  uint64_t off = 0;
  for (int i = 0; i < 3; ++i) {
    out->offset[i] = off;
    out->bytes[i] = bytes[i];
    uint64_t a = 0;
    if (!align_up(bytes[i], kRegionAlign, &a) || off > UINT64_MAX - a) return false;
    off += a;
  }
  out->total = off;
  return true;
}

bool pack_workspace_bytes(int64_t b, int64_t r, int64_t k, uint64_t* out) {
  *out = 0;
  if (b == 0 || r == 0 || k == 0) return true;
  const u128 v = (static_cast<u128>(r) + k + b) * 8;
  if (v >> 63) return false;
  return align_up(static_cast<uint64_t>(v), kRegionAlign, out);
}

uint64_t key_digest(const std::vector<int64_t>& key) {
  uint64_t h = 0xcbf29ce484222325ull;  // FNV-1a over the key's bytes, little-endian words
  for (const int64_t w : key)
    for (int i = 0; i < 8; ++i) {
      h ^= (static_cast<uint64_t>(w) >> (8 * i)) & 0xffu;
      h *= 0x100000001b3ull;
    }
  return h;
}

imd_status_t pack_lower(const imd_pack_desc_t& d, PackLowered* out) {
  *out = PackLowered{};
  if (d.struct_size < sizeof(imd_pack_desc_t)) return IMD_STATUS_INVALID_VALUE;
  if (d.num_moduli < kMinModuli || d.num_moduli > kMaxModuli ||
      (d.rounding != IMD_RN && d.rounding != IMD_TRUNC) ||
      (d.order != IMD_PACK_ORDER_AUTO && d.order != IMD_PACK_ORDER_GIVEN))
    return IMD_STATUS_INVALID_VALUE;
  if (d.tensor == nullptr) return IMD_STATUS_INVALID_VALUE;
  const imd_tensor_t& X = *d.tensor;
  if (X.rank < 0 || (X.rank > 0 && (X.extent == nullptr || X.stride == nullptr || X.label == nullptr)))
    return IMD_STATUS_INVALID_VALUE;
  for (int p = 0; p < X.rank; ++p)
    if (X.extent[p] < 0) return IMD_STATUS_INVALID_VALUE;
  if (d.num_contracted < 0 || d.num_batch < 0 || d.num_rows < 0 ||
      (d.num_contracted > 0 && d.contracted == nullptr) || (d.num_batch > 0 && d.batch == nullptr) ||
      (d.num_rows > 0 && d.rows == nullptr))
    return IMD_STATUS_INVALID_VALUE;
  if (d.order == IMD_PACK_ORDER_AUTO && d.num_rows != 0) return IMD_STATUS_INVALID_VALUE;

  std::vector<XLabel> labs;
  bool stride_overflow = false;
  for (int32_t p = 0; p < X.rank; ++p) {
    XLabel* l = find(labs, X.label[p]);
    if (l == nullptr) {
      labs.push_back({X.label[p], X.extent[p], 0, p, -1});
      l = &labs.back();
    } else if (l->extent != X.extent[p]) {
      return IMD_STATUS_INVALID_VALUE;
    }
    const i128 sum = static_cast<i128>(l->stride) + X.stride[p];
    if (sum > INT64_MAX || sum < INT64_MIN) stride_overflow = true;
    else l->stride = static_cast<int64_t>(sum);
  }
  const auto mark = [&](const int32_t* list, int32_t n, int cls) {
    for (int32_t i = 0; i < n; ++i) {
      XLabel* l = find(labs, list[i]);
      if (l == nullptr || l->cls != -1) return false;  // not X's, or listed twice
      l->cls = cls;
    }
    return true;
  };
  if (!mark(d.contracted, d.num_contracted, kPackK) || !mark(d.batch, d.num_batch, kPackL) ||
      (d.order == IMD_PACK_ORDER_GIVEN && !mark(d.rows, d.num_rows, kPackR)))
    return IMD_STATUS_INVALID_VALUE;
  for (XLabel& l : labs) {
    if (l.cls != -1) continue;
    if (d.order == IMD_PACK_ORDER_GIVEN) return IMD_STATUS_INVALID_VALUE;  // a row label not listed
    l.cls = kPackR;
  }
  // span and class sizes in int64
  bool empty = false;
  for (int p = 0; p < X.rank; ++p) empty = empty || X.extent[p] == 0;
  if (!empty) {
    i128 span = 0;
    for (int p = 0; p < X.rank; ++p)
      if (X.extent[p] > 1) span += static_cast<i128>(mag(X.stride[p])) * (X.extent[p] - 1);
    if (span > INT64_MAX) return IMD_STATUS_INVALID_VALUE;
  }
  if (stride_overflow) return IMD_STATUS_INVALID_VALUE;
  int64_t size[3] = {1, 1, 1};
  bool zero[3] = {false, false, false};
  for (const XLabel& l : labs)
    if (l.extent == 0) zero[l.cls] = true;
  for (int cl = 0; cl < 3; ++cl) {
    if (zero[cl]) {
      size[cl] = 0;
      continue;
    }
    i128 prod = 1;
    for (const XLabel& l : labs)
      if (l.cls == cl && l.extent > 1) {
        prod *= l.extent;
        if (prod > INT64_MAX) return IMD_STATUS_INVALID_VALUE;
      }
    size[cl] = static_cast<int64_t>(prod);
  }
  PackLowered& o = *out;
  o.N = d.num_moduli;
  o.rounding = d.rounding;
  o.b = size[kPackL], o.r = size[kPackR], o.k = size[kPackK];
  o.k_align = k_align_of(o.k);
  o.format = o.k_align == 64 ? IMD_PACK_FORMAT_A64 : IMD_PACK_FORMAT_A16;
  o.k_hat = (o.k + o.k_align - 1) / o.k_align * o.k_align;
  if (!pack_regions(o.b, o.r, o.k, o.N, o.k_align, &o.layout) ||
      !pack_workspace_bytes(o.b, o.r, o.k, &o.ws_bytes))
    return IMD_STATUS_INVALID_VALUE;
  o.kappa = o.k >= 1 ? ceil_sqrt_u64(static_cast<uint64_t>(o.k)) : 0;
  o.sized = true;

  const bool k_kept = std::any_of(labs.begin(), labs.end(),
                                  [](const XLabel& l) { return l.cls == kPackK && l.extent != 1; });
  if (!k_kept) return IMD_STATUS_NOT_SUPPORTED;  // every contraction with it would be DIRECT
  if (o.rounding == IMD_RN && o.k >= 2 && kappa_at_least_T(o.kappa, o.N)) return IMD_STATUS_NOT_SUPPORTED;

  const int32_t* lists[3] = {d.contracted, d.batch, d.rows};
  const int32_t counts[3] = {d.num_contracted, d.num_batch, d.num_rows};
  for (int cl = 0; cl < 3; ++cl) {
    std::vector<const XLabel*> grp;
    if (d.order == IMD_PACK_ORDER_GIVEN) {
      for (int32_t i = 0; i < counts[cl]; ++i) grp.push_back(find(labs, lists[cl][i]));
    } else {
      for (const XLabel& l : labs)
        if (l.cls == cl) grp.push_back(&l);
      std::sort(grp.begin(), grp.end(), [](const XLabel* x, const XLabel* y) {
        return std::array<uint64_t, 2>{mag(x->stride), static_cast<uint64_t>(x->first)} <
               std::array<uint64_t, 2>{mag(y->stride), static_cast<uint64_t>(y->first)};
      });
    }
    for (const XLabel* l : grp) {
      if (l->extent == 1) continue;
      o.order[cl].push_back(l->id);
      fuse_append(o.fused[cl], l->extent, l->stride);
    }
  }
  o.key = make_key(o.format, o.N, o.rounding, o.b, o.r, o.k, o.fused[kPackL], o.fused[kPackR],
                   o.fused[kPackK]);
  return IMD_STATUS_SUCCESS;
}

imd_status_t match_packs(const imd_tensor_t* A, const imd_tensor_t* B,
                         const PackSource* const src[2], Analysis* an) {
  an->packed = PackedSlots{};
  if (src[0] == nullptr && src[1] == nullptr) return IMD_STATUS_SUCCESS;
  GemmView& v = an->view;
  PackedSlots& ps = an->packed;
  const imd_tensor_t* X[2] = {A, B};
  int role[2];
  for (int x = 0; x < 2; ++x) {
    role[x] = ((x == 0) != v.swapped) ? 0 : 1;
    if (src[x] != nullptr) {
      ps.caller |= 1 << x;
      ps.role |= 1 << role[x];
    }
  }
  if (!workspace_regions(v, an->options, an->k_align, ps.role, &an->layout)) return IMD_STATUS_INVALID_VALUE;
  const auto mismatch = [&](int32_t reason) {
    ps.mismatch = reason;
    return IMD_STATUS_PACK_MISMATCH;
  };
  std::vector<int32_t> adopted[2][3];
  for (int x = 0; x < 2; ++x) {
    if (src[x] == nullptr) continue;
    const PackLowered& pl = *src[x]->pl;
    if (pl.key.empty() || (pl.key[0] != IMD_PACK_FORMAT_A16 && pl.key[0] != IMD_PACK_FORMAT_A64))
      return mismatch(IMD_PACK_MISMATCH_FORMAT);
    if (pl.N != an->options.num_moduli) return mismatch(IMD_PACK_MISMATCH_MODULI);
    if (pl.rounding != an->options.rounding) return mismatch(IMD_PACK_MISMATCH_ROUNDING);
    const imd_tensor_t& T = *X[x];
    if (src[x]->rank != T.rank) return mismatch(IMD_PACK_MISMATCH_CLASSES);
    // pack label -> plan label must be a bijection that agrees at every mode position
    std::vector<std::pair<int32_t, int32_t>> map;
    for (int32_t p = 0; p < T.rank; ++p) {
      const int32_t lp = src[x]->label[p], lx = T.label[p];
      bool seen = false;
      for (const auto& ab : map) {
        if ((ab.first == lp) != (ab.second == lx)) return mismatch(IMD_PACK_MISMATCH_CLASSES);
        seen = seen || ab.first == lp;
      }
      if (!seen) map.emplace_back(lp, lx);
    }
    const auto to_plan = [&](int32_t lp) {
      for (const auto& ab : map)
        if (ab.first == lp) return ab.second;
      return lp;
    };
    for (const int32_t id : v.order[kClsK])  // a contracted label X does not carry
      if (find_label(v, id)->count[role[x]] == 0) return mismatch(IMD_PACK_MISMATCH_CLASSES);
    const int plan_cls[3] = {kClsK, kClsL, role[x] == 0 ? kClsI : kClsJ};
    for (int cl = 0; cl < 3; ++cl) {
      for (const int32_t lp : pl.order[cl]) adopted[x][cl].push_back(to_plan(lp));
      std::vector<int32_t> a = adopted[x][cl], b = v.order[plan_cls[cl]];
      std::sort(a.begin(), a.end());
      std::sort(b.begin(), b.end());
      if (a != b) return mismatch(IMD_PACK_MISMATCH_CLASSES);
    }
  }
  if (src[0] != nullptr && src[1] != nullptr &&
      (adopted[0][kPackK] != adopted[1][kPackK] || adopted[0][kPackL] != adopted[1][kPackL]))
    return mismatch(IMD_PACK_MISMATCH_ORDER);
  for (int x = 0; x < 2; ++x) {
    if (src[x] == nullptr) continue;
    adopt_order(&v, kClsK, adopted[x][kPackK]);
    adopt_order(&v, kClsL, adopted[x][kPackL]);
    adopt_order(&v, role[x] == 0 ? kClsI : kClsJ, adopted[x][kPackR]);
  }
  int32_t reason[2] = {0, 0};
  const int64_t plan_format = an->k_align == 64 ? IMD_PACK_FORMAT_A64 : IMD_PACK_FORMAT_A16;
  for (int x = 0; x < 2; ++x) {
    if (src[x] == nullptr) continue;
    std::vector<PackMode> f[3];
    const int plan_cls[3] = {kClsK, kClsL, role[x] == 0 ? kClsI : kClsJ};
    for (int cl = 0; cl < 3; ++cl)
      for (const int32_t id : v.order[plan_cls[cl]]) {
        const Label& li = *find_label(v, id);
        fuse_append(f[cl], li.extent, li.stride[role[x]]);
      }
    const int64_t rows = role[x] == 0 ? v.m : v.n;
    ps.key[x] = make_key(plan_format, an->options.num_moduli, an->options.rounding, v.b, rows, v.k,
                         f[kPackL], f[kPackR], f[kPackK]);
    reason[x] = key_difference(ps.key[x], src[x]->pl->key);
  }
  for (const bool format_pass : {false, true})
    for (int x = 0; x < 2; ++x)
      if (reason[x] != 0 && (reason[x] == IMD_PACK_MISMATCH_FORMAT) == format_pass) {
        ps.key[0].clear(), ps.key[1].clear();
        return mismatch(reason[x]);
      }
  const int64_t plan_k_hat = (v.k + an->k_align - 1) / an->k_align * an->k_align;
  for (int x = 0; x < 2; ++x)
    if (src[x] != nullptr && src[x]->pl->k_hat != plan_k_hat) {
      ps.key[0].clear(), ps.key[1].clear();
      return mismatch(IMD_PACK_MISMATCH_FORMAT);
    }
  for (int x = 0; x < 2; ++x)
    if (src[x] != nullptr) ps.layout[role[x]] = src[x]->pl->layout;
  return IMD_STATUS_SUCCESS;
}

void pack_exec(const PackLowered& pl, ExecPlan* out) {
  ExecPlan e;
  e.path = Path::kGemm;
  e.m = pl.r, e.n = 0, e.k = pl.k, e.b = pl.b;
  e.k_hat = pl.k_hat;
  e.k_align = pl.k_align;
  e.N = pl.N;
  e.g = pl.N;
  e.trunc = pl.rounding == IMD_TRUNC;
  if (pl.k >= 2) {
    e.rhs = shift_rhs(pl.N, pl.rounding == IMD_RN, static_cast<uint64_t>(pl.k));
    e.lhs_shift = pl.rounding == IMD_RN ? 2 : 0;
    e.fast = shift_fast(e.rhs, static_cast<uint64_t>(pl.k));
  }
  // X as operand A: rows = R (class I), K, batch = L; strides in slot A only
  const int cls[3] = {kClsK, kClsL, kClsI};
  int at = 0;
  for (int g = 0; g < 4; ++g) {
    e.modes.first[g] = at;
    e.modes.count[g] = 0;
    for (int cl = 0; cl < 3; ++cl) {
      if (cls[cl] != g) continue;
      for (const PackMode& pm : pl.fused[cl]) {
        if (at >= kMaxVecModes) break;
        e.modes.extent[at] = pm.extent;
        e.modes.stride[at][kTenA] = pm.stride;
        e.modes.stride[at][kTenB] = e.modes.stride[at][kTenC] = 0;
        ++at;
        ++e.modes.count[g];
      }
    }
  }
  // rows contiguous rather than K?
  auto smallest = [&](int cl) {
    uint64_t best = UINT64_MAX;
    for (const PackMode& pm : pl.fused[cl])
      if (pm.stride != 0 && mag(pm.stride) < best) best = mag(pm.stride);
    return best;
  };
  const uint64_t rs = std::min(smallest(kPackR), smallest(kPackL));
  const uint64_t ks = pl.fused[kPackK].empty() ? 0 : mag(pl.fused[kPackK].front().stride);
  e.rows_fast[0] = rs != UINT64_MAX && (ks == 0 || rs < ks);
  e.vec_count = pl.r + pl.k + pl.b;
  *out = e;
}

}  // namespace imd
