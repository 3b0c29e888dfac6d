#include "lowering.hpp"

#include <algorithm>
#include <array>

namespace imd {
namespace {

using i128 = __int128;
constexpr i128 kI64Max = INT64_MAX;

uint64_t mag(int64_t s) { return s < 0 ? 0 - static_cast<uint64_t>(s) : static_cast<uint64_t>(s); }

bool well_formed(const imd_tensor_t& t) {
  if (t.rank < 0) return false;
  if (t.rank > 0 && (t.extent == nullptr || t.stride == nullptr || t.label == nullptr)) return false;
  for (int d = 0; d < t.rank; ++d)
    if (t.extent[d] < 0) return false;
  return true;
}

bool has_zero_extent(const imd_tensor_t& t) {
  for (int d = 0; d < t.rank; ++d)
    if (t.extent[d] == 0) return true;
  return false;
}

// Writes through C are injective if, over modes with extent > 1 in increasing |stride|, each
// |stride| exceeds the span of all smaller ones.
bool strides_nest(const imd_tensor_t& t) {
  std::vector<int> idx;
  for (int d = 0; d < t.rank; ++d)
    if (t.extent[d] > 1) idx.push_back(d);
  std::stable_sort(idx.begin(), idx.end(),
                   [&](int x, int y) { return mag(t.stride[x]) < mag(t.stride[y]); });
  unsigned __int128 span = 0;
  for (int d : idx) {
    const unsigned __int128 s = mag(t.stride[d]);
    if (s <= span) return false;
    span += s * static_cast<uint64_t>(t.extent[d] - 1);
    if (span >> 64) span = static_cast<unsigned __int128>(1) << 64;  // already beyond any stride
  }
  return true;
}

bool span_in_int64(const imd_tensor_t& t) {
  if (has_zero_extent(t)) return true;
  i128 span = 0;
  for (int d = 0; d < t.rank; ++d) {
    if (t.extent[d] <= 1) continue;
    span += static_cast<i128>(mag(t.stride[d])) * (t.extent[d] - 1);
    if (span > kI64Max) return false;
  }
  return true;
}

}  // namespace

imd_status_t lower(const imd_tensor_t& A, const imd_tensor_t& B, const imd_tensor_t& C,
                   GemmView* out) {
  const imd_tensor_t* ten[3] = {&A, &B, &C};
  for (const imd_tensor_t* t : ten)
    if (!well_formed(*t)) return IMD_STATUS_INVALID_VALUE;

  // One record per distinct label; a label repeated inside one tensor is a diagonal whose
  // stride is the sum of its strides.
  std::vector<Label> labels;
  bool diag_overflow = false;
  int pos = 0;
  for (int x = 0; x < 3; ++x)
    for (int d = 0; d < ten[x]->rank; ++d, ++pos) {
      const int32_t id = ten[x]->label[d];
      Label* rec = nullptr;
      for (Label& l : labels)
        if (l.id == id) rec = &l;
      if (rec == nullptr) {
        labels.emplace_back();
        rec = &labels.back();
        rec->id = id;
        rec->extent = ten[x]->extent[d];
        rec->first = pos;
      } else if (rec->extent != ten[x]->extent[d]) {
        return IMD_STATUS_INVALID_VALUE;
      }
      rec->count[x] += 1;
      const i128 sum = static_cast<i128>(rec->stride[x]) + ten[x]->stride[d];
      if (sum > kI64Max || sum < -kI64Max - 1) diag_overflow = true;
      else rec->stride[x] = static_cast<int64_t>(sum);
    }

  for (const Label& l : labels)
    if (l.count[kTenC] > 1) return IMD_STATUS_NOT_SUPPORTED;  // diagonal in the output
  for (const Label& l : labels)
    if (l.count[kTenC] > 0 && l.count[kTenA] == 0 && l.count[kTenB] == 0 && l.extent > 1)
      return IMD_STATUS_NOT_SUPPORTED;                        // broadcast into the output

  const bool c_empty = has_zero_extent(C);
  if (!c_empty && !strides_nest(C)) return IMD_STATUS_INVALID_VALUE;
  if (diag_overflow) return IMD_STATUS_INVALID_VALUE;
  for (const imd_tensor_t* t : ten)
    if (!span_in_int64(*t)) return IMD_STATUS_INVALID_VALUE;

  bool zero[4] = {false, false, false, false};
  for (Label& l : labels) {
    const bool a = l.count[kTenA] > 0, b = l.count[kTenB] > 0, c = l.count[kTenC] > 0;
    l.cls = (a && b && c) ? kClsL : (a && c) ? kClsI : (b && c) ? kClsJ : c ? kClsI : kClsK;
    if (l.extent == 0) zero[l.cls] = true;
  }
  int64_t size[4] = {1, 1, 1, 1};
  for (int g = 0; g < 4; ++g) {
    if (zero[g]) {
      size[g] = 0;
      continue;
    }
    i128 prod = 1;
    for (const Label& l : labels)
      if (l.cls == g && l.extent > 1) {
        prod *= l.extent;
        if (prod > kI64Max) return IMD_STATUS_INVALID_VALUE;
      }
    size[g] = static_cast<int64_t>(prod);
  }

  GemmView v;
  v.m = size[kClsI], v.n = size[kClsJ], v.k = size[kClsK], v.b = size[kClsL];

  // Role swap: the GEMM's column index must run along C's fastest mode.
  if (!c_empty) {
    int fastest = -1;
    for (int d = 0; d < C.rank; ++d)
      if (C.extent[d] > 1 && (fastest < 0 || mag(C.stride[d]) < mag(C.stride[fastest])))
        fastest = d;
    if (fastest >= 0)
      for (const Label& l : labels)
        if (l.id == C.label[fastest] && l.cls == kClsI) v.swapped = true;
  }
  if (v.swapped) {
    std::swap(v.m, v.n);
    for (Label& l : labels) {
      std::swap(l.count[kTenA], l.count[kTenB]);
      std::swap(l.stride[kTenA], l.stride[kTenB]);
      if (l.cls == kClsI) l.cls = kClsJ;
      else if (l.cls == kClsJ) l.cls = kClsI;
    }
  }

  const i128 bb = v.b;
  if (bb * v.m * static_cast<i128>(v.k) > kI64Max || bb * v.n * static_cast<i128>(v.k) > kI64Max ||
      bb * v.m * static_cast<i128>(v.n) > kI64Max)
    return IMD_STATUS_INVALID_VALUE;

  // Canonical orders (first = fastest) and fusion, in the post-swap frame.
  const int big = v.m >= v.n ? kTenA : kTenB, oth = big == kTenA ? kTenB : kTenA;
  for (int g = 0; g < 4; ++g) {
    std::vector<const Label*> grp;
    for (const Label& l : labels)
      if (l.cls == g && l.extent != 1) grp.push_back(&l);
    auto key = [&](const Label* l) {
      const uint64_t a = mag(l->stride[kTenA]), b = mag(l->stride[kTenB]),
                     c = mag(l->stride[kTenC]), p = static_cast<uint64_t>(l->first);
      if (g == kClsI) return std::array<uint64_t, 4>{c, a, p, 0};
      if (g == kClsJ) return std::array<uint64_t, 4>{c, b, p, 0};
      if (g == kClsL) return std::array<uint64_t, 4>{c, a, b, p};
      return std::array<uint64_t, 4>{mag(l->stride[big]), mag(l->stride[oth]), p, 0};
    };
    std::sort(grp.begin(), grp.end(),
              [&](const Label* x, const Label* y) { return key(x) < key(y); });
    for (const Label* l : grp) {
      v.order[g].push_back(l->id);
      std::vector<Mode>& ms = v.modes[g];
      bool fuse = !ms.empty();
      for (int x = 0; fuse && x < 3; ++x)
        fuse = static_cast<i128>(ms.back().stride[x]) * ms.back().extent == l->stride[x];
      if (fuse) {
        ms.back().extent *= l->extent;
      } else {
        Mode md;
        md.extent = l->extent;
        for (int x = 0; x < 3; ++x) md.stride[x] = l->stride[x];
        ms.push_back(md);
      }
    }
  }
  v.labels = std::move(labels);
  *out = std::move(v);
  return IMD_STATUS_SUCCESS;
}

const Label* find_label(const GemmView& v, int32_t id) {
  for (const Label& l : v.labels)
    if (l.id == id) return &l;
  return nullptr;
}

void adopt_order(GemmView* v, int cls, const std::vector<int32_t>& order) {
  v->order[cls] = order;
  std::vector<Mode>& ms = v->modes[cls];
  ms.clear();
  for (const int32_t id : order) {
    const Label* l = find_label(*v, id);
    bool fuse = !ms.empty();
    for (int x = 0; fuse && x < 3; ++x)
      fuse = static_cast<__int128>(ms.back().stride[x]) * ms.back().extent == l->stride[x];
    if (fuse) {
      ms.back().extent *= l->extent;
    } else {
      Mode md;
      md.extent = l->extent;
      for (int x = 0; x < 3; ++x) md.stride[x] = l->stride[x];
      ms.push_back(md);
    }
  }
}

void scatter_vector(const GemmView& v, int cls, int X, int64_t* out) {
  const int64_t size = cls == kClsI ? v.m : cls == kClsJ ? v.n : cls == kClsK ? v.k : v.b;
  const std::vector<Mode>& ms = v.modes[cls];
  std::vector<int64_t> digit(ms.size(), 0);
  int64_t cur = 0;
  for (int64_t q = 0; q < size; ++q) {
    out[q] = cur;
    for (size_t t = 0; t < ms.size(); ++t) {
      if (digit[t] + 1 < ms[t].extent) {
        ++digit[t];
        cur += ms[t].stride[X];
        break;
      }
      cur -= ms[t].stride[X] * (ms[t].extent - 1);
      digit[t] = 0;
    }
  }
}

void scatter_vectors(const GemmView& v, int64_t* out) {
  const struct { int cls, X; int64_t n; } parts[9] = {
      {kClsI, kTenA, v.m}, {kClsK, kTenA, v.k}, {kClsL, kTenA, v.b},
      {kClsK, kTenB, v.k}, {kClsJ, kTenB, v.n}, {kClsL, kTenB, v.b},
      {kClsI, kTenC, v.m}, {kClsJ, kTenC, v.n}, {kClsL, kTenC, v.b}};
  for (const auto& p : parts) {
    scatter_vector(v, p.cls, p.X, out);
    out += p.n;
  }
}

}  // namespace imd
