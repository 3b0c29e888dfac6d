// Fixed-width unsigned integers on 32-bit limbs (little-endian), usable from host and device
// code. Only what the plan-time constants and the per-row shift rule need: compare, add,
// subtract, multiply, shifts, bit length.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#  define IMD_HD __host__ __device__ __forceinline__
#else
#  define IMD_HD inline
#endif

namespace imd {

template <int W>
struct Wide {
  uint32_t w[W];
};

template <int W>
IMD_HD Wide<W> wide_zero() {
  Wide<W> r;
  for (int i = 0; i < W; ++i) r.w[i] = 0;
  return r;
}
template <int W>
IMD_HD Wide<W> wide_u64(uint64_t x) {
  Wide<W> r = wide_zero<W>();
  r.w[0] = static_cast<uint32_t>(x);
  if (W > 1) r.w[1] = static_cast<uint32_t>(x >> 32);
  return r;
}
template <int W>
IMD_HD int wide_cmp(const Wide<W>& a, const Wide<W>& b) {
  for (int i = W - 1; i >= 0; --i)
    if (a.w[i] != b.w[i]) return a.w[i] > b.w[i] ? 1 : -1;
  return 0;
}
template <int W>
IMD_HD bool wide_is_zero(const Wide<W>& a) {
  uint32_t o = 0;
  for (int i = 0; i < W; ++i) o |= a.w[i];
  return o == 0;
}
template <int W>
IMD_HD Wide<W> wide_add(const Wide<W>& a, const Wide<W>& b) {
  Wide<W> r;
  uint64_t c = 0;
  for (int i = 0; i < W; ++i) {
    c += static_cast<uint64_t>(a.w[i]) + b.w[i];
    r.w[i] = static_cast<uint32_t>(c);
    c >>= 32;
  }
  return r;
}
template <int W>
IMD_HD Wide<W> wide_sub(const Wide<W>& a, const Wide<W>& b) {  // a >= b
  Wide<W> r;
  int64_t c = 0;
  for (int i = 0; i < W; ++i) {
    c += static_cast<int64_t>(a.w[i]) - static_cast<int64_t>(b.w[i]);
    r.w[i] = static_cast<uint32_t>(c);
    c >>= 32;  // arithmetic: -1 on borrow
  }
  return r;
}
template <int W>
IMD_HD Wide<W> wide_mul_small(const Wide<W>& a, uint32_t m) {
  Wide<W> r;
  uint64_t c = 0;
  for (int i = 0; i < W; ++i) {
    c += static_cast<uint64_t>(a.w[i]) * m;
    r.w[i] = static_cast<uint32_t>(c);
    c >>= 32;
  }
  return r;
}
template <int W>
IMD_HD Wide<W> wide_mul(const Wide<W>& a, const Wide<W>& b) {  // product must fit
  Wide<W> r = wide_zero<W>();
  for (int i = 0; i < W; ++i) {
    uint64_t c = 0;
    for (int j = 0; i + j < W; ++j) {
      c += static_cast<uint64_t>(a.w[i]) * b.w[j] + r.w[i + j];
      r.w[i + j] = static_cast<uint32_t>(c);
      c >>= 32;
    }
  }
  return r;
}
template <int W>
IMD_HD uint32_t wide_divmod_small(Wide<W>* a, uint32_t d) {
  uint64_t rem = 0;
  for (int i = W - 1; i >= 0; --i) {
    const uint64_t cur = (rem << 32) | a->w[i];
    a->w[i] = static_cast<uint32_t>(cur / d);
    rem = cur % d;
  }
  return static_cast<uint32_t>(rem);
}
template <int W>
IMD_HD Wide<W> wide_shl(const Wide<W>& a, int s) {  // s >= 0; bits shifted out are lost
  Wide<W> r;
  const int ws = s >> 5, bs = s & 31;
  for (int i = W - 1; i >= 0; --i) {
    const int src = i - ws;
    uint32_t v = 0;
    if (src >= 0) v = a.w[src] << bs;
    if (src >= 1 && bs) v |= a.w[src - 1] >> (32 - bs);
    r.w[i] = v;
  }
  return r;
}
template <int W>
IMD_HD Wide<W> wide_shr(const Wide<W>& a, int s) {
  Wide<W> r;
  const int ws = s >> 5, bs = s & 31;
  for (int i = 0; i < W; ++i) {
    const int src = i + ws;
    uint32_t v = 0;
    if (src < W) v = a.w[src] >> bs;
    if (src + 1 < W && bs) v |= a.w[src + 1] << (32 - bs);
    r.w[i] = v;
  }
  return r;
}
template <int W>
IMD_HD int wide_bitlen(const Wide<W>& a) {
  for (int i = W - 1; i >= 0; --i)
    if (a.w[i]) {
      int b = 0;
      uint32_t v = a.w[i];
      while (v) {
        ++b;
        v >>= 1;
      }
      return 32 * i + b;
    }
  return 0;
}
template <int W>
IMD_HD Wide<W> wide_isqrt(const Wide<W>& a) {
  Wide<W> r = wide_zero<W>();
  for (int bit = (wide_bitlen(a) + 1) / 2; bit >= 0; --bit) {
    Wide<W> cand = r;
    cand.w[bit >> 5] |= 1u << (bit & 31);
    if (2 * wide_bitlen(cand) <= 32 * W) {
      const Wide<W> sq = wide_mul(cand, cand);
      if (wide_cmp(sq, a) <= 0) r = cand;
    }
  }
  return r;
}

}  // namespace imd
