// Exact device numerics of the emulated contraction: everything here is integer arithmetic on
// FP64 bit patterns (the only floating-point operations are the native FMA chain of flagged
// outputs and the alpha / beta epilogue). Each function states the rule it implements; the rules
// are those of the reference's specification (spec/oracle.py: scale_vector :361-408, quantize
// :415-435, residue :438-448, crt :498-512, round_dyadic :257-283), realised with this
// engine's own algorithms (byte-weight residues, unreduced CRT sum with a fixed-point quotient
// estimate).
#pragma once
#include <cstdint>

#include "common/wide.hpp"
#include "kernels.hpp"

namespace imd {
namespace dev {

// finite nonzero x = (-1)^neg M 2^E with 2^52 <= M < 2^53 (subnormals normalised).
// Returns -1 non-finite, 0 zero, 1 finite nonzero.
__device__ __forceinline__ int decompose(uint64_t u, uint64_t* M, int* E) {
  const int ef = static_cast<int>((u >> 52) & 0x7FF);
  const uint64_t frac = u & 0xFFFFFFFFFFFFFull;
  if (ef == 0x7FF) return -1;
  if (ef == 0) {
    if (frac == 0) return 0;
    const int sh = __clzll(static_cast<long long>(frac)) - 11;
    *M = frac << sh;
    *E = -1074 - sh;
    return 1;
  }
  *M = frac | (1ull << 52);
  *E = ef - 1075;
  return 1;
}

// ceil(M^2 2^(2 (E - gamma) + 60)) for E + 52 <= gamma: a right shift by sh >= 44 with ceiling.
__device__ __forceinline__ void square_term(uint64_t M, int E, int gamma, uint64_t* hi,
                                            uint64_t* lo) {
  const int sh = -(2 * (E - gamma) + kFracBits);
  const uint64_t ph = __umul64hi(M, M), pl = M * M;  // M^2 < 2^106
  uint64_t rl, rh = 0;
  bool inexact;
  if (sh >= 128) {
    rl = 0;
    inexact = true;
  } else if (sh >= 64) {
    rl = ph >> (sh - 64);
    inexact = pl != 0 || (sh > 64 && (ph & ((1ull << (sh - 64)) - 1)) != 0);
  } else {  // 44 <= sh < 64
    rl = (pl >> sh) | (ph << (64 - sh));
    rh = ph >> sh;
    inexact = (pl & ((1ull << sh) - 1)) != 0;
  }
  if (inexact) {
    rl += 1;
    if (rl == 0) rh += 1;
  }
  *hi = rh;
  *lo = rl;
}

// sigma = u - gamma with u the largest integer such that (S << lhs_shift) 4^u <= rhs.
__device__ inline int shift_from_sum(uint64_t S_hi, uint64_t S_lo, int lhs_shift,
                                     const Wide<8>& rhs, int gamma) {
  Wide<8> L = wide_zero<8>();
  L.w[0] = static_cast<uint32_t>(S_lo), L.w[1] = static_cast<uint32_t>(S_lo >> 32);
  L.w[2] = static_cast<uint32_t>(S_hi), L.w[3] = static_cast<uint32_t>(S_hi >> 32);
  L = wide_shl(L, lhs_shift);
  const int d = wide_bitlen(rhs) - wide_bitlen(L);
  int u = d >> 1;  // floor; within one of the answer
  auto ok = [&](int uu) {
    if (uu >= 0) {
      if (wide_bitlen(L) + 2 * uu > 256) return false;
      return wide_cmp(wide_shl(L, 2 * uu), rhs) <= 0;
    }
    if (wide_bitlen(rhs) - 2 * uu > 256) return true;  // rhs 4^-uu exceeds any L < 2^256
    return wide_cmp(L, wide_shl(rhs, -2 * uu)) <= 0;
  };
  for (int it = 0; it < 8 && !ok(u); ++it) --u;
  for (int it = 0; it < 8 && ok(u + 1); ++it) ++u;
  return u - gamma;
}

// |a'| = RN_even(|a| 2^sigma) (or truncation) as a 96-bit integer (lo, hi); neg = sign of a'.
__device__ __forceinline__ void quantize(uint64_t bits, int sigma, bool trunc, uint64_t* lo,
                                         uint32_t* hi, bool* neg) {
  uint64_t M;
  int E;
  *lo = 0;
  *hi = 0;
  *neg = false;
  if (decompose(bits, &M, &E) != 1) return;
  const int s = E + sigma;
  if (s >= 0) {
    // M 2^s <= T < 2^78 by the shift rule, so s <= 25
    *lo = M << s;
    *hi = s == 0 ? 0u : static_cast<uint32_t>(M >> (64 - s));
  } else {
    const int sh = -s;
    if (sh < 64) {
      uint64_t r = M >> sh;
      if (!trunc) {
        const uint64_t rem = M & ((1ull << sh) - 1), half = 1ull << (sh - 1);
        if (rem > half || (rem == half && (r & 1))) r += 1;
      }
      *lo = r;
    }
  }
  *neg = (bits >> 63) != 0 && (*lo | *hi) != 0;
}

// Symmetric residue of +-|a'| for modulus index l: in [-floor(p/2), ceil(p/2) - 1].
template <int WORDS>
__device__ __forceinline__ int residue(const ResidueTables& t, int l, uint32_t w0, uint32_t w1,
                                       uint32_t w2, bool neg) {
  uint32_t s = __dp4a(w0, t.weight[0][l], 0u);
  s = __dp4a(w1, t.weight[1][l], s);
  if (WORDS > 2) s = __dp4a(w2, t.weight[2][l], s);  // s <= 12 * 255^2 < 2^20
  uint32_t v = neg ? t.lift[l] - s : s;              // >= 0, congruent to a'
  v += t.half[l];
  const uint32_t r = v - t.p[l] * __umulhi(v, t.magic[l]);  // v mod p, exact for v < 2^24
  return static_cast<int>(r) - static_cast<int>(t.half[l]);
}

// ---- CRT ------------------------------------------------------------------------------------
// z = centred representative of the residues, as sign + magnitude on LIMBS 32-bit limbs.
// S = sum_l M_l y_l (y_l = q_l W_l mod p_l) is not reduced on the way: S / P = sum y_l / p_l, so
// the multiple of P to subtract is the rounding of a fixed-point estimate of that sum, followed
// by one exact correction.
// Residue l is byte `lane` of packed[l].
template <int LIMBS>
__device__ __forceinline__ void crt(const CrtTables& t, const uint32_t* packed, int lane,
                                    uint32_t* mag, bool* neg) {
  uint32_t S[LIMBS];
#pragma unroll
  for (int i = 0; i < LIMBS; ++i) S[i] = 0;
  uint32_t est = 0;  // sum y_l floor(2^26 / p_l): below the true sum by less than N 2^-18
#pragma unroll
  for (int l = 0; l < kMaxModuli; ++l) {
    if (l >= t.N) break;
    const uint32_t v = t.q[l] * ((packed[l] >> (8 * lane)) & 0xFFu);
    const uint32_t y = v - t.p[l] * __umulhi(v, t.magic[l]);
    est += y * (t.frac[l] >> 1);
    uint64_t c = 0;
#pragma unroll
    for (int i = 0; i < LIMBS; ++i) {
      c += static_cast<uint64_t>(t.M[l][i]) * y + S[i];
      S[i] = static_cast<uint32_t>(c);
      c >>= 32;
    }
  }
  const uint32_t q = (est + (1u << 25)) >> 26;
  uint32_t Q[LIMBS];
  {
    uint64_t c = 0;
#pragma unroll
    for (int i = 0; i < LIMBS; ++i) {
      c += static_cast<uint64_t>(t.P[i]) * q;
      Q[i] = static_cast<uint32_t>(c);
      c >>= 32;
    }
  }
  // d = S - Q (two's complement); negative iff S < Q
  int64_t b = 0;
  uint32_t d[LIMBS];
#pragma unroll
  for (int i = 0; i < LIMBS; ++i) {
    b += static_cast<int64_t>(S[i]) - static_cast<int64_t>(Q[i]);
    d[i] = static_cast<uint32_t>(b);
    b >>= 32;
  }
  bool ng = b < 0;
  if (ng) {  // magnitude = -d
    uint64_t c = 1;
#pragma unroll
    for (int i = 0; i < LIMBS; ++i) {
      c += static_cast<uint32_t>(~d[i]);
      d[i] = static_cast<uint32_t>(c);
      c >>= 32;
    }
  } else {
    // d in [0, P/2 + small): if d > H the representative is d - P
    bool gt = false, decided = false;
#pragma unroll
    for (int i = LIMBS - 1; i >= 0; --i) {
      const uint32_t hv = i < kCrtLimbs ? t.H[i] : 0u;
      if (!decided && d[i] != hv) {
        gt = d[i] > hv;
        decided = true;
      }
    }
    if (gt) {
      int64_t bb = 0;
#pragma unroll
      for (int i = 0; i < LIMBS; ++i) {
        bb += static_cast<int64_t>(t.P[i]) - static_cast<int64_t>(d[i]);
        d[i] = static_cast<uint32_t>(bb);
        bb >>= 32;
      }
      ng = true;
    }
  }
#pragma unroll
  for (int i = 0; i < LIMBS; ++i) mag[i] = d[i];
  *neg = ng;
}

// 64 bits of mag starting at bit position pos (pos >= 0).
template <int LIMBS>
__device__ __forceinline__ uint64_t bits_at(const uint32_t* mag, int pos) {
  const int w = pos >> 5, s = pos & 31;
  uint64_t lo = 0, mid = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < LIMBS; ++i) {
    if (i == w) lo = mag[i];
    if (i == w + 1) mid = mag[i];
    if (i == w + 2) hi = mag[i];
  }
  uint64_t v = (lo >> s) | (mid << (32 - s));
  if (s) v |= hi << (64 - s);
  return v;
}

// any bit of mag strictly below position pos
template <int LIMBS>
__device__ __forceinline__ bool any_below(const uint32_t* mag, int pos) {
  bool any = false;
#pragma unroll
  for (int i = 0; i < LIMBS; ++i) {
    if (32 * (i + 1) <= pos) any |= mag[i] != 0;
    else if (32 * i < pos) any |= (mag[i] & ((1u << (pos - 32 * i)) - 1)) != 0;
  }
  return any;
}

// RN-even binary64 of (+-mag) 2^e with a single rounding: gradual underflow and overflow exact;
// mag == 0 gives +0; a nonzero value that rounds to zero keeps its sign.
template <int LIMBS>
__device__ __forceinline__ double round_scaled(const uint32_t* mag, bool neg, int e) {
  int bl = 0;
#pragma unroll
  for (int i = 0; i < LIMBS; ++i)
    if (mag[i]) bl = 32 * i + 32 - __clz(static_cast<int>(mag[i]));
  if (bl == 0) return 0.0;
  const int top = bl - 1 + e;
  int q = top - 52;
  if (q < -1074) q = -1074;
  uint64_t r;
  if (q <= e) {
    r = bits_at<LIMBS>(mag, 0) << (e - q);  // bl <= 53 here
  } else {
    const int sh = q - e;
    if (sh > 32 * LIMBS) {
      r = 0;  // below half of the smallest subnormal
    } else {
      r = sh >= 32 * LIMBS ? 0 : bits_at<LIMBS>(mag, sh);
      const bool halfbit = (bits_at<LIMBS>(mag, sh - 1) & 1) != 0;
      if (halfbit && (any_below<LIMBS>(mag, sh - 1) || (r & 1))) r += 1;
    }
  }
  const uint64_t sign = neg ? 0x8000000000000000ull : 0ull;
  if (r == 0) return __longlong_as_double(static_cast<long long>(sign));
  if (r == (1ull << 53)) {
    r >>= 1;
    q += 1;
  }
  const int rb = 64 - __clzll(static_cast<long long>(r));
  if (rb - 1 + q >= 1024) return __longlong_as_double(static_cast<long long>(sign | 0x7FF0000000000000ull));
  uint64_t out;
  if (rb == 53) out = (static_cast<uint64_t>(q + 1075) << 52) | (r & 0xFFFFFFFFFFFFFull);
  else out = r;  // subnormal: q == -1074
  return __longlong_as_double(static_cast<long long>(sign | out));
}

}  // namespace dev
}  // namespace imd
