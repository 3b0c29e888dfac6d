// Exact device numerics of the emulated contraction: everything here is integer arithmetic on
// FP64 bit patterns (the only floating-point operations are the native FMA chain of flagged
// outputs and the alpha / beta epilogue). Each function states the rule it implements; the rules
// are those of the reference's specification (spec/oracle.py: scale_vector :361-408, quantize
// :415-435, residue :438-448, crt :498-512, round_dyadic :257-283), realised with this
// engine's own algorithms (byte-weight residues, unreduced CRT sum with a fixed-point quotient
// estimate).
#pragma once
#include <cstdint>

#include "carry.cuh"
#include "common/crtfast.hpp"
#include "common/modred.hpp"
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

// The shift from one floating-point pass over a row. mx = the largest high word of |a_h| (sign
// cleared), acc = the FP64 sum of the squares a_h^2 in any order. With gamma = ilogb of the
// largest entry, S 2^(2 gamma - 60) lies in [acc lo_scale, acc hi_scale] (see ShiftFast), so
// t = rhs / (S << lhs_shift) is enclosed by two directed divisions; u = floor(log4 t) is decided
// when both ends agree. Rows with a non-finite entry, without a normal entry, or with
// |gamma| > 400 (squares could leave the normal range) are left to the exact integer path.
__device__ __forceinline__ bool fast_shift(uint32_t mx, double acc, const ShiftFast& c,
                                           int lhs_shift, int* sigma) {
  const int ef = static_cast<int>(mx >> 20);
  if (!c.usable || ef < 1023 - 400 || ef > 1023 + 400 || !(acc > 0.0)) return false;
  const int gamma = ef - 1023;
  const double lo = __dmul_rd(acc, c.lo_scale), hi = __dmul_ru(acc, c.hi_scale);
  const double t_lo = __ddiv_rd(c.rm_lo, hi), t_hi = __ddiv_ru(c.rm_hi, lo);
  const int E = c.re - kFracBits + 2 * gamma - lhs_shift;
  const int e_lo = (static_cast<int>(__double_as_longlong(t_lo) >> 52) & 0x7FF) - 1023 + E;
  const int e_hi = (static_cast<int>(__double_as_longlong(t_hi) >> 52) & 0x7FF) - 1023 + E;
  if ((e_lo >> 1) != (e_hi >> 1)) return false;
  *sigma = (e_lo >> 1) - gamma;
  return true;
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

// Quantised value as a two's complement integer, fast path for N <= 16 (|a'| < 2^63): scale the
// double by 2^sigma exactly (exponent add) and let the conversion unit round to nearest even (or
// toward zero). Zeros, subnormals and non-finite inputs take the integer path.
__device__ __forceinline__ int64_t quantize_i64(uint64_t bits, int sigma, bool trunc) {
  const int ef = static_cast<int>((bits >> 52) & 0x7FF);
  if (ef == 0 || ef == 0x7FF) {
    uint64_t lo;
    uint32_t hi;
    bool neg;
    quantize(bits, sigma, trunc, &lo, &hi, &neg);
    return neg ? -static_cast<int64_t>(lo) : static_cast<int64_t>(lo);
  }
  const int en = ef + sigma;
  if (en <= 0) return 0;  // |a 2^sigma| < 2^-1022
  const uint64_t scaled = (bits & 0x800FFFFFFFFFFFFFull) | (static_cast<uint64_t>(en) << 52);
  const double v = __longlong_as_double(static_cast<long long>(scaled));
  return trunc ? __double2ll_rz(v) : __double2ll_rn(v);
}

// Signed base-256 digits of a two's complement integer: adding 0x80 to every byte but the top one
// (with carries) and flipping those bits back turns each byte into a digit in [-128, 127].
__device__ __forceinline__ void signed_digits64(int64_t x, uint32_t* d0, uint32_t* d1) {
  imd::signed_digits64(x, d0, d1);
}
__device__ __forceinline__ void signed_digits96(uint64_t lo, uint32_t hi, bool neg, uint32_t* d0,
                                                uint32_t* d1, uint32_t* d2) {
  if (neg) {  // two's complement on 96 bits
    lo = ~lo + 1;
    hi = ~hi + (lo == 0 ? 1u : 0u);
  }
  const uint64_t k = 0x8080808080808080ull;
  const uint64_t ylo = lo + k;
  const uint32_t yhi = hi + 0x00808080u + (ylo < lo ? 1u : 0u);
  *d0 = static_cast<uint32_t>(ylo ^ k);
  *d1 = static_cast<uint32_t>((ylo ^ k) >> 32);
  *d2 = yhi ^ 0x00808080u;
}

// Nonnegative residue u in [0, p) of the integer with signed digits (d0, d1, d2), modulus index l.
template <int WORDS>
__device__ __forceinline__ uint32_t residue_u(const ResidueTables& t, int l, uint32_t d0,
                                              uint32_t d1, uint32_t d2) {
  int s = __dp4a(static_cast<int>(d0), static_cast<int>(t.weight[0][l]), static_cast<int>(t.lift[l]));
  s = __dp4a(static_cast<int>(d1), static_cast<int>(t.weight[1][l]), s);
  if (WORDS > 2) s = __dp4a(static_cast<int>(d2), static_cast<int>(t.weight[2][l]), s);
  const uint32_t v = static_cast<uint32_t>(s);  // 0 < v < 2^24
  return v - t.p[l] * __umulhi(v, t.magic[l]);
}

// Four residues u (one per byte, each < p) -> four symmetric residues as two's complement bytes.
__device__ __forceinline__ uint32_t symmetric4(const ResidueTables& t, int l, uint32_t packed) {
  const uint32_t above = ((packed + t.fix_add[l]) >> 7) & 0x01010101u;  // 1 where u > ceil(p/2) - 1
  return above * t.fix_mul[l] + packed;                                 // u + 256 - p there
}

using imd::reduce_sym;

// ---- CRT ------------------------------------------------------------------------------------
// z = centred representative of the residues, as sign + magnitude on WORDS 32-bit words.
// The product planes already hold y_l = (q_l W_l) mod p_l (the GEMM epilogue multiplies by q_l).
// S = sum_l M_l y_l is accumulated on NL carry-free limbs (limb sums < 2^32), normalised once,
// and not reduced on the way: the multiple of P to subtract is floor(x_lo + 1/2) for an
// underestimate x_lo of S / P taken from the top 32 bits of S (within 2^-20), so that
// S - q P lies in [-P/2, P/2 + P 2^-20) and one exact comparison with H finishes the centring.
// Limbs of the unreduced sum per N (20-bit limbs up to N = 16, 19-bit above): ceil(bitlen(N P) / lw).
__host__ __device__ constexpr int crt_limbs_of(int N) {
  constexpr int t[21] = {0, 0, 1, 2, 2, 3, 3, 3, 4, 4, 5, 5, 5, 6, 6, 7, 7, 8, 8, 9, 9};
  return t[N];
}
template <int N>
struct CrtShape {
  static constexpr int kNl = crt_limbs_of(N);
  static constexpr int kLw = N <= 16 ? 20 : 19;
  static constexpr int kWords = (kNl * kLw + 31) / 32;
};

// Residue l is byte LANE of packed[l]. Returns the magnitude of z in mag[] and its sign.
template <int N, int LANE>
__device__ __forceinline__ bool crt(const CrtTables& t, const uint32_t* packed, uint32_t* mag) {
  constexpr int NL = CrtShape<N>::kNl, LW = CrtShape<N>::kLw, WORDS = CrtShape<N>::kWords;
  uint32_t acc[NL];
#pragma unroll
  for (int i = 0; i < NL; ++i) acc[i] = 0;
#pragma unroll
  for (int l = 0; l < N; ++l) {
    const uint32_t y = (packed[l] >> (8 * LANE)) & 0xFFu;
#pragma unroll
    for (int i = 0; i < NL; ++i) acc[i] += t.M[l][i] * y;
  }
  // limbs -> 32-bit words
  uint32_t S[WORDS];
  {
    uint64_t carry = 0;  // bits of the running sum at and above the current word
    int word = 0;
#pragma unroll
    for (int i = 0; i < NL; ++i) {
      const int off = i * LW - 32 * word;  // bit offset of limb i inside `carry` (0 <= off < 32)
      carry += static_cast<uint64_t>(acc[i]) << off;
      if ((i + 1) * LW >= 32 * (word + 1) || i == NL - 1) {
        if (word < WORDS) S[word] = static_cast<uint32_t>(carry);
        carry >>= 32;
        ++word;
      }
    }
#pragma unroll
    for (int wd = word; wd < WORDS; ++wd) {
      S[wd] = static_cast<uint32_t>(carry);
      carry >>= 32;
    }
  }
  // multiple of P to subtract
  uint32_t top;
  {
    const int w = t.qshift >> 5, sh = t.qshift & 31;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < WORDS; ++i) {
      if (i == w) lo = S[i];
      if (i == w + 1) hi = S[i];
    }
    top = __funnelshift_r(lo, hi, sh);
  }
  const uint32_t q = (__umulhi(top, t.rinv) + (1u << (t.rshift - 1))) >> t.rshift;
  uint32_t Q[WORDS];
  {
    uint64_t mul = 0;
#pragma unroll
    for (int i = 0; i < WORDS; ++i) {
      mul += static_cast<uint64_t>(t.P[i]) * q;
      Q[i] = static_cast<uint32_t>(mul);
      mul >>= 32;
    }
  }
  uint32_t d1[WORDS], d2[WORDS];
  const uint32_t below = Words<WORDS>::sub(d1, S, Q);  // S - Q
  Words<WORDS>::sub(d2, Q, S);                         // Q - S
#pragma unroll
  for (int i = 0; i < WORDS; ++i) mag[i] = below ? d2[i] : d1[i];
  bool neg = below != 0;
  if (!neg) {
    // S - Q in [0, P/2 + P 2^-20): above H only at the very edge of the range
    uint32_t tmp[WORDS], Hw[WORDS];
#pragma unroll
    for (int i = 0; i < WORDS; ++i) Hw[i] = t.H[i];
    if (Words<WORDS>::sub(tmp, Hw, mag)) {
      uint32_t Pw[WORDS];
#pragma unroll
      for (int i = 0; i < WORDS; ++i) Pw[i] = t.P[i];
      Words<WORDS>::sub(tmp, Pw, mag);
#pragma unroll
      for (int i = 0; i < WORDS; ++i) mag[i] = tmp[i];
      neg = true;
    }
  }
  return neg;
}

// Residue l of the thread's output x (byte x of packed[l]) as the double 256 + y: exponent 2^8, y
// in the top eight bits of the fraction. One shift and one mask-or (x is a constant after unrolling).
struct PackedDigit {
  const uint32_t* packed;
  __device__ __forceinline__ double operator()(int l, int x) const {
    const uint32_t at12 = x == 0 ? packed[l] << 12 : x == 1 ? packed[l] << 4
                        : x == 2 ? packed[l] >> 4 : packed[l] >> 12;
    return __hiloint2double(static_cast<int>((at12 & 0x000FF000u) | 0x40700000u), 0);
  }
};

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

// The same value by the conversion unit when the result is a normal number: the magnitude is
// shifted left until its leading bit is bit 32 LIMBS - 1; the top 64 bits, with every lower bit
// folded into a sticky last bit, are rounded once by the u64 -> f64 conversion (64 bits leave 11
// guard bits, so the sticky bit decides ties correctly), and the power of two is an exponent add.
// Zero, subnormal and overflowing results take the exact integer path.
template <int LIMBS>
__device__ __noinline__ double round_scaled_slow(const uint32_t* mag, bool neg, int e) {
  return round_scaled<LIMBS>(mag, neg, e);
}

template <int LIMBS>
__device__ __forceinline__ double round_scaled_fast(const uint32_t* mag, bool neg, int e) {
  uint32_t w[LIMBS];
#pragma unroll
  for (int i = 0; i < LIMBS; ++i) w[i] = mag[i];
  int lz = 0;  // leading zero bits of the LIMBS-word number
  // whole words first (static cascade), then bits
#pragma unroll
  for (int step = 0; step < LIMBS - 1; ++step) {
    if (w[LIMBS - 1] == 0) {
#pragma unroll
      for (int i = LIMBS - 1; i > 0; --i) w[i] = w[i - 1];
      w[0] = 0;
      lz += 32;
    }
  }
  if (w[LIMBS - 1] == 0) return 0.0;
  const int s = __clz(static_cast<int>(w[LIMBS - 1]));
  lz += s;
  uint32_t hi, mid, rest = 0;
  if (LIMBS == 1) {
    hi = w[0] << s;
    mid = 0;
  } else {
    hi = __funnelshift_l(w[LIMBS - 2], w[LIMBS - 1], s);
    mid = __funnelshift_l(LIMBS > 2 ? w[LIMBS - 3] : 0u, w[LIMBS - 2], s);
    if (LIMBS > 2) rest = w[LIMBS - 3] << s;
#pragma unroll
    for (int i = 0; i < LIMBS - 3; ++i) rest |= w[i];
  }
  const uint64_t top = (static_cast<uint64_t>(hi) << 32) | mid | (rest != 0 ? 1u : 0u);
  const double v = __ull2double_rn(top);                    // in [2^63, 2^64]
  const long long vb = __double_as_longlong(v);
  const int shift = 32 * LIMBS - 64 - lz + e;               // value = v 2^shift
  const int ex = static_cast<int>(vb >> 52) + shift;        // biased exponent of the result
  if (ex >= 1 && ex <= 2046) {
    const long long out = vb + (static_cast<long long>(shift) << 52);
    return __longlong_as_double(neg ? (out | static_cast<long long>(0x8000000000000000ull)) : out);
  }
  return round_scaled_slow<LIMBS>(mag, neg, e);
}

}  // namespace dev
}  // namespace imd
