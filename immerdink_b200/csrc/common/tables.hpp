// Plan-time constants of the residue number system, derived at run time from first principles
// (no generated header): the greedy pairwise-coprime moduli from 256 downwards, P, H = P/2 - 1,
// T = floor(sqrt(H)), the CRT weights M_l = P / p_l and q_l = M_l^-1 mod p_l, and the 32-bit
// magic numbers of the modular reductions. Semantics follow the reference's constants
// (include/immerdink/detail/constants.hpp:43-66; rule in docs/DESIGN.md:153-169).
#pragma once
#include <cstdint>

#include "wide.hpp"

namespace imd {

constexpr int kMinModuli = 2;
constexpr int kMaxModuli = 20;
constexpr int kFracBits = 60;            // fixed-point fraction bits of the sum of squares S
constexpr int64_t kChunkMax = 131071;    // floor((2^31 - 1) / 128^2): int32 cannot overflow
constexpr int64_t kChunk = 130944;       // chunk length used: 1023 K blocks of 128 (<= kChunkMax)
constexpr int kRegionAlign = 256;
constexpr int kCrtLimbs = 5;             // 32-bit limbs of the widest unreduced CRT sum (N P < 2^160)
constexpr int kBigLimbs = 10;            // 320-bit scratch for plan-time arithmetic

constexpr int kModuli[kMaxModuli] = {256, 255, 253, 251, 247, 241, 239, 233, 229, 227,
                                     223, 217, 211, 199, 197, 193, 191, 181, 179, 173};

using Big = Wide<kBigLimbs>;

// Everything the kernels need for one N; passed to kernels by value inside their parameters.
struct CrtTables {
  int32_t N;
  int32_t limbs;                       // 32-bit limbs that hold N * P
  uint32_t p[kMaxModuli];
  uint32_t q[kMaxModuli];              // M_l^-1 mod p_l
  uint32_t magic[kMaxModuli];          // ceil(2^32 / p_l): floor(v / p) = umulhi(v, magic), v < 2^24
  uint32_t frac[kMaxModuli];           // floor(2^27 / p_l): fixed-point 1 / p_l for the quotient estimate
  uint32_t M[kMaxModuli][kCrtLimbs];   // P / p_l
  uint32_t P[kCrtLimbs];
  uint32_t H[kCrtLimbs];               // P / 2 - 1: the largest representable |z|
};

// Constants of the residue emitter for one N (uniform across a warp: kernels take them by value
// and read them from the constant bank).
struct ResidueTables {
  int32_t N;
  int32_t words;                         // 32-bit words of |a'|: 2 (N <= 16) or 3
  uint32_t p[kMaxModuli];
  uint32_t half[kMaxModuli];             // floor(p / 2)
  uint32_t magic[kMaxModuli];            // ceil(2^32 / p)
  uint32_t lift[kMaxModuli];             // a multiple of p >= 2^20: makes negated sums nonnegative
  uint32_t weight[3][kMaxModuli];        // 4 packed byte weights 2^(8 (4 j + i)) mod p
};

inline ResidueTables residue_tables(int N) {
  ResidueTables t{};
  t.N = N;
  t.words = N <= 16 ? 2 : 3;
  for (int l = 0; l < N; ++l) {
    const uint32_t p = static_cast<uint32_t>(kModuli[l]);
    t.p[l] = p;
    t.half[l] = p / 2;
    t.magic[l] = static_cast<uint32_t>(((uint64_t{1} << 32) + p - 1) / p);
    t.lift[l] = ((1u << 20) + p - 1) / p * p;
    uint32_t pw = 1 % p;
    for (int j = 0; j < 3; ++j) {
      uint32_t word = 0;
      for (int i = 0; i < 4; ++i) {
        word |= pw << (8 * i);
        pw = (pw * 256u) % p;
      }
      t.weight[j][l] = word;
    }
  }
  return t;
}

struct PlanConstants {
  Big P, H, T;
};

inline PlanConstants plan_constants(int N) {
  PlanConstants c;
  c.P = wide_u64<kBigLimbs>(1);
  for (int l = 0; l < N; ++l) c.P = wide_mul_small(c.P, static_cast<uint32_t>(kModuli[l]));
  c.H = wide_sub(wide_shr(c.P, 1), wide_u64<kBigLimbs>(1));
  c.T = wide_isqrt(c.H);
  return c;
}

inline CrtTables crt_tables(int N) {
  CrtTables t{};
  const PlanConstants c = plan_constants(N);
  t.N = N;
  const Big NP = wide_mul_small(c.P, static_cast<uint32_t>(N));
  t.limbs = (wide_bitlen(NP) + 31) / 32;
  for (int i = 0; i < kCrtLimbs; ++i) {
    t.P[i] = c.P.w[i];
    t.H[i] = c.H.w[i];
  }
  for (int l = 0; l < N; ++l) {
    const uint32_t p = static_cast<uint32_t>(kModuli[l]);
    t.p[l] = p;
    t.magic[l] = static_cast<uint32_t>(((uint64_t{1} << 32) + p - 1) / p);
    t.frac[l] = (1u << 27) / p;
    Big M = c.P;
    wide_divmod_small(&M, p);
    for (int i = 0; i < kCrtLimbs; ++i) t.M[l][i] = M.w[i];
    Big tmp = M;
    const uint32_t r = wide_divmod_small(&tmp, p);
    for (uint32_t x = 1; x < p; ++x)
      if ((r * x) % p == 1) {
        t.q[l] = x;
        break;
      }
  }
  return t;
}

inline uint64_t ceil_sqrt_u64(uint64_t k) {
  if (k == 0) return 0;
  uint64_t lo = 0, hi = uint64_t{1} << 32;  // smallest r with r * r >= k
  while (lo < hi) {
    const uint64_t mid = lo + (hi - lo) / 2;
    if (static_cast<unsigned __int128>(mid) * mid >= k) hi = mid;
    else lo = mid + 1;
  }
  return lo;
}

// RN acceptance: a plan is rejected when ceil(sqrt k) >= T.
inline bool kappa_at_least_T(uint64_t kappa, int N) {
  return wide_cmp(wide_u64<kBigLimbs>(kappa), plan_constants(N).T) >= 0;
}

// Right-hand side of the shift rule: (2T - kappa)^2 2^60 (RN) or T^2 2^60 (TRUNC), 256 bits.
inline Wide<8> shift_rhs(int N, bool rn, uint64_t k) {
  const PlanConstants c = plan_constants(N);
  Big base = c.T;
  if (rn) base = wide_sub(wide_shl(c.T, 1), wide_u64<kBigLimbs>(ceil_sqrt_u64(k)));
  const Big r = wide_shl(wide_mul(base, base), kFracBits);
  Wide<8> out;
  for (int i = 0; i < 8; ++i) out.w[i] = r.w[i];
  return out;
}

}  // namespace imd
