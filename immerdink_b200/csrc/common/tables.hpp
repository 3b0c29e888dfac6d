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
// Chunk of K the int8 GEMM accumulates before its epilogue adds into the planes mod p: 64 K blocks of
// 128 (far below kChunkMax). A 256-row tile of one chunk is 2 MB, so the tile rows of A and B that
// one wave of CTA pairs works on stay in L2 (16384^3: 67.5 ms with one chunk, 58.5 ms with two).
constexpr int64_t kChunk = 8192;
constexpr int kRegionAlign = 256;
constexpr int kBigLimbs = 10;            // 320-bit scratch for plan-time arithmetic

constexpr int kModuli[kMaxModuli] = {256, 255, 253, 251, 247, 241, 239, 233, 229, 227,
                                     223, 217, 211, 199, 197, 193, 191, 181, 179, 173};

using Big = Wide<kBigLimbs>;

// Everything the CRT kernel needs for one N; passed by value inside the kernel parameters.
// The unreduced sum S = sum_l M_l y_l is accumulated on `nl` carry-free limbs of `lw` bits (each
// limb sum stays below 2^32), then normalised to `words` 32-bit words.
constexpr int kCrtWords = 6;     // 32-bit words of the widest S (N P < 2^160, limbs up to 171 bits)
constexpr int kCrtMaxLimbs = 9;

// Constants of the CRT kernel's floating-point shortcut (dev::crt_fast). With 1 / p_l = rh_l + rl_l,
// rh_l a multiple of 2^-46, the centred fraction f = sum_l y_l / p_l - Q (Q the nearest integer)
// is fh + sl: fh = sum_l y_l rh_l - Q comes out exactly in binary64 (every partial sum is a
// multiple of 2^-46 below 64), sl = sum_l y_l rl_l is tiny (below 2^-33) and rounded. The digits
// enter as 256 + y_l (one shift and one mask build that double), and k0h, k0l take the 256 out
// again. z = P f is then formed in double-double; `eabs` bounds its absolute error, rmax_hi is the
// high word of a magnitude safely inside P / 2.
struct CrtFast {
  double rh[kMaxModuli], rl[kMaxModuli];
  double k0h, k0l;
  double Ph, Pl;       // P = Ph + Pl + (less than 2^-105 P)
  double eabs;
  int32_t rmax_hi;
};

struct CrtTables {
  int32_t N;
  int32_t nl, lw;                      // limbs and limb width: 20 bits for N <= 16, else 19
  int32_t words;                       // 32-bit words = ceil(nl * lw / 32)
  int32_t qshift;                      // S >> qshift and rinv give the multiple of P to subtract
  uint32_t rinv;                       // floor(2^(qshift + 57 - ...) / P), see crt_tables()
  int32_t rshift;                      // final right shift of umulhi(S >> qshift, rinv)
  uint32_t p[kMaxModuli];
  uint32_t q[kMaxModuli];              // M_l^-1 mod p_l (applied by the GEMM epilogue)
  uint32_t M[kMaxModuli][kCrtMaxLimbs];  // limbs of P / p_l
  uint32_t P[kCrtWords];
  uint32_t H[kCrtWords];               // P / 2 - 1: the largest representable |z|
  CrtFast fast;
};

// Constants of the residue emitter for one N (uniform across a warp: kernels take them by value
// and read them from the constant bank). The quantised integer is split into signed base-256
// digits d_j in [-128, 127]; s = sum_j d_j w_j with signed weights w_j = SMod(256^j, p) is formed
// by dp4a on top of `lift`, a multiple of p that keeps the sum positive; u = (s + lift) mod p is
// the nonnegative residue, and the symmetric representative is u - p when u > ceil(p / 2) - 1.
struct ResidueTables {
  int32_t N;
  int32_t words;                         // 32-bit words of the quantised integer: 2 (N <= 16) or 3
  uint32_t p[kMaxModuli];
  uint32_t magic[kMaxModuli];            // ceil(2^32 / p): floor(v / p) = umulhi(v, magic), v < 2^24
  uint32_t lift[kMaxModuli];             // multiple of p, >= 2^18 > max |s|
  uint32_t fix_add[kMaxModuli];          // (127 - (ceil(p/2) - 1)) in every byte
  uint32_t fix_mul[kMaxModuli];          // 256 - p (0 for p = 256): added to bytes above the half
  uint32_t weight[3][kMaxModuli];        // 4 packed signed weights SMod(256^(4 j + i), p)
};

inline ResidueTables residue_tables(int N) {
  ResidueTables t{};
  t.N = N;
  t.words = N <= 16 ? 2 : 3;
  for (int l = 0; l < N; ++l) {
    const uint32_t p = static_cast<uint32_t>(kModuli[l]);
    t.p[l] = p;
    t.magic[l] = static_cast<uint32_t>(((uint64_t{1} << 32) + p - 1) / p);
    t.lift[l] = ((1u << 18) + p - 1) / p * p;
    const uint32_t top = (p + 1) / 2 - 1;  // largest nonnegative symmetric residue
    t.fix_add[l] = (127u - top) * 0x01010101u;
    t.fix_mul[l] = 256u - p;
    uint32_t pw = 1 % p;
    for (int j = 0; j < 3; ++j) {
      uint32_t word = 0;
      for (int i = 0; i < 4; ++i) {
        const int sym = static_cast<int>((pw + p / 2) % p) - static_cast<int>(p / 2);
        word |= (static_cast<uint32_t>(sym) & 0xFFu) << (8 * i);
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

// 53 bits of x starting `skip` bits below its leading bit, as an exact double (0 when x has fewer).
inline double wide_bits_as_double(const Big& x, int skip) {
  const int B = wide_bitlen(x);
  if (B <= skip) return 0.0;
  const int low = B - skip - 53;  // position of the last bit taken
  const Big sh = low >= 0 ? wide_shr(x, low) : wide_shl(x, -low);
  const uint64_t m = (sh.w[0] | (static_cast<uint64_t>(sh.w[1]) << 32)) & ((uint64_t{1} << 53) - 1);
  double v = static_cast<double>(m);  // exact: 53 bits
  for (int i = 0; i < (low >= 0 ? low : -low); ++i) v = low >= 0 ? v * 2.0 : v * 0.5;
  return v;
}

inline CrtFast crt_fast_tables(int N, const Big& P) {
  CrtFast f{};
  int64_t ksum = 0;
  __int128 nsum = 0;  // sum_l n_l 2^64 / p_l, each term within one unit
  for (int l = 0; l < N; ++l) {
    const int64_t p = kModuli[l];
    const int64_t k = ((int64_t{1} << 46) + p / 2) / p;
    const int64_t n = (int64_t{1} << 46) - k * p;  // 1 / p = (k + n / p) 2^-46, |n| <= p / 2
    f.rh[l] = static_cast<double>(k) * 0x1p-46;
    f.rl[l] = static_cast<double>(n) / static_cast<double>(p) * 0x1p-46;
    ksum += k;
    nsum += (static_cast<__int128>(n) << 64) / p;
  }
  f.k0h = -static_cast<double>(ksum * 256) * 0x1p-46;                    // exact: below 2^52
  f.k0l = -static_cast<double>(nsum) * 0x1p-64 * 256.0 * 0x1p-46;
  f.Ph = wide_bits_as_double(P, 0);
  f.Pl = wide_bits_as_double(P, 53);
  // Error of fh + sl against the exact f. The partial sums of sl stay below maxpart, so each of
  // its N fused multiply-adds errs by at most half an ulp of `ub`; the stored rl_l and k0l carry
  // their own roundings. z adds the roundings of the double-double product.
  const double maxpart = N * 767.0 * 0x1p-47;
  double ub = 0x1p-60;
  while (ub < maxpart) ub *= 2.0;
  const double ef = N * ub * 0x1p-53 + N * 511.0 * 0x1p-100 + N * 256.0 * 0x1p-100 + N * 0x1p-102;
  const double ex = ef + 4.0 * 0x1p-53 * (maxpart + 0x1p-50) + 0x1p-104;
  f.eabs = 2.0 * f.Ph * ex;
  const double rmax = f.Ph * (0.5 - 0x1p-20);
  uint64_t bits;
  static_assert(sizeof(bits) == sizeof(rmax), "binary64");
  __builtin_memcpy(&bits, &rmax, 8);
  f.rmax_hi = static_cast<int32_t>(bits >> 32);
  return f;
}

inline CrtTables crt_tables(int N) {
  CrtTables t{};
  const PlanConstants c = plan_constants(N);
  t.fast = crt_fast_tables(N, c.P);
  t.N = N;
  const Big NP = wide_mul_small(c.P, static_cast<uint32_t>(N));
  t.lw = N <= 16 ? 20 : 19;
  t.nl = (wide_bitlen(NP) + t.lw - 1) / t.lw;
  t.words = (t.nl * t.lw + 31) / 32;
  for (int i = 0; i < kCrtWords; ++i) {
    t.P[i] = c.P.w[i];
    t.H[i] = c.H.w[i];
  }
  // Quotient estimate: x_lo = ((S >> qshift) * rinv) >> (32 + rshift) <= S / P, within 2^-20.
  // S >> qshift < 2^32 because S < N P < 2^(bitlen(P) + 5) and qshift = bitlen(P) - 27.
  const int B = wide_bitlen(c.P);
  t.qshift = B > 27 ? B - 27 : 0;
  {
    // rinv = floor(2^(qshift + F) / P) with F chosen so that rinv has 31 bits
    int F = 31 + B - t.qshift;          // 2^(qshift + F) / P is about 2^(31 + (B - log2 P)) < 2^32
    Big num = wide_shl(wide_u64<kBigLimbs>(1), t.qshift + F);
    // long division by P via bitwise restoring division (plan time only)
    Big quo = wide_zero<kBigLimbs>(), rem = wide_zero<kBigLimbs>();
    for (int bit = wide_bitlen(num) - 1; bit >= 0; --bit) {
      rem = wide_shl(rem, 1);
      rem.w[0] |= (num.w[bit >> 5] >> (bit & 31)) & 1u;
      if (wide_cmp(rem, c.P) >= 0) {
        rem = wide_sub(rem, c.P);
        quo.w[bit >> 5] |= 1u << (bit & 31);
      }
    }
    while (quo.w[1] != 0) {  // keep it in 32 bits
      quo = wide_shr(quo, 1);
      --F;
    }
    t.rinv = quo.w[0];
    t.rshift = F - 32;                  // x_lo 2^rshift = umulhi(S >> qshift, rinv)
  }
  for (int l = 0; l < N; ++l) {
    const uint32_t p = static_cast<uint32_t>(kModuli[l]);
    t.p[l] = p;
    Big M = c.P;
    wide_divmod_small(&M, p);
    for (int i = 0; i < t.nl; ++i)
      t.M[l][i] = wide_shr(M, i * t.lw).w[0] & ((1u << t.lw) - 1);
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

// Plan-time constants of the FP64 shortcut of the shift rule (dev::fast_shift): the right-hand
// side as rm 2^re with rm in [rm_lo, rm_hi] (both in [1, 2]), and the factors that turn a
// floating-point sum of k squares into an enclosure of the exact fixed-point sum S (each of the
// k additions errs by at most 2^-53 relative, every ceiling adds less than one unit of 2^-60 to
// a sum that is at least 1).
struct ShiftFast {
  double rm_lo, rm_hi;
  double lo_scale, hi_scale;
  int32_t re;
  int32_t usable;  // 0: always take the exact path (k beyond 2^36)
};

inline ShiftFast shift_fast(const Wide<8>& rhs, uint64_t k) {
  ShiftFast f{};
  const int B = wide_bitlen(rhs);
  if (B < 54 || k > (uint64_t{1} << 36)) return f;
  const Wide<8> top = wide_shr(rhs, B - 53);
  const uint64_t mant = top.w[0] | (static_cast<uint64_t>(top.w[1]) << 32);  // 2^52 <= mant < 2^53
  f.rm_lo = static_cast<double>(mant) * 0x1p-52;
  f.rm_hi = static_cast<double>(mant + 1) * 0x1p-52;
  f.re = B - 1;
  const double kd = static_cast<double>(k);
  f.lo_scale = 1.0 - (kd + 512.0) * 0x1p-51;
  f.hi_scale = 1.0 + (kd + 512.0) * 0x1p-51 + (kd + 1.0) * 0x1p-59;
  f.usable = 1;
  return f;
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
