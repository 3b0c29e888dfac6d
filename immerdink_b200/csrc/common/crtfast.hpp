// Floating-point shortcut of the CRT kernel as a host + device function, so that a host program can
// run it against exact integer arithmetic (tests/test_crt_fast.py).
//
// The planes hold y_l = q_l acc_l mod p_l, so the centred value is z = P f with
// f = sum_l y_l / p_l - Q, Q the nearest integer (rule: spec/oracle.py:498-512; the reference's
// kernel, src/kernels/numerics.cuh:268-334, works on integer words throughout). Here f comes out of two
// FP64 sums (CrtFast in tables.hpp), z out of a double-double product, and the kernel's integer
// path remains for every output whose rounding this arithmetic cannot vouch for.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

#include "tables.hpp"

namespace imd {

IMD_HD double f64_from_words(int32_t hi, int32_t lo) {
#if defined(__CUDA_ARCH__)
  return __hiloint2double(hi, lo);
#else
  const uint64_t b = (static_cast<uint64_t>(static_cast<uint32_t>(hi)) << 32) | static_cast<uint32_t>(lo);
  double d;
  std::memcpy(&d, &b, 8);
  return d;
#endif
}
IMD_HD void f64_words(double d, int32_t* hi, int32_t* lo) {
#if defined(__CUDA_ARCH__)
  *hi = __double2hiint(d);
  *lo = __double2loint(d);
#else
  uint64_t b;
  std::memcpy(&b, &d, 8);
  *hi = static_cast<int32_t>(b >> 32);
  *lo = static_cast<int32_t>(b);
#endif
}
IMD_HD double f64_fma(double a, double b, double c) {
#if defined(__CUDA_ARCH__)
  return __fma_rn(a, b, c);
#else
  return std::fma(a, b, c);
#endif
}
IMD_HD double f64_add(double a, double b) {  // never contracted into a neighbouring multiply
#if defined(__CUDA_ARCH__)
  return __dadd_rn(a, b);
#else
  volatile double s = a + b;
  return s;
#endif
}
IMD_HD double f64_mul(double a, double b) {
#if defined(__CUDA_ARCH__)
  return __dmul_rn(a, b);
#else
  volatile double s = a * b;
  return s;
#endif
}

// The two sums of LANES outputs side by side (every constant is fetched once per modulus and used
// for all of them): digit(l, x) returns the double 256 + y_l of output x. `off` is zero; a kernel
// passes a zero the compiler cannot see through, so that the constants are fetched where they are
// used instead of being held in registers across its row loop.
template <int N, int LANES, class Digit>
IMD_HD void crt_fast_sums(const CrtFast& f, Digit digit, int off, double* sh, double* sl) {
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int x = 0; x < LANES; ++x) sh[x] = f.k0h, sl[x] = f.k0l;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int l = 0; l < N; ++l) {
    const double rh = f.rh[l + off], rl = f.rl[l + off];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int x = 0; x < LANES; ++x) {
      const double d = digit(l, x);
      sh[x] = f64_fma(d, rh, sh[x]);
      sl[x] = f64_fma(d, rl, sl[x]);
    }
  }
}

// xh + xl is the double-double value of z = P f, within f.eabs of it, with |xl| <= 2^-30 P.
IMD_HD void crt_fast_value(const CrtFast& f, double sh, double sl, double* xh_out, double* xl_out) {
  const double Q = f64_add(f64_add(sh, 6755399441055744.0), -6755399441055744.0);
  const double fh = f64_add(sh, -Q);                        // exact, |fh| <= 1/2
  const double xh = f64_mul(f.Ph, fh);
  const double xe = f64_fma(f.Ph, fh, -xh);                 // exact
  *xh_out = xh;
  *xl_out = f64_fma(f.Ph, sl, f64_fma(f.Pl, fh, xe));
}

// e is the power of two applied to z. Writes RN-even(z 2^e) and returns true when that value is
// certain. With s = xh + xl, r = RN(s) and t = s - r (exact: |xh| > |xl| whenever the test can
// pass): z rounds to r as well if |t| + eabs stays below the distance from r to the nearer end of
// its rounding interval (half an ulp; a quarter below a power of two). Everything else returns
// false and is left to the integer path: ties, |z| below eabs 2^53, z within 2^-20 P of +-P / 2,
// results outside the normal range.
IMD_HD bool crt_fast_round(const CrtFast& f, double sh, double sl, int e, double* out) {
  double xh, xl;
  crt_fast_value(f, sh, sl, &xh, &xl);
  const double r = f64_add(xh, xl);
  const double t = f64_add(xl, -f64_add(r, -xh));
  int32_t rhi, rlo;
  f64_words(r, &rhi, &rlo);
  const int32_t mag_hi = rhi & 0x7FFFFFFF;
  const bool pow2 = ((rhi & 0x000FFFFF) | rlo) == 0;
  const int32_t hu_hi = (rhi & 0x7FF00000) - (pow2 ? (54 << 20) : (53 << 20));
  const double thr = f64_add(f64_from_words(hu_hi > 0 ? hu_hi : 0, 0), -f.eabs);
  const int ex = (mag_hi >> 20) + e;                        // biased exponent of the result
  *out = f64_from_words(static_cast<int32_t>(static_cast<uint32_t>(rhi) +
                                              static_cast<uint32_t>(e) * (1u << 20)), rlo);
  return std::fabs(t) < thr && mag_hi < f.rmax_hi && ex >= 1 && ex <= 2046;
}

}  // namespace imd
