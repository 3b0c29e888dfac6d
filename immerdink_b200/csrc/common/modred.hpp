// The modular reductions of the kernels as host + device functions, so that a host program can
// run them over every reachable input (tests/mod_exhaustive.cpp):
//
//   reduce_sym     digit-weight sum of the quantise kernel -> symmetric residue (low byte)
//   mod_epilogue   int32 accumulator of the int8 GEMM -> CRT digit y = (q acc) mod p in [0, p)
//   signed_digits64  two's complement integer -> signed base-256 digits
//
// Counterparts in the reference: src/device/modp.hpp:53-66 (mod_p_barrett_neg), :111-148
// (mod_p_words32); rules spec/oracle.py:438-448 (residue) and :469-487 (modular GEMM).
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>

#include "wide.hpp"

namespace imd {

constexpr int32_t kSumMagic = 0x4B400000;  // bit pattern of 1.5 * 2^23: ulp 1, low 22 bits zero

IMD_HD uint32_t umulhi32(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __umulhi(a, b);
#else
  return static_cast<uint32_t>((static_cast<uint64_t>(a) * b) >> 32);
#endif
}

// X = kSumMagic + s with |s| < 2^21 (the tensor-core accumulator started at kSumMagic): as a float
// X is 1.5 * 2^23 + s exactly. q = round(s / p) comes out of one fused multiply-add in the same
// form (the product with the rounded reciprocal is off by far less than the distance 1 / (2 p) of
// s / p from the nearest half-integer, and for p = 256 a tie changes q by one and r by 256), and
// s - q p is one integer multiply-add on the bit patterns: kSumMagic (1 - p) vanishes mod 2^22.
// The low byte of the result is the symmetric residue of s in two's complement.
IMD_HD uint32_t reduce_sym(int32_t X, float inv_p, int32_t neg_p) {
#if defined(__CUDA_ARCH__)
  const float f = __int_as_float(X) - 12582912.0f;
  const float qm = __fmaf_rn(f, inv_p, 12582912.0f);
  return static_cast<uint32_t>(__float_as_int(qm) * neg_p + X);
#else
  float xf;
  std::memcpy(&xf, &X, 4);
  const float f = xf - 12582912.0f;
  const float qm = std::fmaf(f, inv_p, 12582912.0f);
  int32_t qb;
  std::memcpy(&qb, &qm, 4);
  return static_cast<uint32_t>(qb) * static_cast<uint32_t>(neg_p) + static_cast<uint32_t>(X);
#endif
}

// One accumulator of the int8 GEMM (|acc| < 2^31 - 2^20) -> y = (q (acc mod p)) mod p.
// bias = the multiple of p in [2^31, 2^31 + p); magic = floor(2^32 / p); magic_up = ceil(2^32 / p).
IMD_HD uint32_t mod_epilogue(uint32_t acc, uint32_t p, uint32_t magic, uint32_t magic_up,
                             uint32_t bias, uint32_t q) {
  const uint32_t u = acc + bias;                    // in [0, 2^32)
  uint32_t r = u - umulhi32(u, magic) * p;          // in [0, 2 p)
  const uint32_t r2 = r - p;                        // unsigned wrap: huge when r < p
  r = r < r2 ? r : r2;
  const uint32_t v = r * q;                         // < 2^16
  return v - umulhi32(v, magic_up) * p;             // exact quotient for v < 2^24
}

// Signed base-256 digits of a two's complement integer: adding 0x80 to every byte but the top one
// (with carries) and flipping those bits back turns each byte into a digit in [-128, 127].
IMD_HD void signed_digits64(int64_t x, uint32_t* d0, uint32_t* d1) {
  const uint64_t k = 0x0080808080808080ull;
  const uint64_t y = (static_cast<uint64_t>(x) + k) ^ k;
  *d0 = static_cast<uint32_t>(y);
  *d1 = static_cast<uint32_t>(y >> 32);
}

}  // namespace imd
