// Host program of tests/test_mod_exhaustive.py: runs the kernels' modular reductions
// (immerdink_b200/csrc/common/modred.hpp, compiled here for the host) over every reachable input
// and compares with plain integer arithmetic. Prints "ok <checks>" or the first mismatch.
// Follows the reference's tests/test_mod_exhaustive.cpp:1-40 in intent.
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include "common/modred.hpp"
#include "common/tables.hpp"

using namespace imd;

static int64_t smod(int64_t s, int64_t p) {  // representative in [-floor(p/2), ceil(p/2) - 1]
  int64_t r = ((s % p) + p) % p;
  if (r > (p + 1) / 2 - 1) r -= p;
  return r;
}

int main() {
  uint64_t checks = 0;
  // 1. digit-weight sums: every s the tensor-core dot can produce (12 digits x 128 x 128), every modulus
  for (int l = 0; l < kMaxModuli; ++l) {
    const int32_t p = kModuli[l];
    const float inv = 1.0f / static_cast<float>(p);
    for (int32_t s = -(1 << 18); s <= (1 << 18); ++s, ++checks) {
      const uint32_t got = reduce_sym(kSumMagic + s, inv, -p) & 0xFFu;
      const uint32_t want = static_cast<uint32_t>(smod(s, p)) & 0xFFu;
      if (got != want) {
        std::printf("reduce_sym p=%d s=%d got %u want %u\n", p, s, got, want);
        return 1;
      }
    }
  }
  // 2. GEMM epilogue, first stage over the accumulator range (stride 257 walks every residue class
  //    of every modulus and both ends of the range), with the CRT weight of each modulus ...
  for (int N = kMinModuli; N <= kMaxModuli; N += 6) {
    const CrtTables t = crt_tables(N);
    for (int l = 0; l < N; ++l) {
      const uint32_t p = static_cast<uint32_t>(kModuli[l]);
      const uint32_t magic = static_cast<uint32_t>((uint64_t{1} << 32) / p);
      const uint32_t magic_up = static_cast<uint32_t>(((uint64_t{1} << 32) + p - 1) / p);
      const uint32_t bias = static_cast<uint32_t>(((uint64_t{1} << 31) + p - 1) / p * p);
      const int64_t lim = (int64_t{1} << 31) - (1 << 20);
      for (int64_t acc = -lim; acc <= lim; acc += (acc > -lim + 70000 && acc < lim - 70000) ? 257 : 1, ++checks) {
        const uint32_t got = mod_epilogue(static_cast<uint32_t>(static_cast<int32_t>(acc)), p, magic,
                                          magic_up, bias, t.q[l]);
        const int64_t r = ((acc % p) + p) % p;
        const uint32_t want = static_cast<uint32_t>((r * t.q[l]) % p);
        if (got != want) {
          std::printf("mod_epilogue p=%u acc=%lld got %u want %u\n", p, static_cast<long long>(acc), got, want);
          return 1;
        }
      }
    }
  }
  //    ... and its second stage for every residue and every multiplier
  for (int l = 0; l < kMaxModuli; ++l) {
    const uint32_t p = static_cast<uint32_t>(kModuli[l]);
    const uint32_t magic = static_cast<uint32_t>((uint64_t{1} << 32) / p);
    const uint32_t magic_up = static_cast<uint32_t>(((uint64_t{1} << 32) + p - 1) / p);
    const uint32_t bias = static_cast<uint32_t>(((uint64_t{1} << 31) + p - 1) / p * p);
    for (uint32_t r = 0; r < p; ++r)
      for (uint32_t q = 0; q < p; ++q, ++checks)
        if (mod_epilogue(r, p, magic, magic_up, bias, q) != (r * q) % p) {
          std::printf("mod_epilogue stage 2 p=%u r=%u q=%u\n", p, r, q);
          return 1;
        }
  }
  // 3. signed digits: the digits are in [-128, 127] and sum back to the integer (|x| < 2^62:
  //    quantised entries are bounded by T < 2^62.2 when two words carry them)
  uint64_t z = 0x9E3779B97F4A7C15ull;
  for (int it = 0; it < 2000000; ++it, ++checks) {
    z ^= z << 13, z ^= z >> 7, z ^= z << 17;
    int64_t x = static_cast<int64_t>(z) >> (1 + it % 63);
    if (it < 63) x = (int64_t{1} << it) - 1;
    if (it >= 64 && it < 127) x = -(int64_t{1} << (it - 64));
    uint32_t d0, d1;
    signed_digits64(x, &d0, &d1);
    const uint64_t both = d0 | (static_cast<uint64_t>(d1) << 32);
    __int128 sum = 0;
    for (int j = 7; j >= 0; --j) sum = sum * 256 + static_cast<int8_t>(both >> (8 * j));
    if (sum != x) {
      std::printf("signed_digits64 x=%lld\n", static_cast<long long>(x));
      return 1;
    }
  }
  std::printf("ok %llu\n", static_cast<unsigned long long>(checks));
  return 0;
}
