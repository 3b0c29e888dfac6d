// Host shim of tests/test_crt_fast.py: the CRT kernel's floating-point shortcut
// (immerdink_b200/csrc/common/crtfast.hpp) compiled for the host behind two plain C functions.
#include <cstdint>

#include "common/crtfast.hpp"

using namespace imd;

namespace {
struct ByteDigit {
  const uint8_t* y;
  double operator()(int l, int) const { return 256.0 + static_cast<double>(y[l]); }
};

template <int N>
int run(const CrtFast& f, const uint8_t* y, int e, double* out, double* xh, double* xl) {
  double sh, sl;
  crt_fast_sums<N, 1>(f, ByteDigit{y}, 0, &sh, &sl);
  crt_fast_value(f, sh, sl, xh, xl);
  return crt_fast_round(f, sh, sl, e, out) ? 1 : 0;
}
}  // namespace

extern "C" {

// cases x N digits -> ok[cases] (1 = the shortcut vouches for out[case]) and the double-double
// value xh + xl of z behind it.
int crt_fast_batch(int N, int64_t cases, const uint8_t* y, const int32_t* e, double* out, uint8_t* ok,
                   double* xh, double* xl) {
  if (N < kMinModuli || N > kMaxModuli) return 1;
  const CrtTables t = crt_tables(N);
  for (int64_t c = 0; c < cases; ++c) {
    const uint8_t* d = y + c * N;
    int r = 0;
    switch (N) {
#define CASE(n) case n: r = run<n>(t.fast, d, e[c], out + c, xh + c, xl + c); break;
      CASE(2) CASE(3) CASE(4) CASE(5) CASE(6) CASE(7) CASE(8) CASE(9) CASE(10) CASE(11) CASE(12)
      CASE(13) CASE(14) CASE(15) CASE(16) CASE(17) CASE(18) CASE(19) CASE(20)
#undef CASE
    }
    ok[c] = static_cast<uint8_t>(r);
  }
  return 0;
}

// The plan constants the shortcut uses, for the test's own error analysis.
int crt_fast_constants(int N, double* eabs, double* Ph, double* Pl, uint32_t* q) {
  if (N < kMinModuli || N > kMaxModuli) return 1;
  const CrtTables t = crt_tables(N);
  *eabs = t.fast.eabs;
  *Ph = t.fast.Ph;
  *Pl = t.fast.Pl;
  for (int l = 0; l < N; ++l) q[l] = t.q[l];
  return 0;
}
}
