/* CPU oracle of the emulated FP64 contraction (Ozaki scheme II, CRT over int8 residues).
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker for the CUDA library: tests, the smoke
 * check and the benchmark's CPU-baseline leg may call it; the shipped library never does.
 *
 * It restates, in plain C with exact integer arithmetic, the algorithm of the reference's
 * executable specification spec/oracle.py (one batch of the GEMM view, C = alpha A B + beta C):
 *   constants          oracle.py:172-213  (Plan: moduli, P, H, T, M_l, q_l, shift right-hand side)
 *   scale_row          oracle.py:361-408  (scale_vector / _shift_of_dyadics / largest_u :346-358)
 *   quantize           oracle.py:415-435
 *   residue            oracle.py:438-448
 *   modular gemm       oracle.py:469-487  (K chunks, store-mod / add-mod)
 *   crt                oracle.py:498-512
 *   round_scaled       oracle.py:257-283  (round_dyadic)
 *   native dot, alpha/beta  oracle.py:519-524, 553-604
 * Two evaluation modes produce the same bits: "literal" walks residues -> int32 GEMM per
 * modulus -> CRT exactly like the specification; "direct" accumulates z = sum a'_h b'_h as a
 * wide integer, which the CRT returns exactly because sum |a'||b'| <= H (the reference's
 * numpy engine bench/accuracy/kw_engine.py:338-358 takes the same shortcut).
 *
 * Parity is pinned: tests/golden holds outputs of the reference's own spec/oracle.py for
 * seeded and adversarial inputs (tests/golden/make_golden.py), and this file must match them.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef unsigned __int128 u128;
typedef __int128 i128;

#define IMDO_MAXN 20
#define IMDO_F 60
#define BIGW 6 /* 384-bit unsigned integers, little-endian u64 limbs */

static const int kModuli[IMDO_MAXN] = {256, 255, 253, 251, 247, 241, 239, 233, 229, 227,
                                       223, 217, 211, 199, 197, 193, 191, 181, 179, 173};

typedef struct {
  uint64_t w[BIGW];
} big_t;

static big_t big_u64(uint64_t x) {
  big_t r;
  memset(&r, 0, sizeof r);
  r.w[0] = x;
  return r;
}
static big_t big_u128(u128 x) {
  big_t r = big_u64((uint64_t)x);
  r.w[1] = (uint64_t)(x >> 64);
  return r;
}
static int big_cmp(const big_t* a, const big_t* b) {
  for (int i = BIGW - 1; i >= 0; --i)
    if (a->w[i] != b->w[i]) return a->w[i] > b->w[i] ? 1 : -1;
  return 0;
}
static int big_is_zero(const big_t* a) {
  for (int i = 0; i < BIGW; ++i)
    if (a->w[i]) return 0;
  return 1;
}
static big_t big_add(const big_t* a, const big_t* b) {
  big_t r;
  u128 c = 0;
  for (int i = 0; i < BIGW; ++i) {
    c += (u128)a->w[i] + b->w[i];
    r.w[i] = (uint64_t)c;
    c >>= 64;
  }
  return r;
}
static big_t big_sub(const big_t* a, const big_t* b) { /* a >= b */
  big_t r;
  uint64_t borrow = 0;
  for (int i = 0; i < BIGW; ++i) {
    u128 t = (u128)a->w[i] - b->w[i] - borrow;
    r.w[i] = (uint64_t)t;
    borrow = (uint64_t)(t >> 64) & 1;
  }
  return r;
}
static big_t big_mul_small(const big_t* a, uint64_t m) {
  big_t r;
  u128 c = 0;
  for (int i = 0; i < BIGW; ++i) {
    c += (u128)a->w[i] * m;
    r.w[i] = (uint64_t)c;
    c >>= 64;
  }
  return r;
}
static big_t big_mul(const big_t* a, const big_t* b) { /* product must fit */
  big_t r;
  memset(&r, 0, sizeof r);
  for (int i = 0; i < BIGW; ++i) {
    u128 c = 0;
    for (int j = 0; i + j < BIGW; ++j) {
      c += (u128)a->w[i] * b->w[j] + r.w[i + j];
      r.w[i + j] = (uint64_t)c;
      c >>= 64;
    }
  }
  return r;
}
static uint64_t big_divmod_small(big_t* a, uint64_t d) { /* a /= d, returns remainder */
  u128 rem = 0;
  for (int i = BIGW - 1; i >= 0; --i) {
    u128 cur = (rem << 64) | a->w[i];
    a->w[i] = (uint64_t)(cur / d);
    rem = cur % d;
  }
  return (uint64_t)rem;
}
static big_t big_shl(const big_t* a, int s) { /* 0 <= s, result must fit */
  big_t r;
  memset(&r, 0, sizeof r);
  const int ws = s / 64, bs = s % 64;
  for (int i = BIGW - 1; i >= 0; --i) {
    const int src = i - ws;
    uint64_t v = 0;
    if (src >= 0) v = a->w[src] << bs;
    if (src >= 1 && bs) v |= a->w[src - 1] >> (64 - bs);
    r.w[i] = v;
  }
  return r;
}
static big_t big_shr(const big_t* a, int s) {
  big_t r;
  memset(&r, 0, sizeof r);
  const int ws = s / 64, bs = s % 64;
  for (int i = 0; i < BIGW; ++i) {
    const int src = i + ws;
    uint64_t v = 0;
    if (src < BIGW) v = a->w[src] >> bs;
    if (src + 1 < BIGW && bs) v |= a->w[src + 1] << (64 - bs);
    r.w[i] = v;
  }
  return r;
}
static int big_bitlen(const big_t* a) {
  for (int i = BIGW - 1; i >= 0; --i)
    if (a->w[i]) return 64 * i + 64 - __builtin_clzll(a->w[i]);
  return 0;
}
static int big_bit(const big_t* a, int i) {
  return i >= 64 * BIGW ? 0 : (int)((a->w[i / 64] >> (i % 64)) & 1);
}
/* any bit set below position s */
static int big_low_nonzero(const big_t* a, int s) {
  for (int i = 0; i < BIGW; ++i) {
    if (64 * (i + 1) <= s) {
      if (a->w[i]) return 1;
    } else if (64 * i < s) {
      if (a->w[i] & ((((uint64_t)1) << (s - 64 * i)) - 1)) return 1;
    }
  }
  return 0;
}
static big_t big_isqrt(const big_t* a) {
  big_t r = big_u64(0);
  for (int bit = (big_bitlen(a) + 1) / 2; bit >= 0; --bit) {
    big_t one = big_u64(1);
    big_t t = big_shl(&one, bit);
    big_t cand = big_add(&r, &t);
    big_t sq = big_mul(&cand, &cand);
    if (big_cmp(&sq, a) <= 0) r = cand;
  }
  return r;
}

/* ---- plan constants (oracle.py:172-213) ------------------------------------------------ */
typedef struct {
  int N, trunc;
  int p[IMDO_MAXN], q[IMDO_MAXN];
  big_t P, H, T, M[IMDO_MAXN];
  big_t rhs;   /* (2T - kappa)^2 2^F (RN) or T^2 2^F (TRUNC) */
  int lhs_mul; /* 4 (RN) or 1 (TRUNC) */
  uint64_t kappa;
} plan_t;

static uint64_t ceil_sqrt_u64(uint64_t k) {
  uint64_t r = (uint64_t)sqrtl((long double)k);
  while (r * r > k) --r;
  while ((r + 1) * (r + 1) <= k) ++r;
  return r * r == k ? r : r + 1;
}

/* returns 0 ok, 1 invalid option, 2 not supported (kappa >= T under RN) */
static int plan_init(plan_t* pl, int N, int trunc, int64_t k) {
  if (N < 2 || N > IMDO_MAXN || (trunc != 0 && trunc != 1) || k < 0) return 1;
  memset(pl, 0, sizeof *pl);
  pl->N = N;
  pl->trunc = trunc;
  pl->P = big_u64(1);
  for (int l = 0; l < N; ++l) {
    pl->p[l] = kModuli[l];
    pl->P = big_mul_small(&pl->P, (uint64_t)kModuli[l]);
  }
  big_t one = big_u64(1);
  big_t pm1 = big_sub(&pl->P, &one);
  pl->H = big_shr(&pm1, 1);
  pl->T = big_isqrt(&pl->H);
  for (int l = 0; l < N; ++l) {
    big_t Ml = pl->P;
    big_divmod_small(&Ml, (uint64_t)pl->p[l]);
    pl->M[l] = Ml;
    big_t tmp = Ml;
    const int r = (int)big_divmod_small(&tmp, (uint64_t)pl->p[l]);
    int inv = 0;
    for (int c = 1; c < pl->p[l]; ++c)
      if ((r * c) % pl->p[l] == 1) {
        inv = c;
        break;
      }
    pl->q[l] = inv;
  }
  pl->kappa = k > 0 ? ceil_sqrt_u64((uint64_t)k) : 0;
  big_t kap = big_u64(pl->kappa);
  if (!trunc && k > 0 && big_cmp(&kap, &pl->T) >= 0) return 2;
  big_t base;
  if (!trunc) {
    big_t t2 = big_shl(&pl->T, 1);
    base = big_sub(&t2, &kap);
    pl->lhs_mul = 4;
  } else {
    base = pl->T;
    pl->lhs_mul = 1;
  }
  big_t sq = big_mul(&base, &base);
  pl->rhs = big_shl(&sq, IMDO_F);
  return 0;
}

/* ---- binary64 decomposition ------------------------------------------------------------- */
static uint64_t dbits(double x) {
  uint64_t u;
  memcpy(&u, &x, 8);
  return u;
}
static double from_bits(uint64_t u) {
  double x;
  memcpy(&x, &u, 8);
  return x;
}
/* finite nonzero x = (-1)^neg * M * 2^E with 2^52 <= M < 2^53 (subnormals normalised) */
static int decompose(double x, int* neg, uint64_t* M, int* E) {
  const uint64_t u = dbits(x);
  const int ef = (int)((u >> 52) & 0x7FF);
  uint64_t frac = u & 0xFFFFFFFFFFFFFull;
  *neg = (int)(u >> 63);
  if (ef == 0x7FF) return -1; /* non-finite */
  if (ef == 0) {
    if (frac == 0) return 0; /* zero */
    const int sh = __builtin_clzll(frac) - 11;
    *M = frac << sh;
    *E = -1074 - sh;
    return 1;
  }
  *M = frac | (1ull << 52);
  *E = ef - 1075;
  return 1;
}

/* ---- scale (oracle.py:361-408) ---------------------------------------------------------- */
/* Largest integer u with L * 4^u <= R (L, R > 0). */
static int largest_u(const big_t* L, const big_t* R) {
  int u = (big_bitlen(R) - big_bitlen(L)) / 2; /* any start: the loops below settle it */
#define OK_AT(uu, res)                                   \
  do {                                                   \
    if ((uu) >= 0) {                                     \
      big_t l2 = big_shl(L, 2 * (uu));                   \
      res = big_cmp(&l2, R) <= 0;                        \
    } else {                                             \
      big_t r2 = big_shl(R, -2 * (uu));                  \
      res = big_cmp(L, &r2) <= 0;                        \
    }                                                    \
  } while (0)
  int ok;
  OK_AT(u, ok);
  while (!ok) {
    --u;
    OK_AT(u, ok);
  }
  for (;;) {
    OK_AT(u + 1, ok);
    if (!ok) break;
    ++u;
  }
#undef OK_AT
  return u;
}

/* One row: `len` entries at row[h * stride]. Writes sigma (int16 range asserted by caller). */
static void scale_row(const plan_t* pl, const double* row, int64_t len, int64_t stride,
                      int* sigma, int* flag) {
  int fl = 0, any = 0, gamma = -100000;
  for (int64_t h = 0; h < len; ++h) {
    int neg, E;
    uint64_t M;
    const int c = decompose(row[h * stride], &neg, &M, &E);
    if (c < 0) fl = 1;
    if (c == 1) {
      any = 1;
      if (E + 52 > gamma) gamma = E + 52;
    }
  }
  *flag = fl;
  if (!any) {
    *sigma = 0;
    return;
  }
  u128 S = 0;
  for (int64_t h = 0; h < len; ++h) {
    int neg, E;
    uint64_t M;
    if (decompose(row[h * stride], &neg, &M, &E) != 1) continue;
    /* ceil(M^2 * 2^t), t = 2 (E - gamma) + F <= -44 because E + 52 <= gamma */
    const int sh = -(2 * (E - gamma) + IMDO_F);
    const u128 sq = (u128)M * M;
    u128 term;
    if (sh >= 128) {
      term = 1;
    } else {
      term = sq >> sh;
      if (sq & ((((u128)1) << sh) - 1)) term += 1;
    }
    S += term;
  }
  big_t L = big_u128(S);
  L = big_mul_small(&L, (uint64_t)pl->lhs_mul);
  const int u = largest_u(&L, &pl->rhs);
  *sigma = u - gamma;
}

/* ---- quantize (oracle.py:415-435): |a'| < 2^78 as u128 --------------------------------- */
static void quantize(double v, int sigma, int trunc, int* neg, u128* mag) {
  uint64_t M;
  int E;
  *mag = 0;
  *neg = 0;
  if (decompose(v, neg, &M, &E) != 1) {
    *neg = 0;
    return;
  }
  const int s = E + sigma;
  if (s >= 0) {
    *mag = (u128)M << s; /* guaranteed <= T by the scale rule */
  } else {
    const int sh = -s;
    if (sh >= 64) {
      *mag = 0;
    } else {
      uint64_t r = M >> sh;
      if (!trunc) {
        const uint64_t rem = M & ((1ull << sh) - 1), half = 1ull << (sh - 1);
        if (rem > half || (rem == half && (r & 1))) r += 1;
      }
      *mag = r;
    }
  }
  if (*mag == 0) *neg = 0;
}

/* ---- residue (oracle.py:438-448): SMod(a', p) in [-floor(p/2), ceil(p/2) - 1] ---------- */
static int residue(int neg, u128 mag, int p) {
  int r = (int)(mag % (u128)p);
  if (neg && r) r = p - r;
  const int h = p / 2;
  return (r + h) % p - h;
}

/* ---- signed wide integer: sign + magnitude --------------------------------------------- */
typedef struct {
  int neg;
  big_t mag;
} sbig_t;

/* ---- CRT (oracle.py:498-512) ------------------------------------------------------------ */
static sbig_t crt(const plan_t* pl, const uint8_t* W /* N residues */) {
  big_t x = big_u64(0);
  for (int l = 0; l < pl->N; ++l) {
    const uint64_t y = ((uint64_t)pl->q[l] * W[l]) % (uint64_t)pl->p[l];
    big_t t = big_mul_small(&pl->M[l], y);
    x = big_add(&x, &t);
    if (big_cmp(&x, &pl->P) >= 0) x = big_sub(&x, &pl->P);
  }
  sbig_t z;
  if (big_cmp(&x, &pl->H) <= 0) {
    z.neg = 0;
    z.mag = x;
  } else {
    z.neg = 1;
    z.mag = big_sub(&pl->P, &x);
  }
  return z;
}

/* ---- round_dyadic (oracle.py:257-283): RN-even of (+-mag) 2^e, one rounding ------------- */
static double round_scaled(int neg, const big_t* mag, int e) {
  if (big_is_zero(mag)) return 0.0; /* exact integer zero: +0 */
  const int top = big_bitlen(mag) - 1 + e;
  int q = top - 52;
  if (q < -1074) q = -1074;
  uint64_t r;
  if (q <= e) {
    big_t s = big_shl(mag, e - q); /* fits: at most 53 bits */
    r = s.w[0];
  } else {
    const int sh = q - e;
    big_t s = big_shr(mag, sh);
    r = s.w[0];
    const int halfbit = big_bit(mag, sh - 1);
    const int low = big_low_nonzero(mag, sh - 1);
    if (halfbit && (low || (r & 1))) r += 1;
  }
  const uint64_t sign = neg ? 0x8000000000000000ull : 0;
  if (r == 0) return from_bits(sign);
  int blen = 64 - __builtin_clzll(r); /* <= 54 */
  if (blen - 1 + q >= 1024) return from_bits(sign | 0x7FF0000000000000ull);
  /* r * 2^q exactly representable: r <= 2^53, q >= -1074 */
  if (r == (1ull << 53)) {
    r >>= 1;
    q += 1;
    blen = 53;
  }
  uint64_t bits;
  if (blen == 53) {
    bits = ((uint64_t)(q + 1075) << 52) | (r & 0xFFFFFFFFFFFFFull);
  } else { /* subnormal: q == -1074 */
    bits = r;
  }
  return from_bits(sign | bits);
}

static double finish(double D, double alpha, double beta, const double* Cold) {
  const double E = (alpha == 1.0) ? D : alpha * D;
  if (beta == 0.0) return E;
  return fma(beta, *Cold, E);
}

/* ---- public entry points ---------------------------------------------------------------- */

/* Plan constants for tests: P, H, T as 6 u64 limbs each, M[l] 6 limbs each, q[l]. */
int imdo_constants(int N, uint64_t* P, uint64_t* H, uint64_t* T, uint64_t* M, int32_t* q) {
  plan_t pl;
  const int st = plan_init(&pl, N, 1, 0);
  if (st) return st;
  memcpy(P, pl.P.w, sizeof pl.P.w);
  memcpy(H, pl.H.w, sizeof pl.H.w);
  memcpy(T, pl.T.w, sizeof pl.T.w);
  for (int l = 0; l < N; ++l) {
    memcpy(M + (size_t)l * BIGW, pl.M[l].w, sizeof pl.M[l].w);
    q[l] = pl.q[l];
  }
  return 0;
}

/* sigma and flag of `rows` rows; row r entry h at X[r * row_stride + h * k_stride]. */
int imdo_scale(int N, int trunc, int64_t k_plan, const double* X, int64_t rows, int64_t len,
               int64_t row_stride, int64_t k_stride, int16_t* sigma, uint8_t* flag) {
  plan_t pl;
  const int st = plan_init(&pl, N, trunc, k_plan);
  if (st) return st;
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t r = 0; r < rows; ++r) {
    int s, f;
    scale_row(&pl, X + r * row_stride, len, k_stride, &s, &f);
    sigma[r] = (int16_t)s;
    flag[r] = (uint8_t)f;
  }
  return 0;
}

/* int8 residues of all N moduli: R[(l * rows + r) * len + h]. */
int imdo_residues(int N, int trunc, const double* X, int64_t rows, int64_t len,
                  int64_t row_stride, int64_t k_stride, const int16_t* sigma, int8_t* R) {
  if (N < 2 || N > IMDO_MAXN) return 1;
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t r = 0; r < rows; ++r)
    for (int64_t h = 0; h < len; ++h) {
      int neg;
      u128 mag;
      quantize(X[r * row_stride + h * k_stride], sigma[r], trunc, &neg, &mag);
      for (int l = 0; l < N; ++l)
        R[((size_t)l * rows + r) * len + h] = (int8_t)residue(neg, mag, kModuli[l]);
    }
  return 0;
}

/* One batch: C[m x n] = alpha A[m x k] Bt[n x k]^T + beta C.
 *   A row i entry h at A[i * lda + h]; B column j entry h at Bt[j * ldb + h].
 *   Cin may be NULL when beta == 0; Cout[i * ldc + j].
 *   literal != 0: residues -> chunked int32 GEMM -> CRT, with chunk length `chunk`
 *   (0 = 131008); literal == 0: direct wide-integer z.
 *   Optional traces (NULL to skip): sigma[m], tau[n], fA[m], fB[n], W[N * m * n] (literal only).
 * Returns 0, 1 (invalid), 2 (not supported: kappa >= T under RN). */
int imdo_gemm(int N, int trunc, int64_t m, int64_t n, int64_t k, const double* A, int64_t lda,
              const double* Bt, int64_t ldb, double alpha, double beta, const double* Cin,
              double* Cout, int64_t ldc, int literal, int64_t chunk, int16_t* sigma_out,
              int16_t* tau_out, uint8_t* fA_out, uint8_t* fB_out, uint8_t* W_out) {
  if (m < 0 || n < 0 || k < 0) return 1;
  if (m == 0 || n == 0) return 0;
  if (alpha == 0.0 || k == 0) {
    for (int64_t i = 0; i < m; ++i)
      for (int64_t j = 0; j < n; ++j)
        Cout[i * ldc + j] = (beta == 0.0) ? 0.0 : beta * Cin[i * ldc + j];
    return 0;
  }
  plan_t pl;
  const int st = plan_init(&pl, N, trunc, k);
  if (st) return st;
  if (chunk <= 0) chunk = 131008;
  if (chunk > 131071) return 1;

  int16_t* sg = (int16_t*)malloc(sizeof(int16_t) * (size_t)(m + n));
  uint8_t* fl = (uint8_t*)malloc((size_t)(m + n));
  int16_t* tu = sg + m;
  uint8_t* fb = fl + m;
  imdo_scale(N, trunc, k, A, m, k, lda, 1, sg, fl);
  imdo_scale(N, trunc, k, Bt, n, k, ldb, 1, tu, fb);
  if (sigma_out) memcpy(sigma_out, sg, sizeof(int16_t) * (size_t)m);
  if (tau_out) memcpy(tau_out, tu, sizeof(int16_t) * (size_t)n);
  if (fA_out) memcpy(fA_out, fl, (size_t)m);
  if (fB_out) memcpy(fB_out, fb, (size_t)n);

  const int narrow = (N <= 16); /* |a'| <= T < 2^63 and |z| <= H < 2^125 */
  if (literal) {
    int8_t* RA = (int8_t*)malloc((size_t)N * m * k);
    int8_t* RB = (int8_t*)malloc((size_t)N * n * k);
    uint8_t* W = W_out ? W_out : (uint8_t*)malloc((size_t)N * m * n);
    imdo_residues(N, trunc, A, m, k, lda, 1, sg, RA);
    imdo_residues(N, trunc, Bt, n, k, ldb, 1, tu, RB);
    for (int l = 0; l < N; ++l) {
      const int p = kModuli[l];
#pragma omp parallel for schedule(dynamic, 4)
      for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
          const int8_t* ra = RA + ((size_t)l * m + i) * k;
          const int8_t* rb = RB + ((size_t)l * n + j) * k;
          int w = 0;
          for (int64_t c0 = 0; c0 < k; c0 += chunk) {
            const int64_t c1 = c0 + chunk < k ? c0 + chunk : k;
            int32_t acc = 0; /* cannot overflow: chunk * 128^2 <= 2^31 - 1 */
            for (int64_t h = c0; h < c1; ++h) acc += (int32_t)ra[h] * (int32_t)rb[h];
            int64_t v = (int64_t)w + acc;
            v %= p;
            if (v < 0) v += p;
            w = (int)v;
          }
          W[((size_t)l * m + i) * n + j] = (uint8_t)w;
        }
    }
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t i = 0; i < m; ++i)
      for (int64_t j = 0; j < n; ++j) {
        double D;
        if (fl[i] || fb[j]) {
          double acc = 0.0;
          for (int64_t h = 0; h < k; ++h) acc = fma(A[i * lda + h], Bt[j * ldb + h], acc);
          D = acc;
        } else {
          uint8_t w[IMDO_MAXN];
          for (int l = 0; l < N; ++l) w[l] = W[((size_t)l * m + i) * n + j];
          const sbig_t z = crt(&pl, w);
          D = round_scaled(z.neg, &z.mag, -((int)sg[i] + (int)tu[j]));
        }
        Cout[i * ldc + j] = finish(D, alpha, beta, Cin ? &Cin[i * ldc + j] : NULL);
      }
    free(RA);
    free(RB);
    if (!W_out) free(W);
  } else if (narrow) {
    int64_t* QA = (int64_t*)malloc(sizeof(int64_t) * (size_t)m * k);
    int64_t* QB = (int64_t*)malloc(sizeof(int64_t) * (size_t)n * k);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m + n; ++i) {
      const int isA = i < m;
      const int64_t r = isA ? i : i - m;
      const double* row = isA ? A + r * lda : Bt + r * ldb;
      int64_t* out = isA ? QA + r * k : QB + r * k;
      const int s = isA ? sg[r] : tu[r];
      for (int64_t h = 0; h < k; ++h) {
        int neg;
        u128 mag;
        quantize(row[h], s, trunc, &neg, &mag);
        out[h] = neg ? -(int64_t)mag : (int64_t)mag;
      }
    }
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t i = 0; i < m; ++i)
      for (int64_t j = 0; j < n; ++j) {
        double D;
        if (fl[i] || fb[j]) {
          double acc = 0.0;
          for (int64_t h = 0; h < k; ++h) acc = fma(A[i * lda + h], Bt[j * ldb + h], acc);
          D = acc;
        } else {
          const int64_t* qa = QA + i * k;
          const int64_t* qb = QB + j * k;
          i128 z = 0;
          for (int64_t h = 0; h < k; ++h) z += (i128)qa[h] * qb[h];
          const int neg = z < 0;
          big_t mag = big_u128(neg ? (u128)(-z) : (u128)z);
          D = round_scaled(neg, &mag, -((int)sg[i] + (int)tu[j]));
        }
        Cout[i * ldc + j] = finish(D, alpha, beta, Cin ? &Cin[i * ldc + j] : NULL);
      }
    free(QA);
    free(QB);
  } else {
    /* N >= 17: |a'| < 2^78. Split a' = hi 2^39 + lo and accumulate three exact partial sums. */
#pragma omp parallel for schedule(dynamic, 4)
    for (int64_t i = 0; i < m; ++i)
      for (int64_t j = 0; j < n; ++j) {
        double D;
        if (fl[i] || fb[j]) {
          double acc = 0.0;
          for (int64_t h = 0; h < k; ++h) acc = fma(A[i * lda + h], Bt[j * ldb + h], acc);
          D = acc;
        } else {
          i128 s2 = 0, s1 = 0, s0 = 0;
          for (int64_t h = 0; h < k; ++h) {
            int na, nb;
            u128 ma, mb;
            quantize(A[i * lda + h], sg[i], trunc, &na, &ma);
            quantize(Bt[j * ldb + h], tu[j], trunc, &nb, &mb);
            const i128 ah = (i128)(ma >> 39), al = (i128)(ma & ((((u128)1) << 39) - 1));
            const i128 bh = (i128)(mb >> 39), bl = (i128)(mb & ((((u128)1) << 39) - 1));
            const i128 sgn = (na != nb) ? -1 : 1;
            s2 += sgn * ah * bh;
            s1 += sgn * (ah * bl + al * bh);
            s0 += sgn * al * bl;
          }
          /* z = s2 2^78 + s1 2^39 + s0 as sign + magnitude: sum positives and negatives */
          big_t pos = big_u64(0), ngv = big_u64(0);
          const i128 parts[3] = {s0, s1, s2};
          for (int t = 0; t < 3; ++t) {
            const int ng = parts[t] < 0;
            big_t v = big_u128(ng ? (u128)(-parts[t]) : (u128)parts[t]);
            v = big_shl(&v, 39 * t);
            if (ng) ngv = big_add(&ngv, &v);
            else pos = big_add(&pos, &v);
          }
          sbig_t z;
          if (big_cmp(&pos, &ngv) >= 0) {
            z.neg = 0;
            z.mag = big_sub(&pos, &ngv);
          } else {
            z.neg = 1;
            z.mag = big_sub(&ngv, &pos);
          }
          D = round_scaled(z.neg, &z.mag, -((int)sg[i] + (int)tu[j]));
        }
        Cout[i * ldc + j] = finish(D, alpha, beta, Cin ? &Cin[i * ldc + j] : NULL);
      }
  }
  free(sg);
  free(fl);
  return 0;
}

/* Native path for every element (DIRECT dispatch, oracle.py:937-944). */
int imdo_direct(int64_t m, int64_t n, int64_t k, const double* A, int64_t lda, const double* Bt,
                int64_t ldb, double alpha, double beta, const double* Cin, double* Cout,
                int64_t ldc) {
#pragma omp parallel for schedule(dynamic, 4)
  for (int64_t i = 0; i < m; ++i)
    for (int64_t j = 0; j < n; ++j) {
      double acc = 0.0;
      for (int64_t h = 0; h < k; ++h) acc = fma(A[i * lda + h], Bt[j * ldb + h], acc);
      Cout[i * ldc + j] = finish(acc, alpha, beta, Cin ? &Cin[i * ldc + j] : NULL);
    }
  return 0;
}

/* round_scaled exposed for known-answer tests: magnitude as 6 u64 limbs. */
double imdo_round_scaled(int neg, const uint64_t* mag6, int e) {
  big_t m;
  memcpy(m.w, mag6, sizeof m.w);
  return round_scaled(neg, &m, e);
}

int imdo_crt(int N, const uint8_t* W, int* neg, uint64_t* mag6) {
  plan_t pl;
  const int st = plan_init(&pl, N, 1, 0);
  if (st) return st;
  const sbig_t z = crt(&pl, W);
  *neg = z.neg;
  memcpy(mag6, z.mag.w, sizeof z.mag.w);
  return 0;
}
