// The kernel sequence of one imd_contract on the caller's stream (enqueue only: no allocation,
// no synchronisation, no global state written):
//
//   vectors   nine int64 scatter vectors from the fused-mode table      (unless plan-resident)
//   scale     per row of A / column of B: non-finite flag, exponent, exact sum of squares,
//             shift sigma                                                     (one launch each)
//   residues  gather FP64 through the vectors, quantise with sigma, reduce to the int8 residues
//             of one group of moduli, K-contiguous planes                     (per group, each)
//   gemm      int8 GEMM per modulus on tcgen05 tensor cores with a mod-p epilogue into u8 planes
//   crt       exact CRT over the N planes, one rounding, alpha / beta, scatter into C
//
// plus the two degenerate paths: C <- beta C (alpha = 0 or k = 0) and the native FP64 FMA dot
// (DIRECT mode or k = 1). The sequence replaces the reference's enqueue_contract
// (src/contract.cu:1334-1485) and its kernels K0, K1, K2/K3, KF, KL, K5, k_direct,
// k5_beta_only; the numerics are in numerics.cuh.
#include <atomic>
#include <cstdint>
#include <mutex>
#include <vector>

#include "kernels.hpp"
#include "numerics.cuh"
#include "quantize.cuh"

namespace imd {

namespace {

__device__ unsigned int g_error_word = 0;

constexpr int kThreads = 256;

// ---- scatter vectors -------------------------------------------------------------------------
struct VecParams {
  ModeTable modes;
  int64_t m, n, k, b;
  int32_t segments;  // 9: all vectors of a contraction; 3: rows, K and batches of operand A only
};

__device__ __forceinline__ int64_t radix_offset(const ModeTable& t, int cls, int X, int64_t q) {
  int64_t off = 0;
  const int first = t.first[cls], cnt = t.count[cls];
  for (int i = 0; i < cnt; ++i) {
    const int64_t e = t.extent[first + i];
    const int64_t d = q % e;
    q /= e;
    off += d * t.stride[first + i][X];
  }
  return off;
}

__global__ void __launch_bounds__(kThreads) k_vectors(const __grid_constant__ VecParams p,
                                                      int64_t* __restrict__ vec) {
  const int64_t total = p.segments == 3 ? p.m + p.k + p.b : 2 * p.m + 2 * p.n + 2 * p.k + 3 * p.b;
  const int64_t seg[9] = {p.m, p.k, p.b, p.k, p.n, p.b, p.m, p.n, p.b};
  const int cls[9] = {kClsI, kClsK, kClsL, kClsK, kClsJ, kClsL, kClsI, kClsJ, kClsL};
  const int ten[9] = {kTenA, kTenA, kTenA, kTenB, kTenB, kTenB, kTenC, kTenC, kTenC};
  for (int64_t e = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * kThreads) {
    int64_t q = e;
    int s = 0;
    while (s < 8 && q >= seg[s]) {
      q -= seg[s];
      ++s;
    }
    vec[e] = radix_offset(p.modes, cls[s], ten[s], q);
  }
}

struct Vectors {
  const int64_t *a_row, *a_k, *a_bat, *b_k, *b_col, *b_bat, *c_row, *c_col, *c_bat;
};

Vectors split_vectors(const int64_t* v, const ExecPlan& e) {
  Vectors r;
  r.a_row = v, v += e.m;
  r.a_k = v, v += e.k;
  r.a_bat = v, v += e.b;
  r.b_k = v, v += e.k;
  r.b_col = v, v += e.n;
  r.b_bat = v, v += e.b;
  r.c_row = v, v += e.m;
  r.c_col = v, v += e.n;
  r.c_bat = v;
  return r;
}

// ---- scale (launches of its own: operands that are contiguous along their rows) -------------------
// A CTA owns 2^lg_rt rows completely (a row's shift is produced and consumed inside one CTA);
// its 256 threads are 2^lg_rt rows x KT lanes along K. `rows_fast` picks which of the two runs
// along consecutive threads, so that global loads coalesce along the operand's fast direction.
// One pass over the row gives the flag, the largest exponent and the FP64 sum of squares that
// decides the shift (dev::fast_shift); rows it cannot decide redo the sum with exact integers.
struct ScaleParams {
  const double* X;
  const int64_t *row, *kv, *bat;
  int64_t rows, batches, k;
  int32_t lg_rt;
  int32_t rows_fast;
  int32_t lhs_shift;
  int32_t force_exact;
  Wide<8> rhs;
  ShiftFast fast;
  // Outputs: row i of batch lambda at index lambda * out_rows + out_row0 + i of every destination
  // (one destination and out_rows = rows, out_row0 = 0 inside a contraction; several, possibly
  // in other GPUs' memory, when a piece of a slab is packed for all its consumers).
  int64_t out_rows, out_row0;
  int32_t n_out;
  int16_t* sigma[kMaxDests];
  uint8_t* flag[kMaxDests];
};

__global__ void __launch_bounds__(kThreads) k_scale(const __grid_constant__ ScaleParams p) {
  __shared__ uint32_t s_max[kThreads];
  __shared__ uint64_t s_hi[kThreads], s_lo[kThreads];
  const int RT = 1 << p.lg_rt, KT = kThreads >> p.lg_rt;
  const int tid = threadIdx.x;
  const int r = p.rows_fast ? (tid & (RT - 1)) : (tid / KT);
  const int kl = p.rows_fast ? (tid >> p.lg_rt) : (tid % KT);
  const int64_t total = p.rows * p.batches;
  const int64_t rho = static_cast<int64_t>(blockIdx.x) * RT + r;
  const bool live = rho < total;
  const double* base = p.X;
  if (live) base += p.bat[rho / p.rows] + p.row[rho % p.rows];

  // the pass: largest high word of |a| (exponent and non-finite test in one) and sum of squares
  uint32_t mx = 0;
  double acc = 0.0;
  if (live)
    for (int64_t h = kl; h < p.k; h += 4 * KT) {
      uint64_t u[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // four independent loads in flight
        const int64_t hj = h + static_cast<int64_t>(j) * KT;
        u[j] = hj < p.k ? static_cast<uint64_t>(__double_as_longlong(base[p.kv[hj]])) : 0ull;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mx = max(mx, static_cast<uint32_t>(u[j] >> 32) & 0x7FFFFFFFu);
        const double x = __longlong_as_double(static_cast<long long>(u[j]));
        acc = __fma_rn(x, x, acc);
      }
    }
  const int slot = r * KT + kl;
  double* s_acc = reinterpret_cast<double*>(s_hi);
  s_max[slot] = mx;
  s_acc[slot] = acc;
  __syncthreads();
  for (int s = KT >> 1; s > 0; s >>= 1) {
    if (kl < s) {
      s_max[slot] = max(s_max[slot], s_max[slot + s]);
      s_acc[slot] += s_acc[slot + s];
    }
    __syncthreads();
  }
  int sg = 0, fl = 0, exact = 0;
  if (live && kl == 0)
    if (p.force_exact || !dev::fast_shift(s_max[slot], s_acc[slot], p.fast, p.lhs_shift, &sg)) exact = 1;

  // exact integer passes, for every row of the CTA, when any of its rows could not be decided
  if (__syncthreads_or(exact)) {
    // non-finite flag and largest exponent. Encoding: bit 30 = flag; low bits = gamma + 2048
    // (0 = no finite nonzero entry).
    int g = 0;
    if (live)
      for (int64_t h = kl; h < p.k; h += KT) {
        uint64_t M;
        int E;
        const int kind = dev::decompose(static_cast<uint64_t>(__double_as_longlong(base[p.kv[h]])), &M, &E);
        if (kind < 0) g |= 1 << 30;
        else if (kind > 0) g = (g & (1 << 30)) | max(g & 0xFFFF, E + 52 + 2048);
      }
    s_max[slot] = static_cast<uint32_t>(g);
    __syncthreads();
    for (int s = KT >> 1; s > 0; s >>= 1) {
      if (kl < s) {
        const int a = static_cast<int>(s_max[slot]), b = static_cast<int>(s_max[slot + s]);
        s_max[slot] = static_cast<uint32_t>(((a | b) & (1 << 30)) | max(a & 0xFFFF, b & 0xFFFF));
      }
      __syncthreads();
    }
    const int gf = static_cast<int>(s_max[r * KT]);
    const bool any = (gf & 0xFFFF) != 0;
    const int gamma = (gf & 0xFFFF) - 2048;
    __syncthreads();  // s_hi doubles as the sum of squares above: every read of it is done
    uint64_t hi = 0, lo = 0;
    if (live && any)
      for (int64_t h = kl; h < p.k; h += KT) {
        const uint64_t u = static_cast<uint64_t>(__double_as_longlong(base[p.kv[h]]));
        uint64_t M;
        int E;
        if (dev::decompose(u, &M, &E) == 1) {
          uint64_t th, tl;
          dev::square_term(M, E, gamma, &th, &tl);
          lo += tl;
          hi += th + (lo < tl ? 1 : 0);
        }
      }
    s_hi[slot] = hi;
    s_lo[slot] = lo;
    __syncthreads();
    for (int s = KT >> 1; s > 0; s >>= 1) {
      if (kl < s) {
        const uint64_t bl = s_lo[slot + s];
        const uint64_t nl = s_lo[slot] + bl;
        s_hi[slot] += s_hi[slot + s] + (nl < bl ? 1 : 0);
        s_lo[slot] = nl;
      }
      __syncthreads();
    }
    sg = 0;
    if (live && kl == 0 && any)
      sg = dev::shift_from_sum(s_hi[slot], s_lo[slot], p.lhs_shift, p.rhs, gamma);
    fl = (gf >> 30) & 1;
  }
  if (live && kl == 0) {
    const int64_t lam = rho / p.rows;
    const int64_t at = lam * p.out_rows + p.out_row0 + (rho - lam * p.rows);
    for (int dst = 0; dst < p.n_out; ++dst) {
      p.sigma[dst][at] = static_cast<int16_t>(sg);
      p.flag[dst][at] = static_cast<uint8_t>(fl);
    }
  }
}

// ---- CRT + output ------------------------------------------------------------------------------
struct CrtParams {
  const uint8_t* W;            // [N][b][m][n_hat]
  const int16_t *sigma, *tau;  // [b][m], [b][n]
  const uint8_t *fA, *fB;
  const double *A, *B;         // post-swap operands (native path of flagged outputs)
  double* C;
  Vectors v;
  int64_t m, n, n_hat, k, b;
  int32_t lg_fast;
  int32_t part;  // 0 all outputs, 1 emulated outputs only, 2 native-path outputs only
  int32_t exact_only;  // verification: every output takes the integer path
  double alpha, beta;
  CrtTables t;
};

__device__ __forceinline__ double finish(double D, double alpha, double beta, const double* c) {
  const double E = (alpha == 1.0) ? D : __dmul_rn(alpha, D);
  return (beta == 0.0) ? E : __fma_rn(beta, *c, E);
}

__device__ __noinline__ double native_dot(const double* a, const double* b, const int64_t* ak,
                                          const int64_t* bk, int64_t k) {
  double acc = 0.0;
  for (int64_t h = 0; h < k; ++h) acc = __fma_rn(a[ak[h]], b[bk[h]], acc);
  return acc;
}

// The integer path of one output (exact CRT on limbs, one rounding): taken by the few outputs whose
// floating-point shortcut cannot vouch for its rounding. Out of line, and it reads its digits from
// the planes again, so that nothing of it weighs on the registers of the common path.
template <int N>
__device__ __noinline__ double crt_exact(const CrtTables* t, const uint8_t* w, int64_t plane, int e) {
  constexpr int WORDS = dev::CrtShape<N>::kWords;
  uint32_t y[N], mag[WORDS];
#pragma unroll
  for (int l = 0; l < N; ++l) y[l] = w[l * plane];
  const bool neg = dev::crt<N, 0>(*t, y, mag);
  return dev::round_scaled_fast<WORDS>(mag, neg, e);
}

// One thread = 4 consecutive columns of one row of one batch. Grid: x (with 2^lg_fast threads of a
// CTA) covers the column quads of a row, y and the remaining threads stride over the rows of one
// batch, z strides over the batches. Every output first goes through the floating-point shortcut
// (straight-line code for the thread's four); the outputs it cannot vouch for and those of
// flagged rows / columns (native FMA chain) are redone one by one afterwards.
constexpr int kCrtCtasPerSm = 4;  // 64 registers: measured against 2, 3 and 5 CTAs per SM
template <int N>
__global__ void __launch_bounds__(kThreads, kCrtCtasPerSm) k_crt(const __grid_constant__ CrtParams p) {
  const int64_t quads = p.n_hat >> 2;
  const int F = 1 << p.lg_fast, per = kThreads >> p.lg_fast;
  const int64_t jq = static_cast<int64_t>(blockIdx.x) * F + (threadIdx.x & (F - 1));
  const int64_t j0 = jq << 2;
  if (jq >= quads || j0 >= p.n) return;
  const int64_t plane = p.b * p.m * p.n_hat;
  const int64_t left = p.n - j0;  // >= 1
  const unsigned inside = left > 3 ? 15u : (1u << left) - 1u;
  // the thread's four outputs are adjacent in C and 16-byte aligned relative to the row start?
  const int64_t c0 = p.v.c_col[j0];
  const bool adjacent = left > 3 && p.v.c_col[j0 + 3] == c0 + 3 && p.v.c_col[j0 + 1] == c0 + 1 &&
                        p.v.c_col[j0 + 2] == c0 + 2;
  const int64_t c1 = left > 1 ? p.v.c_col[j0 + 1] : 0, c2 = left > 2 ? p.v.c_col[j0 + 2] : 0,
                c3 = left > 3 ? p.v.c_col[j0 + 3] : 0;
  const int64_t row_step = static_cast<int64_t>(gridDim.y) * per;
  for (int64_t lam = blockIdx.z; lam < p.b; lam += gridDim.z) {
    const int16_t* tau = p.tau + lam * p.n + j0;
    const uint8_t* fb = p.fB + lam * p.n + j0;
    const int t0 = tau[0], t1 = left > 1 ? tau[1] : 0, t2 = left > 2 ? tau[2] : 0,
              t3 = left > 3 ? tau[3] : 0;
    unsigned col_flags = fb[0] != 0 ? 1u : 0u;
    if (left > 1 && fb[1] != 0) col_flags |= 2u;
    if (left > 2 && fb[2] != 0) col_flags |= 4u;
    if (left > 3 && fb[3] != 0) col_flags |= 8u;
    double* cbat = p.C + p.v.c_bat[lam];
    const int64_t i0 = static_cast<int64_t>(blockIdx.y) * per + (threadIdx.x >> p.lg_fast);
    const uint8_t* w = p.W + (lam * p.m + i0) * p.n_hat + j0;
    for (int64_t i = i0; i < p.m; i += row_step, w += row_step * p.n_hat) {
      const int64_t rho = lam * p.m + i;
      const unsigned fa = p.fA[rho];
      // outputs of flagged rows / columns take the native path
      unsigned native = (fa != 0 ? 15u : col_flags) & inside;
      // part 0: every output. part 1: only the outputs of the emulated path (A and B are not
      // read); part 2: only the outputs of the native path.
      unsigned wanted = inside;
      if (p.part == 1) wanted &= ~native, native = 0;
      if (p.part == 2) {
        wanted &= native;
        if (wanted == 0) continue;
      }
      uint32_t packed[N];
#pragma unroll
      for (int l = 0; l < N; ++l) packed[l] = *reinterpret_cast<const uint32_t*>(w + l * plane);
      const int si = p.sigma[rho];
      double D0, D1, D2, D3;
      unsigned redo = 0;
      {
        // a zero the compiler cannot fold: with a known offset it holds all the constants of the
        // sums in registers across the row loop and spills
        int zero;
        asm volatile("mov.u32 %0, 0;" : "=r"(zero));
        double sh[4], sl[4];
        crt_fast_sums<N, 4>(p.t.fast, dev::PackedDigit{packed}, zero, sh, sl);
        if (!crt_fast_round(p.t.fast, sh[0], sl[0], -(si + t0), &D0)) redo |= 1u;
        if (!crt_fast_round(p.t.fast, sh[1], sl[1], -(si + t1), &D1)) redo |= 2u;
        if (!crt_fast_round(p.t.fast, sh[2], sl[2], -(si + t2), &D2)) redo |= 4u;
        if (!crt_fast_round(p.t.fast, sh[3], sl[3], -(si + t3), &D3)) redo |= 8u;
      }
      if (p.exact_only) redo = 15u;
      redo = (redo | native) & wanted;
      if (redo) {
        const double* arow = p.A + p.v.a_bat[lam] + p.v.a_row[i];
        const double* bbat = p.B + p.v.b_bat[lam];
#define IMD_REDO(x, D, tx)                                                                     \
  if (redo & (1u << x))                                                                          \
    D = (native & (1u << x)) ? native_dot(arow, bbat + p.v.b_col[j0 + x], p.v.a_k, p.v.b_k, p.k) \
                             : crt_exact<N>(&p.t, w + x, plane, -(si + tx));
        IMD_REDO(0, D0, t0) IMD_REDO(1, D1, t1) IMD_REDO(2, D2, t2) IMD_REDO(3, D3, t3)
#undef IMD_REDO
      }
      double* crow = cbat + p.v.c_row[i];
      double* c = crow + c0;
      if (adjacent && wanted == 15u && (reinterpret_cast<uintptr_t>(c) & 15) == 0) {
        double2* cv = reinterpret_cast<double2*>(c);
        double2 lo = make_double2(0.0, 0.0), hi = lo;
        if (p.beta != 0.0) {
          lo = cv[0];
          hi = cv[1];
        }
        lo.x = finish(D0, p.alpha, p.beta, &lo.x);
        lo.y = finish(D1, p.alpha, p.beta, &lo.y);
        hi.x = finish(D2, p.alpha, p.beta, &hi.x);
        hi.y = finish(D3, p.alpha, p.beta, &hi.y);
        cv[0] = lo;
        cv[1] = hi;
      } else {
        if (wanted & 1u) *c = finish(D0, p.alpha, p.beta, c);
        if (wanted & 2u) crow[c1] = finish(D1, p.alpha, p.beta, crow + c1);
        if (wanted & 4u) crow[c2] = finish(D2, p.alpha, p.beta, crow + c2);
        if (wanted & 8u) crow[c3] = finish(D3, p.alpha, p.beta, crow + c3);
      }
    }
  }
}

}  // namespace
}  // namespace imd
#include "small.cuh"
namespace imd {
namespace {

template <int N>
void launch_crt(const CrtParams& p, dim3 grid, cudaStream_t stream) {
  k_crt<N><<<grid, kThreads, 0, stream>>>(p);
}

// ---- degenerate paths --------------------------------------------------------------------------
struct EpilogueOnlyParams {
  const double *A, *B;
  double* C;
  Vectors v;
  int64_t m, n, k, b;
  double alpha, beta;
};

__global__ void __launch_bounds__(kThreads) k_direct(const __grid_constant__ EpilogueOnlyParams p) {
  const int64_t total = p.b * p.m * p.n;
  for (int64_t e = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t j = e % p.n, i = (e / p.n) % p.m, lam = e / (p.n * p.m);
    const double D = native_dot(p.A + p.v.a_bat[lam] + p.v.a_row[i],
                                p.B + p.v.b_bat[lam] + p.v.b_col[j], p.v.a_k, p.v.b_k, p.k);
    double* c = p.C + p.v.c_bat[lam] + p.v.c_row[i] + p.v.c_col[j];
    *c = finish(D, p.alpha, p.beta, c);
  }
}

__global__ void __launch_bounds__(kThreads) k_beta(const __grid_constant__ EpilogueOnlyParams p) {
  const int64_t total = p.b * p.m * p.n;
  for (int64_t e = blockIdx.x * static_cast<int64_t>(kThreads) + threadIdx.x; e < total;
       e += static_cast<int64_t>(gridDim.x) * kThreads) {
    const int64_t j = e % p.n, i = (e / p.n) % p.m, lam = e / (p.n * p.m);
    double* c = p.C + p.v.c_bat[lam] + p.v.c_row[i] + p.v.c_col[j];
    *c = (p.beta == 0.0) ? 0.0 : __dmul_rn(p.beta, *c);
  }
}

// ---- reference int8 GEMM (verification only) ----------------------------------------------------
__global__ void __launch_bounds__(kThreads) k_gemm_reference(const __grid_constant__ GemmShape s,
                                                             const int8_t* __restrict__ RA,
                                                             const int8_t* __restrict__ RB,
                                                             uint8_t* __restrict__ W) {
  const int64_t per_plane = static_cast<int64_t>(s.m) * s.n_hat;
  const int64_t item = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x;
  if (item >= per_plane * s.planes) return;
  const int64_t z = item / per_plane, rem = item % per_plane;
  const int64_t i = rem / s.n_hat, j = rem % s.n_hat;
  const int slot = static_cast<int>(z / s.batches);
  const int8_t* a = RA + (z * s.m + i) * static_cast<int64_t>(s.k_hat) + s.k0;
  const int8_t* b = RB + (z * s.b_rows + j) * static_cast<int64_t>(s.k_hat) + s.k0;
  int acc = 0;
  for (int h = 0; h < s.klen && j < s.b_rows; h += 4)
    acc = __dp4a(*reinterpret_cast<const int*>(a + h), *reinterpret_cast<const int*>(b + h), acc);
  uint8_t* w = W + ((static_cast<int64_t>(s.mod0 + slot) * s.batches + z % s.batches) * s.m + i) * s.n_hat + j;
  const int64_t pm = s.p[slot];
  int64_t r = static_cast<int64_t>(acc) % pm;
  if (r < 0) r += pm;
  r = (r * s.q[slot] + (s.add ? *w : 0)) % pm;  // planes hold y = q (A'B') mod p
  *w = static_cast<uint8_t>(r);
}

unsigned int grid_for(int64_t items, int64_t cap = int64_t{1} << 30) {
  int64_t g = (items + kThreads - 1) / kThreads;
  if (g < 1) g = 1;
  if (g > cap) g = cap;
  return static_cast<unsigned int>(g);
}

bool launched() { return cudaPeekAtLastError() == cudaSuccess; }

// log2 of the rows a CTA of the scale kernel owns. Rows contiguous: 32 rows x 8 K lanes (256-byte
// segments per K step), fewer rows (down to 4: one 32-byte sector per step) and more K lanes when
// that leaves fewer than two CTAs per SM. K contiguous: as many K lanes as k can feed.
int scale_lg_rt(bool rows_fast, int64_t k, int64_t rows_total) {
  if (rows_fast) {
    int lg = 5;
    while (lg > 2 && (rows_total >> lg) < 2 * kDefaultSms) --lg;
    return lg;
  }
  int lanes = 1;
  while (lanes < 256 && lanes < k) lanes <<= 1;
  int lg = 0;
  while ((256 >> lg) > lanes) ++lg;
  return lg;
}

}  // namespace

unsigned int* device_error_word() {
  unsigned int* p = nullptr;
  cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_error_word);
  return p;
}

imd_status_t generate_vectors(const ExecPlan& e, int64_t* vec, cudaStream_t stream) {
  VecParams p;
  p.modes = e.modes;
  p.m = e.m, p.n = e.n, p.k = e.k, p.b = e.b;
  p.segments = 9;
  k_vectors<<<grid_for(e.vec_count, 1 << 20), kThreads, 0, stream>>>(p, vec);
  return launched() ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
}

imd_status_t gemm_reference_launch(const GemmShape& s, const int8_t* RA, const int8_t* RB,
                                   uint8_t* W, cudaStream_t stream) {
  const int64_t items = static_cast<int64_t>(s.m) * s.n_hat * s.planes;
  k_gemm_reference<<<grid_for(items), kThreads, 0, stream>>>(s, RA, RB, W);
  return launched() ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
}

GemmShape gemm_shape(const ExecPlan& e, const uint32_t* crt_q, int mod0, int mods, int chunk) {
  GemmShape s{};
  s.m = static_cast<int32_t>(e.m);
  s.n_hat = static_cast<int32_t>(e.n_hat);
  s.b_rows = static_cast<int32_t>((e.packed & 2) ? e.n : e.n_hat);
  s.k_hat = static_cast<int32_t>(e.k_hat);
  s.k0 = static_cast<int32_t>(chunk * kChunk);
  s.klen = static_cast<int32_t>(e.k_hat - s.k0 < kChunk ? e.k_hat - s.k0 : kChunk);
  s.batches = static_cast<int32_t>(e.b);
  s.planes = static_cast<int32_t>(mods * e.b);
  s.mod0 = mod0;
  s.add = chunk > 0;
  for (int i = 0; i < mods; ++i) {
    const uint32_t p = static_cast<uint32_t>(kModuli[mod0 + i]);
    s.p[i] = p;
    s.magic[i] = static_cast<uint32_t>((uint64_t{1} << 32) / p);
    s.magic_up[i] = static_cast<uint32_t>(((uint64_t{1} << 32) + p - 1) / p);
    s.bias[i] = static_cast<uint32_t>(((uint64_t{1} << 31) + p - 1) / p * p);
    s.q[i] = crt_q[mod0 + i];
  }
  return s;
}

constexpr int kSmallSmemMax = 200 * 1024;

// Plan time: the fused quantise launches may use up to kQStageMax units of dynamic shared memory,
// the small-contraction kernel up to kSmallSmemMax bytes.
imd_status_t quantize_setup() {
  const int bytes = kQStageMax * kQStageBytes;
  const bool ok =
      cudaFuncSetAttribute(k_quantize<2, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess &&
      cudaFuncSetAttribute(k_quantize<2, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess &&
      cudaFuncSetAttribute(k_quantize<3, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess &&
      cudaFuncSetAttribute(k_quantize<3, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) == cudaSuccess;
  if (!ok) cudaGetLastError();
  if (ok && cudaFuncSetAttribute(k_small, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kSmallSmemMax) != cudaSuccess) {
    cudaGetLastError();
    return IMD_STATUS_CUDA_ERROR;
  }
  return ok ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
}

namespace {

// One post-swap operand as the scale and residue kernels read it.
struct OperandView {
  const double* X;
  const int64_t *row, *kv, *bat;
  int64_t rows, rows_pad;  // rows per batch; rows per batch of the residue planes
  bool rows_fast;
  int64_t k_run;
  // Where the rows land in the outputs (see ScaleParams / ResidueParams); 0 = the defaults.
  int64_t out_rows = 0, out_row0 = 0;
};

// Destinations of a scale / residue launch.
struct PackDests {
  int n = 1;
  int16_t* sigma[kMaxDests] = {};
  uint8_t* flag[kMaxDests] = {};
  int8_t* res[kMaxDests] = {};
};

OperandView operand_view(const ExecPlan& e, const Vectors& v, int x, const double* X) {
  OperandView o;
  o.X = X;
  o.row = x == 0 ? v.a_row : v.b_col;
  o.kv = x == 0 ? v.a_k : v.b_k;
  o.bat = x == 0 ? v.a_bat : v.b_bat;
  o.rows = x == 0 ? e.m : e.n;
  o.rows_pad = x == 0 ? e.m : e.n_hat;
  o.rows_fast = e.rows_fast[x];
  o.k_run = e.modes.count[kClsK] > 0 && e.modes.stride[e.modes.first[kClsK]][x] == 1
                ? e.modes.extent[e.modes.first[kClsK]]
                : 0;
  return o;
}

bool launch_scale(const ExecPlan& e, const OperandView& o, const PackDests& d, cudaStream_t stream) {
  ScaleParams p{};
  p.X = o.X;
  p.row = o.row, p.kv = o.kv, p.bat = o.bat;
  p.rows = o.rows;
  p.batches = e.b;
  p.k = e.k;
  p.rows_fast = o.rows_fast;
  p.lg_rt = scale_lg_rt(o.rows_fast, e.k, o.rows * e.b);
  p.lhs_shift = e.lhs_shift;
  p.force_exact = hooks().force_exact_shift;
  p.rhs = e.rhs;
  p.fast = e.fast;
  p.out_rows = o.out_rows > 0 ? o.out_rows : o.rows;
  p.out_row0 = o.out_row0;
  p.n_out = d.n;
  for (int i = 0; i < d.n; ++i) p.sigma[i] = d.sigma[i], p.flag[i] = d.flag[i];
  const int64_t rt = int64_t{1} << p.lg_rt;
  const int64_t blocks = (p.rows * p.batches + rt - 1) / rt;
  k_scale<<<static_cast<unsigned int>(blocks), kThreads, 0, stream>>>(p);
  return launched();
}

// An operand whose K direction is the contiguous one is quantised by fused launches (shift and
// residues of the first group in one kernel, the row read from HBM once); one that is contiguous
// along its rows gets its shifts from k_scale first, and tiles of 8 adjacent rows afterwards.
bool fuses(const OperandView& o) { return !o.rows_fast; }

// Residue planes of moduli [mod0, mod0 + mods) of one operand into R[slot][batch][rows_pad][k_hat];
// with `fused` also the operand's shifts and flags (into every destination).
bool launch_quantize(const ExecPlan& e, const ResidueTables& t, const OperandView& o,
                     const PackDests& d, int mod0, int mods, bool fused, cudaStream_t stream) {
  QuantParams p{};
  p.X = o.X;
  p.row = o.row, p.kv = o.kv, p.bat = o.bat;
  p.rows = o.rows;
  p.rows_pad = o.rows_pad;
  p.batches = e.b;
  p.k = e.k;
  p.k_hat = e.k_hat;
  p.contig = o.k_run >= e.k ? 2 : (o.k_run >= 8 ? 1 : 0);
  p.trunc = e.trunc;
  p.mod0 = mod0;
  p.mods = mods;
  p.force_exact = hooks().force_exact_shift;
  p.lhs_shift = e.lhs_shift;
  p.rhs = e.rhs;
  p.fast = e.fast;
  const bool placed = o.out_rows > 0;  // rows of a larger packed buffer
  p.plane_rows = placed ? o.out_rows : o.rows_pad;
  p.sigma_rows = placed ? o.out_rows : o.rows;
  p.row0 = o.out_row0;
  p.sigma_in = d.sigma[0];
  p.flag_in = d.flag[0];
  p.n_out = d.n;
  for (int i = 0; i < d.n; ++i) p.sigma[i] = d.sigma[i], p.flag[i] = d.flag[i], p.R[i] = d.res[i];
  p.t = t;
  const int64_t chunks = (e.k_hat + kQChunk - 1) / kQChunk;
  const int64_t span_all = chunks * kQChunk;
  if (o.rows_fast) {
    p.lg_wpr = 0;  // a warp per row: the rows of a CTA are adjacent in memory
    p.k_span = span_all < 1024 ? span_all : 1024;
  } else {
    p.lg_wpr = 0;
    while (p.lg_wpr < kQLgWarps && (int64_t{2} << p.lg_wpr) <= chunks) ++p.lg_wpr;
    p.k_span = span_all;
  }
  size_t smem = 0;
  if (fused) {
    const int64_t per_thread = (e.k_hat + (int64_t{256} << p.lg_wpr) - 1) / (int64_t{256} << p.lg_wpr);
    p.stage_units = static_cast<int32_t>(per_thread < kQStageMax ? per_thread : kQStageMax);
    smem = static_cast<size_t>(p.stage_units) * kQStageBytes;
  }
  const int64_t rows_per = kQWarps >> p.lg_wpr;
  const int64_t gx = (p.rows_pad * p.batches + rows_per - 1) / rows_per;
  const int64_t gy = fused ? 1 : (span_all + p.k_span - 1) / p.k_span;
  if (gx > INT32_MAX || gy > 65535) return false;
  const dim3 grid(static_cast<unsigned int>(gx), static_cast<unsigned int>(gy));
  const int variant = (t.words == 2 ? 0 : 4) + (fused ? 2 : 0) + (e.trunc ? 1 : 0);
  switch (variant) {
    case 0: k_quantize<2, false, false><<<grid, kQThreads, smem, stream>>>(p); break;
    case 1: k_quantize<2, false, true><<<grid, kQThreads, smem, stream>>>(p); break;
    case 2: k_quantize<2, true, false><<<grid, kQThreads, smem, stream>>>(p); break;
    case 3: k_quantize<2, true, true><<<grid, kQThreads, smem, stream>>>(p); break;
    case 4: k_quantize<3, false, false><<<grid, kQThreads, smem, stream>>>(p); break;
    case 5: k_quantize<3, false, true><<<grid, kQThreads, smem, stream>>>(p); break;
    case 6: k_quantize<3, true, false><<<grid, kQThreads, smem, stream>>>(p); break;
    default: k_quantize<3, true, true><<<grid, kQThreads, smem, stream>>>(p); break;
  }
  return launched();
}

}  // namespace

imd_status_t enqueue_contract(const imd_plan_st& plan, double alpha, const double* A,
                              const double* B, double beta, double* C, void* ws,
                              cudaStream_t stream, const void* const packed[2], int part) {
  const ExecPlan& e = plan.exec;
  char* base = static_cast<char*>(ws);
  auto region = [&](int r) { return base + e.layout.offset[r]; };
  phase_mark(0, stream);
  const int64_t* vec = e.vec_resident ? static_cast<const int64_t*>(plan.vec_dev)
                                      : reinterpret_cast<const int64_t*>(region(IMD_REGION_VEC));
  if (!e.vec_resident)
    if (generate_vectors(e, const_cast<int64_t*>(vec), stream) != IMD_STATUS_SUCCESS)
      return IMD_STATUS_CUDA_ERROR;
  const Vectors v = split_vectors(vec, e);

  if (alpha == 0.0 || e.k == 0 || e.path == Path::kDirect) {
    EpilogueOnlyParams p{A, B, C, v, e.m, e.n, e.k, e.b, alpha, beta};
    const unsigned int grid = grid_for(e.b * e.m * e.n, 1 << 20);
    if (alpha == 0.0 || e.k == 0) k_beta<<<grid, kThreads, 0, stream>>>(p);
    else k_direct<<<grid, kThreads, 0, stream>>>(p);
    phase_mark(5, stream);
    return launched() ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
  }

  const void* const no_packs[2] = {nullptr, nullptr};
  if (packed == nullptr) packed = no_packs;
  // shifts, flags and residue planes of each post-swap operand: workspace regions, or the regions
  // of its packed buffer (then nothing is computed for that operand here)
  const int16_t* sX[2];
  const uint8_t* fX[2];
  const int8_t* RX[2];
  const int sreg[2] = {IMD_REGION_SA, IMD_REGION_SB}, freg[2] = {IMD_REGION_FA, IMD_REGION_FB},
            rreg[2] = {IMD_REGION_RA, IMD_REGION_RB};
  bool from_pack[2];
  for (int x = 0; x < 2; ++x) {
    from_pack[x] = (e.packed >> x) & 1;
    if (from_pack[x]) {
      if (packed[x] == nullptr) return IMD_STATUS_INVALID_VALUE;
      const char* pk = static_cast<const char*>(packed[x]);
      sX[x] = reinterpret_cast<const int16_t*>(pk + e.pack_off[x][0]);
      fX[x] = reinterpret_cast<const uint8_t*>(pk + e.pack_off[x][1]);
      RX[x] = reinterpret_cast<const int8_t*>(pk + e.pack_off[x][2]);
    } else {
      sX[x] = reinterpret_cast<const int16_t*>(region(sreg[x]));
      fX[x] = reinterpret_cast<const uint8_t*>(region(freg[x]));
      RX[x] = reinterpret_cast<const int8_t*>(region(rreg[x]));
    }
  }
  uint8_t* W = reinterpret_cast<uint8_t*>(region(IMD_REGION_W));
  const OperandView ov[2] = {operand_view(e, v, 0, A), operand_view(e, v, 1, B)};

  if (e.small() && part == 0 && hooks().small_path) {
    SmallParams sp{};
    sp.A = A, sp.B = B, sp.C = C;
    sp.v = v;
    sp.m = e.m, sp.n = e.n, sp.k = e.k, sp.b = e.b;
    sp.kh = static_cast<int32_t>((e.k + 31) / 32 * 32);
    sp.N = e.N, sp.trunc = e.trunc ? 1 : 0, sp.lhs_shift = e.lhs_shift;
    sp.force_exact_shift = hooks().force_exact_shift, sp.exact_crt = hooks().force_exact_crt;
    sp.rhs = e.rhs, sp.fast = e.fast;
    sp.alpha = alpha, sp.beta = beta;
    sp.sigma_a = const_cast<int16_t*>(sX[0]), sp.sigma_b = const_cast<int16_t*>(sX[1]);
    sp.flag_a = const_cast<uint8_t*>(fX[0]), sp.flag_b = const_cast<uint8_t*>(fX[1]);
    sp.t = plan.res, sp.crt = plan.crt;
    // as many moduli per pass as the residues' share of shared memory holds
    const int64_t fixed = static_cast<int64_t>(small_smem_bytes(sp.kh, 0, e.N));
    const int64_t per_modulus = static_cast<int64_t>(kSmRows) * (sp.kh + kSmPad);
    int64_t group = (kSmallSmemMax - fixed) / per_modulus;
    if (group > e.N) group = e.N;
    if (group < 1) return IMD_STATUS_CUDA_ERROR;  // cannot happen: k <= 128 leaves room for 8 moduli
    sp.group = static_cast<int32_t>(group);
    const int64_t tiles = ((e.m + kSmTM - 1) / kSmTM) * ((e.n + kSmTN - 1) / kSmTN) * e.b;
    k_small<<<static_cast<unsigned int>(tiles), kSmThreads, small_smem_bytes(sp.kh, sp.group, e.N), stream>>>(sp);
    phase_mark(7, stream);
    return launched() ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
  }

  PackDests dest[2];
  // Parts (imd_contract_packed_part): 0 everything; 1 everything but the native-path outputs;
  // 2 only those; 3 the CRT of the emulated outputs alone; 16 + i the GEMM of residue group i alone
  // (with the shifts of in-line operands when i = 0 and their residues of that group).
  const int only_group = part >= 16 ? part - 16 : -1;
  const bool run_groups = part == 0 || part == 1 || only_group >= 0;
  const bool run_scale = part == 0 || part == 1 || only_group == 0;
  const bool run_crt = only_group < 0;
  const int crt_part = part == 3 ? 1 : part;
  if (only_group >= 0 && static_cast<int64_t>(only_group) * e.g >= e.N) return IMD_STATUS_INVALID_VALUE;
  for (int x = 0; x < 2; ++x) {
    dest[x].sigma[0] = const_cast<int16_t*>(sX[x]);
    dest[x].flag[0] = const_cast<uint8_t*>(fX[x]);
    dest[x].res[0] = const_cast<int8_t*>(RX[x]);
    if (run_scale && !from_pack[x] && !fuses(ov[x]) && !launch_scale(e, ov[x], dest[x], stream))
      return IMD_STATUS_CUDA_ERROR;
  }

  phase_mark(1, stream);
  GemmPlanInfo info;
  info.encode_tiled = plan.encode_tiled;
  info.error_word = static_cast<unsigned int*>(plan.error_word);
  info.sms = plan.sms;
  for (int g0 = 0; run_groups && g0 < e.N; g0 += e.g) {
    if (only_group >= 0 && g0 != only_group * e.g) continue;
    const int mods = e.N - g0 < e.g ? e.N - g0 : e.g;
    const int8_t* Rg[2];
    for (int x = 0; x < 2; ++x) {
      if (from_pack[x]) {  // a packed buffer holds all N planes: the group's start at plane g0
        Rg[x] = RX[x] + static_cast<int64_t>(g0) * e.b * ov[x].rows * e.k_hat;
        continue;
      }
      Rg[x] = RX[x];
      // the launch of the first group of a call also computes the shifts of a fusing operand
      const bool fused = run_scale && g0 == 0 && fuses(ov[x]);
      if (!launch_quantize(e, plan.res, ov[x], dest[x], g0, mods, fused, stream))
        return IMD_STATUS_CUDA_ERROR;
    }
    phase_mark(2, stream);
    for (int64_t c = 0; c < e.k_chunks; ++c) {
      const GemmShape s = gemm_shape(e, plan.crt.q, g0, mods, static_cast<int>(c));
      const imd_status_t st = hooks().reference_gemm
                                  ? gemm_reference_launch(s, Rg[0], Rg[1], W, stream)
                                  : gemm_launch(info, s, Rg[0], Rg[1], W, stream);
      if (st != IMD_STATUS_SUCCESS) return st;
    }
    phase_mark(3, stream);
  }

  if (!run_crt) return launched() ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
  CrtParams p{};
  p.W = W;
  p.sigma = sX[0], p.tau = sX[1], p.fA = fX[0], p.fB = fX[1];
  p.A = A, p.B = B, p.C = C;
  p.v = v;
  p.m = e.m, p.n = e.n, p.n_hat = e.n_hat, p.k = e.k, p.b = e.b;
  p.alpha = alpha, p.beta = beta;
  p.part = crt_part;
  p.exact_only = hooks().force_exact_crt;
  p.t = plan.crt;
  const int64_t quads = e.n_hat >> 2;
  p.lg_fast = 0;
  while (p.lg_fast < 8 && (int64_t{1} << p.lg_fast) < quads) ++p.lg_fast;
  const int64_t Fq = int64_t{1} << p.lg_fast, perq = kThreads / Fq;
  const int64_t gxq = (quads + Fq - 1) / Fq;
  // A thread's set-up (its columns' shifts, flags and C offsets) is paid once and used for all the
  // rows it walks: about twelve CTAs per SM in all, rows of one batch over y, batches over z.
  const int64_t want_ctas = int64_t{12} * plan.sms;
  int64_t gyq = (e.m + perq - 1) / perq;
  const int64_t gy_cap = (want_ctas + gxq - 1) / gxq;
  if (gyq > gy_cap) gyq = gy_cap;
  if (gyq > 65535) gyq = 65535;
  int64_t gzq = (want_ctas + gxq * gyq - 1) / (gxq * gyq);
  if (gzq > e.b) gzq = e.b;
  if (gzq > 65535) gzq = 65535;
  if (gzq < 1) gzq = 1;
  const dim3 grid(static_cast<unsigned int>(gxq), static_cast<unsigned int>(gyq),
                  static_cast<unsigned int>(gzq));
  if (plan.crt.nl != dev::crt_limbs_of(e.N)) return IMD_STATUS_CUDA_ERROR;  // tables out of step
  switch (e.N) {
#define IMD_CRT_CASE(n) case n: launch_crt<n>(p, grid, stream); break;
    IMD_CRT_CASE(2) IMD_CRT_CASE(3) IMD_CRT_CASE(4) IMD_CRT_CASE(5) IMD_CRT_CASE(6)
    IMD_CRT_CASE(7) IMD_CRT_CASE(8) IMD_CRT_CASE(9) IMD_CRT_CASE(10) IMD_CRT_CASE(11)
    IMD_CRT_CASE(12) IMD_CRT_CASE(13) IMD_CRT_CASE(14) IMD_CRT_CASE(15) IMD_CRT_CASE(16)
    IMD_CRT_CASE(17) IMD_CRT_CASE(18) IMD_CRT_CASE(19) IMD_CRT_CASE(20)
#undef IMD_CRT_CASE
    default: return IMD_STATUS_INVALID_VALUE;
  }
  phase_mark(4, stream);
  return launched() ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
}

// ---- imd_pack --------------------------------------------------------------------------------
namespace {

struct ZeroRanges {
  uint64_t begin[4], end[4];
};

// The bytes of a packed buffer that no row owns: the alignment gaps behind each region and the
// tail behind the last residue plane. A few hundred bytes plus at most 15 rows of k_hat.
__global__ void __launch_bounds__(kThreads) k_zero_ranges(const __grid_constant__ ZeroRanges z,
                                                          uint8_t* __restrict__ out) {
  for (int r = 0; r < 4; ++r)
    for (uint64_t at = z.begin[r] + blockIdx.x * static_cast<uint64_t>(kThreads) + threadIdx.x;
         at < z.end[r]; at += static_cast<uint64_t>(gridDim.x) * kThreads)
      out[at] = 0;
}

}  // namespace

imd_status_t enqueue_pack(const ExecPlan& e, const ResidueTables& tables, const PackRegions& layout,
                          const double* X, void* packed, void* ws, cudaStream_t stream) {
  void* const one[1] = {packed};
  return enqueue_pack_scatter(e, tables, layout, e.m, 0, X, one, 1, ws, stream);
}

// The rows of X (a piece) as rows [row0, row0 + e.m) of packed buffers whose batches have
// slab_rows rows and the byte layout `layout`; every destination gets the same bytes (they may be
// other GPUs' memory: plain stores). Gaps and tail are zeroed in dest[0], the caller's own buffer.
imd_status_t enqueue_pack_scatter(const ExecPlan& e, const ResidueTables& tables,
                                  const PackRegions& layout, int64_t slab_rows, int64_t row0,
                                  const double* X, void* const* dest, int n_dest, void* ws,
                                  cudaStream_t stream) {
  if (layout.total == 0 || e.m == 0) return IMD_STATUS_SUCCESS;
  if (n_dest < 1 || n_dest > kMaxDests) return IMD_STATUS_INVALID_VALUE;
  uint8_t* out = static_cast<uint8_t*>(dest[0]);
  int64_t* vec = static_cast<int64_t*>(ws);
  phase_mark(0, stream);
  VecParams vp;
  vp.modes = e.modes;
  vp.m = e.m, vp.n = 0, vp.k = e.k, vp.b = e.b;
  vp.segments = 3;
  k_vectors<<<grid_for(e.vec_count, 1 << 20), kThreads, 0, stream>>>(vp, vec);
  if (!launched()) return IMD_STATUS_CUDA_ERROR;

  const uint64_t planes = static_cast<uint64_t>(e.N) * e.b * slab_rows * e.k_hat;
  ZeroRanges z{};
  uint64_t longest = 0;
  for (int r = 0; r < 3; ++r) {
    z.begin[r] = layout.offset[r] + layout.bytes[r];
    z.end[r] = r < 2 ? layout.offset[r + 1] : layout.total;
  }
  z.begin[3] = layout.offset[2] + planes;          // the tail: part of region 2's byte count
  z.end[3] = layout.offset[2] + layout.bytes[2];
  for (int r = 0; r < 4; ++r)
    if (z.end[r] - z.begin[r] > longest) longest = z.end[r] - z.begin[r];
  if (longest > 0) {
    k_zero_ranges<<<grid_for(static_cast<int64_t>(longest), 1 << 16), kThreads, 0, stream>>>(z, out);
    if (!launched()) return IMD_STATUS_CUDA_ERROR;
  }

  OperandView o;  // X as operand A of a one-operand view: rows, K, batches
  o.X = X;
  o.row = vec, o.kv = vec + e.m, o.bat = vec + e.m + e.k;
  o.rows = e.m, o.rows_pad = e.m;
  o.rows_fast = e.rows_fast[0];
  o.k_run = e.modes.count[kClsK] > 0 && e.modes.stride[e.modes.first[kClsK]][kTenA] == 1
                ? e.modes.extent[e.modes.first[kClsK]]
                : 0;
  o.out_rows = slab_rows, o.out_row0 = row0;
  PackDests d;
  d.n = n_dest;
  for (int i = 0; i < n_dest; ++i) {
    uint8_t* base = static_cast<uint8_t*>(dest[i]);
    d.sigma[i] = reinterpret_cast<int16_t*>(base + layout.offset[0]);
    d.flag[i] = base + layout.offset[1];
    d.res[i] = reinterpret_cast<int8_t*>(base + layout.offset[2]);
  }
  if (!fuses(o) && !launch_scale(e, o, d, stream)) return IMD_STATUS_CUDA_ERROR;
  if (!launch_quantize(e, tables, o, d, 0, e.N, fuses(o), stream)) return IMD_STATUS_CUDA_ERROR;
  phase_mark(6, stream);
  return IMD_STATUS_SUCCESS;
}

// ---- bounded wait on flags --------------------------------------------------------------------------
// For exchanges in which a peer's copy engine writes data into this GPU's memory and then a 32-bit
// flag: one thread per flag polls (system-scope acquire loads) until the flag holds `expect`, for at
// most `limit` polls; a thread that gives up sets bit 2 of the device error word and returns, so
// the stream always moves on. Kernels launched after this one see the data the flags announce.
namespace {

struct WaitParams {
  const unsigned int* flag[kMaxWaitFlags];
  int n;
  unsigned int expect;
  unsigned long long limit;
  unsigned long long max_ns;
  unsigned int* error_word;
};

__global__ void k_wait_flags(WaitParams p) {
  const int i = threadIdx.x;
  if (i >= p.n) return;
  // bounded twice: by the poll count and by about two seconds of the global timer, whichever
  // comes first (a poll takes longer when the GPU is busy, the timer does not)
  unsigned long long t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (unsigned long long it = 0; it < p.limit; ++it) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p.flag[i]) : "memory");
    if (v == p.expect) return;
    __nanosleep(200);
    if ((it & 1023) == 1023) {
      unsigned long long t1;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t1));
      if (t1 - t0 > p.max_ns) break;
    }
  }
  atomicOr(p.error_word, 4u);
}

}  // namespace

imd_status_t enqueue_wait_flags(const unsigned int* const* flags, int n, unsigned int expect,
                                unsigned long long limit, cudaStream_t stream) {
  WaitParams p;
  for (int i = 0; i < kMaxWaitFlags; ++i) p.flag[i] = i < n ? flags[i] : nullptr;
  p.n = n, p.expect = expect, p.limit = limit;
  p.max_ns = 2000000000ull;
  p.error_word = device_error_word();
  if (p.error_word == nullptr) return IMD_STATUS_CUDA_ERROR;
  k_wait_flags<<<1, kMaxWaitFlags, 0, stream>>>(p);
  return launched() ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
}

// ---- pushes by a small copy kernel --------------------------------------------------------------
// The residue exchange of the multi-GPU driver sends a rank's rows of the residue planes into
// the other consumers' slab buffers while the GEMM of the previous residue group runs. One launch
// of a few CTAs (they share the SMs with the persistent GEMM, which leaves threads and registers
// free) copies every range with 16-byte loads and plain stores (destinations may be peers' memory
// mapped into this process) and, after the last CTA has finished, writes `value` into the flag
// words that tell the consumers. Order: every CTA fences its stores at system scope before it
// counts itself done; the last one fences again and then stores the flags.
namespace {

constexpr int kPushTickets = 64;
__device__ unsigned int g_push_done[kPushTickets];

struct PushParams {
  uint4* dst[kMaxPushRanges];
  const uint4* src[kMaxPushRanges];
  long long units[kMaxPushRanges];   // 16-byte units
  int ranges;
  unsigned int* flag[kMaxPushFlags];
  int flags;
  unsigned int value;
  int ticket;
};

__global__ void __launch_bounds__(kThreads) k_push(const __grid_constant__ PushParams p) {
  const long long step = static_cast<long long>(gridDim.x) * kThreads;
  const long long first = static_cast<long long>(blockIdx.x) * kThreads + threadIdx.x;
  for (int r = 0; r < p.ranges; ++r) {
    const uint4* __restrict__ src = p.src[r];
    uint4* __restrict__ dst = p.dst[r];
    const long long n = p.units[r];
    long long i = first;
    for (; i + 3 * step < n; i += 4 * step) {  // four loads in flight per thread
      // streaming loads: the planes are read once here and must not push the GEMM's operand
      // tiles out of L2
      const uint4 a = __ldcs(src + i), b = __ldcs(src + i + step), c = __ldcs(src + i + 2 * step),
                  d = __ldcs(src + i + 3 * step);
      dst[i] = a, dst[i + step] = b, dst[i + 2 * step] = c, dst[i + 3 * step] = d;
    }
    for (; i < n; i += step) dst[i] = __ldcs(src + i);
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(&g_push_done[p.ticket], 1u) + 1;
    if (done == gridDim.x) {
      g_push_done[p.ticket] = 0;  // the ticket is free again once this launch has ended
      __threadfence_system();
      for (int f = 0; f < p.flags; ++f)
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flag[f]), "r"(p.value) : "memory");
    }
  }
}

std::atomic<unsigned int> g_push_ticket{0};

}  // namespace

imd_status_t enqueue_push(void* const* dst, const void* const* src, const int64_t* bytes, int ranges,
                          unsigned int* const* flags, int num_flags, unsigned int value, int ctas,
                          cudaStream_t stream) {
  PushParams p = {};
  p.ranges = ranges, p.flags = num_flags, p.value = value;
  for (int r = 0; r < ranges; ++r) {
    p.dst[r] = static_cast<uint4*>(dst[r]);
    p.src[r] = static_cast<const uint4*>(src[r]);
    p.units[r] = bytes[r] / 16;
  }
  for (int f = 0; f < num_flags; ++f) p.flag[f] = flags[f];
  // launches that may overlap (different streams) count on different words
  p.ticket = static_cast<int>(g_push_ticket.fetch_add(1) % kPushTickets);
  k_push<<<ctas, kThreads, 0, stream>>>(p);
  return launched() ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
}

imd_status_t enqueue_error_peek(unsigned int* host_word, cudaStream_t stream) {
  unsigned int* p = device_error_word();
  if (p == nullptr) return IMD_STATUS_CUDA_ERROR;
  if (cudaMemcpyAsync(host_word, p, sizeof(unsigned int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) {
    cudaGetLastError();
    return IMD_STATUS_CUDA_ERROR;
  }
  return IMD_STATUS_SUCCESS;
}

// ---- copies that run only when a row is flagged ----------------------------------------------------
// The native path of non-finite rows is the only reader of a slab's FP64 values. A rank of the
// multi-GPU driver therefore fetches the other ranks' FP64 pieces only when a row flag of its slabs
// is set: every CTA scans the (few KB of) flags; if none is set the kernel ends, else the grid
// copies the ranges with 8-byte loads and stores (sources may be peers' memory).
namespace {

struct CopyIfParams {
  const unsigned char* flags[kMaxFlagRanges];
  long long flag_bytes[kMaxFlagRanges];
  int ranges;
  unsigned long long* dst[kMaxCondCopies];
  const unsigned long long* src[kMaxCondCopies];
  long long vecs[kMaxCondCopies];   // 8-byte units
  int copies;
};

__global__ void __launch_bounds__(kThreads) k_copy_if_flagged(CopyIfParams p) {
  int mine = 0;
  for (int r = 0; r < p.ranges; ++r)
    for (long long i = threadIdx.x; i < p.flag_bytes[r]; i += blockDim.x) mine |= p.flags[r][i];
  if (!__syncthreads_or(mine)) return;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (int c = 0; c < p.copies; ++c)
    for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.vecs[c];
         i += step)
      p.dst[c][i] = p.src[c][i];
}

}  // namespace

imd_status_t enqueue_copy_if_flagged(const unsigned char* const* flags, const int64_t* flag_bytes,
                                     int ranges, void* const* dst, const void* const* src,
                                     const int64_t* bytes, int copies, cudaStream_t stream) {
  CopyIfParams p = {};
  p.ranges = ranges, p.copies = copies;
  for (int r = 0; r < ranges; ++r) p.flags[r] = flags[r], p.flag_bytes[r] = flag_bytes[r];
  for (int c = 0; c < copies; ++c) {
    p.dst[c] = static_cast<unsigned long long*>(dst[c]);
    p.src[c] = static_cast<const unsigned long long*>(src[c]);
    p.vecs[c] = bytes[c] / 8;
  }
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) {
    cudaGetLastError();
    return IMD_STATUS_CUDA_ERROR;
  }
  k_copy_if_flagged<<<sms * 4, kThreads, 0, stream>>>(p);
  return launched() ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
}

// ---- built-in workspace ---------------------------------------------------------------------------
// A fixed workspace that lives in the library image, for callers that are not in a position to
// allocate device memory. The name below is only a handle on the host side: its device address is
// looked up once per device (with that device current) and that pointer is what the kernels get.
namespace {

constexpr size_t kBuiltinWorkspaceBytes = IMD_BUILTIN_WS_BYTES;  // per GPU that loads the library
constexpr int kBuiltinMaxDevices = 64;
static __device__ __align__(256) unsigned char g_builtin_workspace[kBuiltinWorkspaceBytes];

std::mutex g_builtin_lock;
void* g_builtin_ptr[kBuiltinMaxDevices] = {};

}  // namespace

// Device address of the built-in workspace on the current device; looked up on the first call per
// device, cached afterwards. No allocation.
imd_status_t builtin_workspace(void** ptr, size_t* bytes) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kBuiltinMaxDevices) {
    cudaGetLastError();
    return IMD_STATUS_CUDA_ERROR;
  }
  std::lock_guard<std::mutex> hold(g_builtin_lock);
  if (g_builtin_ptr[device] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_builtin_workspace) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return IMD_STATUS_CUDA_ERROR;
    }
    g_builtin_ptr[device] = p;
  }
  *ptr = g_builtin_ptr[device];
  *bytes = kBuiltinWorkspaceBytes;
  return IMD_STATUS_SUCCESS;
}

}  // namespace imd

extern "C" {

// imd_contract on the library's built-in workspace (see immerdink.h). Allocates nothing.
IMD_API imd_status_t imd_contract_builtin_ws(imd_plan_t plan, double alpha, const double* A,
                                             const double* B, double beta, double* C,
                                             cudaStream_t stream) {
  if (plan == nullptr) return IMD_STATUS_INVALID_VALUE;
  void* ws = nullptr;
  size_t bytes = 0;
  if (const imd_status_t st = imd::builtin_workspace(&ws, &bytes); st != IMD_STATUS_SUCCESS)
    return st;
  // imd_contract's own checks in their documented order: a plan that needs more than the fixed
  // 32 MiB fails its size test there (INSUFFICIENT_WORKSPACE), after the earlier checks
  return imd_contract(plan, alpha, A, B, beta, C, ws, bytes, stream);
}

}  // extern "C"
