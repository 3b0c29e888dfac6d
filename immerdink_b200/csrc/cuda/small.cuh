// Small contractions in one launch: shift, quantise, residues, int8 products, CRT and output of a
// 32 x 32 tile of C inside one CTA of 16 warps, for k <= 128. At such sizes the general sequence (vectors,
// quantise A, quantise B, GEMM, CRT) is bound by its launches and by the round trips of tiny
// intermediates through HBM. Every CTA scales and quantises the rows of A and the columns of B of
// its own tile (other tiles repeat some of that work, which is cheap here), keeps the residues in
// shared memory, multiplies them with mma.sync (m16n8k32, int8; a warp takes a quarter of the tile
// and every fourth modulus), reduces every product mod p_l into a digit in shared memory, and
// every thread then runs the CRT of two outputs: the FP64 shortcut over the digits in the order
// of the moduli, the integer CRT where the shortcut cannot vouch. The arithmetic is that of the general
// path, function by function (numerics.cuh, modred.hpp, crtfast.hpp): results are bit-identical.
//
// Counterpart in the reference: the fused small-shape path of src/contract.cu:800-926 (KF) and its
// dispatch, src/contract.cu:1411-1434.
#pragma once
#include <cstdint>

#include "kernels.hpp"
#include "numerics.cuh"

namespace imd {
namespace {

constexpr int kSmThreads = 512;  // measured on 64 x 32 x 48 . 48 x 40: 256 / 512 / 1024 threads 46 / 34 / 32 us
constexpr int kSmTM = 32, kSmTN = 32, kSmRows = kSmTM + kSmTN;
constexpr int kSmKMax = 128;
constexpr int64_t kSmDead = INT64_MIN;
constexpr int kSmPad = 16;  // bytes added to a residue row: fragment loads of 8 rows hit 8 banks

struct SmallParams {
  const double *A, *B;
  double* C;
  Vectors v;
  int64_t m, n, k, b;
  int32_t kh;      // k rounded up to a multiple of 32
  int32_t group;   // moduli whose residues fit in shared memory at once
  int32_t N, trunc, lhs_shift, force_exact_shift, exact_crt;
  Wide<8> rhs;
  ShiftFast fast;
  double alpha, beta;
  int16_t *sigma_a, *sigma_b;  // the call's shift and flag regions, written as the general path does
  uint8_t *flag_a, *flag_b;
  ResidueTables t;
  CrtTables crt;
};

inline size_t small_smem_bytes(int kh, int group, int N) {
  return static_cast<size_t>(kSmRows) * kh * 8 + static_cast<size_t>(group) * kSmRows * (kh + kSmPad) +
         static_cast<size_t>(N) * kSmTM * kSmTN;
}

// The shift and flag of one row, decided by eight adjacent lanes (lane x of the eight reads entries
// x, x + 8, ... of the row's bit patterns in shared memory; four rows per warp at a time), exactly
// as the quantise kernel decides them: FP64 shortcut, else exact 128-bit sum of squares. All 32
// lanes call it together; the shuffles stay inside a group of eight.
__device__ __forceinline__ void small_row_shift(const SmallParams& p, const uint64_t* row, int l8,
                                                bool live, int* sigma_out, bool* flag_out) {
  uint32_t mx = 0;
  double acc = 0.0;
  for (int h = l8; h < p.kh; h += 8) {
    const uint64_t u = row[h];
    mx = max(mx, static_cast<uint32_t>(u >> 32) & 0x7FFFFFFFu);
    const double x = __longlong_as_double(static_cast<long long>(u));
    acc = __fma_rn(x, x, acc);
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
  }
  int sg = 0;
  // rows outside the tensor (all zero) need no decision
  const bool quick = !live || (!p.force_exact_shift && dev::fast_shift(mx, acc, p.fast, p.lhs_shift, &sg));
  *sigma_out = sg;
  *flag_out = false;
  if (__all_sync(0xFFFFFFFFu, quick)) return;
  int g = 0;  // bit 30: a non-finite entry; low bits: gamma + 2048 (0: no finite nonzero entry)
  for (int h = l8; h < p.kh; h += 8) {
    uint64_t M;
    int E;
    const int kind = dev::decompose(row[h], &M, &E);
    if (kind < 0) g |= 1 << 30;
    else if (kind > 0) g = (g & (1 << 30)) | max(g & 0xFFFF, E + 52 + 2048);
  }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    const int other = __shfl_xor_sync(0xFFFFFFFFu, g, o);
    g = ((g | other) & (1 << 30)) | max(g & 0xFFFF, other & 0xFFFF);
  }
  const bool any = (g & 0xFFFF) != 0;
  const int gamma = (g & 0xFFFF) - 2048;
  uint64_t hi = 0, lo = 0;
  if (any)
    for (int h = l8; h < p.kh; h += 8) {
      uint64_t M;
      int E;
      if (dev::decompose(row[h], &M, &E) == 1) {
        uint64_t th, tl;
        dev::square_term(M, E, gamma, &th, &tl);
        lo += tl;
        hi += th + (lo < tl ? 1 : 0);
      }
    }
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) {
    const uint64_t oh = __shfl_xor_sync(0xFFFFFFFFu, hi, o), ol = __shfl_xor_sync(0xFFFFFFFFu, lo, o);
    lo += ol;
    hi += oh + (lo < ol ? 1 : 0);
  }
  if (!quick) {
    *sigma_out = any ? dev::shift_from_sum(hi, lo, p.lhs_shift, p.rhs, gamma) : 0;
    *flag_out = ((g >> 30) & 1) != 0;
  }
}

// The integer CRT of one output from digits `plane` bytes apart (any N; the instances are those of
// the CRT kernel).
__device__ __noinline__ double small_crt_exact(const CrtTables* t, const uint8_t* w, int64_t plane, int e) {
  switch (t->N) {
#define IMD_SM_CASE(n) case n: return crt_exact<n>(t, w, plane, e);
    IMD_SM_CASE(2) IMD_SM_CASE(3) IMD_SM_CASE(4) IMD_SM_CASE(5) IMD_SM_CASE(6) IMD_SM_CASE(7)
    IMD_SM_CASE(8) IMD_SM_CASE(9) IMD_SM_CASE(10) IMD_SM_CASE(11) IMD_SM_CASE(12) IMD_SM_CASE(13)
    IMD_SM_CASE(14) IMD_SM_CASE(15) IMD_SM_CASE(16) IMD_SM_CASE(17) IMD_SM_CASE(18) IMD_SM_CASE(19)
    IMD_SM_CASE(20)
#undef IMD_SM_CASE
  }
  return 0.0;
}

__global__ void __launch_bounds__(kSmThreads) k_small(const __grid_constant__ SmallParams p) {
  extern __shared__ __align__(16) unsigned char s_dyn[];
  __shared__ int s_sigma[kSmRows];
  __shared__ unsigned char s_flag[kSmRows];
  __shared__ uint32_t s_pm[kMaxModuli][5];  // p, floor(2^32 / p), ceil(2^32 / p), bias, q
  uint64_t* s_raw = reinterpret_cast<uint64_t*>(s_dyn);                        // [row][kh] bit patterns
  const int pitch = p.kh + kSmPad;
  int8_t* s_res = reinterpret_cast<int8_t*>(s_dyn) + static_cast<size_t>(kSmRows) * p.kh * 8;  // [l][row][pitch]
  uint8_t* s_w = reinterpret_cast<uint8_t*>(s_res) + static_cast<size_t>(p.group) * kSmRows * pitch;  // [l][TM][TN]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t tiles_n = (p.n + kSmTN - 1) / kSmTN, tiles_m = (p.m + kSmTM - 1) / kSmTM;
  int64_t tile = blockIdx.x;
  const int64_t tn = tile % tiles_n;
  tile /= tiles_n;
  const int64_t tm = tile % tiles_m, lam = tile / tiles_m;
  const int64_t i0 = tm * kSmTM, j0 = tn * kSmTN;

  if (tid < p.N) {
    const uint32_t pm = p.t.p[tid];
    s_pm[tid][0] = pm;
    s_pm[tid][1] = static_cast<uint32_t>((1ull << 32) / pm);
    s_pm[tid][2] = static_cast<uint32_t>(((1ull << 32) + pm - 1) / pm);
    s_pm[tid][3] = static_cast<uint32_t>(((1ull << 31) + pm - 1) / pm * pm);
    s_pm[tid][4] = p.crt.q[tid];
  }
  // ---- the tile's rows of A and columns of B: values, shifts, flags ----
  // row r < TM: row i0 + r of A; row TM + c: column j0 + c of B; rows outside the tensor are zero.
  // All loads of the tile are issued together (one row offset per row first), then eight lanes
  // decide the shift of a row.
  __shared__ int64_t s_off[kSmRows];
  if (tid < kSmRows) {
    const bool is_a = tid < kSmTM;
    const int64_t idx = is_a ? i0 + tid : j0 + (tid - kSmTM);
    int64_t off = kSmDead;  // offsets may be negative (negative strides): a value no row can have
    if (idx < (is_a ? p.m : p.n)) off = is_a ? p.v.a_bat[lam] + p.v.a_row[idx] : p.v.b_bat[lam] + p.v.b_col[idx];
    s_off[tid] = off;
  }
  __syncthreads();
  for (int e = tid; e < kSmRows * p.kh; e += kSmThreads) {
    const int r = e / p.kh, h = e - r * p.kh;
    const int64_t off = s_off[r];
    uint64_t bits = 0;
    if (off != kSmDead && h < p.k)
      bits = static_cast<uint64_t>(__double_as_longlong(
          r < kSmTM ? p.A[off + p.v.a_k[h]] : p.B[off + p.v.b_k[h]]));
    s_raw[e] = bits;
  }
  __syncthreads();
  {
    const int l8 = lane & 7;
    for (int r = 4 * warp + (lane >> 3); r < kSmRows; r += 4 * (kSmThreads / 32)) {
      int sg = 0;
      bool fl = false;
      const bool live = s_off[r] != kSmDead;
      small_row_shift(p, s_raw + static_cast<size_t>(r) * p.kh, l8, live, &sg, &fl);
      const bool is_a = r < kSmTM;
      const int64_t idx = is_a ? i0 + r : j0 + (r - kSmTM);
      if (l8 == 0) {
        s_sigma[r] = live ? sg : 0;
        s_flag[r] = live && fl ? 1 : 0;
        if (live && is_a && tn == 0) {
          p.sigma_a[lam * p.m + idx] = static_cast<int16_t>(sg);
          p.flag_a[lam * p.m + idx] = fl ? 1 : 0;
        }
        if (live && !is_a && tm == 0) {
          p.sigma_b[lam * p.n + idx] = static_cast<int16_t>(sg);
          p.flag_b[lam * p.n + idx] = fl ? 1 : 0;
        }
      }
    }
  }
  __syncthreads();

  // ---- per group of moduli: residues into shared memory, products, digits ----
  // warp w: quarter w & 3 of the tile (16 rows x 16 columns: two n-tiles of the mma) and the moduli
  // w >> 2, w >> 2 + 4, ... of the group; a thread's accumulators: rows g8 and g8 + 8, columns
  // 2 t4, 2 t4 + 1 of either n-tile
  const int g8 = lane >> 2, t4 = lane & 3;
  const int wr = 16 * (warp & 1), wc = 16 * ((warp >> 1) & 1);
  for (int l0 = 0; l0 < p.N; l0 += p.group) {
    const int mods = min(p.group, p.N - l0);
    for (int e = tid; e < kSmRows * p.kh; e += kSmThreads) {
      const int r = e / p.kh, h = e - r * p.kh;
      uint64_t bits = s_raw[e];
      if (s_flag[r] && ((bits >> 52) & 0x7FF) == 0x7FF) bits = 0;  // non-finite entries count as 0
      uint32_t d0, d1, d2 = 0;
      if (p.t.words == 2) {
        dev::signed_digits64(dev::quantize_i64(bits, s_sigma[r], p.trunc != 0), &d0, &d1);
      } else {
        uint64_t lo;
        uint32_t hi;
        bool neg;
        dev::quantize(bits, s_sigma[r], p.trunc != 0, &lo, &hi, &neg);
        dev::signed_digits96(lo, hi, neg, &d0, &d1, &d2);
      }
      for (int l = 0; l < mods; ++l) {
        const uint32_t u = p.t.words == 2 ? dev::residue_u<2>(p.t, l0 + l, d0, d1, d2)
                                          : dev::residue_u<3>(p.t, l0 + l, d0, d1, d2);
        const uint32_t pm = p.t.p[l0 + l], top = (pm + 1) / 2 - 1;
        s_res[(static_cast<size_t>(l) * kSmRows + r) * pitch + h] = static_cast<int8_t>(u > top ? u - pm : u);
      }
    }
    __syncthreads();
    for (int l = warp >> 2; l < mods; l += kSmThreads / 128) {
      const int8_t* ra = s_res + (static_cast<size_t>(l) * kSmRows + wr) * pitch;
      const int8_t* rb = s_res + (static_cast<size_t>(l) * kSmRows + kSmTM + wc) * pitch;
      int acc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
      for (int kk = 0; kk < p.kh; kk += 32) {
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(ra + g8 * pitch + kk + 4 * t4);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(ra + (g8 + 8) * pitch + kk + 4 * t4);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(ra + g8 * pitch + kk + 16 + 4 * t4);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(ra + (g8 + 8) * pitch + kk + 16 + 4 * t4);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          const int8_t* col = rb + (8 * nt + g8) * pitch + kk;
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(col + 4 * t4);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(col + 16 + 4 * t4);
          int c[4];
          mma_s8(c, a0, a1, a2, a3, b0, b1, acc[nt]);
#pragma unroll
          for (int x = 0; x < 4; ++x) acc[nt][x] = c[x];
        }
      }
      const int lg = l0 + l;
      const uint32_t pm = s_pm[lg][0], magic = s_pm[lg][1], magic_up = s_pm[lg][2], bias = s_pm[lg][3],
                     q = s_pm[lg][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const uint32_t y = mod_epilogue(static_cast<uint32_t>(acc[nt][x]), pm, magic, magic_up, bias, q);
          const int row = wr + g8 + 8 * (x >> 1), colx = wc + 8 * nt + 2 * t4 + (x & 1);
          s_w[(static_cast<size_t>(lg) * kSmTM + row) * kSmTN + colx] = static_cast<uint8_t>(y);
        }
    }
    __syncthreads();  // the next group overwrites the residues; the digits are complete after the last
  }

  // ---- CRT, alpha / beta, output: adjacent outputs of a row per thread ----
  constexpr int kPer = kSmTM * kSmTN / kSmThreads;
  const int64_t plane = static_cast<int64_t>(kSmTM) * kSmTN;
  const int row = tid * kPer / kSmTN;
  const int64_t i = i0 + row;
#pragma unroll
  for (int x = 0; x < kPer; ++x) {
    const int colx = tid * kPer % kSmTN + x;
    const int64_t j = j0 + colx;
    if (i >= p.m || j >= p.n) continue;
    const uint8_t* digits = s_w + static_cast<size_t>(row) * kSmTN + colx;
    const int e = -(s_sigma[row] + s_sigma[kSmTM + colx]);
    double D;
    if (s_flag[row] || s_flag[kSmTM + colx]) {
      D = native_dot(p.A + p.v.a_bat[lam] + p.v.a_row[i], p.B + p.v.b_bat[lam] + p.v.b_col[j], p.v.a_k,
                     p.v.b_k, p.k);
    } else {
      double sh = p.crt.fast.k0h, sl = p.crt.fast.k0l;
      for (int l = 0; l < p.N; ++l) {
        const uint32_t y = digits[l * plane];
        const double d = __hiloint2double(static_cast<int>(0x40700000u | (y << 12)), 0);  // 256 + y
        sh = __fma_rn(d, p.crt.fast.rh[l], sh);
        sl = __fma_rn(d, p.crt.fast.rl[l], sl);
      }
      if (p.exact_crt || !crt_fast_round(p.crt.fast, sh, sl, e, &D))
        D = small_crt_exact(&p.crt, digits, plane, e);
    }
    double* c = p.C + p.v.c_bat[lam] + p.v.c_row[i] + p.v.c_col[j];
    *c = finish(D, p.alpha, p.beta, c);
  }
}

}  // namespace
}  // namespace imd
