// The quantise kernel: per row of an operand the non-finite flag, the exact shift sigma, and the
// int8 residues of a group of moduli, with each FP64 element read from HBM once.
//
//   phase 1 (fused launches)  one pass over the row: largest magnitude, any non-finite entry, and
//            the plain FP64 sum of squares. The sum encloses the exact fixed-point sum S of the
//            shift rule tightly enough to decide the shift in all but a vanishing share of rows
//            (fast_shift); the others redo the row with exact 128-bit integers.
//   phase 2  the row is read again (it is still in L2: a CTA owns its rows for both phases),
//            scaled by 2^sigma, rounded to an integer once by the conversion unit, split into
//            signed base-256 digits, and the digit x weight dot products of every element and
//            modulus are formed by the int8 tensor path (mma.sync m16n8k32: 4 elements x 8
//            digits along K, 8 (element, modulus) columns). Each sum s (|s| <= 2^17.6) is reduced
//            to the symmetric residue by one float multiply-add (quotient) and one integer
//            multiply-add, and 16 K-contiguous residues leave as one 16-byte store.
//
// Replaces the reference's K1 / K2 / K3 and the fused KF / KL pack kernels
// (src/contract.cu:91-161, 320-384, 800-926, 1027-1189; emitter src/kernels/pack_emitter.cuh:34-116);
// the arithmetic rules are those of spec/oracle.py:361-448.
#pragma once
#include <cstdint>

#include "kernels.hpp"
#include "numerics.cuh"

namespace imd {
namespace {

// Four warps per CTA, five CTAs of 96 registers per SM, in different phases (one waits for DRAM,
// the others compute). Measured at the 8000 x 8000 shape against 4 and 6 CTAs per SM and 0 to 6
// staged units: 5 CTAs with 3 units is the fastest (more staging takes the L1 cache's room).
constexpr int kQLgWarps = 2;
constexpr int kQWarps = 1 << kQLgWarps;
constexpr int kQThreads = 32 * kQWarps;
constexpr int kQCtasPerSm = 5;
constexpr int kQMaxSlots = (kMaxModuli + 1) / 2;  // a slot = two moduli (one mma column group)
constexpr int kQChunk = 256;                      // K positions a warp handles per step
constexpr int kMaxDests = 8;  // buffers one pack launch can write (the consumers of a slab)
constexpr int kQStageBytes = kQThreads * 64;  // one unit (8 entries) of every thread
constexpr int kQStageMax = 3;                 // units per thread: 24 KB per CTA

struct QuantParams {
  const double* X;
  const int64_t *row, *kv, *bat;
  int64_t rows, rows_pad, batches, k, k_hat;
  // Output rows: a batch's planes have plane_rows rows, the rows of this launch start at row0
  // (plane_rows = rows_pad, row0 = 0 inside a contraction); sigma has sigma_rows rows per batch
  // (rows inside a contraction, plane_rows in a packed buffer) and the same row0.
  int64_t plane_rows, row0, sigma_rows;
  int64_t k_span;      // K positions per CTA (a multiple of 256; the whole row when fused)
  int32_t contig;      // how 8 adjacent K positions are found in memory (see load8)
  int32_t lg_wpr;      // log2 of the warps that share a row (kQWarps >> lg_wpr rows per CTA)
  int32_t stage_units; // fused: units of 8 entries per thread kept in shared memory for phase 2
  int32_t trunc;
  int32_t mod0, mods;  // first modulus and number of moduli of the group
  int32_t force_exact; // verification: never take the FP64 shortcut of the shift
  int32_t lhs_shift;
  Wide<8> rhs;
  ShiftFast fast;
  const int16_t* sigma_in;  // launches without phase 1: the shifts and flags computed earlier
  const uint8_t* flag_in;
  int32_t n_out;
  int16_t* sigma[kMaxDests];
  uint8_t* flag[kMaxDests];
  int8_t* R[kMaxDests];
  ResidueTables t;
};

// Eight consecutive K positions of a row starting at Kt (a multiple of 8) as bit patterns; zeros
// beyond k. contig = 2: K is one stride-1 run (offset = position); contig = 1: the fastest K mode
// has stride 1 and at least 8 entries, so eight positions are adjacent in memory exactly when
// the offsets of the first and the last differ by 7; contig = 0: gather through the K vector.
__device__ __forceinline__ void load8(const QuantParams& p, const double* base, int64_t Kt,
                                      uint64_t (&raw)[8]) {
  if (p.contig && Kt + 8 <= p.k) {
    int64_t o0 = Kt;
    bool adjacent = true;
    if (p.contig == 1) {
      o0 = p.kv[Kt];
      adjacent = p.kv[Kt + 7] - o0 == 7;
    }
    if (adjacent) {
      const double* src = base + o0;
      if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        const ulonglong2* v = reinterpret_cast<const ulonglong2*>(src);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const ulonglong2 t = v[e];
          raw[2 * e] = t.x;
          raw[2 * e + 1] = t.y;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) raw[e] = static_cast<uint64_t>(__double_as_longlong(src[e]));
      }
      return;
    }
  }
  if (Kt >= p.k) {
#pragma unroll
    for (int e = 0; e < 8; ++e) raw[e] = 0;
    return;
  }
  int64_t idx[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) idx[e] = Kt + e < p.k ? p.kv[Kt + e] : 0;
#pragma unroll
  for (int e = 0; e < 8; ++e)
    raw[e] = Kt + e < p.k ? static_cast<uint64_t>(__double_as_longlong(base[idx[e]])) : 0ull;
}

// d = a b (int8 x int8, m16n8k32) with a zero accumulator.
__device__ __forceinline__ void mma_s8_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%10, %10, %10, %10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

__device__ __forceinline__ void mma_s8(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                       uint32_t a3, uint32_t b0, uint32_t b1, const int (&c)[4]) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%10, %11, %12, %13};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]),
        "r"(c[3]));
}

// Low bytes of four words -> one word (a's byte first).
__device__ __forceinline__ uint32_t pack4(uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  const uint32_t ab = __byte_perm(a, b, 0x0040), cd = __byte_perm(c, d, 0x0040);
  return __byte_perm(ab, cd, 0x5410);
}

template <int WORDS, bool FUSED, bool TRUNC>
__global__ void __launch_bounds__(kQThreads, kQCtasPerSm) k_quantize(const __grid_constant__ QuantParams p) {
  __shared__ uint32_t s_b[WORDS][kQMaxSlots][32];  // B fragments (digit weights) by slot and lane
  __shared__ float s_inv[kQMaxSlots][2];
  __shared__ int s_negp[kQMaxSlots][2];
  __shared__ uint32_t s_max[kQWarps];
  __shared__ double s_acc[kQWarps];
  __shared__ uint64_t s_hi[kQWarps], s_lo[kQWarps];
  __shared__ int s_sigma[kQWarps], s_flag[kQWarps];
  extern __shared__ uint4 s_stage[];  // fused launches: [unit][quarter][thread] of raw entries

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int W = 1 << p.lg_wpr;  // warps per row
  const int rr = warp >> p.lg_wpr, sub = warp & (W - 1);
  const int slots = (p.mods + 1) >> 1;

  // digit weights as the B operand: column c of slot s is (element c % 4, modulus 2 s + c / 4);
  // thread (g, t) holds rows 4 t .. 4 t + 3 (the low digits of element t) and 16 + 4 t .. of
  // column g: nonzero only for its own element.
  for (int idx = tid; idx < slots * 32; idx += kQThreads) {
    const int s = idx >> 5, ln = idx & 31, g = ln >> 2, t = ln & 3;
    const int rel = 2 * s + (g >> 2);
    const bool on = rel < p.mods && t == (g & 3);
#pragma unroll
    for (int w = 0; w < WORDS; ++w) s_b[w][s][ln] = on ? p.t.weight[w][p.mod0 + rel] : 0u;
  }
  if (tid < 2 * slots) {
    const int s = tid >> 1, rel = 2 * s + (tid & 1);
    const uint32_t pm = rel < p.mods ? p.t.p[p.mod0 + rel] : 1u;
    s_inv[s][tid & 1] = 1.0f / static_cast<float>(pm);
    s_negp[s][tid & 1] = -static_cast<int>(pm);
  }

  const int64_t total_rows = p.rows_pad * p.batches;
  const int64_t rho = static_cast<int64_t>(blockIdx.x) * (kQWarps >> p.lg_wpr) + rr;
  int64_t lam = 0, i = rho;
  if (p.batches != 1) {
    lam = rho / p.rows_pad;
    i = rho - lam * p.rows_pad;
  }
  const bool inside = rho < total_rows;
  const bool live = inside && i < p.rows;  // rows beyond `rows` are the zero padding of the planes
  const double* base = p.X;
  if (live) base += p.bat[lam] + p.row[i];
  const int64_t srow = lam * p.sigma_rows + p.row0 + i;

  int sigma = 0;
  bool flagged = false;
  if (FUSED) {
    // ---- phase 1: one pass over the row ----
    uint32_t mx = 0;
    double acc = 0.0;
    if (live) {
      // unit j of this thread = K positions 8 (32 (sub + W j) + lane) .. + 7: the same units it
      // quantises in phase 2, so the first stage_units of them are parked in shared memory
      // (thread-private slots) and phase 2 does not go back to L2 for them. Four units in flight.
      const int64_t stride = 8 * 32 * W;
      const int64_t Kfirst = 8 * static_cast<int64_t>(sub * 32 + lane);
      const int units = static_cast<int>((p.k_hat + stride - 1) / stride);  // zeros beyond k
      int64_t Kt = Kfirst;
      for (int j = 0; j < units; j += 4, Kt += 4 * stride) {
        uint64_t ru[4][8];
#pragma unroll
        for (int u = 0; u < 4; ++u) load8(p, base, Kt + u * stride, ru[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            mx = max(mx, static_cast<uint32_t>(ru[u][e] >> 32) & 0x7FFFFFFFu);
            const double x = __longlong_as_double(static_cast<long long>(ru[u][e]));
            acc = __fma_rn(x, x, acc);
          }
          if (j + u < p.stage_units) {
#pragma unroll
            for (int q = 0; q < 4; ++q)
              s_stage[((j + u) * 4 + q) * kQThreads + tid] = make_uint4(
                  static_cast<uint32_t>(ru[u][2 * q]), static_cast<uint32_t>(ru[u][2 * q] >> 32),
                  static_cast<uint32_t>(ru[u][2 * q + 1]), static_cast<uint32_t>(ru[u][2 * q + 1] >> 32));
          }
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = max(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
      acc += __shfl_xor_sync(0xFFFFFFFFu, acc, o);
    }
    if (lane == 0) {
      s_max[warp] = mx;
      s_acc[warp] = acc;
    }
    __syncthreads();
    int exact = 0;
    if (sub == 0 && lane == 0) {
      for (int w = 1; w < W; ++w) {
        mx = max(mx, s_max[warp + w]);
        acc += s_acc[warp + w];
      }
      int sg = 0;
      if (live && (p.force_exact || !dev::fast_shift(mx, acc, p.fast, p.lhs_shift, &sg))) exact = 1;
      s_sigma[rr] = sg;
      s_flag[rr] = 0;  // the shortcut is only taken for rows without non-finite entries
    }
    if (__syncthreads_or(exact)) {
      // ---- exact integers, for every row of the CTA ----
      int g = 0;  // bit 30: a non-finite entry; low bits: gamma + 2048 (0: no finite nonzero entry)
      if (live)
        for (int64_t Kt = 8 * static_cast<int64_t>(sub * 32 + lane); Kt < p.k; Kt += 8 * 32 * W) {
          uint64_t raw[8];
          load8(p, base, Kt, raw);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            uint64_t M;
            int E;
            const int kind = dev::decompose(raw[e], &M, &E);
            if (kind < 0) g |= 1 << 30;
            else if (kind > 0) g = (g & (1 << 30)) | max(g & 0xFFFF, E + 52 + 2048);
          }
        }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const int other = __shfl_xor_sync(0xFFFFFFFFu, g, o);
        g = ((g | other) & (1 << 30)) | max(g & 0xFFFF, other & 0xFFFF);
      }
      if (lane == 0) s_max[warp] = static_cast<uint32_t>(g);
      __syncthreads();
      for (int w = 0; w < W; ++w) {
        const int other = static_cast<int>(s_max[(rr << p.lg_wpr) + w]);
        g = ((g | other) & (1 << 30)) | max(g & 0xFFFF, other & 0xFFFF);
      }
      const bool any = (g & 0xFFFF) != 0;
      const int gamma = (g & 0xFFFF) - 2048;
      uint64_t hi = 0, lo = 0;
      if (live && any)
        for (int64_t Kt = 8 * static_cast<int64_t>(sub * 32 + lane); Kt < p.k; Kt += 8 * 32 * W) {
          uint64_t raw[8];
          load8(p, base, Kt, raw);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            uint64_t M;
            int E;
            if (dev::decompose(raw[e], &M, &E) == 1) {
              uint64_t th, tl;
              dev::square_term(M, E, gamma, &th, &tl);
              lo += tl;
              hi += th + (lo < tl ? 1 : 0);
            }
          }
        }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const uint64_t oh = __shfl_xor_sync(0xFFFFFFFFu, hi, o), ol = __shfl_xor_sync(0xFFFFFFFFu, lo, o);
        lo += ol;
        hi += oh + (lo < ol ? 1 : 0);
      }
      if (lane == 0) {
        s_hi[warp] = hi;
        s_lo[warp] = lo;
      }
      __syncthreads();
      if (sub == 0 && lane == 0) {
        for (int w = 1; w < W; ++w) {
          const uint64_t ol = s_lo[warp + w];
          lo += ol;
          hi += s_hi[warp + w] + (lo < ol ? 1 : 0);
        }
        s_sigma[rr] = live && any ? dev::shift_from_sum(hi, lo, p.lhs_shift, p.rhs, gamma) : 0;
        s_flag[rr] = (g >> 30) & 1;
      }
      __syncthreads();
    }
    sigma = s_sigma[rr];
    flagged = s_flag[rr] != 0;
    if (live && sub == 0 && lane == 0)
      for (int dst = 0; dst < p.n_out; ++dst) {
        p.sigma[dst][srow] = static_cast<int16_t>(sigma);
        p.flag[dst][srow] = flagged ? 1 : 0;
      }
  } else {
    __syncthreads();  // the tables above
    if (live) {
      sigma = p.sigma_in[srow];
      flagged = p.flag_in[srow] != 0;
    }
  }
  if (!inside) return;

  // ---- phase 2: quantise and emit the residues ----
  const int g8 = lane >> 2, t4 = lane & 3;
  const int half = t4 >> 1;  // which modulus of a slot this thread's result columns belong to
  const int s1 = sigma >> 1, s2 = sigma - s1;
  const double f1 = __longlong_as_double(static_cast<long long>(1023 + s1) << 52);
  const double f2 = __longlong_as_double(static_cast<long long>(1023 + s2) << 52);
  const int64_t plane = p.batches * p.plane_rows * p.k_hat;
  const int64_t kbeg = FUSED ? 0 : static_cast<int64_t>(blockIdx.y) * p.k_span;
  int64_t kend = kbeg + p.k_span;
  if (FUSED || kend > p.k_hat) kend = p.k_hat;
  // this thread's 16 output bytes of a chunk start at K0 + kofs in the plane of modulus
  // 2 s + half of slot s; the last slot of an odd group has no second modulus
  const int kofs = 32 * g8 + 16 * (t4 & 1);
  const int64_t out0 = (lam * p.plane_rows + p.row0 + i) * p.k_hat + kofs + half * plane;
  const int last_slot = ((p.mods & 1) && half) ? slots - 1 : slots;  // slots this thread stores
  const int64_t step = static_cast<int64_t>(kQChunk) * W;
  // the accumulators start at the float magic (see reduce_sym); the four registers are opaque to
  // the compiler so that it keeps them instead of rebuilding the constant in front of every mma
  int mg[4];
#pragma unroll
  for (int x = 0; x < 4; ++x) asm volatile("mov.u32 %0, 0x4B400000;" : "=r"(mg[x]));

  uint64_t raw[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) raw[e] = 0;
  int64_t K0 = kbeg + static_cast<int64_t>(kQChunk) * sub;
  const int staged = FUSED ? p.stage_units : 0;
  // chunk c of this warp is unit c of phase 1; unstaged chunks are loaded one step ahead
  if (live && K0 < kend && staged == 0) load8(p, base, K0 + 8 * lane, raw);
  for (int c = 0; K0 < kend; K0 += step, ++c) {
    if (FUSED && c < staged && live) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 v = s_stage[(c * 4 + q) * kQThreads + tid];
        raw[2 * q] = v.x | (static_cast<uint64_t>(v.y) << 32);
        raw[2 * q + 1] = v.z | (static_cast<uint64_t>(v.w) << 32);
      }
    }
    // element e of this thread: K position K0 + 8 lane + e = tile e / 2, row g8 + 8 (e & 1),
    // element slot t4 of the mma operand
    uint32_t dl[8], dh[8], dt[8];
    if (flagged) {  // rare: non-finite entries count as 0
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (((raw[e] >> 52) & 0x7FF) == 0x7FF) raw[e] = 0;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (WORDS == 2) {
        const double x = __longlong_as_double(static_cast<long long>(raw[e]));
        const double v = __dmul_rn(__dmul_rn(x, f1), f2);  // exact: two powers of two of one sign
        const long long q = TRUNC ? __double2ll_rz(v) : __double2ll_rn(v);
        dev::signed_digits64(q, &dl[e], &dh[e]);
        dt[e] = 0;
      } else {
        uint64_t lo;
        uint32_t hi;
        bool neg;
        dev::quantize(raw[e], sigma, TRUNC, &lo, &hi, &neg);
        dev::signed_digits96(lo, hi, neg, &dl[e], &dh[e], &dt[e]);
      }
    }
    // the next chunk's loads travel while this one is reduced
    if (live && K0 + step < kend && c + 1 >= staged) load8(p, base, K0 + step + 8 * lane, raw);
    const bool in_k = K0 + kofs < p.k_hat;
    int64_t at = out0 + K0;
#pragma unroll 1  // measured: 1.10 ms against 1.13 (unroll 2) and 1.11 (unroll 4) at the 8000 x 8000 shape
    for (int s = 0; s < slots; ++s, at += 2 * plane) {
      const uint32_t b0 = s_b[0][s][lane], b1 = s_b[1][s][lane];
      const float inv = s_inv[s][half];
      const int negp = s_negp[s][half];
      uint32_t r[4][4];
#pragma unroll
      for (int T = 0; T < 4; ++T) {
        int c[4];
        mma_s8(c, dl[2 * T], dl[2 * T + 1], dh[2 * T], dh[2 * T + 1], b0, b1, mg);
        if (WORDS == 3) {
          int c2[4];
          mma_s8(c2, dt[2 * T], dt[2 * T + 1], 0u, 0u, s_b[WORDS - 1][s][lane], 0u, c);
#pragma unroll
          for (int x = 0; x < 4; ++x) c[x] = c2[x];
        }
#pragma unroll
        for (int x = 0; x < 4; ++x) r[T][x] = dev::reduce_sym(c[x], inv, negp);
      }
      // c0 = (row g8, column 2 t4), c1 = (g8, 2 t4 + 1), c2 / c3 = row g8 + 8: byte offset of
      // (column jj, tile T, row half h) in the 16 bytes = 8 jj + 2 T + h
      const uint4 out = make_uint4(pack4(r[0][0], r[0][2], r[1][0], r[1][2]),
                                   pack4(r[2][0], r[2][2], r[3][0], r[3][2]),
                                   pack4(r[0][1], r[0][3], r[1][1], r[1][3]),
                                   pack4(r[2][1], r[2][3], r[3][1], r[3][3]));
      if (in_k && s < last_slot) {
        *reinterpret_cast<uint4*>(p.R[0] + at) = out;
        for (int dst = 1; dst < p.n_out; ++dst) *reinterpret_cast<uint4*>(p.R[dst] + at) = out;
      }
    }
  }
}

}  // namespace
}  // namespace imd
