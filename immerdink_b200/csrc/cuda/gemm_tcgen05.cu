// Batched int8 GEMM with a modular epilogue on Blackwell tensor cores (sm_100a only).
//
//   W[l][lambda][i][j] = (q_l * sum_h RA[z][i][h] * RB[z][j][h]  (+ W))  mod p_l      z = slot * b + lambda
//   (q_l = (P / p_l)^-1 mod p_l: the planes hold the CRT digits y_l directly)
//
// One persistent CTA per SM walks (plane, 128 x 256 tile) work items. Per CTA:
//   warp 0   TMA producer: cp.async.bulk.tensor loads of 128-byte-swizzled K-major tiles of A
//            (128 rows x 128 bytes) and B (256 rows x 128 bytes) into a 4-stage shared-memory ring;
//            rows and K positions outside the planes are filled with zeros by the TMA unit
//   warp 1   MMA issuer: one elected lane issues tcgen05.mma.cta_group::1.kind::i8 (M 128, N 256,
//            K 32 per instruction) with the int32 accumulator in tensor memory, double-buffered
//            (2 x 256 columns) so that the epilogue of a tile overlaps the main loop of the next
//   warps 2-5  epilogue: tcgen05.ld of the accumulator, exact reduction mod p, 32-byte stores of
//            u8 residues
// Synchronisation is by mbarriers; every wait is bounded: a wait that gives up sets a sticky
// error word and the CTA drains and exits instead of hanging.
//
// int32 accumulation is exact in any order because a K chunk is at most 130944 long and
// |residue| <= 128 (130944 * 128^2 < 2^31). This kernel replaces the reference's CUTLASS-based
// mma.sync kernel K4 (src/kernels/k4_gemm.cuh:268-319) and its epilogue (:192-264).
#include <cstdint>

#include <cuda.h>

#include "common/modred.hpp"
#include "kernels.hpp"

namespace imd {
namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kTileK = 128;   // bytes of K per pipeline stage = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kMmaK = 32;     // K of one tcgen05.mma kind::i8
constexpr int kBytesA = kTileM * kTileK;
constexpr int kBytesB = kTileN * kTileK;
constexpr int kStageBytes = kBytesA + kBytesB;
constexpr int kGemmThreads = 192;
constexpr int kAccCols = 256;  // TMEM columns of one accumulator
constexpr int kTmemCols = 512;
constexpr uint32_t kSpinLimit = 1u << 26;  // try_wait polls before a wait gives up
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /* alignment slack */ + 256 /* barriers */;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false (and raises *abort) when the phase did not complete in time or
// another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 1023u) == 1023u && *abort) return false;
  }
  *abort = 1;
  return false;
}

// L2 eviction policy of an operand load.
__device__ __forceinline__ uint64_t l2_policy(int kind) {  // 0 normal, 1 evict last, 2 evict first
  uint64_t pol;
  if (kind == 1) asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  else if (kind == 2) asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  else asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2),
        "l"(policy)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes with the 128-byte
// swizzle: groups of 8 rows are 1024 bytes apart (stride byte offset); the leading byte offset is
// unused for this layout; bits 46-47 carry the descriptor version of this architecture (1); bits
// 61-63 the swizzle mode (2 = 128 bytes).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;               // leading byte offset (ignored), 16 bytes
  d |= static_cast<uint64_t>(1024 >> 4) << 32;       // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;               // version
  d |= static_cast<uint64_t>(2) << 61;               // SWIZZLE_128B
  return d;
}

// Instruction descriptor of kind::i8: D = s32, A = B = s8, both K-major, N / 8 at bit 17, M / 16
// at bit 24.
constexpr uint32_t kInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) |
                                (static_cast<uint32_t>(kTileN >> 3) << 17) |
                                (static_cast<uint32_t>(kTileM >> 4) << 24);

struct GemmParams {
  GemmShape s;
  int32_t tiles_m, tiles_n;
  int32_t k_blocks;
  int32_t band_rows;  // tile rows walked together (see tile_of)
  int32_t l2_hints;   // eviction policy of A's loads (bits 0-1) and B's (bits 2-3): 0 normal, 1 last, 2 first
  uint8_t* W;
  unsigned int* error_word;
};

// Work item -> (plane, tile row, tile column). Tile rows are walked in bands of `band_rows`, tile
// row fastest: the band's rows of A stay in L2 while the rows of B stream through once per band,
// so DRAM reads A once and B (tile rows / band_rows) times per plane. The host sizes the band to
// about a quarter of L2.
struct TileCoord {
  int plane, tm, tn;
};
__device__ __forceinline__ TileCoord tile_of(const GemmParams& p, int64_t w) {
  const int per_plane = p.tiles_m * p.tiles_n;
  TileCoord c;
  c.plane = static_cast<int>(w / per_plane);
  const int t = static_cast<int>(w % per_plane);
  const int band = p.band_rows * p.tiles_n;
  const int first = (t / band) * p.band_rows;
  const int rows = min(p.tiles_m - first, p.band_rows);
  const int r = t % band;
  c.tm = first + r % rows;
  c.tn = r / rows;
  return c;
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 16 accumulators -> 16 residues in [0, p), packed into a uint4 (column order = byte order).
__device__ __forceinline__ uint4 reduce16(const uint32_t* acc, uint4 prev, bool add, uint32_t p,
                                          uint32_t magic, uint32_t magic_up, uint32_t bias,
                                          uint32_t q) {
  uint32_t out[4];
  const uint32_t pv[4] = {prev.x, prev.y, prev.z, prev.w};
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    uint32_t word = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      uint32_t y = mod_epilogue(acc[4 * wd + b], p, magic, magic_up, bias, q);  // (q acc) mod p
      if (add) {
        y += (pv[wd] >> (8 * b)) & 0xFFu;              // both < p
        y = min(y, y - p);
      }
      word |= y << (8 * b);
    }
    out[wd] = word;
  }
  return make_uint4(out[0], out[1], out[2], out[3]);
}

__global__ void __launch_bounds__(kGemmThreads, 1)
k_gemm_i8(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
          const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;          // 1024-byte aligned tile ring
  uint8_t* ctrl = smem_raw + (tiles - raw) + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);      // full[4] empty[4] tfull[2] tempty[2] drain
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 128);
  volatile int* abort = reinterpret_cast<volatile int*>(ctrl + 136);
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull = [&](int a) { return bar0 + 8u * (2 * kStages + a); };
  auto tempty = [&](int a) { return bar0 + 8u * (2 * kStages + 2 + a); };
  const uint32_t drain = bar0 + 8u * (2 * kStages + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull(a), 1);
      mbar_init(tempty(a), 4);
    }
    mbar_init(drain, 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int64_t total = static_cast<int64_t>(p.s.planes) * p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued = 0;  // bit s: a load into stage s is (or was) in flight
      bool okay = true;
      const uint64_t pol_a = l2_policy(p.l2_hints & 3), pol_b = l2_policy((p.l2_hints >> 2) & 3);
      for (int64_t w = blockIdx.x; w < total && okay; w += gridDim.x) {
        const TileCoord c = tile_of(p, w);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty(stage), phase ^ 1u, abort)) {
            okay = false;
            break;
          }
          mbar_expect_tx(full(stage), kStageBytes);
          const uint32_t dst = tiles + stage * kStageBytes;
          const int kx = p.s.k0 + kb * kTileK;
          tma_load_3d(dst, &map_a, full(stage), kx, c.tm * kTileM, c.plane, pol_a);
          tma_load_3d(dst + kBytesA, &map_b, full(stage), kx, c.tn * kTileN, c.plane, pol_b);
          issued |= 1u << stage;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!okay) {
        // give the copies still in flight a bounded time to land before the CTA exits
        for (int s = 0; s < kStages; ++s)
          if (issued & (1u << s))
            for (uint32_t it = 0; it < (1u << 20); ++it)
              if (mbar_try_wait(full(s), 0) || mbar_try_wait(full(s), 1)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool okay = true;
      for (int64_t w = blockIdx.x; w < total && okay; w += gridDim.x) {
        if (!mbar_wait(tempty(acc), acc_phase ^ 1u, abort)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full(stage), phase, abort)) {
            okay = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = tiles + stage * kStageBytes, b_addr = a_addr + kBytesA;
#pragma unroll
          for (int k4 = 0; k4 < kTileK / kMmaK; ++k4)
            tc_mma_i8(d_tmem, smem_desc(a_addr + k4 * kMmaK), smem_desc(b_addr + k4 * kMmaK),
                      kInstrDesc, (kb | k4) != 0 ? 1u : 0u);
          tc_commit(empty(stage));
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!okay) break;
        tc_commit(tfull(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      // every MMA issued above has retired once this commit arrives
      tc_commit(drain);
      for (uint32_t it = 0; it < kSpinLimit; ++it)
        if (mbar_try_wait(drain, 0)) break;
    }
  } else {
    // ---------------- epilogue ----------------
    const int quarter = warp & 3;  // TMEM lanes 32 * quarter .. + 31 belong to this warp
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int64_t w = blockIdx.x; w < total; w += gridDim.x) {
      const TileCoord c = tile_of(p, w);
      if (!mbar_wait(tfull(acc), acc_phase, abort)) break;
      tc_fence_after();
      const int slot = c.plane / p.s.batches, lam = c.plane % p.s.batches;
      const uint32_t pm = p.s.p[slot], magic = p.s.magic[slot], bias = p.s.bias[slot];
      const uint32_t magic_up = p.s.magic_up[slot], qm = p.s.q[slot];
      const int row = c.tm * kTileM + quarter * 32 + lane;
      const int64_t wplane = static_cast<int64_t>(p.s.mod0 + slot) * p.s.batches + lam;
      uint8_t* wrow = p.W + (wplane * p.s.m + row) * static_cast<int64_t>(p.s.n_hat);
      const uint32_t taddr = tmem_base + acc * kAccCols + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int cc = 0; cc < kTileN / 32; ++cc) {
        const int col = c.tn * kTileN + cc * 32;
        if (col >= p.s.n_hat) break;  // warp-uniform
        uint32_t v[32];
        tmem_load_32(taddr + cc * 32, v);
        if (row < p.s.m) {
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            if (col + 16 * hf < p.s.n_hat) {
              uint4* dst = reinterpret_cast<uint4*>(wrow + col + 16 * hf);
              uint4 prev = make_uint4(0, 0, 0, 0);
              if (p.s.add) prev = *dst;
              *dst = reduce16(v + 16 * hf, prev, p.s.add != 0, pm, magic, magic_up, bias, qm);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort) atomicOr(p.error_word, 1u);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

// ---- CTA-pair variant ---------------------------------------------------------------------------
// Two CTAs of a cluster (two SMs) share one 256 x 256 tile: each loads its own 128 rows of A and its
// own 128 of the 256 rows of B, and one tcgen05.mma.cta_group::2 of the leader CTA (rank 0) drives
// both tensor cores, each accumulating its 128 rows in its own tensor memory. Per SM this halves
// the B bytes that are written to and read from shared memory, which is what bounds the 1-CTA
// kernel (TMA writes plus operand reads exceed the shared-memory port). Signals:
//   full[s]    in the leader: its producer arms it with the bytes of both CTAs; every TMA load of
//              either CTA completes on it (cp.async.bulk.tensor with .cta_group::2, no multicast)
//   empty[s]   in each CTA: tcgen05.commit of the leader arrives on both (commit multicast)
//   tfull[a]   in each CTA: same commit multicast after the last K block of a tile
//   tempty[a]  in the leader: the eight epilogue warps of both CTAs arrive (the peer's remotely)
constexpr int kPairStages = 6;
constexpr int kPairBytesB = 128 * kTileK;
constexpr int kPairStageBytes = kBytesA + kPairBytesB;
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 1024 + 256;
constexpr uint32_t kPairInstrDesc = (2u << 4) | (1u << 7) | (1u << 10) |
                                    (static_cast<uint32_t>(256 >> 3) << 17) |
                                    (static_cast<uint32_t>(256 >> 4) << 24);

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map,
                                                 uint32_t leader_bar, int c0, int c1, int c2,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(leader_bar), "r"(c0), "r"(c1), "r"(c2),
        "l"(policy)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in the CTAs of `mask` (bit r = CTA rank r)
// once every tcgen05.mma issued so far by this thread has retired.
__device__ __forceinline__ void tc_commit_pair(uint32_t bar, uint16_t mask = 3) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;" ::"r"(bar), "h"(mask)
      : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Work item -> (plane, 256-row tile, 256-column tile), bands as in tile_of.
__device__ __forceinline__ TileCoord pair_tile_of(const GemmParams& p, int64_t w) {
  const int per_plane = p.tiles_m * p.tiles_n;
  TileCoord c;
  c.plane = static_cast<int>(w / per_plane);
  const int t = static_cast<int>(w % per_plane);
  const int band = p.band_rows * p.tiles_n;
  const int first = (t / band) * p.band_rows;
  const int rows = min(p.tiles_m - first, p.band_rows);
  const int r = t % band;
  c.tm = first + r % rows;
  c.tn = r / rows;
  return c;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
k_gemm_i8_pair(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  uint8_t* ctrl = smem_raw + (tiles - raw) + kPairStages * kPairStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl);  // full[6] empty[6] tfull[2] tempty[2] drain
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(ctrl + 160);
  volatile int* abort = reinterpret_cast<volatile int*>(ctrl + 168);
  const uint32_t bar0 = smem_u32(bars);
  auto full = [&](int s) { return bar0 + 8u * s; };
  auto empty = [&](int s) { return bar0 + 8u * (kPairStages + s); };
  auto tfull = [&](int a) { return bar0 + 8u * (2 * kPairStages + a); };
  auto tempty = [&](int a) { return bar0 + 8u * (2 * kPairStages + 2 + a); };
  const uint32_t drain = bar0 + 8u * (2 * kPairStages + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const bool leader = rank == 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(full(s), 1);
      mbar_init(empty(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull(a), 1);
      mbar_init(tempty(a), 8);
    }
    mbar_init(drain, 1);
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // every tcgen05 instruction of this kernel names cta_group::2; the allocation is made by one
  // warp of each CTA of the pair, which gives both the same columns
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int64_t total = static_cast<int64_t>(p.s.planes) * p.tiles_m * p.tiles_n;
  const int64_t first = blockIdx.x >> 1, step = gridDim.x >> 1;
  // a role that gives up also raises the other CTA's abort flag, so that both leave promptly
  const uint32_t peer_abort = map_to_cta(smem_u32(const_cast<int*>(abort)), rank ^ 1u);
  auto tell_peer = [&]() {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer_abort), "r"(1u) : "memory");
  };

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t issued = 0;  // bit s: a load into stage s is (or was) in flight
      bool okay = true;
      const uint64_t pol_a = l2_policy(p.l2_hints & 3), pol_b = l2_policy((p.l2_hints >> 2) & 3);
      for (int64_t w = first; w < total && okay; w += step) {
        const TileCoord c = pair_tile_of(p, w);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(empty(stage), phase ^ 1u, abort)) {
            okay = false;
            tell_peer();
            break;
          }
          const uint32_t leader_full = map_to_cta(full(stage), 0);
          if (leader) mbar_expect_tx(full(stage), 2 * kPairStageBytes);
          const uint32_t dst = tiles + stage * kPairStageBytes;
          const int kx = p.s.k0 + kb * kTileK;
          tma_load_3d_pair(dst, &map_a, leader_full, kx, c.tm * 256 + static_cast<int>(rank) * 128,
                           c.plane, pol_a);
          tma_load_3d_pair(dst + kBytesA, &map_b, leader_full, kx,
                           c.tn * 256 + static_cast<int>(rank) * 128, c.plane, pol_b);
          issued |= 1u << stage;
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!okay && leader) {
        // give the copies of both CTAs still in flight a bounded time to land (they complete on
        // the leader's barriers) before the pair passes its final cluster barrier and exits
        for (int s = 0; s < kPairStages; ++s)
          if (issued & (1u << s))
            for (uint32_t it = 0; it < (1u << 20); ++it)
              if (mbar_try_wait(full(s), 0) || mbar_try_wait(full(s), 1)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA only) ----------------
    if (lane == 0 && leader) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool okay = true;
      for (int64_t w = first; w < total && okay; w += step) {
        if (!mbar_wait(tempty(acc), acc_phase ^ 1u, abort)) {
          tell_peer();
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kAccCols;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(full(stage), phase, abort)) {
            okay = false;
            tell_peer();
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = tiles + stage * kPairStageBytes, b_addr = a_addr + kBytesA;
#pragma unroll
          for (int k4 = 0; k4 < kTileK / kMmaK; ++k4)
            tc_mma_i8_pair(d_tmem, smem_desc(a_addr + k4 * kMmaK), smem_desc(b_addr + k4 * kMmaK),
                           kPairInstrDesc, (kb | k4) != 0 ? 1u : 0u);
          tc_commit_pair(empty(stage));
          if (++stage == kPairStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!okay) break;
        tc_commit_pair(tfull(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      tc_commit_pair(drain, 1);  // every MMA issued above has retired once this arrives
      for (uint32_t it = 0; it < kSpinLimit; ++it)
        if (mbar_try_wait(drain, 0)) break;
    }
  } else {
    // ---------------- epilogue (both CTAs, own 128 rows) ----------------
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int64_t w = first; w < total; w += step) {
      const TileCoord c = pair_tile_of(p, w);
      if (!mbar_wait(tfull(acc), acc_phase, abort)) {
        if (lane == 0) tell_peer();
        break;
      }
      tc_fence_after();
      const int slot = c.plane / p.s.batches, lam = c.plane % p.s.batches;
      const uint32_t pm = p.s.p[slot], magic = p.s.magic[slot], bias = p.s.bias[slot];
      const uint32_t magic_up = p.s.magic_up[slot], qm = p.s.q[slot];
      const int row = c.tm * 256 + static_cast<int>(rank) * 128 + quarter * 32 + lane;
      const int64_t wplane = static_cast<int64_t>(p.s.mod0 + slot) * p.s.batches + lam;
      uint8_t* wrow = p.W + (wplane * p.s.m + row) * static_cast<int64_t>(p.s.n_hat);
      const uint32_t taddr = tmem_base + acc * kAccCols + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
      for (int cc = 0; cc < 256 / 32; ++cc) {
        const int col = c.tn * 256 + cc * 32;
        if (col >= p.s.n_hat) break;
        uint32_t v[32];
        tmem_load_32(taddr + cc * 32, v);
        if (row < p.s.m) {
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            if (col + 16 * hf < p.s.n_hat) {
              uint4* dst = reinterpret_cast<uint4*>(wrow + col + 16 * hf);
              uint4 prev = make_uint4(0, 0, 0, 0);
              if (p.s.add) prev = *dst;
              *dst = reduce16(v + 16 * hf, prev, p.s.add != 0, pm, magic, magic_up, bias, qm);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty(acc), 0));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  tc_fence_before();
  cluster_sync_all();  // no CTA leaves while its peer may still signal it or write its tensor memory
  if (threadIdx.x == 0 && *abort) atomicOr(p.error_word, 2u);
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"(kTmemCols)
                 : "memory");
  }
}

// ---- tensor-pipe probe ---------------------------------------------------------------------------
// Issues tcgen05.mma.kind::i8 back to back on whatever the shared memory holds (no loads, results
// discarded): the time gives the ceiling of the int8 tensor pipe for the tile shapes used above,
// the denominator of the GEMM roofline. PAIR = false: M128 N256 per CTA; PAIR = true: M256 N256
// per CTA pair (every tcgen05 instruction of an instantiation names one cta_group).
template <bool PAIR>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(64, 1) k_mma_probe(int iters) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_slot;
  const uint32_t rank = cluster_rank();
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x < 32) {
    if (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(&tmem_slot)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(&tmem_slot)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tc_fence_before();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  if (threadIdx.x == 0 && (!PAIR || rank == 0)) {
    uint32_t phase = 0;
    for (int it = 0; it < iters; it += 64) {
      for (int j = 0; j < 64; ++j) {
        const uint32_t a = tiles + (j & 3) * kMmaK, b = tiles + kBytesA + (j & 3) * kMmaK;
        if (PAIR) tc_mma_i8_pair(tmem_base + (j & 1) * kAccCols, smem_desc(a), smem_desc(b), kPairInstrDesc, 1u);
        else tc_mma_i8(tmem_base + (j & 1) * kAccCols, smem_desc(a), smem_desc(b), kInstrDesc, 1u);
      }
      if (PAIR) tc_commit_pair(smem_u32(&bar), 1);
      else tc_commit(smem_u32(&bar));
      for (uint32_t spin = 0; spin < kSpinLimit; ++spin)
        if (mbar_try_wait(smem_u32(&bar), phase)) break;
      phase ^= 1u;
    }
  }
  tc_fence_before();
  cluster_sync_all();
  if (threadIdx.x < 32) {
    tc_fence_after();
    if (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(kTmemCols)
                   : "memory");
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                   "r"(kTmemCols)
                   : "memory");
  }
}

using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                 const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                 const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Residue planes [planes][rows][k_hat] as a 3-D tensor of bytes, boxes of box_rows x 128 bytes.
bool encode_planes(EncodeTiled fn, CUtensorMap* map, const int8_t* base, int64_t k_hat,
                   int64_t rows, int64_t planes, int box_rows) {
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(k_hat), static_cast<cuuint64_t>(rows),
                              static_cast<cuuint64_t>(planes)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(k_hat),
                                 static_cast<cuuint64_t>(rows) * static_cast<cuuint64_t>(k_hat)};
  const cuuint32_t box[3] = {kTileK, static_cast<cuuint32_t>(box_rows), 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<int8_t*>(base), dims, strides, box,
            elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

imd_status_t gemm_setup(GemmPlanInfo* info) {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
      q != cudaDriverEntryPointSuccess || fn == nullptr) {
    cudaGetLastError();
    return IMD_STATUS_CUDA_ERROR;
  }
  if (cudaFuncSetAttribute(k_gemm_i8, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
          cudaSuccess ||
      cudaFuncSetAttribute(k_gemm_i8_pair, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kPairSmemBytes) != cudaSuccess) {
    cudaGetLastError();
    return IMD_STATUS_CUDA_ERROR;
  }
  info->encode_tiled = fn;
  info->error_word = device_error_word();
  if (info->error_word == nullptr) {
    cudaGetLastError();
    return IMD_STATUS_CUDA_ERROR;
  }
  return IMD_STATUS_SUCCESS;
}

imd_status_t gemm_launch(const GemmPlanInfo& info, const GemmShape& s, const int8_t* RA,
                         const int8_t* RB, uint8_t* W, cudaStream_t stream) {
  if (info.encode_tiled == nullptr || info.error_word == nullptr) return IMD_STATUS_CUDA_ERROR;
  const EncodeTiled fn = reinterpret_cast<EncodeTiled>(info.encode_tiled);
  const int variant = hooks().gemm_variant;
  const bool pair = variant == 2 || (variant == 0 && s.m > kTileM);
  CUtensorMap map_a, map_b;
  if (!encode_planes(fn, &map_a, RA, s.k_hat, s.m, s.planes, kTileM) ||
      !encode_planes(fn, &map_b, RB, s.k_hat, s.b_rows, s.planes, pair ? 128 : kTileN))
    return IMD_STATUS_CUDA_ERROR;
  GemmParams p{};
  p.s = s;
  p.tiles_m = (s.m + (pair ? 256 : kTileM) - 1) / (pair ? 256 : kTileM);
  p.tiles_n = (s.n_hat + kTileN - 1) / kTileN;
  p.k_blocks = (s.klen + kTileK - 1) / kTileK;
  {
    // rows of A that stay resident: about 32 MB of the 126 MB L2 (the B rows in flight, the
    // product tiles being written and the other die's copies share the rest)
    const int64_t tile_bytes = static_cast<int64_t>(pair ? 256 : kTileM) * (s.klen > 0 ? s.klen : 1);
    int64_t rows = (static_cast<int64_t>(hooks().gemm_band_mb) << 20) / tile_bytes;
    rows = rows < 4 ? 4 : rows;
    p.band_rows = static_cast<int32_t>(rows < p.tiles_m ? rows : p.tiles_m);
    if (p.band_rows < 1) p.band_rows = 1;
  }
  p.l2_hints = hooks().gemm_l2_hints;
  p.W = W;
  p.error_word = info.error_word;
  const int64_t total = static_cast<int64_t>(s.planes) * p.tiles_m * p.tiles_n;
  const int sms = info.sms > 0 ? info.sms : kDefaultSms;
  if (pair) {
    const int64_t pairs = total < sms / 2 ? total : sms / 2;
    k_gemm_i8_pair<<<static_cast<unsigned int>(2 * pairs), kGemmThreads, kPairSmemBytes, stream>>>(
        map_a, map_b, p);
  } else {
    const unsigned int grid = static_cast<unsigned int>(total < sms ? total : sms);
    k_gemm_i8<<<grid, kGemmThreads, kSmemBytes, stream>>>(map_a, map_b, p);
  }
  return cudaPeekAtLastError() == cudaSuccess ? IMD_STATUS_SUCCESS : IMD_STATUS_CUDA_ERROR;
}

// int8 ops per second of the bare tensor pipe (see k_mma_probe); 0 on failure. Synchronises.
double mma_probe_tops(int pair, int sms) {
  const int smem = kBytesA + kBytesB + 2048;
  if (cudaFuncSetAttribute(k_mma_probe<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
      cudaFuncSetAttribute(k_mma_probe<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
    return 0.0;
  const int iters = 64 * 256;
  const int grid = sms / 2 * 2;
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return 0.0;
  if (pair) k_mma_probe<true><<<grid, 64, smem>>>(64);  // warm-up
  else k_mma_probe<false><<<grid, 64, smem>>>(64);
  cudaEventRecord(e0);
  if (pair) k_mma_probe<true><<<grid, 64, smem>>>(iters);
  else k_mma_probe<false><<<grid, 64, smem>>>(iters);
  cudaEventRecord(e1);
  float ms = 0;
  const bool ok = cudaEventSynchronize(e1) == cudaSuccess && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (!ok || ms <= 0) return 0.0;
  const double issuers = pair ? grid / 2 : grid;
  const double ops = 2.0 * (pair ? 256.0 : 128.0) * 256.0 * 32.0 * iters * issuers;
  return ops / (ms * 1e-3);
}

}  // namespace imd
