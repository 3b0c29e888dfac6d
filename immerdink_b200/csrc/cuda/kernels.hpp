// Declarations shared by the C ABI (api.cpp), the pipeline (pipeline.cu) and the tcgen05 GEMM
// (gemm_tcgen05.cu). Everything a kernel needs is passed by value in its parameters, so a plan
// may be destroyed as soon as imd_contract has returned and a captured graph replays without it.
#pragma once
#include <cstdint>

#include <cuda.h>
#include <cuda_runtime_api.h>

#include "common/tables.hpp"
#include "host/plan.hpp"
#include "immerdink/immerdink.h"

namespace imd {

// One GEMM launch: `planes` planes of the residue buffers, K range [k0, k0 + klen) of every row,
// into the product planes starting at modulus mod0. A product plane holds
// y = (q_l * sum_h RA RB) mod p_l, the form the CRT consumes.
struct GemmShape {
  int32_t m, n_hat;        // rows of A per plane; row pitch of W (columns of C, padded to 16)
  int32_t b_rows;          // rows of B per plane: n_hat in the workspace, n in a packed buffer
  int32_t k_hat;           // row pitch of the residue planes (bytes)
  int32_t k0, klen;        // K chunk
  int32_t planes;          // slots x batches in this launch
  int32_t batches;         // b
  int32_t mod0;            // first modulus of the group
  int32_t add;             // 0: W = acc mod p; 1: W = (W + acc) mod p
  uint32_t p[kMaxModuli];      // moduli of the group's slots (index = slot)
  uint32_t magic[kMaxModuli];     // floor(2^32 / p): quotient within one of floor(v / p)
  uint32_t magic_up[kMaxModuli];  // ceil(2^32 / p): exact quotient for v < 2^24
  uint32_t bias[kMaxModuli];      // the multiple of p in [2^31, 2^31 + p)
  uint32_t q[kMaxModuli];         // CRT weight inverse M_l^-1 mod p_l: the planes store q (A'B') mod p
};

struct GemmPlanInfo {
  void* encode_tiled = nullptr;
  unsigned int* error_word = nullptr;
  int sms = 0;
};

imd_status_t quantize_setup();                 // plan / pack creation: function attributes
imd_status_t gemm_setup(GemmPlanInfo* info);   // plan time: function attributes, driver entry point
imd_status_t gemm_launch(const GemmPlanInfo& info, const GemmShape& s, const int8_t* RA,
                         const int8_t* RB, uint8_t* W, cudaStream_t stream);
// Slow exact int8 GEMM with the same contract: a second, independent implementation used only
// by the verification hooks to cross-check the tensor-core kernel at sizes a CPU cannot reach.
imd_status_t gemm_reference_launch(const GemmShape& s, const int8_t* RA, const int8_t* RB,
                                   uint8_t* W, cudaStream_t stream);

// `packed[x]`: the packed buffer of the post-swap operand x of a plan with that slot packed.
// `part`: 0 the whole call; 1 everything but the outputs of the native path (A and B are not
// read); 2 only those outputs, from the shifts and flags already in the packs / workspace.
imd_status_t enqueue_contract(const imd_plan_st& plan, double alpha, const double* A,
                              const double* B, double beta, double* C, void* ws,
                              cudaStream_t stream, const void* const packed[2] = nullptr,
                              int part = 0);
// imd_pack: shifts, flags and all N residue planes of X into `packed` (every byte written).
imd_status_t enqueue_pack(const ExecPlan& e, const ResidueTables& tables, const PackRegions& layout,
                          const double* X, void* packed, void* ws, cudaStream_t stream);
// imd_pack_scatter: the rows of a piece into rows [row0, row0 + rows) of up to 8 packed buffers of
// a slab with slab_rows rows per batch (layout = that slab's).
imd_status_t enqueue_pack_scatter(const ExecPlan& e, const ResidueTables& tables,
                                  const PackRegions& layout, int64_t slab_rows, int64_t row0,
                                  const double* X, void* const* dest, int n_dest, void* ws,
                                  cudaStream_t stream);
imd_status_t generate_vectors(const ExecPlan& e, int64_t* vec, cudaStream_t stream);

// Bounded wait (one launch of one warp) until every flags[i] (device addresses, n <= kMaxWaitFlags)
// holds `expect`; gives up after `limit` polls per flag and sets bit 2 of the device error word.
constexpr int kMaxFlagRanges = 4;
constexpr int kMaxCondCopies = 16;
// One launch: copies the ranges src[c] -> dst[c] (8-byte aligned, bytes[c] multiples of 8) only if
// a byte of the flag ranges is nonzero.
imd_status_t enqueue_copy_if_flagged(const unsigned char* const* flags, const int64_t* flag_bytes,
                                     int ranges, void* const* dst, const void* const* src,
                                     const int64_t* bytes, int copies, cudaStream_t stream);
// One launch of `ctas` CTAs: copies the ranges src[r] -> dst[r] (16-byte aligned, bytes[r] multiples
// of 16; destinations may be peers' memory), then stores `value` into the flag words (release,
// system scope).
constexpr int kMaxPushRanges = 96;
constexpr int kMaxPushFlags = 8;
imd_status_t enqueue_push(void* const* dst, const void* const* src, const int64_t* bytes, int ranges,
                          unsigned int* const* flags, int num_flags, unsigned int value, int ctas,
                          cudaStream_t stream);
// Copies the device error word into *host_word (pinned host memory) on `stream`, without clearing it.
imd_status_t enqueue_error_peek(unsigned int* host_word, cudaStream_t stream);
constexpr int kMaxWaitFlags = 32;
imd_status_t enqueue_wait_flags(const unsigned int* const* flags, int n, unsigned int expect,
                                unsigned long long limit, cudaStream_t stream);

// Knobs of the verification and tuning hooks. The production library links a constant copy of the
// defaults (nothing in it can change them: imd_contract consults no mutable process state); the
// instrumented library used by the tests and by phase timing links a mutable copy with the
// imd_test_* / imd_prof_* entry points (hooks.cpp, compiled twice).
struct Hooks {
  bool reference_gemm = false;  // run the slow exact GEMM instead of the tensor-core kernel
  int gemm_variant = 0;         // 0 = by shape, 1 = one CTA per 128 x 256 tile, 2 = CTA pairs
  int gemm_band_mb = 32;        // MB of operand A's tile rows the tile order keeps in L2
  int gemm_l2_hints = 5;        // eviction hints of the GEMM's operand loads (evict last on both)
  int force_exact_shift = 0;    // 1 = the scale step never takes its FP64 shortcut
  int force_exact_crt = 0;      // 1 = the CRT step never takes its FP64 shortcut
  int small_path = 1;           // 0 = small contractions take the general kernel sequence too
};
const Hooks& hooks();
// Phase boundary of a call (tags: 1 vectors + scale, 2 quantise, 3 GEMM, 4 CRT, 5 degenerate path,
// 6 imd_pack, 7 the one fused launch of a small contraction): records an event in the instrumented library, nothing in the production one.
void phase_mark(int tag, cudaStream_t stream);
// Benchmark hook: int8 ops per second of back-to-back tcgen05.mma.kind::i8 with no loads.
double mma_probe_tops(int pair, int sms);

// Sticky device-side error word (bounded waits that gave up); read by the verification hook.
unsigned int* device_error_word();

}  // namespace imd
