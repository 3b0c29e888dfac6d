// Plan-time analysis shared by libimmerdink_host (the queries) and libimmerdink (plan creation):
// options, legality, workspace regions, the constants of the shift rule, the gather orientation of
// each operand and the launch structure of one imd_contract. CUDA-free. Everything the kernels
// size or index with comes from here, so the host queries report what the kernels really use.
//
// Counterparts in the reference: src/host/analysis.cpp:93-120 (analyze), :292-356 (plan_data),
// src/host/workspace.cpp:21-81 (workspace_layout), src/host/plan_data.hpp:41-99 (ExecPlan).
#pragma once
#include <cstdint>
#include <vector>

#include "../common/tables.hpp"
#include "immerdink/immerdink_host.h"
#include "lowering.hpp"

#define IMD_INTERNAL __attribute__((visibility("default")))

namespace imd {

constexpr int kDefaultSms = 148;      // B200
constexpr int kMaxVecModes = 64;      // fused modes a kernel parameter block can carry

struct Layout {
  uint64_t offset[IMD_REGION_COUNT] = {};
  uint64_t bytes[IMD_REGION_COUNT] = {};
  uint64_t total = 0;
};

// Regions of a packed operand's buffer (shifts, flags, residue planes).
struct PackRegions {
  uint64_t offset[3] = {0, 0, 0}, bytes[3] = {0, 0, 0};
  uint64_t total = 0;
};

// Which operands of a plan are read from packs, and their keys.
struct PackedSlots {
  int32_t caller = 0;    // bit 0 / 1: the caller's A / B
  int32_t role = 0;      // bit 0 / 1: the post-swap A / B
  int32_t mismatch = 0;  // IMD_PACK_MISMATCH_* of a PACK_MISMATCH status
  std::vector<int64_t> key[2];  // by caller operand; empty = in-line
  PackRegions layout[2];        // by post-swap role
};

struct Analysis {
  imd_options_t options{};
  GemmView view;
  int k_align = 16;
  Layout layout;
  PackedSlots packed;
};

enum class Path : int { kNoop = 0, kGemm = 1, kDirect = 2 };

// Fused modes of the four classes, flattened; passed by value to the vector-generation kernel.
struct ModeTable {
  int32_t first[4] = {0, 0, 0, 0};
  int32_t count[4] = {0, 0, 0, 0};
  int64_t extent[kMaxVecModes] = {};
  int64_t stride[kMaxVecModes][3] = {};
};

struct ExecPlan {
  Path path = Path::kNoop;
  bool swapped = false;
  int64_t m = 0, n = 0, k = 0, b = 0, n_hat = 0, k_hat = 0;
  int32_t k_align = 16;
  int32_t N = 0, g = 0;
  bool trunc = false;
  Layout layout;
  Wide<8> rhs{};            // (2T - kappa)^2 2^60 or T^2 2^60
  int32_t lhs_shift = 0;    // S is multiplied by 4 (RN) or 1 (TRUNC): a left shift of 2 or 0
  ShiftFast fast{};         // the same right-hand side for the FP64 shortcut of the shift rule
  bool rows_fast[2] = {false, false};  // operand is contiguous along its rows rather than along K
  bool c_batch_fast = false;           // C's batch mode is faster than its column mode
  int64_t vec_count = 0;
  uint64_t device_bytes = 0;
  bool vec_resident = false;
  int64_t k_chunks = 0;
  int32_t packed = 0;                 // bit 0 / 1: the post-swap A / B comes from a packed buffer
  uint64_t pack_off[2][3] = {};       // by role: offsets of shifts, flags, planes in that buffer
  uint64_t pack_bytes[2] = {0, 0};
  ModeTable modes;
  bool emulated() const { return path == Path::kGemm && k >= 2; }
  // Small contractions take one fused launch (k_small): short rows and at most 256 tiles of
  // 32 x 32 outputs, no packed operand. The same test decides the lowering's launch count.
  bool small() const {
    if (!emulated() || packed != 0 || k > 128) return false;
    const int64_t tiles = ((m + 31) / 32) * ((n + 31) / 32);
    return tiles <= 256 && b <= 256 && tiles * b <= 256;
  }
};

IMD_INTERNAL imd_status_t analyze(const imd_tensor_t* A, const imd_tensor_t* B,
                                  const imd_tensor_t* C, const imd_options_t* options,
                                  Analysis* out);
IMD_INTERNAL imd_status_t make_plan(const Analysis& an, ExecPlan* out);
// The eight regions; `packed_roles` (bit 0 / 1) drops sX, fX, RX of a packed post-swap A / B.
IMD_INTERNAL bool workspace_regions(const GemmView& v, const imd_options_t& o, int k_align,
                                    int packed_roles, Layout* L);

// K chunks of the int8 GEMM, GEMM launches and all kernel launches of one call (alpha != 0).
IMD_INTERNAL int64_t plan_k_chunks(const ExecPlan& e);
IMD_INTERNAL int64_t plan_gemm_launches(const ExecPlan& e);
IMD_INTERNAL int64_t plan_kernel_launches(const ExecPlan& e);
// Bytes of the plan record and its tables (allocator overhead excluded).
IMD_INTERNAL uint64_t plan_host_bytes(const imd_tensor_t& A, const imd_tensor_t& B,
                                      const imd_tensor_t& C, const Analysis& an, const ExecPlan& e);

// The plan record of libimmerdink; defined here so that the host library can size it.
struct TensorCopy {
  std::vector<int64_t> extent, stride;
  std::vector<int32_t> label;
  TensorCopy() = default;
  explicit TensorCopy(const imd_tensor_t& t)
      : extent(t.extent, t.extent + t.rank), stride(t.stride, t.stride + t.rank),
        label(t.label, t.label + t.rank) {}
};

}  // namespace imd

struct imd_plan_st {
  imd_options_t options{};
  imd::GemmView view;
  imd::TensorCopy A, B, C;   // the caller's descriptors (aliasing intervals)
  imd::ExecPlan exec;
  imd::CrtTables crt{};
  imd::ResidueTables res{};
  int device = 0;
  int sms = 0;
  void* vec_dev = nullptr;   // IMD_VEC_RESIDENT: plan-owned scatter vectors
  void* encode_tiled = nullptr;  // driver entry point for TMA descriptor encoding
  void* error_word = nullptr;    // device address of the sticky error word of bounded waits
  std::vector<int64_t> slot_key[2];
};
