// Packed operands, host side: one operand X scaled and reduced once to all N residue planes in a
// caller-owned buffer, reused by many contractions. This file sizes the buffer, derives the
// compatibility key and matches packs against plans. CUDA-free.
//
// Behaviour follows the reference (src/host/pack.cpp:35-244 for the pack itself,
// src/host/analysis.cpp:136-258 for the plan-side match; byte layout in
// include/immerdink/immerdink_host.h:259-283):
//   sig   int16 shift of row (lambda, rho) at index lambda r + rho
//   flag  u8 non-finite flag, same index
//   res   int8 residue planes, plane l at l b r k_hat + (lambda r + rho) k_hat + k-bar, zero K padding,
//         followed by a zero tail of (ceil(r)_16 - r) k_hat bytes
// each region 256-byte aligned; every byte of the buffer is written by imd_pack.
#pragma once
#include <cstdint>
#include <vector>

#include "immerdink/immerdink_host.h"
#include "plan.hpp"

namespace imd {

enum : int { kPackK = 0, kPackL = 1, kPackR = 2 };
enum : int { kPackSig = 0, kPackFlag = 1, kPackRes = 2 };

struct PackMode {
  int64_t extent = 0, stride = 0;
};

struct PackLowered {
  bool sized = false;  // sizes and layout valid (SUCCESS or NOT_SUPPORTED)
  int N = 0;
  int32_t rounding = IMD_RN;
  int64_t b = 0, r = 0, k = 0, k_hat = 0;
  int32_t k_align = 0;
  int64_t format = 0;
  uint64_t kappa = 0;
  PackRegions layout;
  uint64_t ws_bytes = 0;
  std::vector<int32_t> order[3];   // kept labels per class (K, L, R), first fastest
  std::vector<PackMode> fused[3];  // X's modes fused over X's strides alone
  std::vector<int64_t> key;
};

// A pack as a plan sees it: X's labels by position and the lowered pack.
struct PackSource {
  int32_t rank = 0;
  const int32_t* label = nullptr;
  const PackLowered* pl = nullptr;
};

IMD_INTERNAL bool pack_regions(int64_t b, int64_t r, int64_t k, int N, int32_t k_align,
                               PackRegions* out);
IMD_INTERNAL bool pack_workspace_bytes(int64_t b, int64_t r, int64_t k, uint64_t* out);
IMD_INTERNAL imd_status_t pack_lower(const imd_pack_desc_t& d, PackLowered* out);
IMD_INTERNAL uint64_t key_digest(const std::vector<int64_t>& key);
// Plan-side match: adopts the packs' orders into an->view, recomputes the workspace without the
// packed roles' regions, fills an->packed. PACK_MISMATCH with an->packed.mismatch set otherwise.
IMD_INTERNAL imd_status_t match_packs(const imd_tensor_t* A, const imd_tensor_t* B,
                                      const PackSource* const src[2], Analysis* an);
// The launch data of imd_pack: X as operand A of a one-operand view (rows = R, K, batch = L).
IMD_INTERNAL void pack_exec(const PackLowered& pl, ExecPlan* out);

}  // namespace imd
