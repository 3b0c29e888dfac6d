// C ABI of libimmerdink.so. Argument checks follow the order the reference documents and
// implements (src/api.cpp:293-334 for imd_contract, :120-199 for plan creation): a failing call
// touches nothing. No exception leaves a function. All sizing and legality come from
// libimmerdink_host (host/plan.hpp); this file adds the device-side parts of a plan.
#include <cstdint>
#include <memory>
#include <new>

#include <cuda_runtime_api.h>

#include "immerdink/immerdink.h"
#include "host/pack.hpp"
#include "kernels.hpp"

struct imd_handle_st {
  int device = 0;
};
// A pack handle: host-only (no GPU work reads it), immutable after creation.
struct imd_pack_s {
  imd::TensorCopy tensor;   // X's descriptor (aliasing interval, labels for the plan-side match)
  imd::PackLowered pl;
  imd::ExecPlan exec;       // the launch data of imd_pack
  imd::ResidueTables res{};
};

namespace {

using i128 = __int128;

bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Bytes a strided FP64 view can address, [lo, hi); empty for a null pointer or an empty tensor.
struct Interval {
  i128 lo = 0, hi = 0;
};
Interval tensor_bytes(const imd::TensorCopy& t, const void* p) {
  Interval r;
  if (p == nullptr) return r;
  i128 below = 0, above = 0;
  for (size_t d = 0; d < t.extent.size(); ++d) {
    if (t.extent[d] == 0) return r;
    const i128 span = static_cast<i128>(t.stride[d]) * (t.extent[d] - 1);
    (span < 0 ? below : above) += span;
  }
  const i128 base = static_cast<i128>(reinterpret_cast<uintptr_t>(p));
  r.lo = base + 8 * below;
  r.hi = base + 8 * above + 8;
  return r;
}
Interval raw_bytes(const void* p, uint64_t n) {
  Interval r;
  if (p == nullptr || n == 0) return r;
  r.lo = static_cast<i128>(reinterpret_cast<uintptr_t>(p));
  r.hi = r.lo + static_cast<i128>(n);
  return r;
}
bool overlap(const Interval& x, const Interval& y) {
  return x.lo < x.hi && y.lo < y.hi && x.lo < y.hi && y.lo < x.hi;
}

imd_status_t plan_create(imd_handle_t handle, const imd_tensor_t* A, const imd_tensor_t* B,
                         const imd_tensor_t* C, const imd_options_t* options,
                         const imd_pack_t pack[2], imd_plan_t* plan) {
  if (handle == nullptr || plan == nullptr) return IMD_STATUS_INVALID_VALUE;
  try {
    imd::Analysis an;
    if (const imd_status_t st = imd::analyze(A, B, C, options, &an); st != IMD_STATUS_SUCCESS)
      return st;
    if (pack[0] != nullptr || pack[1] != nullptr) {
      imd::PackSource ps[2];
      const imd::PackSource* src[2] = {nullptr, nullptr};
      for (int x = 0; x < 2; ++x) {
        if (pack[x] == nullptr) continue;
        ps[x] = imd::PackSource{static_cast<int32_t>(pack[x]->tensor.label.size()),
                                pack[x]->tensor.label.data(), &pack[x]->pl};
        src[x] = &ps[x];
      }
      if (const imd_status_t st = imd::match_packs(A, B, src, &an); st != IMD_STATUS_SUCCESS)
        return st;
    }
    imd::ExecPlan e;
    if (const imd_status_t st = imd::make_plan(an, &e); st != IMD_STATUS_SUCCESS) return st;
    auto p = std::make_unique<imd_plan_st>();
    p->options = an.options;
    p->view = an.view;
    p->A = imd::TensorCopy(*A), p->B = imd::TensorCopy(*B), p->C = imd::TensorCopy(*C);
    p->exec = e;
    for (int x = 0; x < 2; ++x) p->slot_key[x] = an.packed.key[x];
    p->crt = imd::crt_tables(e.N);
    p->res = imd::residue_tables(e.N);
    if (e.path != imd::Path::kNoop) {
      if (cudaGetDevice(&p->device) != cudaSuccess ||
          cudaDeviceGetAttribute(&p->sms, cudaDevAttrMultiProcessorCount, p->device) != cudaSuccess) {
        cudaGetLastError();
        return IMD_STATUS_CUDA_ERROR;
      }
    }
    if (e.emulated()) {
      imd::GemmPlanInfo info;
      if (const imd_status_t st = imd::gemm_setup(&info); st != IMD_STATUS_SUCCESS) return st;

      p->encode_tiled = info.encode_tiled;
      p->error_word = info.error_word;
    }
    if (e.vec_resident) {
      void* dev = nullptr;
      const cudaError_t err = cudaMalloc(&dev, static_cast<size_t>(e.device_bytes));
      if (err != cudaSuccess) {
        cudaGetLastError();
        return err == cudaErrorMemoryAllocation ? IMD_STATUS_ALLOC_FAILED : IMD_STATUS_CUDA_ERROR;
      }
      p->vec_dev = dev;
      if (imd::generate_vectors(e, static_cast<int64_t*>(dev), cudaStreamPerThread) !=
              IMD_STATUS_SUCCESS ||
          cudaStreamSynchronize(cudaStreamPerThread) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(dev);
        return IMD_STATUS_CUDA_ERROR;
      }
    }
    *plan = p.release();
    return IMD_STATUS_SUCCESS;
  } catch (const std::bad_alloc&) {
    return IMD_STATUS_ALLOC_FAILED;
  } catch (...) {
    return IMD_STATUS_INVALID_VALUE;
  }
}

}  // namespace

extern "C" {

imd_status_t imd_create(imd_handle_t* handle) {
  if (handle == nullptr) return IMD_STATUS_INVALID_VALUE;
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    cudaGetLastError();
    return IMD_STATUS_CUDA_ERROR;
  }
  // per-device function attributes of the kernels are set here, never inside imd_contract / imd_pack
  if (const imd_status_t st = imd::quantize_setup(); st != IMD_STATUS_SUCCESS) return st;
  auto* h = new (std::nothrow) imd_handle_st{device};
  if (h == nullptr) return IMD_STATUS_ALLOC_FAILED;
  *handle = h;
  return IMD_STATUS_SUCCESS;
}

imd_status_t imd_destroy(imd_handle_t handle) {
  delete handle;
  return IMD_STATUS_SUCCESS;
}

imd_status_t imd_plan_create(imd_handle_t handle, const imd_tensor_t* A, const imd_tensor_t* B,
                             const imd_tensor_t* C, const imd_options_t* options,
                             imd_plan_t* plan) {
  const imd_pack_t none[2] = {nullptr, nullptr};
  return plan_create(handle, A, B, C, options, none, plan);
}

imd_status_t imd_plan_destroy(imd_plan_t plan) {
  if (plan != nullptr && plan->vec_dev != nullptr) cudaFree(plan->vec_dev);
  delete plan;
  return IMD_STATUS_SUCCESS;
}

imd_status_t imd_plan_device_bytes(imd_plan_t plan, size_t* bytes) {
  if (plan == nullptr || bytes == nullptr) return IMD_STATUS_INVALID_VALUE;
  *bytes = plan->exec.vec_resident ? static_cast<size_t>(plan->exec.device_bytes) : 0;
  return IMD_STATUS_SUCCESS;
}

imd_status_t imd_contract(imd_plan_t plan, double alpha, const double* A, const double* B,
                          double beta, double* C, void* ws, size_t ws_bytes, cudaStream_t stream) {
  if (plan == nullptr) return IMD_STATUS_INVALID_VALUE;
  if (!plan->slot_key[0].empty() || !plan->slot_key[1].empty()) return IMD_STATUS_PACK_MISMATCH;
  const imd::ExecPlan& e = plan->exec;
  const bool reads_ab = alpha != 0.0 && e.k != 0;
  const uint64_t need = e.layout.total;
  if (C == nullptr || (reads_ab && (A == nullptr || B == nullptr)) || (need > 0 && ws == nullptr))
    return IMD_STATUS_INVALID_VALUE;
  if (e.path == imd::Path::kNoop) return IMD_STATUS_SUCCESS;
  const Interval iA = tensor_bytes(plan->A, A), iB = tensor_bytes(plan->B, B),
                 iC = tensor_bytes(plan->C, C), iW = raw_bytes(ws, need);
  if (overlap(iC, iA) || overlap(iC, iB) || overlap(iW, iA) || overlap(iW, iB) || overlap(iW, iC))
    return IMD_STATUS_ALIASING;
  if (!aligned(A, 8) || !aligned(B, 8) || !aligned(C, 8) || (need > 0 && !aligned(ws, imd::kRegionAlign)))
    return IMD_STATUS_MISALIGNED;
  if (ws_bytes < need) return IMD_STATUS_INSUFFICIENT_WORKSPACE;
  const double* gA = e.swapped ? B : A;
  const double* gB = e.swapped ? A : B;
  try {
    return imd::enqueue_contract(*plan, alpha, gA, gB, beta, C, ws, stream);
  } catch (...) {
    return IMD_STATUS_CUDA_ERROR;
  }
}

/* ---- packed operands (ref: src/api.cpp:211-276 and :336-394) ---------------------------------- */
imd_status_t imd_pack_create(imd_handle_t handle, const imd_pack_desc_t* desc, imd_pack_t* pack) {
  if (handle == nullptr || desc == nullptr || pack == nullptr) return IMD_STATUS_INVALID_VALUE;
  try {
    imd::PackLowered pl;
    if (const imd_status_t st = imd::pack_lower(*desc, &pl); st != IMD_STATUS_SUCCESS) return st;
    auto p = std::make_unique<imd_pack_s>();
    p->tensor = imd::TensorCopy(*desc->tensor);
    p->pl = std::move(pl);
    imd::pack_exec(p->pl, &p->exec);
    p->res = imd::residue_tables(p->pl.N);
    *pack = p.release();
    return IMD_STATUS_SUCCESS;
  } catch (const std::bad_alloc&) {
    return IMD_STATUS_ALLOC_FAILED;
  } catch (...) {
    return IMD_STATUS_INVALID_VALUE;
  }
}

imd_status_t imd_pack_destroy(imd_pack_t pack) {
  delete pack;
  return IMD_STATUS_SUCCESS;
}

imd_status_t imd_pack_bytes(imd_pack_t pack, size_t* pack_bytes, size_t* pack_ws_bytes) {
  if (pack == nullptr) return IMD_STATUS_INVALID_VALUE;
  if (pack_bytes != nullptr) *pack_bytes = static_cast<size_t>(pack->pl.layout.total);
  if (pack_ws_bytes != nullptr) *pack_ws_bytes = static_cast<size_t>(pack->pl.ws_bytes);
  return IMD_STATUS_SUCCESS;
}

imd_status_t imd_pack(imd_pack_t pack, const double* X, void* packed, size_t packed_bytes,
                      void* ws, size_t ws_bytes, cudaStream_t stream) {
  // order: null pointers; an empty pack; ALIASING; MISALIGNED; sizes
  if (pack == nullptr) return IMD_STATUS_INVALID_VALUE;
  const uint64_t need = pack->pl.layout.total, need_ws = pack->pl.ws_bytes;
  if ((need > 0 && (X == nullptr || packed == nullptr)) || (need_ws > 0 && ws == nullptr))
    return IMD_STATUS_INVALID_VALUE;
  if (need == 0) return IMD_STATUS_SUCCESS;
  const Interval iX = tensor_bytes(pack->tensor, X), iP = raw_bytes(packed, need),
                 iW = raw_bytes(ws, need_ws);
  if (overlap(iP, iX) || overlap(iW, iX) || overlap(iW, iP)) return IMD_STATUS_ALIASING;
  if (!aligned(X, 8) || !aligned(packed, imd::kRegionAlign) ||
      (need_ws > 0 && !aligned(ws, imd::kRegionAlign)))
    return IMD_STATUS_MISALIGNED;
  if (packed_bytes < need || ws_bytes < need_ws) return IMD_STATUS_INSUFFICIENT_WORKSPACE;
  try {
    return imd::enqueue_pack(pack->exec, pack->res, pack->pl.layout, X, packed, ws, stream);
  } catch (...) {
    return IMD_STATUS_CUDA_ERROR;
  }
}

/* Extension (no counterpart in the reference): imd_pack of a PIECE of a slab for all the slab's
 * consumers at once. The pack handle describes the piece X (r rows per batch); its rows land as
 * rows [row_offset, row_offset + r) of packed buffers whose batches have slab_rows rows, in the
 * byte layout imd_pack_layout reports for that slab (same K, batches, N, rounding), and every one
 * of the num_dest buffers (1..8, dest[0] the caller's own, the others possibly other GPUs' memory
 * mapped into this process) receives the same bytes by plain stores. Gaps and tail are zeroed in
 * dest[0] only. Checks: null pointers, ranges -> INVALID_VALUE; 256-byte alignment -> MISALIGNED;
 * dest_bytes below the slab's pack_bytes, ws_bytes below the piece's pack_ws_bytes ->
 * INSUFFICIENT_WORKSPACE. Enqueue only. */
IMD_API imd_status_t imd_pack_scatter(imd_pack_t piece, const double* X, int64_t slab_rows,
                                      int64_t row_offset, int32_t num_dest, void* const* dest,
                                      size_t dest_bytes, void* ws, size_t ws_bytes,
                                      cudaStream_t stream) {
  if (piece == nullptr || dest == nullptr || num_dest < 1 || num_dest > 8 || row_offset < 0 ||
      slab_rows < 0)
    return IMD_STATUS_INVALID_VALUE;
  const imd::PackLowered& pl = piece->pl;
  if (pl.r > slab_rows || row_offset > slab_rows - pl.r) return IMD_STATUS_INVALID_VALUE;
  imd::PackRegions slab;
  if (!imd::pack_regions(pl.b, slab_rows, pl.k, pl.N, pl.k_align, &slab)) return IMD_STATUS_INVALID_VALUE;
  const uint64_t need_ws = pl.ws_bytes;
  if (pl.layout.total == 0) return IMD_STATUS_SUCCESS;  // an empty piece
  if (X == nullptr || (need_ws > 0 && ws == nullptr)) return IMD_STATUS_INVALID_VALUE;
  for (int32_t i = 0; i < num_dest; ++i)
    if (dest[i] == nullptr) return IMD_STATUS_INVALID_VALUE;
  if (!aligned(X, 8) || (need_ws > 0 && !aligned(ws, imd::kRegionAlign))) return IMD_STATUS_MISALIGNED;
  for (int32_t i = 0; i < num_dest; ++i)
    if (!aligned(dest[i], imd::kRegionAlign)) return IMD_STATUS_MISALIGNED;
  if (dest_bytes < slab.total || ws_bytes < need_ws) return IMD_STATUS_INSUFFICIENT_WORKSPACE;
  try {
    return imd::enqueue_pack_scatter(piece->exec, piece->res, slab, slab_rows, row_offset, X, dest,
                                     num_dest, ws, stream);
  } catch (...) {
    return IMD_STATUS_CUDA_ERROR;
  }
}

imd_status_t imd_plan_create_packed(imd_handle_t handle, const imd_tensor_t* A,
                                    const imd_tensor_t* B, const imd_tensor_t* C,
                                    const imd_options_t* options, imd_pack_t packA,
                                    imd_pack_t packB, imd_plan_t* plan) {
  const imd_pack_t packs[2] = {packA, packB};
  return plan_create(handle, A, B, C, options, packs, plan);
}

IMD_API imd_status_t imd_contract_packed_part(imd_plan_t plan, double alpha,
                                              const imd_operand_t* A, const imd_operand_t* B,
                                              double beta, double* C, void* ws, size_t ws_bytes,
                                              cudaStream_t stream, int32_t part) {
  if (part < 0 || (part > 3 && part < 16) || part >= 16 + imd::kMaxModuli) return IMD_STATUS_INVALID_VALUE;
  // order: operands and packed slots; null pointers; empty output; ALIASING; MISALIGNED; sizes
  if (plan == nullptr || A == nullptr || B == nullptr) return IMD_STATUS_INVALID_VALUE;
  const imd::ExecPlan& e = plan->exec;
  const imd_operand_t* op[2] = {A, B};
  int role[2];  // post-swap role of the caller's operand x
  for (int x = 0; x < 2; ++x) {
    role[x] = (x == 0) != e.swapped ? 0 : 1;
    if (plan->slot_key[x].empty()) {
      if (op[x]->packed != nullptr || op[x]->pack != nullptr) return IMD_STATUS_PACK_MISMATCH;
    } else if (op[x]->pack == nullptr || op[x]->pack->pl.key != plan->slot_key[x]) {
      return IMD_STATUS_PACK_MISMATCH;
    }
  }
  const bool reads_ab = alpha != 0.0 && e.k != 0;
  const bool reads_pack = reads_ab && e.emulated();
  const uint64_t need = e.layout.total;
  // a part is defined for the emulated GEMM only; part 1 never reads the FP64 operands
  if (part != 0 && !reads_pack) return IMD_STATUS_INVALID_VALUE;
  const bool native = part == 0 || part == 2;  // the parts that read the FP64 operands
  if (C == nullptr || (reads_ab && native && (A->data == nullptr || B->data == nullptr)) ||
      (need > 0 && ws == nullptr))
    return IMD_STATUS_INVALID_VALUE;
  for (int x = 0; x < 2; ++x)
    if (!plan->slot_key[x].empty() && reads_pack && e.pack_bytes[role[x]] > 0 &&
        op[x]->packed == nullptr)
      return IMD_STATUS_INVALID_VALUE;
  if (e.path == imd::Path::kNoop) return IMD_STATUS_SUCCESS;
  // C against every input range; the workspace against those and C. Packed buffers may overlap
  // each other and the FP64 operands: all are only read.
  const Interval iC = tensor_bytes(plan->C, C), iW = raw_bytes(ws, need);
  Interval in[4] = {tensor_bytes(plan->A, A->data), tensor_bytes(plan->B, B->data), {}, {}};
  for (int x = 0; x < 2; ++x)
    if (!plan->slot_key[x].empty()) in[2 + x] = raw_bytes(op[x]->packed, e.pack_bytes[role[x]]);
  if (overlap(iW, iC)) return IMD_STATUS_ALIASING;
  for (const Interval& r : in)
    if (overlap(iC, r) || overlap(iW, r)) return IMD_STATUS_ALIASING;
  if (!aligned(A->data, 8) || !aligned(B->data, 8) || !aligned(C, 8) ||
      !aligned(A->packed, imd::kRegionAlign) || !aligned(B->packed, imd::kRegionAlign) ||
      (need > 0 && !aligned(ws, imd::kRegionAlign)))
    return IMD_STATUS_MISALIGNED;
  if (ws_bytes < need) return IMD_STATUS_INSUFFICIENT_WORKSPACE;
  for (int x = 0; x < 2; ++x)
    if (op[x]->packed != nullptr && op[x]->packed_bytes < e.pack_bytes[role[x]])
      return IMD_STATUS_INSUFFICIENT_WORKSPACE;
  const double* gA = e.swapped ? B->data : A->data;
  const double* gB = e.swapped ? A->data : B->data;
  const void* packed[2] = {nullptr, nullptr};  // by post-swap role
  for (int x = 0; x < 2; ++x)
    if (!plan->slot_key[x].empty()) packed[role[x]] = op[x]->packed;
  try {
    return imd::enqueue_contract(*plan, alpha, gA, gB, beta, C, ws, stream, packed, part);
  } catch (...) {
    return IMD_STATUS_CUDA_ERROR;
  }
}

imd_status_t imd_contract_packed(imd_plan_t plan, double alpha, const imd_operand_t* A,
                                 const imd_operand_t* B, double beta, double* C, void* ws,
                                 size_t ws_bytes, cudaStream_t stream) {
  return imd_contract_packed_part(plan, alpha, A, B, beta, C, ws, ws_bytes, stream, 0);
}

/* Bounded wait on flags that a peer's copies set (extension; see the header). */
imd_status_t imd_wait_flags(const unsigned int* const* flags, int num_flags, unsigned int expect,
                            uint64_t max_polls, cudaStream_t stream) {
  if (num_flags == 0) return IMD_STATUS_SUCCESS;
  if (flags == nullptr || num_flags < 0 || num_flags > imd::kMaxWaitFlags)
    return IMD_STATUS_INVALID_VALUE;
  for (int i = 0; i < num_flags; ++i) {
    if (flags[i] == nullptr) return IMD_STATUS_INVALID_VALUE;
    if (reinterpret_cast<uintptr_t>(flags[i]) % 4 != 0) return IMD_STATUS_MISALIGNED;
  }
  const unsigned long long limit = max_polls ? max_polls : 4000000ull;  /* about a second */
  return imd::enqueue_wait_flags(flags, num_flags, expect, limit, stream);
}

/* Copies that run only when a row flag is set (extension; see the header). */
imd_status_t imd_copy_if_flagged(const unsigned char* const* flags, const int64_t* flag_bytes,
                                 int32_t num_ranges, void* const* dst, const void* const* src,
                                 const int64_t* bytes, int32_t num_copies, cudaStream_t stream) {
  if (num_ranges < 0 || num_ranges > imd::kMaxFlagRanges || num_copies < 0 ||
      num_copies > imd::kMaxCondCopies)
    return IMD_STATUS_INVALID_VALUE;
  if (num_copies == 0) return IMD_STATUS_SUCCESS;
  if (dst == nullptr || src == nullptr || bytes == nullptr ||
      (num_ranges > 0 && (flags == nullptr || flag_bytes == nullptr)))
    return IMD_STATUS_INVALID_VALUE;
  for (int r = 0; r < num_ranges; ++r)
    if (flag_bytes[r] < 0 || (flag_bytes[r] > 0 && flags[r] == nullptr)) return IMD_STATUS_INVALID_VALUE;
  for (int c = 0; c < num_copies; ++c) {
    if (bytes[c] < 0 || (bytes[c] > 0 && (dst[c] == nullptr || src[c] == nullptr)))
      return IMD_STATUS_INVALID_VALUE;
    if (bytes[c] % 8 != 0 || reinterpret_cast<uintptr_t>(dst[c]) % 8 != 0 ||
        reinterpret_cast<uintptr_t>(src[c]) % 8 != 0)
      return IMD_STATUS_MISALIGNED;
  }
  return imd::enqueue_copy_if_flagged(flags, flag_bytes, num_ranges, dst, src, bytes, num_copies, stream);
}

/* Pushes by a small copy kernel (extension; see the header). */
imd_status_t imd_push_ranges(void* const* dst, const void* const* src, const int64_t* bytes,
                             int32_t num_ranges, unsigned int* const* flags, int32_t num_flags,
                             unsigned int value, int32_t ctas, cudaStream_t stream) {
  if (num_ranges < 0 || num_ranges > imd::kMaxPushRanges || num_flags < 0 ||
      num_flags > imd::kMaxPushFlags || ctas < 0 || ctas > 1024)
    return IMD_STATUS_INVALID_VALUE;
  if (num_ranges == 0 && num_flags == 0) return IMD_STATUS_SUCCESS;
  if ((num_ranges > 0 && (dst == nullptr || src == nullptr || bytes == nullptr)) ||
      (num_flags > 0 && flags == nullptr))
    return IMD_STATUS_INVALID_VALUE;
  for (int r = 0; r < num_ranges; ++r) {
    if (bytes[r] < 0 || (bytes[r] > 0 && (dst[r] == nullptr || src[r] == nullptr)))
      return IMD_STATUS_INVALID_VALUE;
    if (bytes[r] % 16 != 0 || reinterpret_cast<uintptr_t>(dst[r]) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(src[r]) % 16 != 0)
      return IMD_STATUS_MISALIGNED;
  }
  for (int f = 0; f < num_flags; ++f) {
    if (flags[f] == nullptr) return IMD_STATUS_INVALID_VALUE;
    if (reinterpret_cast<uintptr_t>(flags[f]) % 4 != 0) return IMD_STATUS_MISALIGNED;
  }
  return imd::enqueue_push(dst, src, bytes, num_ranges, flags, num_flags, value, ctas > 0 ? ctas : 32,
                           stream);
}

/* The device error word copied to pinned host memory in stream order (extension; see the header). */
imd_status_t imd_device_error_peek(unsigned int* host_word, cudaStream_t stream) {
  if (host_word == nullptr) return IMD_STATUS_INVALID_VALUE;
  return imd::enqueue_error_peek(host_word, stream);
}

/* Extension: reads and clears the sticky device error word of the current device (bit 0 / 1: a
 * bounded wait inside the GEMM kernels gave up, bit 2: imd_wait_flags ran out). Synchronises the
 * device. */
IMD_API imd_status_t imd_device_error(unsigned int* word) {
  if (word == nullptr) return IMD_STATUS_INVALID_VALUE;
  unsigned int v = 0, zero = 0;
  unsigned int* p = imd::device_error_word();
  if (p == nullptr || cudaDeviceSynchronize() != cudaSuccess ||
      cudaMemcpy(&v, p, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess ||
      cudaMemcpy(p, &zero, sizeof zero, cudaMemcpyHostToDevice) != cudaSuccess) {
    cudaGetLastError();
    return IMD_STATUS_CUDA_ERROR;
  }
  *word = v;
  return IMD_STATUS_SUCCESS;
}

}  // extern "C"
