// The verification / tuning knobs and the phase timer, in two flavours of one source file:
//
//   without IMD_HOOKS  (libimmerdink.so, the production library)  hooks() returns a constant
//        copy of the defaults and phase_mark() does nothing: no entry point can change how
//        imd_contract runs, and imd_contract reads or writes no mutable process state.
//   with IMD_HOOKS     (libimmerdink_hooks.so, loaded by the tests and for phase timing)  the
//        knobs are mutable through imd_test_*, and imd_prof_* records CUDA events at the phase
//        boundaries of every call (one caller at a time: the event pool is process-global).
//
// The reference gates its own test entry points the same way (CMakeLists.txt:33-34, 134-141).
#include <cstddef>
#include <vector>

#include <cuda_runtime_api.h>

#include "kernels.hpp"

namespace imd {

#ifndef IMD_HOOKS

const Hooks& hooks() {
  static const Hooks defaults{};
  return defaults;
}
void phase_mark(int, cudaStream_t) {}

#else

namespace {
Hooks g_hooks;
struct PhaseProfile {
  std::vector<cudaEvent_t> events;
  std::vector<int> tags;
  size_t used = 0;
  bool on = false;
} g_prof;
}  // namespace

const Hooks& hooks() { return g_hooks; }

void phase_mark(int tag, cudaStream_t stream) {
  if (!g_prof.on || g_prof.used >= g_prof.events.size()) return;
  cudaEventRecord(g_prof.events[g_prof.used], stream);
  g_prof.tags[g_prof.used++] = tag;
}

#endif

}  // namespace imd

#ifdef IMD_HOOKS
extern "C" {

/* 1: run the slow exact int8 GEMM instead of the tensor-core kernel in later calls (cross-check). */
IMD_API int imd_test_use_reference_gemm(int on) {
  imd::g_hooks.reference_gemm = on != 0;
  return 0;
}
/* 0 = GEMM kernel chosen by shape, 1 = one CTA per 128 x 256 tile, 2 = CTA pairs on 256 x 256. */
IMD_API int imd_test_gemm_variant(int v) {
  imd::g_hooks.gemm_variant = v;
  return 0;
}
IMD_API int imd_test_gemm_band_mb(int mb) {
  if (mb > 0) imd::g_hooks.gemm_band_mb = mb;
  return imd::g_hooks.gemm_band_mb;
}
IMD_API int imd_test_gemm_l2_hints(int on) {
  if (on >= 0) imd::g_hooks.gemm_l2_hints = on;
  return imd::g_hooks.gemm_l2_hints;
}
/* 1: later calls compute every shift from the exact 128-bit sum of squares (no FP64 shortcut). */
IMD_API int imd_test_force_exact_shift(int on) {
  imd::g_hooks.force_exact_shift = on != 0;
  return 0;
}
/* 1: later calls run every output through the integer CRT (no FP64 shortcut). */
IMD_API int imd_test_force_exact_crt(int on) {
  imd::g_hooks.force_exact_crt = on != 0;
  return 0;
}
/* 0: later calls run small contractions through the general kernel sequence (whose intermediate
 * results the tests read from the workspace) instead of the one fused launch; 1: as in production. */
IMD_API int imd_test_small_path(int on) {
  imd::g_hooks.small_path = on != 0;
  return 0;
}
/* The device error word, read and cleared (imd_device_error without the status). */
IMD_API unsigned int imd_test_device_error(void) {
  unsigned int v = 0;
  return imd_device_error(&v) == IMD_STATUS_SUCCESS ? v : 0xFFFFFFFFu;
}
/* Measured ceiling of the int8 tensor pipe (ops/s) for the GEMM's tile shapes. */
IMD_API double imd_prof_mma_peak(int pair) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
    return 0.0;
  return imd::mma_probe_tops(pair, sms);
}
/* Phase timing: enable with an event capacity (0 disables); read sums the milliseconds per phase
 * tag since the last read: ms_by_tag[t] += time of every segment that ENDS with an event tagged t
 * (tag 0 opens a call). Returns the segments read. */
IMD_API int imd_prof_enable(int capacity) {
  using imd::g_prof;
  for (cudaEvent_t e : g_prof.events) cudaEventDestroy(e);
  g_prof = imd::PhaseProfile{};
  if (capacity <= 0) return 0;
  g_prof.events.resize(static_cast<size_t>(capacity));
  g_prof.tags.assign(static_cast<size_t>(capacity), 0);
  for (cudaEvent_t& e : g_prof.events)
    if (cudaEventCreate(&e) != cudaSuccess) return 1;
  g_prof.on = true;
  return 0;
}
IMD_API int imd_prof_read(float* ms_by_tag, int tags) {
  using imd::g_prof;
  if (!g_prof.on || g_prof.used == 0) return 0;
  cudaEventSynchronize(g_prof.events[g_prof.used - 1]);
  int n = 0;
  for (size_t i = 1; i < g_prof.used; ++i) {
    const int t = g_prof.tags[i];
    if (t <= 0 || t >= tags) continue;
    float ms = 0;
    if (cudaEventElapsedTime(&ms, g_prof.events[i - 1], g_prof.events[i]) == cudaSuccess) {
      ms_by_tag[t] += ms;
      ++n;
    }
  }
  g_prof.used = 0;
  return n;
}

}  // extern "C"
#endif
