/* Device-side C ABI of the B200 contraction engine: libimmerdink.so (sm_100a).
 *
 *   C[I,J,L] <- alpha * sum_K A[I,K,L] * B[K,J,L] + beta * C[I,J,L]     (FP64 in, FP64 out)
 *
 * computed by Ozaki scheme II: exact power-of-two row/column scaling, int8 residues for N
 * coprime moduli, one int8 GEMM per modulus on tcgen05 tensor cores, exact CRT, one correctly
 * rounded conversion. Drop-in for the reference's include/immerdink/immerdink.h: the same twelve
 * entry points with the same argument meaning, check order and statuses; each declaration
 * names the reference declaration it replaces as "ref: immerdink.h:<line>".
 *
 * Contract shared by every entry point: status codes only (nothing throws); the caller owns
 * operands, output, workspace, packed buffers and the stream; imd_contract and imd_pack only
 * enqueue kernels (no allocation, no synchronisation, no write to the plan). */
#ifndef IMMERDINK_B200_H
#define IMMERDINK_B200_H

#include <stddef.h>
#include <stdint.h>

#include <cuda_runtime_api.h>

#include "immerdink/immerdink_host.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct imd_handle_st* imd_handle_t;
typedef struct imd_plan_st* imd_plan_t;
typedef struct imd_pack_s* imd_pack_t;

/* Library context, bound to the current device. ref: immerdink.h:28-29 */
IMD_API imd_status_t imd_create(imd_handle_t* handle);
IMD_API imd_status_t imd_destroy(imd_handle_t handle);

/* Lower the contraction, check legality and RN acceptance, and precompute everything the
 * kernels are launched with (including the function attributes of the tcgen05 GEMM and the
 * driver entry point used to encode TMA descriptors), so that imd_contract touches no global
 * state. With IMD_VEC_RESIDENT the plan owns device scatter vectors. ref: immerdink.h:35-38 */
IMD_API imd_status_t imd_plan_create(imd_handle_t handle, const imd_tensor_t* A,
                                     const imd_tensor_t* B, const imd_tensor_t* C,
                                     const imd_options_t* options, imd_plan_t* plan);
IMD_API imd_status_t imd_plan_destroy(imd_plan_t plan);

/* Device bytes owned by the plan (= imd_plan_bytes). ref: immerdink.h:43 */
IMD_API imd_status_t imd_plan_device_bytes(imd_plan_t plan, size_t* bytes);

/* Enqueue one contraction on `stream`. Checks, in order: null pointers (C always; A, B unless
 * alpha == 0 or k == 0; ws when the plan needs one) -> INVALID_VALUE; empty output -> SUCCESS;
 * ALIASING (byte intervals C/A, C/B, ws/A, ws/B, ws/C); MISALIGNED (8 bytes, ws 256);
 * ws_bytes < imd_workspace_size -> INSUFFICIENT_WORKSPACE. A failing call touches nothing.
 * One workspace serves one in-flight call. ref: immerdink.h:49-51 */
IMD_API imd_status_t imd_contract(imd_plan_t plan, double alpha, const double* A,
                                  const double* B, double beta, double* C, void* ws,
                                  size_t ws_bytes, cudaStream_t stream);

/* Packed operands: one operand scaled and reduced to all N residue planes once, reused by many
 * contractions. ref: immerdink.h:64-82, 89-92, 95-102, 119-121 */
IMD_API imd_status_t imd_pack_create(imd_handle_t handle, const imd_pack_desc_t* desc,
                                     imd_pack_t* pack);
IMD_API imd_status_t imd_pack_destroy(imd_pack_t pack);
IMD_API imd_status_t imd_pack_bytes(imd_pack_t pack, size_t* pack_bytes, size_t* pack_ws_bytes);
IMD_API imd_status_t imd_pack(imd_pack_t pack, const double* X, void* packed,
                              size_t packed_bytes, void* ws, size_t ws_bytes,
                              cudaStream_t stream);
IMD_API imd_status_t imd_plan_create_packed(imd_handle_t handle, const imd_tensor_t* A,
                                            const imd_tensor_t* B, const imd_tensor_t* C,
                                            const imd_options_t* options, imd_pack_t packA,
                                            imd_pack_t packB, imd_plan_t* plan);
typedef struct {
  const double* data;  /* the FP64 operand (native path of flagged outputs, DIRECT, in-line) */
  const void* packed;  /* imd_pack's output for a packed slot, else NULL */
  size_t packed_bytes;
  imd_pack_t pack;     /* packed slot: a handle with the plan's key; in-line slot: NULL */
} imd_operand_t;
IMD_API imd_status_t imd_contract_packed(imd_plan_t plan, double alpha, const imd_operand_t* A,
                                         const imd_operand_t* B, double beta, double* C,
                                         void* ws, size_t ws_bytes, cudaStream_t stream);

/* imd_contract without a caller-supplied workspace (no counterpart in the reference).
 *
 * For callers that cannot obtain device memory at the point of the call: a plugin running inside
 * a host application whose device memory pool is closed to cudaMalloc, or code on a
 * latency-critical path where a driver allocation (which may synchronise the whole device) is not
 * acceptable. The workspace is a fixed IMD_BUILTIN_WS_BYTES array inside the library image, so
 * every GPU that loads libimmerdink.so gives up that much memory until the process exits.
 *
 * Same checks in the same order, statuses and results as imd_contract given that array and its
 * size: a plan whose imd_workspace_size exceeds IMD_BUILTIN_WS_BYTES fails the size test at its
 * usual place (IMD_STATUS_INSUFFICIENT_WORKSPACE, nothing touched). The call allocates nothing,
 * neither directly nor through a library.
 *   - The first call on each device looks up the array's device address (the plan's device must be
 *     current, as for imd_contract); make that first call before any stream capture begins.
 *   - All calls on a device share the one array: two calls whose GPU work can overlap (different
 *     streams, or threads) race on it. Order them on one stream or with events.
 *   - The array keeps whatever the previous call left there. Nothing in it needs to start at zero:
 *     every byte a kernel reads is written earlier in the same call.
 *   - The looked-up address is cached per device for the life of the process; after a
 *     cudaDeviceReset the library must be reloaded before this entry point is used again. */
#define IMD_BUILTIN_WS_BYTES (32u << 20)
IMD_API imd_status_t imd_contract_builtin_ws(imd_plan_t plan, double alpha, const double* A,
                                             const double* B, double beta, double* C,
                                             cudaStream_t stream);

/* imd_pack of a PIECE of a slab for all consumers of the slab at once (no counterpart in the
 * reference; used by the multi-GPU driver, where the other destinations are peers' buffers mapped
 * into this process). The pack handle describes the piece X (r rows per batch); its rows land as
 * rows [row_offset, row_offset + r) of packed buffers whose batches have slab_rows rows, laid out
 * as imd_pack_layout describes that slab (same K, batches, N, rounding); every one of the
 * num_dest buffers (1..8) receives the same bytes by plain stores. dest[0] is the caller's own
 * buffer: its alignment gaps and tail are zeroed here. Checks: NULL pointers and ranges ->
 * INVALID_VALUE; an empty piece -> SUCCESS; X 8-byte, dest[] and ws 256-byte aligned -> else
 * MISALIGNED; dest_bytes below the slab's pack_bytes or ws_bytes below the piece's pack_ws_bytes
 * -> INSUFFICIENT_WORKSPACE. Enqueue only: no allocation, no synchronisation. */
IMD_API imd_status_t imd_pack_scatter(imd_pack_t piece, const double* X, int64_t slab_rows,
                                      int64_t row_offset, int32_t num_dest, void* const* dest,
                                      size_t dest_bytes, void* ws, size_t ws_bytes,
                                      cudaStream_t stream);

/* Bounded wait for data that arrives by copies from other GPUs (no counterpart in the reference;
 * used by the multi-GPU driver). A producer copies data into this GPU's memory and then, in the
 * same stream, a 32-bit value into a flag word next to it. This call enqueues on `stream` one
 * small kernel that polls the num_flags (0..32) words flags[i] (device addresses, read at the
 * call) until each holds `expect`; work enqueued on `stream` afterwards sees the announced data.
 * The wait is bounded: after max_polls polls of a flag (0 = the default, about a second) the
 * kernel gives up, sets bit 2 (value 4) of the device error word (imd_device_error) and
 * returns, so the stream always moves on. Checks: NULL -> INVALID_VALUE; num_flags outside 0..32
 * -> INVALID_VALUE; a flag address that is not 4-byte aligned -> MISALIGNED. */
IMD_API imd_status_t imd_wait_flags(const unsigned int* const* flags, int num_flags,
                                    unsigned int expect, uint64_t max_polls, cudaStream_t stream);

/* Copies that run only when a row is flagged (no counterpart in the reference; used by the
 * multi-GPU driver). The native path of non-finite rows is the only reader of a slab's FP64
 * values, so a rank fetches the other ranks' FP64 pieces only when a row flag of its packed slabs
 * is set. Enqueues one kernel on `stream`: if any byte of the num_ranges (0..4) ranges
 * flags[r][0 .. flag_bytes[r]) is nonzero, the num_copies (0..16) ranges src[c] -> dst[c] of
 * bytes[c] bytes are copied (sources may be peers' memory mapped into this process); else nothing
 * is touched. Checks: counts out of range, NULL arrays or NULL pointers of non-empty ranges ->
 * INVALID_VALUE; dst[c], src[c] or bytes[c] not a multiple of 8 (FP64 data) -> MISALIGNED. */
IMD_API imd_status_t imd_copy_if_flagged(const unsigned char* const* flags, const int64_t* flag_bytes,
                                         int32_t num_ranges, void* const* dst,
                                         const void* const* src, const int64_t* bytes,
                                         int32_t num_copies, cudaStream_t stream);

/* imd_contract_packed in parts (no counterpart in the reference; used by the multi-GPU driver to
 * start the GEMM of one residue group while the planes of the next are still arriving, and before
 * the FP64 operands of other GPUs have arrived).
 *   part 0       the whole call.
 *   part 1       everything except the outputs of the native path (outputs whose row of A or
 *                column of B holds a non-finite entry): those elements of C are left untouched
 *                and A->data, B->data are not read (they may be NULL).
 *   part 2       only those outputs, by the native path, from the shifts and flags already in
 *                the packed buffers (in-line operand: in the workspace); no GEMM runs.
 *   part 16 + i  only the GEMM of residue group i into the product planes of the workspace (for
 *                an in-line operand also its shifts, when i = 0, and its residues of the group).
 *   part 3       only the CRT of the emulated outputs, from the product planes in the workspace.
 * Parts 16 + i for every group in order, then 3, then 2, with the same arguments and workspace,
 * write exactly what part 0 writes; so do 1 then 2. Same checks as imd_contract_packed (the FP64
 * pointers are required by parts 0 and 2 only); an unknown part, a group index beyond the
 * plan's groups, or a part other than 0 on a plan whose call would not run the emulated GEMM ->
 * INVALID_VALUE. */
IMD_API imd_status_t imd_contract_packed_part(imd_plan_t plan, double alpha,
                                              const imd_operand_t* A, const imd_operand_t* B,
                                              double beta, double* C, void* ws, size_t ws_bytes,
                                              cudaStream_t stream, int32_t part);

/* Pushes by a small copy kernel (no counterpart in the reference; used by the multi-GPU driver).
 * Enqueues ONE kernel of `ctas` CTAs (0 = 32; at most 1024) on `stream` that copies the
 * num_ranges (0..96) ranges src[r] -> dst[r] of bytes[r] bytes with 16-byte loads and plain stores
 * (destinations may be other GPUs' memory mapped into this process) and then, when every CTA has
 * finished and fenced its stores at system scope, stores `value` into the num_flags (0..8) words
 * flags[f] (release, system scope): what imd_wait_flags on the consumer's side waits for. The few
 * CTAs run beside a persistent GEMM kernel on the same GPU. Checks: counts out of range, NULL
 * arrays or NULL pointers of non-empty ranges -> INVALID_VALUE; a range that is not 16-byte
 * granular or a flag that is not 4-byte aligned -> MISALIGNED. */
IMD_API imd_status_t imd_push_ranges(void* const* dst, const void* const* src, const int64_t* bytes,
                                     int32_t num_ranges, unsigned int* const* flags,
                                     int32_t num_flags, unsigned int value, int32_t ctas,
                                     cudaStream_t stream);

/* The sticky device error word (no counterpart in the reference: its kernels have no waits).
 * Every wait inside this library's kernels is bounded; one that gives up sets a bit of a word in
 * device memory and the kernel ends: bit 0 / bit 1 a barrier wait of the one-CTA / CTA-pair GEMM
 * kernel, bit 2 imd_wait_flags. Reads the word of the current device into *word and clears it.
 * Synchronises the device: a diagnostic, not part of a step. word == NULL -> INVALID_VALUE. */
IMD_API imd_status_t imd_device_error(unsigned int* word);
/* The same word copied into *host_word (pinned host memory) in stream order, without clearing it
 * and without synchronising: a driver that enqueues this at the end of every step sees, a step or
 * two later, that a bounded wait of that step gave up. host_word == NULL -> INVALID_VALUE. */
IMD_API imd_status_t imd_device_error_peek(unsigned int* host_word, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* IMMERDINK_B200_H */
