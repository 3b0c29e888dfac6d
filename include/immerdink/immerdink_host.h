/* Host-side (CUDA-free) C ABI of the B200 contraction engine: libimmerdink_host.so.
 *
 * Drop-in for the reference's include/immerdink/immerdink_host.h: same symbol names, struct
 * layouts, enum values and status precedence, so that callers compiled or bound (ctypes)
 * against the reference keep working. Each declaration names the reference declaration it
 * replaces as "ref: immerdink_host.h:<line>". The numbers these queries report (k_hat, n_hat,
 * workspace regions, launch counts) are the ones the sm_100a kernels of libimmerdink.so use.
 *
 * Pure functions: no GPU, no global state, thread-safe. */
#ifndef IMMERDINK_B200_HOST_H
#define IMMERDINK_B200_HOST_H

#include <stddef.h>
#include <stdint.h>

#define IMD_API __attribute__((visibility("default")))

#ifdef __cplusplus
extern "C" {
#endif

/* ref: immerdink_host.h:30 */
#define IMD_HOST_API_VERSION 13

/* ref: immerdink_host.h:65-79 */
typedef enum {
  IMD_STATUS_SUCCESS = 0,
  IMD_STATUS_INVALID_VALUE = 1,
  IMD_STATUS_NOT_SUPPORTED = 2,
  IMD_STATUS_ALIASING = 3,
  IMD_STATUS_INSUFFICIENT_WORKSPACE = 4,
  IMD_STATUS_MISALIGNED = 5,
  IMD_STATUS_CUDA_ERROR = 6,
  IMD_STATUS_ALLOC_FAILED = 7,
  IMD_STATUS_PACK_MISMATCH = 8
} imd_status_t;

/* ref: immerdink_host.h:82-102 */
enum { IMD_RN = 0, IMD_TRUNC = 1 };
enum { IMD_EMULATE = 0, IMD_DIRECT = 1 };
enum { IMD_VEC_GENERATE = 0, IMD_VEC_RESIDENT = 1 };
/* The reference's four mma.sync tile shapes. This engine has one tcgen05 tile pipeline; the
 * values are accepted and reported for compatibility and select nothing. */
enum { IMD_K4_128x256 = 0, IMD_K4_128x128 = 1, IMD_K4_64x128 = 2, IMD_K4_64x64 = 3,
       IMD_K4_CONFIG_COUNT = 4 };
enum { IMD_K4_TUNE_OFF = 0, IMD_K4_TUNE_ON = 1 };

/* Strided FP64 tensor view; strides in elements, any sign. ref: immerdink_host.h:107-112 */
typedef struct {
  int32_t rank;
  const int64_t* extent;
  const int64_t* stride;
  const int32_t* label;
} imd_tensor_t;

/* Zero-initialised = defaults; residue_group 0 means N. ref: immerdink_host.h:114-121 */
typedef struct {
  int32_t num_moduli;    /* N in 2..20 */
  int32_t residue_group; /* g: how many modulus planes of the operands are resident at once */
  int32_t rounding;      /* IMD_RN | IMD_TRUNC */
  int32_t mode;          /* IMD_EMULATE | IMD_DIRECT */
  int32_t vec_mode;      /* IMD_VEC_GENERATE | IMD_VEC_RESIDENT */
  int32_t k4_tune;       /* accepted, ignored (one GEMM pipeline) */
} imd_options_t;

/* ref: immerdink_host.h:124 */
IMD_API uint32_t imd_host_api_version(void);

/* Exact bytes imd_contract needs. Legality rows only, never the RN acceptance rule.
 * ref: immerdink_host.h:135 */
IMD_API imd_status_t imd_workspace_size(const imd_tensor_t* A, const imd_tensor_t* B,
                                        const imd_tensor_t* C, const imd_options_t* options,
                                        size_t* bytes);

/* Workspace regions, in this order; every offset 256-byte aligned; bytes 0 = absent.
 * ref: immerdink_host.h:140-154 */
enum {
  IMD_REGION_SA = 0,  /* int16 shift per A row         */
  IMD_REGION_SB = 1,  /* int16 shift per B column      */
  IMD_REGION_FA = 2,  /* u8 non-finite flag per A row  */
  IMD_REGION_FB = 3,  /* u8 non-finite flag per B col  */
  IMD_REGION_VEC = 4, /* int64 scatter vectors         */
  IMD_REGION_RA = 5,  /* int8 residue planes of A (one group) */
  IMD_REGION_RB = 6,  /* int8 residue planes of B (one group) */
  IMD_REGION_W = 7,   /* u8 product planes, all N      */
  IMD_REGION_COUNT = 8
};
typedef struct {
  uint64_t offset;
  uint64_t bytes;
} imd_region_t;

/* ref: immerdink_host.h:159 */
IMD_API imd_status_t imd_workspace_layout(const imd_tensor_t* A, const imd_tensor_t* B,
                                          const imd_tensor_t* C, const imd_options_t* options,
                                          imd_region_t* regions, int32_t capacity,
                                          int32_t* num_regions, size_t* total);
/* ref: immerdink_host.h:165 */
IMD_API const char* imd_region_name(int32_t region);

/* Plan-time status plus what a plan would own. ref: immerdink_host.h:175 */
IMD_API imd_status_t imd_plan_bytes(const imd_tensor_t* A, const imd_tensor_t* B,
                                    const imd_tensor_t* C, const imd_options_t* options,
                                    size_t* device_bytes, size_t* host_bytes);

/* ref: immerdink_host.h:185-186 */
enum { IMD_DISPATCH_NOOP = 0, IMD_DISPATCH_EMULATE = 1, IMD_DISPATCH_DIRECT = 2,
       IMD_DISPATCH_SCALE = 3 };

/* Lowering summary, versioned by struct_size (136, 152, 168, 176, 184, 192 bytes); the library
 * writes only the fields that fit. ref: immerdink_host.h:191-248. Kernel-dependent fields
 * describe THIS engine: n_hat = ceil(n)_16; k_hat = ceil(k)_A with A = k_align (64 iff
 * k > 96 else 16); gemm_launches = residue groups x K chunks (one batched tcgen05 launch
 * each); kernel_launches = every launch of one call; fused = 1 when the call is one fused
 * launch (k <= 128, no packed operand and at most 256 tiles of 32 x 32 outputs over all batches:
 * shifts, residues, int8 products and CRT inside one CTA per tile; kernel_launches is then 1,
 * plus the vectors' launch), fused_large is 0 (in the general sequence the quantise kernel is
 * always one fused scale+pack launch per operand and group); k4_config is
 * IMD_K4_128x256 (the 128 x 256 accumulator tile); k4_tune_bytes is 0. */
typedef struct {
  uint32_t struct_size;
  int32_t status;
  int32_t lowered;
  int32_t dispatch;
  int32_t swapped;
  int32_t num_moduli;
  int32_t residue_group;
  int32_t num_groups;
  int64_t m, n, k, b;
  int64_t n_hat, k_hat;
  int64_t vec_entries;
  int64_t k_chunks;
  int64_t gemm_launches;
  uint64_t kappa;
  uint64_t workspace_bytes;
  uint64_t plan_device_bytes;
  uint64_t plan_host_bytes;
  int32_t fused;
  int32_t reserved;
  int64_t kernel_launches;
  int32_t sm_count; /* in/out; 0 = 148 (B200) */
  int32_t k4_config;
  uint64_t k4_tune_bytes;
  int32_t fused_large;
  int32_t reserved4;
  int32_t packed;
  int32_t pack_mismatch;
  int32_t k_align;
  int32_t reserved6;
} imd_lowering_t;
enum { IMD_FUSED_LARGE_A = 1, IMD_FUSED_LARGE_B = 2 };

/* ref: immerdink_host.h:255 */
IMD_API imd_status_t imd_lowering(const imd_tensor_t* A, const imd_tensor_t* B,
                                  const imd_tensor_t* C, const imd_options_t* options,
                                  imd_lowering_t* out);

/* ref: immerdink_host.h:407 */
IMD_API const char* imd_status_string(imd_status_t status);

/* ---- Packed operands. ref: immerdink_host.h:259-404 -------------------------------------- */
#define IMD_PACK_FORMAT_A16 1
#define IMD_PACK_FORMAT_A64 2
#define IMD_PACK_FORMAT 2
enum { IMD_PACK_ORDER_AUTO = 0, IMD_PACK_ORDER_GIVEN = 1 };
enum {
  IMD_PACK_MISMATCH_NONE = 0,
  IMD_PACK_MISMATCH_FORMAT = 1,
  IMD_PACK_MISMATCH_MODULI = 2,
  IMD_PACK_MISMATCH_ROUNDING = 3,
  IMD_PACK_MISMATCH_CLASSES = 4,
  IMD_PACK_MISMATCH_EXTENTS = 5,
  IMD_PACK_MISMATCH_STRIDES = 6,
  IMD_PACK_MISMATCH_ORDER = 7
};
typedef struct {
  uint32_t struct_size;
  int32_t num_moduli;
  int32_t rounding;
  int32_t order;
  const imd_tensor_t* tensor;
  int32_t num_contracted;
  const int32_t* contracted;
  int32_t num_batch;
  const int32_t* batch;
  int32_t num_rows;
  const int32_t* rows;
} imd_pack_desc_t;
typedef struct {
  uint32_t struct_size;
  int32_t status;
  int32_t format;
  int32_t num_moduli, rounding;
  int32_t reserved;
  int64_t b, r, k, k_hat;
  uint64_t kappa;
  imd_region_t sig, flag, res;
  uint64_t pack_bytes;
  uint64_t pack_ws_bytes;
  uint64_t key_digest;
} imd_pack_layout_t;
typedef struct {
  const imd_pack_desc_t* A;
  const imd_pack_desc_t* B;
} imd_packing_t;

/* ref: immerdink_host.h:357, 369, 385, 389, 402 */
IMD_API imd_status_t imd_pack_layout(const imd_pack_desc_t* desc, imd_pack_layout_t* out);
IMD_API imd_status_t imd_pack_desc_for(const imd_tensor_t* A, const imd_tensor_t* B,
                                       const imd_tensor_t* C, const imd_options_t* options,
                                       int32_t operand, imd_pack_desc_t* out, int32_t* labels,
                                       int32_t capacity);
IMD_API imd_status_t imd_workspace_size_packed(const imd_tensor_t* A, const imd_tensor_t* B,
                                               const imd_tensor_t* C,
                                               const imd_options_t* options,
                                               const imd_packing_t* packing, size_t* bytes);
IMD_API imd_status_t imd_workspace_layout_packed(const imd_tensor_t* A, const imd_tensor_t* B,
                                                 const imd_tensor_t* C,
                                                 const imd_options_t* options,
                                                 const imd_packing_t* packing,
                                                 imd_region_t* regions, int32_t capacity,
                                                 int32_t* num_regions, size_t* total);
IMD_API imd_status_t imd_lowering_packed(const imd_tensor_t* A, const imd_tensor_t* B,
                                         const imd_tensor_t* C, const imd_options_t* options,
                                         const imd_packing_t* packing, imd_lowering_t* out);

/* ---- Error estimates. ref: immerdink_host.h:866-918 -------------------------------------- */
enum { IMD_ERR_NORMWISE = 0, IMD_ERR_ELEMENTWISE = 1, IMD_ERR_ABSOLUTE = 2 };
enum { IMD_ERR_BASIS_BOUND = 0, IMD_ERR_BASIS_TYPICAL = 1 };
enum { IMD_ERR_UNCHECKED = 0, IMD_ERR_MET = 1, IMD_ERR_MISSED = 2 };
typedef struct imd_err_request_s {
  uint32_t struct_size;
  int32_t metric;
  double target;
  double cond;
  double norm_product;
  double l1_ratio_a;
  double l1_ratio_b;
  int32_t basis;
  int32_t reserved;
  double fail_prob;
} imd_err_request_t;
typedef struct {
  uint32_t struct_size;
  int32_t status;
  int32_t num_moduli;
  int32_t rounding;
  int32_t dispatch;
  int32_t err_status;
  int64_t k;
  int64_t outputs;
  double bound;
  double typical;
  double unit_bound;
  double unit_typical;
} imd_err_t;
IMD_API imd_status_t imd_err_estimate(int32_t num_moduli, int32_t rounding, int32_t dispatch,
                                      int64_t k, int64_t outputs,
                                      const imd_err_request_t* request, imd_err_t* out);
IMD_API imd_status_t imd_err_min_moduli(const imd_tensor_t* A, const imd_tensor_t* B,
                                        const imd_tensor_t* C, const imd_options_t* options,
                                        int32_t n_lo, int32_t n_hi,
                                        const imd_err_request_t* request, imd_err_t* out);

/* ---- Performance model. ref: immerdink_host.h:409-839 ------------------------------------
 * Predicted time of one imd_contract / imd_pack per phase and in total, and a ranking of the
 * configurations a caller may choose (N, g, vec mode, packed operands) within a memory budget.
 * Struct layouts, enum values, function names, argument checks and the ranking order are the
 * reference's. The MODEL is this engine's: phases are its own kernels, the features x are
 * computed from the plan's lowering, and the shipped calibration (NULL) is a B200 (sm_100a) one.
 *   t_phase = sum_j param[class * 6 + j] * x[j]  (ns); GEMM class: max(terms j != 4, term j = 4).
 * Phase -> kernel of this engine (class):
 *   K0 "K0 vec"        k_vectors                        (k0: launch, byte)
 *   KL_A / KL_B        k_scale of the post-swap A / B   (kl: launch, byte, op = elements)
 *   PACK_A / PACK_B    k_residues of A / B, all groups  (pack: launch, byte, op = residues,
 *                                                        chain = quantisations)
 *   K4                 k_gemm_i8(_pair), all launches   (k4_128x256: round = tile rounds with a main
 *                                                        loop too short to hide the epilogue,
 *                                                        mac1 = MACs of the busiest SM in the
 *                                                        other rounds incl. tile padding,
 *                                                        byte = modelled DRAM bytes)
 *   K5                 k_crt                            (k5: launch, byte, op = outputs x N)
 *   DIRECT, BETA       k_direct, k_beta                 (direct: launch, byte, flop; beta)
 *   CALL               per call and per launch host / gap term
 *   PACK_PREP, PACK_KL, PACK_A   imd_pack: vectors + zero ranges, k_scale, k_residues (g = N)
 * Not modelled (accepted, validated, no effect): clock regimes and the power model (the
 * shipped calibration has power.cap_w = 0: SUSTAINED = BURST, power_w = 0), cache states
 * (warm_bytes = 0), the K4 configurations other than 128x256 (k4_config of a request is
 * validated and ignored: one GEMM kernel per shape class). Calibration text: format 2 only. */
#define IMD_PERF_CALIB_FORMAT 2
#define IMD_PERF_MAX_PARAMS 6
#define IMD_PERF_PARAM_CAPACITY 96
#define IMD_PERF_PARAM_KL_DROP_SLOT (IMD_PERF_PARAM_CAPACITY - 1)
#define IMD_PERF_MAX_PHASES 16
enum {
  IMD_PERF_CLASS_K0 = 0, IMD_PERF_CLASS_KF = 1, IMD_PERF_CLASS_KL = 2, IMD_PERF_CLASS_PACK = 3,
  IMD_PERF_CLASS_K4_128x256 = 4, IMD_PERF_CLASS_K4_128x128 = 5, IMD_PERF_CLASS_K4_64x128 = 6,
  IMD_PERF_CLASS_K4_64x64 = 7, IMD_PERF_CLASS_K5 = 8, IMD_PERF_CLASS_DIRECT = 9,
  IMD_PERF_CLASS_BETA = 10, IMD_PERF_CLASS_CALL = 11, IMD_PERF_CLASS_COUNT = 12
};
enum {
  IMD_PERF_PHASE_K0 = 0, IMD_PERF_PHASE_KF = 1, IMD_PERF_PHASE_KL_A = 2, IMD_PERF_PHASE_KL_B = 3,
  IMD_PERF_PHASE_PACK_A = 4, IMD_PERF_PHASE_PACK_B = 5, IMD_PERF_PHASE_K4 = 6,
  IMD_PERF_PHASE_K5 = 7, IMD_PERF_PHASE_DIRECT = 8, IMD_PERF_PHASE_BETA = 9,
  IMD_PERF_PHASE_CALL = 10, IMD_PERF_PHASE_PACK_PREP = 11, IMD_PERF_PHASE_PACK_KL = 12,
  IMD_PERF_PHASE_COUNT = 13
};
enum { IMD_PERF_BETA_NONZERO = 1, IMD_PERF_ALPHA_ZERO = 2 };
#define IMD_PERF_KERNEL_CAPACITY 128
#define IMD_PERF_CLASS_CAPACITY 16
enum {
  IMD_PERF_KERNEL_K0 = 0, IMD_PERF_KERNEL_KF16 = 1, IMD_PERF_KERNEL_KF4 = 2,
  IMD_PERF_KERNEL_KL8 = 3, IMD_PERF_KERNEL_KL4 = 4, IMD_PERF_KERNEL_PACK = 5,
  IMD_PERF_KERNEL_ZERO_ROWS = 6, IMD_PERF_KERNEL_DIRECT = 7, IMD_PERF_KERNEL_BETA = 8,
  IMD_PERF_KERNEL_PACK_PREP = 9, IMD_PERF_KERNEL_K4 = 10, IMD_PERF_KERNEL_K5 = 14,
  IMD_PERF_KERNEL_COUNT = 90
};
typedef struct {
  int32_t resident, regs, smem_bytes, threads;
} imd_perf_kernel_t;
enum { IMD_PERF_REGIME_DEFAULT = 0, IMD_PERF_REGIME_BURST = 1, IMD_PERF_REGIME_SUSTAINED = 2 };
enum { IMD_PERF_CACHE_COLD = 0, IMD_PERF_CACHE_WARM = 1, IMD_PERF_CACHE_REPEAT = 2,
       IMD_PERF_CACHE_CLEAN = 3 };
enum { IMD_PERF_ORDER_TIME = 0, IMD_PERF_ORDER_TIES_BY_FOOTPRINT = 1 };
enum { IMD_PERF_BAND_SMALL = 0, IMD_PERF_BAND_MID = 1, IMD_PERF_BAND_LARGE = 2 };
typedef struct {
  uint32_t struct_size;
  int32_t format;
  int32_t sm_count;
  int32_t reserved;
  double peak_dram_bytes_per_s, peak_int8_ops_per_s, peak_fp64_flops_per_s, l2_bytes;
  char gpu[64], date[32], version[64], clocks[128], notes[128];
  double param[IMD_PERF_PARAM_CAPACITY];
  imd_perf_kernel_t kernel[IMD_PERF_KERNEL_CAPACITY];
  double clock_eff_mhz, clock_min_mhz, power_cap_w, power_idle_w;
  double energy_tc_pj, energy_alu_pj, energy_byte_pj, energy_gamma;
  double warm_l2_bytes, warm_l2byte_ns;
  double band_call[3][2];
  double band_class[IMD_PERF_CLASS_CAPACITY][2];
  double tie_ratio;
  double energy_byte_f_pj;
  double pack_l2_hit_bytes;
  double clock_boost_mhz, power_act_w, power_act_gap_us, energy_dram_pj, warm_call_ns,
      warm_clean_byte_ns, pack_l2_planes;
} imd_perf_calib_t;
enum { IMD_PERF_CALIB_OK = 0, IMD_PERF_CALIB_ERR_ARGUMENT = 1, IMD_PERF_CALIB_ERR_FILE = 2,
       IMD_PERF_CALIB_ERR_SYNTAX = 3, IMD_PERF_CALIB_ERR_UNKNOWN_KEY = 4,
       IMD_PERF_CALIB_ERR_REPEATED_KEY = 5, IMD_PERF_CALIB_ERR_VALUE = 6,
       IMD_PERF_CALIB_ERR_TOO_LONG = 7, IMD_PERF_CALIB_ERR_MISSING_KEY = 8,
       IMD_PERF_CALIB_ERR_FORMAT2_KEY = 9, IMD_PERF_CALIB_ERR_INCONSISTENT = 10 };
#define IMD_PERF_CALIB_ERR_COUNT 11
typedef struct {
  uint32_t struct_size;
  int32_t line, reason, reserved;
  char key[64];
  char message[192];
} imd_perf_calib_error_t;
typedef struct {
  uint32_t struct_size;
  int32_t flags, k4_config, reserved;
  double eps_fraction;
  int32_t regime, cache;
  double clock_mhz;
  const struct imd_err_request_s* accuracy;
} imd_perf_request_t;
typedef struct {
  int32_t phase, cls;
  int64_t launches;
  double time_s, bytes, ops, bound_s;
  double x[IMD_PERF_MAX_PARAMS];
} imd_perf_phase_t;
typedef struct {
  uint32_t struct_size;
  int32_t status, dispatch, k4_config, sm_count, num_phases;
  double time_s, bound_s, flops_eq, tflops_eq, eps_s, eps_fraction;
  int64_t kernel_launches;
  uint64_t workspace_bytes, plan_device_bytes, pack_bytes, pack_ws_bytes;
  imd_perf_phase_t phase[IMD_PERF_MAX_PHASES];
  int32_t regime, cache;
  double clock_mhz, power_w, warm_bytes, time_lo_s, time_hi_s;
  double phase_lo_s[IMD_PERF_MAX_PHASES], phase_hi_s[IMD_PERF_MAX_PHASES];
  double err_bound, err_typical;
  int32_t err_status, err_metric;
} imd_perf_t;
enum { IMD_PERF_VEC_GENERATE = 1, IMD_PERF_VEC_RESIDENT = 2 };
enum { IMD_PERF_PACK_NONE = 1, IMD_PERF_PACK_A = 2, IMD_PERF_PACK_B = 4, IMD_PERF_PACK_AB = 8 };
typedef struct {
  uint32_t struct_size, candidate_size;
  int32_t num_moduli_count, residue_group_count;
  const int32_t* num_moduli;
  const int32_t* residue_groups;
  int32_t vec_modes, pack_modes, reuse, flags;
  uint64_t budget_bytes;
  double eps_fraction;
  int32_t regime, cache, order, reserved;
  double clock_mhz;
  const struct imd_err_request_s* accuracy;
} imd_perf_rank_request_t;
typedef struct {
  int32_t num_moduli, residue_group, vec_mode, packed, status, feasible, k4_config, dispatch;
  double time_s, contract_s, pack_s, tflops_eq, eps_s, eps_fraction;
  uint64_t workspace_bytes, plan_device_bytes, pack_bytes, pack_ws_bytes, total_bytes;
  int64_t kernel_launches;
  double time_lo_s, time_hi_s, clock_mhz, power_w;
  int32_t tie, raw_rank;
  double err_bound, err_typical;
  int32_t err_status, infeasible;
} imd_perf_candidate_t;
enum { IMD_PERF_INFEASIBLE_STATUS = 1, IMD_PERF_INFEASIBLE_BUDGET = 2,
       IMD_PERF_INFEASIBLE_ACCURACY = 4 };
IMD_API const char* imd_perf_kernel_name(int32_t kernel);
IMD_API imd_status_t imd_perf_calib_default(imd_perf_calib_t* out);
IMD_API imd_status_t imd_perf_calib_parse(const char* text, size_t length, imd_perf_calib_t* out,
                                          int32_t* error_line);
IMD_API imd_status_t imd_perf_calib_load(const char* path, imd_perf_calib_t* out,
                                         int32_t* error_line);
IMD_API imd_status_t imd_perf_calib_parse_ex(const char* text, size_t length,
                                             imd_perf_calib_t* out, imd_perf_calib_error_t* err);
IMD_API imd_status_t imd_perf_calib_load_ex(const char* path, imd_perf_calib_t* out,
                                            imd_perf_calib_error_t* err);
IMD_API imd_status_t imd_perf_calib_default_ex(imd_perf_calib_t* out,
                                               imd_perf_calib_error_t* err);
IMD_API const char* imd_perf_calib_error_name(int32_t reason);
IMD_API imd_status_t imd_perf_calib_format(const imd_perf_calib_t* calib, char* buf,
                                           size_t capacity, size_t* length);
IMD_API const char* imd_perf_class_name(int32_t cls);
IMD_API const char* imd_perf_param_name(int32_t cls, int32_t j);
IMD_API const char* imd_perf_phase_name(int32_t phase);
IMD_API imd_status_t imd_perf_predict(const imd_tensor_t* A, const imd_tensor_t* B,
                                      const imd_tensor_t* C, const imd_options_t* options,
                                      const imd_packing_t* packing,
                                      const imd_perf_request_t* request,
                                      const imd_perf_calib_t* calib, imd_perf_t* out);
IMD_API imd_status_t imd_perf_predict_pack(const imd_pack_desc_t* desc,
                                           const imd_perf_request_t* request,
                                           const imd_perf_calib_t* calib, imd_perf_t* out);
IMD_API imd_status_t imd_perf_rank(const imd_tensor_t* A, const imd_tensor_t* B,
                                   const imd_tensor_t* C, const imd_options_t* base,
                                   const imd_perf_rank_request_t* request,
                                   const imd_perf_calib_t* calib, imd_perf_candidate_t* out,
                                   int32_t capacity, int32_t* num_candidates);

#ifdef __cplusplus
}
#endif
#endif /* IMMERDINK_B200_HOST_H */
