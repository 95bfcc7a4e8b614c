/*
 * ra_spmm_b200.h - C ABI of libra_spmm_b200.so
 *
 * B200 (sm_100a) implementation of the RA-SpMM hot path: the O(M) router
 * feature scan, the seven-rule router, and the five SpMM kernel families
 * (CSR_DIRECT, ZERO_OVERHEAD_CSR, TC_DIRECT, COMMUNITY_TC, SEGMENT_HYBRID with
 * FP16 and TF32 paths) together with their plan builders.
 *
 * Conventions
 *  - every entry point returns an int status (RA_OK == 0); nothing throws
 *    across the boundary; ra_last_error_string() describes the last failure
 *    on the calling thread;
 *  - pointers named d_* are device pointers on the current CUDA device,
 *    h_* are host pointers; `stream` is a cudaStream_t passed as void*
 *    (NULL = the legacy default stream);
 *  - indices are int32, values/B/C are row-major float32 unless stated;
 *  - plan handles own device memory obtained with cudaMalloc and must be
 *    destroyed with the matching *_destroy call; a plan holds lazily grown
 *    scratch, so one plan must not run concurrently on two streams (same
 *    rule as the reference plans, ra_common.h:607-609,704-708).
 *
 * Each declaration cites the reference interface it replaces, by the file's
 * path inside the RA-SpMM project.
 */
#ifndef RA_SPMM_B200_H
#define RA_SPMM_B200_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RA_API __attribute__((visibility("default")))

/* ---- status codes ------------------------------------------------------ */
enum {
    RA_OK                = 0,
    RA_ERR_INVALID_ARG   = 1,  /* null pointer, negative size, bad enum      */
    RA_ERR_CUDA          = 2,  /* a CUDA runtime call failed                 */
    RA_ERR_UNSUPPORTED   = 3,  /* shape outside what the kernel supports     */
    RA_ERR_INACTIVE_PLAN = 4,  /* tile plan built with N<16 or nnz==0        */
    RA_ERR_ALIGNMENT     = 5,  /* device pointer not 16-byte aligned         */
    RA_ERR_TOO_LARGE     = 6   /* exceeds a documented fixed capacity        */
};

/* ---- kernel identifiers: values of NextPath, ra_common.h:76-95 --------- */
enum {
    RA_PATH_CSR_DIRECT        = 0,
    RA_PATH_CSR_ADAPTIVE      = 1,
    RA_PATH_STAGED_REUSE      = 2,
    RA_PATH_TC_SPARSE         = 3,
    RA_PATH_ROW_SPLIT_CUDA    = 4,
    RA_PATH_TC_REORDERED      = 5,
    RA_PATH_HYBRID_TC_CUDA    = 6,
    RA_PATH_CUSPARSE          = 7,
    RA_PATH_RODE_ENHANCED     = 8,
    RA_PATH_VECTORIZED_COARSE = 9,
    RA_PATH_LOCALITY_TILED    = 10,
    RA_PATH_TC_DIRECT         = 11,
    RA_PATH_COMMUNITY_TC      = 12,
    RA_PATH_ZERO_OVERHEAD_CSR = 13,
    RA_PATH_SEGMENT_HYBRID    = 14,
    RA_PATH_COUNT             = 15
};

enum { RA_PORTFOLIO_MAIN = 0 };

/* RA_TILE_TC_DIRECT_ZC: TC_DIRECT with zero-compressed block values (make_ra_tc_direct_zc_plan,
 * tc/ra_tc_direct.cu:792-800): per block a 64-bit occupancy mask, the offset of its first
 * stored value, and the stored fp16 values only, instead of 64 padded halves per block. */
enum { RA_TILE_TC_DIRECT = 0, RA_TILE_COMMUNITY_TC = 1, RA_TILE_SEGMENT_HYBRID = 2,
       RA_TILE_TC_DIRECT_ZC = 3 };
enum { RA_PRECISION_FP16 = 0, RA_PRECISION_TF32 = 1 };
enum { RA_DTYPE_F32 = 0, RA_DTYPE_F16 = 1 };

/* Production router features: the fields of RouterFeatures (ra_common.h:185-231)
 * that compute_production_router_features fills; the remaining 27 floats of the
 * reference struct stay zero on the MAIN portfolio. */
typedef struct RaFeatures {
    float   avg_nnz_per_row;
    float   std_nnz_per_row;
    float   degree_cv;
    int32_t output_dim_N;
    int32_t matrix_M;
    int32_t matrix_K;
    int32_t total_nnz;
    /* exact integer moments behind the floats (device scan only; 0 on host) */
    uint64_t sum_deg;
    uint64_t sum_deg_sq;
} RaFeatures;

/* Routing decision: the RouterPlan fields (ra_common.h:250-268) that the
 * seven-rule block of route_dispatch determines. */
typedef struct RaRoute {
    int32_t chosen_path;                 /* RA_PATH_*                         */
    int32_t use_tf32;                    /* 0/1                               */
    float   estimated_risk;
    uint8_t feasible[RA_PATH_COUNT];     /* indexed by RA_PATH_*              */
    char    decision_reason[64];         /* NUL-terminated                    */
} RaRoute;

/* ---- diagnostics ------------------------------------------------------- */
RA_API const char* ra_last_error_string(void);
RA_API const char* ra_path_name(int path);      /* next_path_name, ra_common.h:116-136 */
RA_API int  ra_version(void);
/* Blocking device-to-host copy of `bytes` bytes (synchronises the device first);
 * lets a host language without a CUDA binding read back the plan arrays that
 * the *_info calls expose. No counterpart in the reference, whose plan arrays
 * are not readable from Python. */
RA_API int  ra_copy_to_host(void* h_dst, const void* d_src, size_t bytes);
/* 64-bit FNV-1a over a host buffer: byte-identity checksums of plan arrays (the
 * RA_PLAN_CHECKSUM hook that the reference's experiments/verify_format_checksums.py
 * expects but the reference does not implement). */
RA_API uint64_t ra_fnv1a64_host(const void* h_data, size_t bytes);

/* ---- router features ---------------------------------------------------
 * Replaces compute_production_router_features (router/router_features.cpp:79-111):
 * two-pass host formula, serial summation order. */
RA_API int ra_features_from_rowptr_host(const int32_t* h_rowptr, int M, int K, int N,
                                        RaFeatures* out);
/* Replaces compute_production_router_features_gpu + row_degree_moments_kernel
 * (router/router_features_cuda.cu:13-92): exact integer moments on the device,
 * one-pass host finish. Blocks until the 16-byte result is on the host. */
RA_API int ra_features_from_rowptr_device(const int32_t* d_rowptr, int M, int K, int N,
                                          void* stream, RaFeatures* out);

/* ---- router ------------------------------------------------------------
 * Replaces route_dispatch's feasibility table and seven-rule block
 * (router/router_dispatch.cpp:107-464, 979-1110) for the MAIN portfolio. */
RA_API int ra_route(const RaFeatures* features, int portfolio, RaRoute* out);

/* Diagnostic half of the decision dict: compute_router_scores (router/router_scores.cpp:27-86)
 * and the per-path rejection code / text that compute_feasible and the legacy selection stage
 * of route_dispatch leave behind (router/router_dispatch.cpp:107-464, 668-966), as plan_to_dict
 * publishes them (bindings/ra_bindings.cpp:650-716). MAIN portfolio only. `route` is the result
 * of ra_route for the same features. */
typedef struct RaRouteDetails {
    float   scores[8];   /* csr_direct, csr_adaptive, staged_reuse, tc_sparse, row_split_cuda,
                            tc_reordered, hybrid_tc_cuda, cusparse                           */
    int32_t rejection_code[RA_PATH_COUNT];          /* RejectReason, ra_common.h:146-160     */
    char    rejection_detail[RA_PATH_COUNT][128];   /* NUL-terminated                        */
    float   gate_margin_raw, gate_margin_norm;
} RaRouteDetails;
RA_API int ra_route_details(const RaFeatures* features, int portfolio, const RaRoute* route,
                            RaRouteDetails* out);
RA_API const char* ra_reject_reason_name(int code);   /* reject_reason_str, ra_common.h:162-179 */

/* ---- structural analysis (the 34 features of the research portfolio) ------------------
 * Replaces compute_router_features (router/router_features.cpp:113-432) as the binding
 * analyze_matrix publishes it (bindings/ra_bindings.cpp:1993-2051): degree statistics, fill
 * statistics of the nonempty 16x16 tiles, 64-bucket column signatures of the rows and the
 * locality / partition proxies derived from them over 16-row windows. Field names, order and
 * arithmetic are the reference's (RouterFeatures, ra_common.h:185-231); every field is
 * bit-exact with it on duplicate-free CSR. The O(nnz) parts (tile counts by radix sort, per-row
 * column sums and signatures, the proxy row order) run on the device and produce integers
 * only; the order-sensitive floating-point reductions over rows and windows run on the host in
 * the reference's order. rowptr/colind: host or device pointers (on_device). Blocks until the
 * result is on the host. RA_ERR_UNSUPPORTED when a 16x16 tile holds more than 256 entries
 * (duplicate (row, column) pairs). */
typedef struct RaMatrixAnalysis {
    float avg_nnz_per_row, std_nnz_per_row, degree_cv, max_to_mean_ratio, frac_dense_rows,
          skew_ratio, long_row_fraction, long_row_nnz_fraction, top_1_row_nnz_fraction,
          top_5_row_nnz_fraction;
    float tile_fill_mean, tile_fill_median, tile_fill_p90, tile_fill_max, tile_fill_variance,
          tile_occupancy, actual_nnz_coverage, avg_nnz_per_tile, row_window_colspan_compactness,
          local_row_similarity_proxy, reordered_locality_proxy, locality_gain_proxy,
          locality_selectivity_proxy, road_likeness_proxy, row_split_affinity_proxy,
          mixedness_proxy;
    float tc_candidate_ratio, tc_synergy_proxy, estimated_tc_partition_ratio,
          estimated_cuda_partition_ratio, irregular_window_fraction, tc_granularity_proxy,
          redundancy_risk_proxy;
    int32_t tc_candidate_tiles;
    int32_t output_dim_N, matrix_M, matrix_K, total_nnz;
} RaMatrixAnalysis;
RA_API int ra_analyze_matrix(const int32_t* rowptr, const int32_t* colind, int on_device,
                             int M, int K, int N, void* stream, RaMatrixAnalysis* out);

/* ---- CSR_DIRECT --------------------------------------------------------
 * Replaces csr_direct_spmm (csr/csr_direct.cu:234-338). C is fully overwritten
 * (empty rows become zero rows). */
RA_API int ra_csr_direct_spmm(const int32_t* d_rowptr, const int32_t* d_colind,
                              const float* d_vals, const float* d_B, float* d_C,
                              int M, int K, int N, int64_t nnz, void* stream);

/* ---- ZERO_OVERHEAD_CSR -------------------------------------------------
 * Replaces make/run/free_ra_zero_overhead_plan (csr/ra_zero_overhead.cu:312-519)
 * and RAZeroOverheadPlan (ra_common.h:507-530). The plan is built on the
 * device; rowptr may live on the host or on the device. */
typedef struct RaZoPlan RaZoPlan;

typedef struct RaZoInfo {
    int32_t M, K;
    int32_t num_tiny, num_short, num_medium, num_long, num_empty;
    int32_t num_small, num_chunks, num_zero_rows, max_long_chunks;
    int64_t plan_bytes;
    /* device arrays with the contents and order of the reference plan */
    const int32_t* d_small_row_ids;   /* [num_small]     */
    const int32_t* d_chunk_rows;      /* [num_chunks]    */
    const int32_t* d_chunk_starts;    /* [num_chunks]    */
    const int32_t* d_zero_row_ids;    /* [num_zero_rows] */
} RaZoInfo;

RA_API int ra_zo_plan_create(const int32_t* rowptr, int rowptr_on_device, int M, int K,
                             void* stream, RaZoPlan** out);
RA_API int ra_zo_plan_info(const RaZoPlan* plan, RaZoInfo* out);
RA_API int ra_zo_plan_run(RaZoPlan* plan, const int32_t* d_rowptr, const int32_t* d_colind,
                          const float* d_vals, const float* d_B, float* d_C, int N,
                          void* stream);
RA_API int ra_zo_plan_destroy(RaZoPlan* plan);
/* Diagnostics: run a subset of the three phases of ra_zo_plan_run so each can
 * be timed on its own (bit 0 long-row chunks, bit 1 small rows, bit 2 finish =
 * merge of multi-chunk rows + zero rows). Bits 0 and 1 together run as the one
 * launch that ra_zo_plan_run uses for both at N in {32,64,128,256,512}. The
 * reference has no counterpart; its three launches are
 * csr/ra_zero_overhead.cu:411-502. Mask 7 == run. */
RA_API int ra_zo_plan_run_phases(RaZoPlan* plan, const int32_t* d_rowptr, const int32_t* d_colind,
                                 const float* d_vals, const float* d_B, float* d_C, int N,
                                 int phase_mask, void* stream);

/* Same result as ra_zo_plan_run, for callers that cannot allocate device memory
 * while they run (HBM fully handed to their own pool, or a cudaMalloc would stall
 * streams that are in flight). It calls no cudaMalloc / cudaFree: the partial rows
 * of multi-chunk long rows go to a 16 MiB array built into the library, which
 * every GPU that loads the library keeps until the process exits.
 *   - limit: (chunks of rows longer than 256 nonzeros) x N <= 4,194,304 floats;
 *     larger plans get RA_ERR_TOO_LARGE and a message naming the sizes;
 *   - the first call on each device looks up the array's device address (that
 *     device must be current); make that first call before any stream capture;
 *   - all calls on a device share the one array: two calls that overlap on the
 *     GPU (different streams) race. Nothing in it has to start at zero - every
 *     slot a plan uses is rewritten by each call before it is read.
 * This entry point has no counterpart in the reference. */
RA_API int ra_zo_plan_run_noalloc(RaZoPlan* plan, const int32_t* d_rowptr, const int32_t* d_colind,
                                  const float* d_vals, const float* d_B, float* d_C, int N,
                                  void* stream);

/* ---- tile plans: TC_DIRECT / COMMUNITY_TC / SEGMENT_HYBRID -------------
 * Replace make_ra_tc_direct_plan (tc/ra_tc_direct.cu:627-790),
 * make_ra_community_tc_plan (tc/ra_community_tc.cu:320-471),
 * make_ra_segment_hybrid_plan (tc/ra_segment_hybrid.cu:371-543) and the
 * matching run_*_plan / run_*_plan_tf32 / free_*_plan. The CSR may live on
 * the host or on the device; the build runs on the device. */
typedef struct RaTilePlan RaTilePlan;

typedef struct RaTileInfo {
    int32_t kind;            /* RA_TILE_*                                   */
    int32_t active;          /* 0 when N<16 or nnz==0 (no arrays)           */
    int32_t M, K;
    int32_t num_windows;
    int64_t num_blocks;      /* num_tc_tiles                                */
    int64_t nnz;
    float   tile_density;    /* nnz / (vectors*8)                           */
    int64_t plan_bytes;
    const int32_t*  d_block_offsets;  /* [num_windows+1]                    */
    const int32_t*  d_atox;           /* [8*num_blocks]                     */
    const uint16_t* d_vals_f16;       /* [64*num_blocks], fragment order    */
    const int32_t*  d_win_rows;       /* COMMUNITY_TC: [8*num_windows]      */
    /* SEGMENT_HYBRID */
    int32_t num_segments, num_split_segs, num_split_windows, num_zero_rows;
    const int32_t* d_seg_window;      /* [num_segments]                     */
    const int32_t* d_seg_bbegin;      /* [num_segments]                     */
    const int32_t* d_seg_bend;        /* [num_segments]                     */
    const int32_t* d_seg_scratch;     /* [num_segments]                     */
    const int32_t* d_split_wins;      /* [num_split_windows]                */
    const int32_t* d_split_off;       /* [num_split_windows+1]              */
    const int32_t* d_zero_rows;       /* [num_zero_rows]                    */
    /* TC_DIRECT_ZC (d_vals_f16 is null): bit k*8+r of a mask = (vector k, window row r) stored;
     * its value sits at base + number of set mask bits below it */
    const uint64_t* d_val_masks;      /* [num_blocks]                       */
    const int32_t*  d_val_base;       /* [num_blocks]                       */
    const uint16_t* d_vals_zc;        /* [nnz], (window, column, row) order */
} RaTileInfo;

RA_API int ra_tile_plan_create(int kind, const int32_t* rowptr, const int32_t* colind,
                               const float* vals, int csr_on_device,
                               int M, int K, int N, void* stream, RaTilePlan** out);
RA_API int ra_tile_plan_info(const RaTilePlan* plan, RaTileInfo* out);
/* precision: RA_PRECISION_FP16 (B rounded to fp16, RNE) or RA_PRECISION_TF32
 * (B rounded to tf32, ties away). b_dtype: RA_DTYPE_F32, or RA_DTYPE_F16 to
 * hand over an fp16 B directly (FP16 precision only). C is float32 [M,N].
 * Every plan kind runs through this call (a zero-compressed TC_DIRECT plan is
 * decoded inside the kernels). The plan's lazily grown scratch (fp16 copy of B,
 * partial tiles of split segments and of windows shared between groups of the
 * TMA ring) makes a plan unsafe for two concurrent runs, as in the reference
 * (ra_common.h:607-609, 704-708); it grows (cudaMalloc) on the first run at a
 * given width, so make that run before any stream capture. */
RA_API int ra_tile_plan_run(RaTilePlan* plan, int precision, const void* d_B, int b_dtype,
                            float* d_C, int N, void* stream);
RA_API int ra_tile_plan_destroy(RaTilePlan* plan);
/* Device status word of the plan's kernels (synchronises the device): 0 = ok; non-zero = a
 * bounded wait inside a kernel gave up (1 = a stage of the bulk-copy ring never filled,
 * 3 = a tensor-core commit never arrived) and the output of that run is not valid. Reading a
 * non-zero status clears it. The reference kernels have no waits and no counterpart. */
RA_API int ra_tile_plan_device_status(RaTilePlan* plan, int* status);

/* ---- plan files ----------------------------------------------------------
 * A built plan written to a file and read back in another process. The reference keeps its
 * plans (ra_common.h:507-530, 593-719) in memory only and rebuilds them per process; its
 * experiments/verify_format_checksums.py compares per-array checksums of the formats across
 * runs. The file stores every plan array with its length and 64-bit FNV-1a checksum; *_load
 * recomputes the checksums while uploading and fails (RA_ERR_INVALID_ARG, nothing returned)
 * on a truncated or altered file. Lazily grown scratch is not part of the file. */
RA_API int ra_zo_plan_save(const RaZoPlan* plan, const char* path);
RA_API int ra_zo_plan_load(const char* path, RaZoPlan** out);
RA_API int ra_tile_plan_save(const RaTilePlan* plan, const char* path);
RA_API int ra_tile_plan_load(const char* path, RaTilePlan** out);

#ifdef __cplusplus
}
#endif
#endif /* RA_SPMM_B200_H */
