"""ctypes binding of libra_spmm_b200.so (the C ABI declared in include/ra_spmm_b200.h).

The library is the product: importing this module fails loudly when the shared
object has not been built, and nothing in the package computes on the CPU in
its place.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "libra_spmm_b200.so"

RA_OK = 0
PATH_NAMES = [
    "CSR_DIRECT", "CSR_ADAPTIVE", "STAGED_REUSE", "TC_SPARSE", "ROW_SPLIT_CUDA",
    "TC_REORDERED", "HYBRID_TC_CUDA", "CUSPARSE", "RODE_ENHANCED", "VECTORIZED_COARSE",
    "LOCALITY_TILED", "TC_DIRECT", "COMMUNITY_TC", "ZERO_OVERHEAD_CSR", "SEGMENT_HYBRID",
]
PATH_COUNT = len(PATH_NAMES)
TILE_TC_DIRECT, TILE_COMMUNITY_TC, TILE_SEGMENT_HYBRID, TILE_TC_DIRECT_ZC = 0, 1, 2, 3
PRECISION_FP16, PRECISION_TF32 = 0, 1
DTYPE_F32, DTYPE_F16 = 0, 1

# Every symbol include/ra_spmm_b200.h declares.
EXPORTED_SYMBOLS = [
    "ra_last_error_string", "ra_path_name", "ra_version", "ra_copy_to_host", "ra_fnv1a64_host",
    "ra_features_from_rowptr_host", "ra_features_from_rowptr_device", "ra_route",
    "ra_route_details", "ra_reject_reason_name", "ra_analyze_matrix",
    "ra_csr_direct_spmm",
    "ra_zo_plan_create", "ra_zo_plan_info", "ra_zo_plan_run", "ra_zo_plan_destroy",
    "ra_zo_plan_run_phases", "ra_zo_plan_run_noalloc",
    "ra_tile_plan_create", "ra_tile_plan_info", "ra_tile_plan_run", "ra_tile_plan_destroy", "ra_tile_plan_device_status",
    "ra_zo_plan_save", "ra_zo_plan_load", "ra_tile_plan_save", "ra_tile_plan_load",
]


class RaFeatures(C.Structure):
    _fields_ = [
        ("avg_nnz_per_row", C.c_float), ("std_nnz_per_row", C.c_float), ("degree_cv", C.c_float),
        ("output_dim_N", C.c_int32), ("matrix_M", C.c_int32), ("matrix_K", C.c_int32),
        ("total_nnz", C.c_int32),
        ("sum_deg", C.c_uint64), ("sum_deg_sq", C.c_uint64),
    ]


class RaRoute(C.Structure):
    _fields_ = [
        ("chosen_path", C.c_int32), ("use_tf32", C.c_int32), ("estimated_risk", C.c_float),
        ("feasible", C.c_uint8 * PATH_COUNT), ("decision_reason", C.c_char * 64),
    ]


SCORE_KEYS = ("csr_direct", "csr_adaptive", "staged_reuse", "tc_sparse", "row_split_cuda",
              "tc_reordered", "hybrid_tc_cuda", "cusparse")


class RaRouteDetails(C.Structure):
    _fields_ = [
        ("scores", C.c_float * 8), ("rejection_code", C.c_int32 * PATH_COUNT),
        ("rejection_detail", (C.c_char * 128) * PATH_COUNT),
        ("gate_margin_raw", C.c_float), ("gate_margin_norm", C.c_float),
    ]


ANALYSIS_FLOAT_KEYS = (
    "avg_nnz_per_row", "std_nnz_per_row", "degree_cv", "max_to_mean_ratio", "frac_dense_rows", "skew_ratio",
    "long_row_fraction", "long_row_nnz_fraction", "top_1_row_nnz_fraction", "top_5_row_nnz_fraction",
    "tile_fill_mean", "tile_fill_median", "tile_fill_p90", "tile_fill_max", "tile_fill_variance",
    "tile_occupancy", "actual_nnz_coverage", "avg_nnz_per_tile", "row_window_colspan_compactness",
    "local_row_similarity_proxy", "reordered_locality_proxy", "locality_gain_proxy",
    "locality_selectivity_proxy", "road_likeness_proxy", "row_split_affinity_proxy", "mixedness_proxy",
    "tc_candidate_ratio", "tc_synergy_proxy", "estimated_tc_partition_ratio", "estimated_cuda_partition_ratio",
    "irregular_window_fraction", "tc_granularity_proxy", "redundancy_risk_proxy")
ANALYSIS_INT_KEYS = ("tc_candidate_tiles", "output_dim_N", "matrix_M", "matrix_K", "total_nnz")


class RaMatrixAnalysis(C.Structure):
    _fields_ = [(k, C.c_float) for k in ANALYSIS_FLOAT_KEYS] + [(k, C.c_int32) for k in ANALYSIS_INT_KEYS]


class RaZoInfo(C.Structure):
    _fields_ = [
        ("M", C.c_int32), ("K", C.c_int32),
        ("num_tiny", C.c_int32), ("num_short", C.c_int32), ("num_medium", C.c_int32),
        ("num_long", C.c_int32), ("num_empty", C.c_int32),
        ("num_small", C.c_int32), ("num_chunks", C.c_int32), ("num_zero_rows", C.c_int32),
        ("max_long_chunks", C.c_int32),
        ("plan_bytes", C.c_int64),
        ("d_small_row_ids", C.c_void_p), ("d_chunk_rows", C.c_void_p),
        ("d_chunk_starts", C.c_void_p), ("d_zero_row_ids", C.c_void_p),
    ]


class RaTileInfo(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("active", C.c_int32), ("M", C.c_int32), ("K", C.c_int32),
        ("num_windows", C.c_int32),
        ("num_blocks", C.c_int64), ("nnz", C.c_int64),
        ("tile_density", C.c_float),
        ("plan_bytes", C.c_int64),
        ("d_block_offsets", C.c_void_p), ("d_atox", C.c_void_p), ("d_vals_f16", C.c_void_p),
        ("d_win_rows", C.c_void_p),
        ("num_segments", C.c_int32), ("num_split_segs", C.c_int32),
        ("num_split_windows", C.c_int32), ("num_zero_rows", C.c_int32),
        ("d_seg_window", C.c_void_p), ("d_seg_bbegin", C.c_void_p), ("d_seg_bend", C.c_void_p),
        ("d_seg_scratch", C.c_void_p), ("d_split_wins", C.c_void_p), ("d_split_off", C.c_void_p),
        ("d_zero_rows", C.c_void_p),
        ("d_val_masks", C.c_void_p), ("d_val_base", C.c_void_p), ("d_vals_zc", C.c_void_p),
    ]


class RaSpmmError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference raises RuntimeError
    from TORCH_CHECK / CUDA_CHECK_NEXT, ra_common.h:53-71)."""


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m ra_spmm_b200.build` "
            "(nvcc, sm_100a). There is no CPU fallback.")
    lib = C.CDLL(str(LIB_PATH))
    vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64
    lib.ra_last_error_string.restype = C.c_char_p
    lib.ra_path_name.restype = C.c_char_p
    lib.ra_path_name.argtypes = [i32]
    lib.ra_version.restype = i32
    lib.ra_copy_to_host.argtypes = [vp, vp, C.c_size_t]
    lib.ra_fnv1a64_host.argtypes = [vp, C.c_size_t]
    lib.ra_fnv1a64_host.restype = C.c_uint64
    lib.ra_features_from_rowptr_host.argtypes = [vp, i32, i32, i32, C.POINTER(RaFeatures)]
    lib.ra_features_from_rowptr_device.argtypes = [vp, i32, i32, i32, vp, C.POINTER(RaFeatures)]
    lib.ra_route.argtypes = [C.POINTER(RaFeatures), i32, C.POINTER(RaRoute)]
    lib.ra_route_details.argtypes = [C.POINTER(RaFeatures), i32, C.POINTER(RaRoute), C.POINTER(RaRouteDetails)]
    lib.ra_reject_reason_name.argtypes = [i32]
    lib.ra_analyze_matrix.argtypes = [vp, vp, i32, i32, i32, i32, vp, C.POINTER(RaMatrixAnalysis)]
    lib.ra_reject_reason_name.restype = C.c_char_p
    lib.ra_csr_direct_spmm.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i64, vp]
    lib.ra_zo_plan_create.argtypes = [vp, i32, i32, i32, vp, C.POINTER(vp)]
    lib.ra_zo_plan_info.argtypes = [vp, C.POINTER(RaZoInfo)]
    lib.ra_zo_plan_run.argtypes = [vp, vp, vp, vp, vp, vp, i32, vp]
    lib.ra_zo_plan_destroy.argtypes = [vp]
    lib.ra_zo_plan_run_phases.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, vp]
    lib.ra_zo_plan_run_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, i32, vp]
    lib.ra_tile_plan_create.argtypes = [i32, vp, vp, vp, i32, i32, i32, i32, vp, C.POINTER(vp)]
    lib.ra_tile_plan_info.argtypes = [vp, C.POINTER(RaTileInfo)]
    lib.ra_tile_plan_run.argtypes = [vp, i32, vp, i32, vp, i32, vp]
    lib.ra_tile_plan_destroy.argtypes = [vp]
    lib.ra_tile_plan_device_status.argtypes = [vp, C.POINTER(C.c_int)]
    lib.ra_zo_plan_save.argtypes = [vp, C.c_char_p]
    lib.ra_zo_plan_load.argtypes = [C.c_char_p, C.POINTER(vp)]
    lib.ra_tile_plan_save.argtypes = [vp, C.c_char_p]
    lib.ra_tile_plan_load.argtypes = [C.c_char_p, C.POINTER(vp)]
    for name in EXPORTED_SYMBOLS:
        fn = getattr(lib, name)
        if fn.restype is C.c_int and name not in ("ra_version",):
            fn.restype = C.c_int
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status != RA_OK:
        msg = load().ra_last_error_string().decode("utf-8", "replace")
        raise RaSpmmError(f"{what} failed (status {status}): {msg}")
