"""ctypes access to the reference's own code built into oracle/_ref/ by
oracle/Makefile, and to the C restatement liboracle_c.so. TEST INFRASTRUCTURE ONLY.

`router()` loads the reference's host router (route_dispatch and the production
feature scan); `kernels()` loads its five kernel families compiled for sm_100a
(needs a GPU to call). Both return None when the file was not built.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PATH_COUNT = 15


class RefRoute(C.Structure):
    _fields_ = [("avg_nnz_per_row", C.c_float), ("std_nnz_per_row", C.c_float),
                ("degree_cv", C.c_float), ("total_nnz", C.c_int),
                ("chosen_path", C.c_int), ("use_tf32", C.c_int), ("estimated_risk", C.c_float),
                ("feasible", C.c_ubyte * PATH_COUNT), ("decision_reason", C.c_char * 64)]


class RefZoInfo(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("num_small", "num_chunks", "num_zero_rows", "num_tiny",
                                       "num_short", "num_medium", "num_long", "num_empty",
                                       "max_long_chunks")] + \
               [(n, C.c_void_p) for n in ("d_small_row_ids", "d_chunk_rows", "d_chunk_starts",
                                          "d_zero_row_ids")]


class RefTileInfo(C.Structure):
    _fields_ = [("active", C.c_int), ("num_windows", C.c_int), ("num_blocks", C.c_int),
                ("d_block_offsets", C.c_void_p), ("d_atox", C.c_void_p),
                ("d_vals_f16", C.c_void_p), ("d_win_rows", C.c_void_p),
                ("num_segments", C.c_int), ("num_split_segs", C.c_int),
                ("num_split_windows", C.c_int), ("num_zero_rows", C.c_int)] + \
               [(n, C.c_void_p) for n in ("d_seg_window", "d_seg_bbegin", "d_seg_bend",
                                          "d_seg_scratch", "d_split_wins", "d_split_off",
                                          "d_zero_rows")] + \
               [(n, C.c_void_p) for n in ("d_val_masks", "d_val_base", "d_vals_zc")]


class RefRouteDetails(C.Structure):
    _fields_ = [("scores", C.c_float * 8), ("rejection_code", C.c_int * PATH_COUNT),
                ("rejection_detail", (C.c_char * 128) * PATH_COUNT),
                ("gate_margin_raw", C.c_float), ("gate_margin_norm", C.c_float)]


_cache = {}


def _load(name: str):
    if name in _cache:
        return _cache[name]
    path = HERE / name
    lib = C.CDLL(str(path)) if path.exists() else None
    _cache[name] = lib
    return lib


def router():
    lib = _load("_ref/libra_ref_router.so")
    if lib is not None and not getattr(lib, "_typed", False):
        lib.ref_route_from_rowptr.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(RefRoute)]
        lib.ref_route_from_features.argtypes = [C.c_float, C.c_float, C.c_float, C.c_int, C.c_int,
                                                C.c_int, C.c_int, C.POINTER(RefRoute)]
        if hasattr(lib, "ref_route_details_from_features"):
            lib.ref_route_details_from_features.argtypes = [C.c_float, C.c_float, C.c_float, C.c_int, C.c_int,
                                                            C.c_int, C.c_int, C.POINTER(RefRouteDetails)]
        if hasattr(lib, "ref_analyze_matrix"):
            lib.ref_analyze_matrix.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
        lib._typed = True
    return lib


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


def ref_analyze_matrix(rowptr, colind, M, K, N) -> dict:
    """compute_router_features of the reference (router/router_features.cpp:113-432): the 33
    float fields as np.float32 and the five int fields, keyed by field name."""
    rp = np.ascontiguousarray(rowptr, dtype=np.int32)
    ci = np.ascontiguousarray(colind, dtype=np.int32)
    f = np.zeros(33, dtype=np.float32)
    i = np.zeros(5, dtype=np.int32)
    router().ref_analyze_matrix(rp.ctypes.data, ci.ctypes.data, M, K, N, f.ctypes.data, i.ctypes.data)
    out = {k: f[j] for j, k in enumerate(ANALYSIS_FLOAT_KEYS)}
    out.update({k: int(i[j]) for j, k in enumerate(ANALYSIS_INT_KEYS)})
    return out


def ref_route_details_from_features(avg, std, cv, M, K, N, nnz) -> RefRouteDetails:
    out = RefRouteDetails()
    router().ref_route_details_from_features(float(avg), float(std), float(cv), M, K, N, nnz, C.byref(out))
    return out


def ref_route_from_rowptr(rowptr: np.ndarray, M, K, N) -> RefRoute:
    rp = np.ascontiguousarray(rowptr, dtype=np.int32)
    out = RefRoute()
    router().ref_route_from_rowptr(rp.ctypes.data, M, K, N, C.byref(out))
    return out


def ref_route_from_features(avg, std, cv, M, K, N, nnz) -> RefRoute:
    out = RefRoute()
    router().ref_route_from_features(float(avg), float(std), float(cv), M, K, N, nnz, C.byref(out))
    return out


def kernels():
    lib = _load("_ref/libra_ref_kernels.so")
    if lib is not None and not getattr(lib, "_typed", False):
        vp, i = C.c_void_p, C.c_int
        lib.ref_last_error.restype = C.c_char_p
        lib.ref_csr_direct.argtypes = [vp, vp, vp, vp, vp, i, i, i, i]
        lib.ref_zo_make.restype = vp
        lib.ref_zo_make.argtypes = [vp, i, i]
        lib.ref_zo_info.argtypes = [vp, C.POINTER(RefZoInfo)]
        lib.ref_zo_run.argtypes = [vp, vp, vp, vp, vp, vp, i]
        lib.ref_zo_free.argtypes = [vp]
        lib.ref_tile_make.restype = vp
        lib.ref_tile_make.argtypes = [i, vp, vp, vp, i, i, i]
        lib.ref_tile_info.argtypes = [vp, C.POINTER(RefTileInfo)]
        lib.ref_tile_run.argtypes = [vp, i, vp, vp, i, vp]
        lib.ref_tile_free.argtypes = [vp]
        lib._typed = True
    return lib


def oracle_c():
    lib = _load("liboracle_c.so")
    if lib is not None and not getattr(lib, "_typed", False):
        vp, i = C.c_void_p, C.c_int
        lib.oc_spmm_f64.argtypes = [vp, vp, vp, vp, vp, i, i, i]
        lib.oc_spmm_f32.argtypes = [vp, vp, vp, vp, vp, i, i]
        lib.oc_f32_to_f16_bits.argtypes = [vp, vp, C.c_int64]
        lib.oc_tile_plan.argtypes = [vp, vp, vp, i, vp, vp, vp, vp]
        lib.oc_tile_plan.restype = i
        lib._typed = True
    return lib


def c_spmm_f64(rowptr, colind, vals, B, mode=0) -> np.ndarray:
    """float64-accumulated SpMM of the C restatement (mode 0 fp32, 1 fp16, 2 tf32)."""
    rp = np.ascontiguousarray(rowptr, dtype=np.int32)
    ci = np.ascontiguousarray(colind, dtype=np.int32)
    va = np.ascontiguousarray(vals, dtype=np.float32)
    Bm = np.ascontiguousarray(B, dtype=np.float32)
    M, N = rp.size - 1, Bm.shape[1]
    out = np.empty((M, N), dtype=np.float64)
    oracle_c().oc_spmm_f64(rp.ctypes.data, ci.ctypes.data, va.ctypes.data, Bm.ctypes.data,
                           out.ctypes.data, M, N, mode)
    return out


def c_tile_plan(rowptr, colind, vals, M, win_rows=None):
    rp = np.ascontiguousarray(rowptr, dtype=np.int32)
    ci = np.ascontiguousarray(colind, dtype=np.int32)
    va = np.ascontiguousarray(vals, dtype=np.float32)
    wr = None if win_rows is None else np.ascontiguousarray(win_rows, dtype=np.int32)
    W = (M + 7) // 8
    bo = np.zeros(W + 1, dtype=np.int32)
    lib = oracle_c()
    wrp = None if wr is None else wr.ctypes.data
    lib.oc_tile_plan(rp.ctypes.data, ci.ctypes.data, va.ctypes.data, M, wrp, bo.ctypes.data, None, None)
    nb = int(bo[-1])
    atox = np.zeros(nb * 8, dtype=np.int32)
    v16 = np.zeros(nb * 64, dtype=np.uint16)
    lib.oc_tile_plan(rp.ctypes.data, ci.ctypes.data, va.ctypes.data, M, wrp, bo.ctypes.data,
                     atox.ctypes.data, v16.ctypes.data)
    return dict(block_offsets=bo, atox=atox, vals_f16=v16, num_blocks=nb, num_windows=W)
