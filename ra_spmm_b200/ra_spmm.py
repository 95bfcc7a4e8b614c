"""Host-side mirror of the reference's `ra_spmm` extension module for the SpMM hot path.

Same entry-point names, argument order and meaning, and error behaviour as the
pybind11 module defined in bindings/ra_bindings.cpp:2318-2899 (hot-path subset),
implemented as a thin layer over the C ABI of libra_spmm_b200.so. torch is used
only for device memory and the current CUDA stream.

Differences that are deliberate:
  * every launch goes to torch's *current* stream (the reference launches
    CSR_DIRECT and ZERO_OVERHEAD_CSR on the legacy default stream,
    csr/csr_direct.cu:273, csr/ra_zero_overhead.cu:421-499);
  * plans are built on the GPU; `make_*_plan` accepts CPU or CUDA tensors;
  * running an inactive tile plan (N < 16 or nnz == 0) raises instead of
    returning uninitialised memory (bindings/ra_bindings.cpp:2155-2166);
  * `run_*_plan` accepts an fp16 B on the FP16 path (skips the per-call
    fp32 -> fp16 conversion pass of tc/ra_tc_direct.cu:823-835).
"""
from __future__ import annotations

import ctypes as C
import os
import sys
import time

import torch

from . import _capi
from ._capi import RaSpmmError

__all__ = [
    "spmm_csr_direct", "make_zero_overhead_plan", "run_zero_overhead_plan",
    "make_tc_direct_plan", "make_tc_direct_zc_plan", "run_tc_direct_plan", "run_tc_direct_plan_tf32",
    "make_community_tc_plan", "run_community_tc_plan", "run_community_tc_plan_tf32",
    "make_segment_hybrid_plan", "run_segment_hybrid_plan", "run_segment_hybrid_plan_tf32",
    "make_router_plan", "run_router_plan", "gpu_info_next", "analyze_matrix",
    "spmm_cusparse", "spmm_cusparse_fp16", "make_cusparse_plan", "run_cusparse_plan",
    "benchmark_cusparse", "benchmark_cusparse_cold", "benchmark_cusparse_fp16", "benchmark_cusparse_fp16_cold",
    "RAZeroOverheadPlan", "RATcDirectPlan", "RACommunityTCPlan", "RASegmentHybridPlan",
    "save_plan", "load_zero_overhead_plan", "load_tile_plan",
]


def _lib():
    return _capi.load()


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _check_gpu_tensor(t: torch.Tensor, name: str) -> None:
    # bindings/ra_bindings.cpp:288-291
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _check_csr_tensors(rowptr, colind, vals) -> None:
    # bindings/ra_bindings.cpp:298-306
    _check_gpu_tensor(rowptr, "rowptr")
    _check_gpu_tensor(colind, "colind")
    _check_gpu_tensor(vals, "vals")
    if rowptr.dtype != torch.int32:
        raise RuntimeError("rowptr must be int32")
    if colind.dtype != torch.int32:
        raise RuntimeError("colind must be int32")
    if vals.dtype != torch.float32:
        raise RuntimeError("vals must be float32")


def _check_dense_b(B: torch.Tensor, allow_half: bool = False) -> None:
    _check_gpu_tensor(B, "B")
    ok = (torch.float32, torch.float16) if allow_half else (torch.float32,)
    if B.dtype not in ok:
        raise RuntimeError("B must be float32" + (" or float16" if allow_half else ""))
    if B.dim() != 2:
        raise RuntimeError("B must be 2-D")


# ---------------------------------------------------------------------------
# CSR_DIRECT  (bindings/ra_bindings.cpp:724-742)
# ---------------------------------------------------------------------------
def spmm_csr_direct(rowptr, colind, vals, B):
    _check_csr_tensors(rowptr, colind, vals)
    _check_dense_b(B)
    M = rowptr.shape[0] - 1
    K, N = B.shape
    # the kernel gathers B[colind]; the binding cannot see K, so the caller's B states it
    C_out = torch.empty((M, N), dtype=torch.float32, device=B.device)
    with torch.cuda.device(B.device):
        st = _lib().ra_csr_direct_spmm(
            rowptr.data_ptr(), colind.data_ptr(), vals.data_ptr(), B.data_ptr(),
            C_out.data_ptr(), M, K, N, colind.numel(), _stream_ptr(B.device))
    _capi.check(st, "spmm_csr_direct")
    return C_out


# ---------------------------------------------------------------------------
# ZERO_OVERHEAD_CSR  (bindings/ra_bindings.cpp:2057-2082, 2731-2750)
# ---------------------------------------------------------------------------
class RAZeroOverheadPlan:
    """Owner of a device-resident degree-binned plan (RAZeroOverheadPlan,
    ra_common.h:507-530). Freed when the object is collected."""

    def __init__(self, handle: int, device: torch.device):
        self._h = handle
        self._device = device
        info = _capi.RaZoInfo()
        _capi.check(_lib().ra_zo_plan_info(handle, C.byref(info)), "ra_zo_plan_info")
        self._info = info
        self.valid = True

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _lib().ra_zo_plan_destroy(h)
            except Exception:
                pass

    M = property(lambda s: s._info.M)
    K = property(lambda s: s._info.K)
    num_tiny = property(lambda s: s._info.num_tiny)
    num_short = property(lambda s: s._info.num_short)
    num_medium = property(lambda s: s._info.num_medium)
    num_long = property(lambda s: s._info.num_long)
    num_empty = property(lambda s: s._info.num_empty)
    plan_bytes = property(lambda s: s._info.plan_bytes)
    # additional read-only diagnostics
    num_small = property(lambda s: s._info.num_small)
    num_chunks = property(lambda s: s._info.num_chunks)
    num_zero_rows = property(lambda s: s._info.num_zero_rows)
    max_long_chunks = property(lambda s: s._info.max_long_chunks)

    def arrays(self) -> dict:
        """Copies of the four plan lists as CPU int32 tensors (for parity checks)."""
        i = self._info
        return {
            "small_row_ids": _copy_i32(i.d_small_row_ids, i.num_small, self._device),
            "chunk_rows": _copy_i32(i.d_chunk_rows, i.num_chunks, self._device),
            "chunk_starts": _copy_i32(i.d_chunk_starts, i.num_chunks, self._device),
            "zero_row_ids": _copy_i32(i.d_zero_row_ids, i.num_zero_rows, self._device),
        }


def _copy_raw(ptr, nbytes: int, device) -> torch.Tensor:
    out = torch.empty(nbytes, dtype=torch.uint8)
    if nbytes == 0 or not ptr:
        return out
    with torch.cuda.device(device):
        _capi.check(_lib().ra_copy_to_host(out.data_ptr(), ptr, nbytes), "ra_copy_to_host")
    return out


def _copy_i32(ptr, n: int, device) -> torch.Tensor:
    return _copy_raw(ptr, 4 * n, device).view(torch.int32)


def _copy_u16(ptr, n: int, device) -> torch.Tensor:
    return _copy_raw(ptr, 2 * n, device).view(torch.int16)


def _default_device(t: torch.Tensor) -> torch.device:
    if t.is_cuda:
        return t.device
    return torch.device("cuda", torch.cuda.current_device())


def make_zero_overhead_plan(rowptr_cpu, M, K):
    rp = rowptr_cpu.contiguous().to(torch.int32)
    dev = _default_device(rp)
    handle = C.c_void_p()
    with torch.cuda.device(dev):
        st = _lib().ra_zo_plan_create(rp.data_ptr(), 1 if rp.is_cuda else 0, int(M), int(K),
                                      _stream_ptr(dev), C.byref(handle))
    _capi.check(st, "make_zero_overhead_plan")
    plan = RAZeroOverheadPlan(handle.value, dev)
    _report_checksum("RAZeroOverheadPlan", plan)
    return plan


def run_zero_overhead_plan(plan, rowptr, colind, vals, B):
    _check_gpu_tensor(rowptr, "rowptr")
    _check_gpu_tensor(colind, "colind")
    _check_gpu_tensor(vals, "vals")
    _check_dense_b(B)
    if plan is None or not getattr(plan, "valid", False):
        raise RuntimeError("Invalid ZeroOverhead plan")
    if B.shape[0] != plan.K:
        raise RuntimeError(f"B has {B.shape[0]} rows but the plan was built for K={plan.K}")
    if rowptr.numel() != plan.M + 1:
        raise RuntimeError(f"rowptr has {rowptr.numel()} entries but the plan was built for M={plan.M}")
    M, N = plan.M, B.shape[1]
    C_out = torch.empty((M, N), dtype=torch.float32, device=B.device)
    with torch.cuda.device(B.device):
        st = _lib().ra_zo_plan_run(plan._h, rowptr.data_ptr(), colind.data_ptr(), vals.data_ptr(),
                                   B.data_ptr(), C_out.data_ptr(), N, _stream_ptr(B.device))
    _capi.check(st, "run_zero_overhead_plan")
    return C_out


# ---------------------------------------------------------------------------
# Tile plans  (bindings/ra_bindings.cpp:2140-2251, 2795-2898)
# ---------------------------------------------------------------------------
class _TilePlan:
    _kind = None

    def __init__(self, handle: int, device: torch.device):
        self._h = handle
        self._device = device
        info = _capi.RaTileInfo()
        _capi.check(_lib().ra_tile_plan_info(handle, C.byref(info)), "ra_tile_plan_info")
        self._info = info
        self.valid = True

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            try:
                _lib().ra_tile_plan_destroy(h)
            except Exception:
                pass

    M = property(lambda s: s._info.M)
    K = property(lambda s: s._info.K)
    active = property(lambda s: bool(s._info.active))
    num_windows = property(lambda s: s._info.num_windows)
    num_tc_tiles = property(lambda s: int(s._info.num_blocks))
    plan_bytes = property(lambda s: s._info.plan_bytes)

    def device_status(self) -> int:
        """Status word written by the plan's kernels (0 = ok); synchronises the device."""
        out = C.c_int(0)
        _capi.check(_lib().ra_tile_plan_device_status(self._h, C.byref(out)), "ra_tile_plan_device_status")
        return out.value

    def arrays(self) -> dict:
        """Copies of the plan's index/value arrays on the CPU (for parity checks)."""
        i = self._info
        nb = int(i.num_blocks)
        out = {}
        if not i.active:
            return out
        out["block_offsets"] = _copy_i32(i.d_block_offsets, i.num_windows + 1, self._device)
        out["atox"] = _copy_i32(i.d_atox, 8 * nb, self._device)
        if i.kind == _capi.TILE_TC_DIRECT_ZC:
            out["val_masks"] = _copy_raw(i.d_val_masks, 8 * nb, self._device).view(torch.int64)
            out["val_base"] = _copy_i32(i.d_val_base, nb, self._device)
            out["vals_zc"] = _copy_u16(i.d_vals_zc, int(i.nnz), self._device)
        else:
            out["vals_f16"] = _copy_u16(i.d_vals_f16, 64 * nb, self._device)
        if i.kind == _capi.TILE_COMMUNITY_TC:
            out["win_rows"] = _copy_i32(i.d_win_rows, 8 * i.num_windows, self._device)
        if i.kind == _capi.TILE_SEGMENT_HYBRID:
            out["seg_window"] = _copy_i32(i.d_seg_window, i.num_segments, self._device)
            out["seg_bbegin"] = _copy_i32(i.d_seg_bbegin, i.num_segments, self._device)
            out["seg_bend"] = _copy_i32(i.d_seg_bend, i.num_segments, self._device)
            out["seg_scratch"] = _copy_i32(i.d_seg_scratch, i.num_segments, self._device)
            out["split_wins"] = _copy_i32(i.d_split_wins, i.num_split_windows, self._device)
            out["split_off"] = _copy_i32(i.d_split_off, i.num_split_windows + 1, self._device)
            out["zero_rows"] = _copy_i32(i.d_zero_rows, i.num_zero_rows, self._device)
        return out


class RATcDirectPlan(_TilePlan):
    _kind = _capi.TILE_TC_DIRECT
    zc = property(lambda s: s._info.kind == _capi.TILE_TC_DIRECT_ZC)
    num_groups = property(lambda s: s._info.num_windows)
    num_fp32_rows = property(lambda s: 0)
    avg_tc_tile_density = property(lambda s: s._info.tile_density)
    fp32_group_fraction = property(lambda s: 0.0)


class RACommunityTCPlan(_TilePlan):
    _kind = _capi.TILE_COMMUNITY_TC
    num_communities = property(lambda s: s._info.num_windows)
    intra_community_nnz_fraction = property(lambda s: s._info.tile_density)


class RASegmentHybridPlan(_TilePlan):
    _kind = _capi.TILE_SEGMENT_HYBRID
    num_tc_groups = property(lambda s: s._info.num_windows)
    tc_nnz_fraction = property(lambda s: 1.0 if s._info.active else 0.0)
    cuda_nnz_fraction = property(lambda s: 0.0)
    num_segments = property(lambda s: s._info.num_segments)
    num_split_windows = property(lambda s: s._info.num_split_windows)


def _report_checksum(what: str, plan) -> None:
    """RA_PLAN_CHECKSUM=1: one stderr line per built plan with the FNV-1a checksum of every plan
    array and of all of them together - the hook that experiments/verify_format_checksums.py
    expects from the plan builders (byte identity of the format across builds and runs)."""
    if os.environ.get("RA_PLAN_CHECKSUM") != "1":
        return
    import numpy as np
    lib = _lib()
    parts, total = [], 0xcbf29ce484222325
    for name, arr in plan.arrays().items():
        b = np.ascontiguousarray(arr.numpy())
        h = int(lib.ra_fnv1a64_host(b.ctypes.data, b.nbytes)) if b.nbytes else 0xcbf29ce484222325
        parts.append(f"{name}={h:016x}")
        total = ((total ^ h) * 0x100000001b3) & 0xffffffffffffffff      # fold the array hashes in order
    print(f"[RA_PLAN_CHECKSUM] {what} {' '.join(parts)} all={total:016x}", file=sys.stderr, flush=True)


def _make_tile_plan(cls, rowptr, colind, vals, M, K, N, kind=None):
    dev = _default_device(rowptr)
    on_dev = rowptr.is_cuda and colind.is_cuda and vals.is_cuda
    if not on_dev:
        rowptr, colind, vals = rowptr.cpu(), colind.cpu(), vals.cpu()
    rp = rowptr.contiguous().to(torch.int32)
    ci = colind.contiguous().to(torch.int32)
    va = vals.contiguous().to(torch.float32)
    handle = C.c_void_p()
    with torch.cuda.device(dev):
        st = _lib().ra_tile_plan_create(cls._kind if kind is None else kind, rp.data_ptr(), ci.data_ptr(), va.data_ptr(),
                                        1 if on_dev else 0, int(M), int(K), int(N),
                                        _stream_ptr(dev), C.byref(handle))
    _capi.check(st, f"make plan ({cls.__name__})")
    plan = cls(handle.value, dev)
    _report_checksum(cls.__name__, plan)
    return plan


def _run_tile_plan(plan, B, precision, what):
    _check_dense_b(B, allow_half=(precision == _capi.PRECISION_FP16))
    if plan is None or not getattr(plan, "valid", False):
        raise RuntimeError(f"Invalid {what} plan")
    if B.shape[0] != plan.K:
        raise RuntimeError(f"B has {B.shape[0]} rows but the plan was built for K={plan.K}")
    M, N = plan.M, B.shape[1]
    C_out = torch.empty((M, N), dtype=torch.float32, device=B.device)
    b_dtype = _capi.DTYPE_F16 if B.dtype == torch.float16 else _capi.DTYPE_F32
    with torch.cuda.device(B.device):
        st = _lib().ra_tile_plan_run(plan._h, precision, B.data_ptr(), b_dtype,
                                     C_out.data_ptr(), N, _stream_ptr(B.device))
    _capi.check(st, f"run {what} plan")
    return C_out


def make_tc_direct_plan(rowptr_cpu, colind_cpu, vals_cpu, M, K, N):
    return _make_tile_plan(RATcDirectPlan, rowptr_cpu, colind_cpu, vals_cpu, M, K, N)


def make_tc_direct_zc_plan(rowptr_cpu, colind_cpu, vals_cpu, M, K, N):
    """TC_DIRECT plan with zero-compressed block values (bindings/ra_bindings.cpp:2817,
    tc/ra_tc_direct.cu:792-800); run with run_tc_direct_plan[_tf32] like the padded plan."""
    return _make_tile_plan(RATcDirectPlan, rowptr_cpu, colind_cpu, vals_cpu, M, K, N,
                           kind=_capi.TILE_TC_DIRECT_ZC)


def run_tc_direct_plan(plan, B):
    return _run_tile_plan(plan, B, _capi.PRECISION_FP16, "TcDirect")


def run_tc_direct_plan_tf32(plan, B):
    return _run_tile_plan(plan, B, _capi.PRECISION_TF32, "TcDirect")


def make_community_tc_plan(rowptr_cpu, colind_cpu, vals_cpu, M, K, N):
    return _make_tile_plan(RACommunityTCPlan, rowptr_cpu, colind_cpu, vals_cpu, M, K, N)


def run_community_tc_plan(plan, B):
    return _run_tile_plan(plan, B, _capi.PRECISION_FP16, "CommunityTC")


def run_community_tc_plan_tf32(plan, B):
    return _run_tile_plan(plan, B, _capi.PRECISION_TF32, "CommunityTC")


def make_segment_hybrid_plan(rowptr_cpu, colind_cpu, vals_cpu, M, K, N):
    return _make_tile_plan(RASegmentHybridPlan, rowptr_cpu, colind_cpu, vals_cpu, M, K, N)


def run_segment_hybrid_plan(plan, colind, vals, B):
    # colind / vals are accepted and ignored, as in the reference
    # (tc/ra_segment_hybrid.cu:548-551).
    return _run_tile_plan(plan, B, _capi.PRECISION_FP16, "SegmentHybrid")


def run_segment_hybrid_plan_tf32(plan, colind, vals, B):
    return _run_tile_plan(plan, B, _capi.PRECISION_TF32, "SegmentHybrid")


# ---------------------------------------------------------------------------
# Plan files (no counterpart in the reference, whose plans live in one process only):
# every array with its length and FNV-1a checksum, verified again on load.
# ---------------------------------------------------------------------------
def save_plan(plan, path) -> None:
    """Write a ZERO_OVERHEAD_CSR or tile plan to `path`."""
    fn = _lib().ra_zo_plan_save if isinstance(plan, RAZeroOverheadPlan) else _lib().ra_tile_plan_save
    with torch.cuda.device(plan._device):
        _capi.check(fn(plan._h, os.fsencode(path)), "save_plan")


def load_zero_overhead_plan(path, device=None) -> "RAZeroOverheadPlan":
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    handle = C.c_void_p()
    with torch.cuda.device(dev):
        _capi.check(_lib().ra_zo_plan_load(os.fsencode(path), C.byref(handle)), "load_zero_overhead_plan")
    return RAZeroOverheadPlan(handle.value, dev)


def load_tile_plan(path, device=None):
    """Plan object of the family stored in the file (RATcDirectPlan, RACommunityTCPlan or
    RASegmentHybridPlan)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    handle = C.c_void_p()
    with torch.cuda.device(dev):
        _capi.check(_lib().ra_tile_plan_load(os.fsencode(path), C.byref(handle)), "load_tile_plan")
    info = _capi.RaTileInfo()
    _capi.check(_lib().ra_tile_plan_info(handle.value, C.byref(info)), "ra_tile_plan_info")
    cls = {_capi.TILE_COMMUNITY_TC: RACommunityTCPlan, _capi.TILE_SEGMENT_HYBRID: RASegmentHybridPlan}.get(
        info.kind, RATcDirectPlan)
    return cls(handle.value, dev)


# ---------------------------------------------------------------------------
# Router  (bindings/ra_bindings.cpp:634-718, 1717-1753)
# ---------------------------------------------------------------------------
_FEATURE_KEYS = [
    "avg_nnz_per_row", "std_nnz_per_row", "degree_cv", "max_to_mean_ratio", "frac_dense_rows",
    "skew_ratio", "long_row_fraction", "long_row_nnz_fraction", "top_1_row_nnz_fraction",
    "top_5_row_nnz_fraction", "tile_fill_mean", "tile_fill_median", "tile_fill_p90",
    "tile_fill_max", "tile_fill_variance", "tile_occupancy", "actual_nnz_coverage",
    "avg_nnz_per_tile", "row_window_colspan_compactness", "local_row_similarity_proxy",
    "reordered_locality_proxy", "locality_gain_proxy", "locality_selectivity_proxy",
    "road_likeness_proxy", "row_split_affinity_proxy", "mixedness_proxy", "tc_candidate_ratio",
    "tc_synergy_proxy", "estimated_tc_partition_ratio", "estimated_cuda_partition_ratio",
    "irregular_window_fraction", "tc_granularity_proxy", "redundancy_risk_proxy",
]


def router_features(rowptr, M, K, N) -> _capi.RaFeatures:
    """Production features of a CSR: device scan for a CUDA rowptr, host scan otherwise."""
    feats = _capi.RaFeatures()
    if rowptr.is_cuda:
        if rowptr.dtype != torch.int32 or not rowptr.is_contiguous():
            raise RuntimeError("rowptr must be a contiguous int32 tensor")
        with torch.cuda.device(rowptr.device):
            st = _lib().ra_features_from_rowptr_device(rowptr.data_ptr(), int(M), int(K), int(N),
                                                       _stream_ptr(rowptr.device), C.byref(feats))
    else:
        rp = rowptr.contiguous().to(torch.int32)
        st = _lib().ra_features_from_rowptr_host(rp.data_ptr(), int(M), int(K), int(N),
                                                 C.byref(feats))
    _capi.check(st, "router_features")
    return feats


def route(feats: _capi.RaFeatures) -> _capi.RaRoute:
    out = _capi.RaRoute()
    _capi.check(_lib().ra_route(C.byref(feats), 0, C.byref(out)), "ra_route")
    return out


def route_details(feats: _capi.RaFeatures, r: _capi.RaRoute) -> _capi.RaRouteDetails:
    out = _capi.RaRouteDetails()
    _capi.check(_lib().ra_route_details(C.byref(feats), 0, C.byref(r), C.byref(out)), "ra_route_details")
    return out


def make_router_plan(rowptr, colind, vals, M, K, N, portfolio="MAIN"):
    """Decision dict with the keys and values of plan_to_dict (bindings/ra_bindings.cpp:634-718)
    for the MAIN portfolio: the decision (`chosen_path`, `use_tf32`, `decision_reason`,
    `estimated_risk`, `feasible_by_path`, `feature_values`) and its diagnostics (`scores`,
    `rejection_codes`, `rejection_details`, gate margins).
    """
    if portfolio != "MAIN":
        raise RaSpmmError("only the MAIN portfolio is implemented (FULL is the "
                          "reference's ablation roster)")
    t0 = time.perf_counter()
    feats = router_features(rowptr, M, K, N)
    r = route(feats)
    det = route_details(feats, r)
    planning_ms = (time.perf_counter() - t0) * 1e3
    names = _capi.PATH_NAMES
    feas = [bool(r.feasible[i]) for i in range(_capi.PATH_COUNT)]
    fv = {k: 0.0 for k in _FEATURE_KEYS}
    fv["avg_nnz_per_row"] = float(feats.avg_nnz_per_row)
    fv["std_nnz_per_row"] = float(feats.std_nnz_per_row)
    fv["degree_cv"] = float(feats.degree_cv)
    fv["tc_candidate_tiles"] = 0
    chosen = names[r.chosen_path]
    return {
        "chosen_path": chosen,
        "use_tf32": bool(r.use_tf32),
        "chosen_path_int": int(r.chosen_path),
        "decision_reason": r.decision_reason.decode(),
        "estimated_risk": float(r.estimated_risk),
        "planning_time_ms": planning_ms,
        "gate_margin_raw": float(det.gate_margin_raw),
        "gate_margin_norm": float(det.gate_margin_norm),
        "path_count": _capi.PATH_COUNT,
        "path_names": list(names),
        "feasible": feas,
        "feasible_by_path": dict(zip(names, feas)),
        "rejection_codes": {n: _lib().ra_reject_reason_name(det.rejection_code[i]).decode()
                            for i, n in enumerate(names)},
        "rejection_details": {n: det.rejection_detail[i].value.decode() for i, n in enumerate(names)},
        "feature_values": fv,
        "scores": {k: float(det.scores[i]) for i, k in enumerate(_capi.SCORE_KEYS)},
        "feature_set": "production_4",
        "feature_backend": "cuda_rowptr_moments" if rowptr.is_cuda else "cpu_rowptr",
        "total_nnz": int(feats.total_nnz),
    }


# ---------------------------------------------------------------------------
# cuSPARSE guardrail and harness reference (bindings/ra_bindings.cpp:431-615, 838-1037,
# 2342-2391): the vendor library behind rule 5's CUSPARSE route, the correctness reference of
# the sweep drivers and their external baseline. Pass-throughs to the cuSPARSE SpMM that torch
# exposes for CSR tensors - library calls, not kernels of this package.
# ---------------------------------------------------------------------------
class CuSparsePlan:
    """Reusable CSR operand (CuSparsePlanWrapper, bindings/ra_bindings.cpp:2374-2386)."""

    def __init__(self, rowptr, colind, vals, K, half=False):
        M = rowptr.shape[0] - 1
        v = vals.to(torch.float16) if half else vals
        self.A = torch.sparse_csr_tensor(rowptr, colind, v, size=(int(M), int(K)))
        self.half = half
        self.valid = True
        self.algorithm = "torch.sparse.mm (cuSPARSE CSR SpMM)"


CusparsePlan = CuSparsePlan


def make_cusparse_plan(rowptr, colind, vals, B):
    """`B` is a same-shape dense operand (only its row count is read), as in the reference."""
    _check_csr_tensors(rowptr, colind, vals)
    K = B.shape[0] if torch.is_tensor(B) else int(B)
    return CuSparsePlan(rowptr, colind, vals, K)


def run_cusparse_plan(plan, B):
    if plan.half:
        return torch.sparse.mm(plan.A, B.to(torch.float16)).float()
    return torch.sparse.mm(plan.A, B)


def spmm_cusparse(rowptr, colind, vals, B):
    return run_cusparse_plan(make_cusparse_plan(rowptr, colind, vals, B), B)


def spmm_cusparse_fp16(rowptr, colind, vals, B):
    """Precision-matched vendor baseline: A and B rounded to fp16, result returned as fp32."""
    _check_csr_tensors(rowptr, colind, vals)
    return run_cusparse_plan(CuSparsePlan(rowptr, colind, vals, B.shape[0], half=True), B)


def _event_ms(fn, warmup, iters):
    # measure_cuda_exec_ms, bench/benchmark.cpp:39-67
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _cusparse_timing(label, plan_ms, exec_ms, nnz, N, main):
    return {"plan_ms": plan_ms, "exec_ms": exec_ms, "total_ms": plan_ms + exec_ms,
            "gflops": (2.0 * nnz * N / (exec_ms * 1e6)) if exec_ms > 0 else 0.0,
            "path": label, "in_main_portfolio": main, "legacy_baseline": False,
            "external_baseline": not main, "cusparse_algorithm": "torch.sparse.mm (cuSPARSE CSR SpMM)",
            "preprocess_ms": plan_ms}


def _bench_cusparse(rowptr, colind, vals, B, half, warmup, iters, cold):
    _check_csr_tensors(rowptr, colind, vals)
    _check_dense_b(B)
    nnz, N = colind.numel(), B.shape[1]
    label = "CUSPARSE_FP16" if half else "CUSPARSE"
    iters = max(1, int(iters))
    if not cold:
        plan = CuSparsePlan(rowptr, colind, vals, B.shape[0], half=half)
        Bop = B.to(torch.float16) if half else B
        ms = _event_ms(lambda: torch.sparse.mm(plan.A, Bop), int(warmup), iters)
        return _cusparse_timing(label, 0.0, ms, nnz, N, False)
    plan_sum = exec_sum = 0.0
    for _ in range(iters):                      # state construction timed on the host, one run on the device
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        plan = CuSparsePlan(rowptr, colind, vals, B.shape[0], half=half)
        Bop = B.to(torch.float16) if half else B
        torch.cuda.synchronize()
        plan_sum += (time.perf_counter() - t0) * 1e3
        exec_sum += _event_ms(lambda: torch.sparse.mm(plan.A, Bop), 0, 1)
    return _cusparse_timing(label, plan_sum / iters, exec_sum / iters, nnz, N, not half)


def benchmark_cusparse(rowptr, colind, vals, B, warmup=3, iters=10):
    return _bench_cusparse(rowptr, colind, vals, B, False, warmup, iters, False)


def benchmark_cusparse_cold(rowptr, colind, vals, B, iters=10):
    return _bench_cusparse(rowptr, colind, vals, B, False, 0, iters, True)


def benchmark_cusparse_fp16(rowptr, colind, vals, B, warmup=3, iters=10):
    return _bench_cusparse(rowptr, colind, vals, B, True, warmup, iters, False)


def benchmark_cusparse_fp16_cold(rowptr, colind, vals, B, iters=10):
    return _bench_cusparse(rowptr, colind, vals, B, True, 0, iters, True)


def run_router_plan(plan_dict, rowptr, colind, vals, B):
    """One-shot convenience path (bindings/ra_bindings.cpp:1762-1879): rebuilds the
    chosen kernel's plan and runs it. Like the reference it always takes the FP16
    tile path (`use_tf32` is ignored) and synchronises before returning."""
    _check_csr_tensors(rowptr, colind, vals)
    _check_dense_b(B)
    path = plan_dict["chosen_path"]
    M = rowptr.shape[0] - 1
    K, N = B.shape
    if path == "CSR_DIRECT":
        out = spmm_csr_direct(rowptr, colind, vals, B)
    elif path == "ZERO_OVERHEAD_CSR":
        out = run_zero_overhead_plan(make_zero_overhead_plan(rowptr, M, K), rowptr, colind, vals, B)
    elif path == "TC_DIRECT":
        out = run_tc_direct_plan(make_tc_direct_plan(rowptr, colind, vals, M, K, N), B)
    elif path == "COMMUNITY_TC":
        out = run_community_tc_plan(make_community_tc_plan(rowptr, colind, vals, M, K, N), B)
    elif path == "SEGMENT_HYBRID":
        out = run_segment_hybrid_plan(make_segment_hybrid_plan(rowptr, colind, vals, M, K, N),
                                      colind, vals, B)
    elif path == "CUSPARSE":
        out = spmm_cusparse(rowptr, colind, vals, B)
    else:
        raise RaSpmmError(f"run_router_plan: path {path} is not part of this library")
    torch.cuda.synchronize(B.device)
    return out


def analyze_matrix(rowptr, colind, M, K, N=128):
    """The 34 structural features as a dict with the keys of the reference's analyze_matrix
    (bindings/ra_bindings.cpp:1993-2051), plus "nnz". rowptr/colind: int32 tensors, both on the
    CPU or both on the current CUDA device; the O(nnz) work runs on the GPU either way."""
    if rowptr.is_cuda != colind.is_cuda:
        raise RuntimeError("rowptr and colind must be on the same device")
    rp = rowptr.contiguous().to(torch.int32)
    ci = colind.contiguous().to(torch.int32)
    out = _capi.RaMatrixAnalysis()
    dev = rp.device if rp.is_cuda else torch.device("cuda", torch.cuda.current_device())
    with torch.cuda.device(dev):
        st = _lib().ra_analyze_matrix(rp.data_ptr(), ci.data_ptr(), 1 if rp.is_cuda else 0, int(M), int(K), int(N),
                                      _stream_ptr(dev), C.byref(out))
    _capi.check(st, "analyze_matrix")
    d = {k: float(getattr(out, k)) for k in _capi.ANALYSIS_FLOAT_KEYS}
    d["tc_candidate_tiles"] = int(out.tc_candidate_tiles)
    d["nnz"] = int(rp[M].item()) if M > 0 else 0
    return d


def gpu_info_next():
    """List of per-device dicts (bindings/ra_bindings.cpp:2719)."""
    out = []
    for i in range(torch.cuda.device_count()):
        p = torch.cuda.get_device_properties(i)
        out.append({"device": i, "name": p.name, "sm_count": p.multi_processor_count,
                    "major": p.major, "minor": p.minor,
                    "total_memory_bytes": p.total_memory})
    return out
