"""Caller-side helpers of the reference module that sit next to the hot path:
timing helpers (run_oracle_warm/cold, run_router_warm/cold,
bindings/ra_bindings.cpp:1888-1965, 2526-2572), the cuSPARSE guardrail
pass-through (bindings/ra_bindings.cpp:431-615: rule 5 of the router returns
CUSPARSE) and FNV-1a checksums of plan arrays (the RA_PLAN_CHECKSUM hook that
experiments/verify_format_checksums.py expects).

Timing protocol = measure_cuda_exec_ms (bench/benchmark.cpp:39-67): warm-ups,
device sync, CUDA events around `iters` back-to-back calls, mean ms;
GFLOP/s = 2*nnz*N / (ms * 1e6) (bench/benchmark.cpp:19-25).
"""
from __future__ import annotations

import time

import numpy as np
import torch

from . import ra_spmm as m

MAIN_KERNELS = ["CSR_DIRECT", "ZERO_OVERHEAD_CSR", "TC_DIRECT", "COMMUNITY_TC", "SEGMENT_HYBRID",
                "TC_DIRECT_TF32", "COMMUNITY_TC_TF32", "SEGMENT_HYBRID_TF32"]


# ---- cuSPARSE pass-through (vendor library; lives beside the entry points it mirrors) ----
CusparsePlan = m.CuSparsePlan
make_cusparse_plan = m.make_cusparse_plan
run_cusparse_plan = m.run_cusparse_plan
spmm_cusparse = m.spmm_cusparse


# ---- plan build / run by kernel label (ra_real_graph_eval.py:247-285) ---------------
def build_kernel_plan(kernel, rowptr, colind, vals, M, K, N):
    fam = kernel.replace("_TF32", "")
    if fam == "CSR_DIRECT":
        return None
    if fam == "ZERO_OVERHEAD_CSR":
        return m.make_zero_overhead_plan(rowptr, M, K)
    if fam == "TC_DIRECT":
        return m.make_tc_direct_plan(rowptr, colind, vals, M, K, N)
    if fam == "COMMUNITY_TC":
        return m.make_community_tc_plan(rowptr, colind, vals, M, K, N)
    if fam == "SEGMENT_HYBRID":
        return m.make_segment_hybrid_plan(rowptr, colind, vals, M, K, N)
    if fam == "CUSPARSE":
        return m.CuSparsePlan(rowptr, colind, vals, K)
    raise ValueError(f"Kernel has no reusable custom plan: {kernel}")


def run_planned_kernel(kernel, plan, rowptr, colind, vals, B):
    tf32 = kernel.endswith("_TF32")
    fam = kernel.replace("_TF32", "")
    if fam == "CSR_DIRECT":
        return m.spmm_csr_direct(rowptr, colind, vals, B)
    if fam == "ZERO_OVERHEAD_CSR":
        return m.run_zero_overhead_plan(plan, rowptr, colind, vals, B)
    if fam == "TC_DIRECT":
        return m.run_tc_direct_plan_tf32(plan, B) if tf32 else m.run_tc_direct_plan(plan, B)
    if fam == "COMMUNITY_TC":
        return m.run_community_tc_plan_tf32(plan, B) if tf32 else m.run_community_tc_plan(plan, B)
    if fam == "SEGMENT_HYBRID":
        return (m.run_segment_hybrid_plan_tf32(plan, colind, vals, B) if tf32
                else m.run_segment_hybrid_plan(plan, colind, vals, B))
    if fam == "CUSPARSE":
        return run_cusparse_plan(plan, B)
    raise ValueError(f"Unknown planned kernel: {kernel}")


# ---- timing ------------------------------------------------------------------------
def measure_cuda_exec_ms(fn, warmup=3, iters=10):
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


def _timing(plan_ms, exec_ms, nnz, N):
    total = plan_ms + exec_ms
    return {"plan_ms": plan_ms, "exec_ms": exec_ms, "total_ms": total,
            "gflops": (2.0 * nnz * N / (exec_ms * 1e6)) if exec_ms > 0 else 0.0}


def measure_path_timing(kernel, rowptr, colind, vals, B, cold, warmup=3, iters=10):
    M, (K, N), nnz = rowptr.shape[0] - 1, B.shape, colind.numel()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    plan = build_kernel_plan(kernel, rowptr, colind, vals, M, K, N)
    torch.cuda.synchronize()
    plan_ms = (time.perf_counter() - t0) * 1e3
    run = lambda: run_planned_kernel(kernel, plan, rowptr, colind, vals, B)
    if cold:
        return _timing(plan_ms, measure_cuda_exec_ms(run, 0, 1), nnz, N)
    return _timing(0.0, measure_cuda_exec_ms(run, warmup, iters), nnz, N)


def _run_oracle(rowptr, colind, vals, B, warmup, iters, portfolio, cold):
    if portfolio != "MAIN":
        raise m.RaSpmmError("only the MAIN portfolio is implemented")
    M, (K, N), nnz = rowptr.shape[0] - 1, B.shape, colind.numel()
    kernels = [k for k in MAIN_KERNELS if N >= 16 or k in ("CSR_DIRECT", "ZERO_OVERHEAD_CSR")]
    results = {k: dict(measure_path_timing(k, rowptr, colind, vals, B, cold, warmup, iters), path=k,
                       in_main_portfolio=True, legacy_baseline=False) for k in kernels}
    best = min(results, key=lambda k: results[k]["total_ms"])
    return {"mode": "cold" if cold else "warm", "portfolio": "MAIN", "path_results": results,
            "path_times": {k: v["total_ms"] for k, v in results.items()}, "oracle_path": best,
            "oracle_time_ms": results[best]["total_ms"], "oracle_plan_ms": results[best]["plan_ms"],
            "oracle_exec_ms": results[best]["exec_ms"], "M": M, "K": K, "N": N, "nnz": nnz}


def run_oracle_warm(rowptr, colind, vals, B, warmup=3, iters=10, portfolio="MAIN"):
    return _run_oracle(rowptr, colind, vals, B, warmup, iters, portfolio, False)


def run_oracle_cold(rowptr, colind, vals, B, warmup=3, iters=10, portfolio="MAIN"):
    return _run_oracle(rowptr, colind, vals, B, warmup, iters, portfolio, True)


def _run_router(rowptr, colind, vals, B, portfolio, warmup, iters, cold):
    M, (K, N), nnz = rowptr.shape[0] - 1, B.shape, colind.numel()
    t0 = time.perf_counter()
    plan = m.make_router_plan(rowptr, colind, vals, M, K, N, portfolio)
    route_ms = (time.perf_counter() - t0) * 1e3
    label = plan["chosen_path"] + ("_TF32" if plan["use_tf32"] else "")
    timing = measure_path_timing(label, rowptr, colind, vals, B, cold, warmup, iters)
    if cold:
        timing["plan_ms"] += route_ms
        timing["total_ms"] = timing["plan_ms"] + timing["exec_ms"]
    return {"mode": "cold" if cold else "warm", "portfolio": portfolio, "router_path": plan["chosen_path"],
            "router_kernel": label, "timing": timing, "plan": plan, "M": M, "K": K, "N": N, "nnz": nnz}


def run_router_warm(rowptr, colind, vals, B, portfolio="MAIN", warmup=3, iters=10):
    return _run_router(rowptr, colind, vals, B, portfolio, warmup, iters, False)


def run_router_cold(rowptr, colind, vals, B, portfolio="MAIN", warmup=3, iters=10):
    return _run_router(rowptr, colind, vals, B, portfolio, warmup, iters, True)


# ---- plan checksums -------------------------------------------------------------------
def fnv1a64(data: np.ndarray) -> int:
    """64-bit FNV-1a over the bytes of an array (computed by the library)."""
    from . import _capi
    b = np.ascontiguousarray(data)
    return int(_capi.load().ra_fnv1a64_host(b.ctypes.data, b.nbytes))


def plan_checksums(plan) -> dict:
    """Checksum per plan array (bit-identity evidence across builds and runs)."""
    return {k: f"{fnv1a64(v.numpy()):016x}" for k, v in plan.arrays().items()}
