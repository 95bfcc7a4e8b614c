"""Caller-side helpers: timing dicts, cuSPARSE pass-through, plan checksums, lifecycle router."""
import json

import numpy as np
import pytest
import torch

from oracle import ra_oracle as O
from ra_spmm_b200 import generators as G
from ra_spmm_b200 import harness as H
from ra_spmm_b200 import ra_spmm
from ra_spmm_b200 import cost_model as CM

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def graph(cuda):
    a = G.chung_lu_power_law(n=20000, seed=3)
    rp, ci, va = a.torch(cuda)
    B = G.dense(a.K, 64, 3).to(cuda)
    return a, rp, ci, va, B


def test_oracle_and_router_timing_dicts(graph):
    a, rp, ci, va, B = graph
    o = H.run_oracle_warm(rp, ci, va, B, warmup=1, iters=2)
    assert set(o["path_results"]) == set(H.MAIN_KERNELS)
    assert o["oracle_path"] in H.MAIN_KERNELS and o["nnz"] == a.nnz and o["mode"] == "warm"
    for k, v in o["path_results"].items():
        assert v["exec_ms"] > 0 and v["plan_ms"] == 0 and v["gflops"] > 0
    c = H.run_oracle_cold(rp, ci, va, B)
    assert all(v["total_ms"] >= v["exec_ms"] for v in c["path_results"].values())
    r = H.run_router_warm(rp, ci, va, B, warmup=1, iters=2)
    want = O.route(r["plan"]["feature_values"]["avg_nnz_per_row"], r["plan"]["feature_values"]["degree_cv"], a.M, 64)
    assert r["router_path"] == want["chosen_path"] and r["timing"]["exec_ms"] > 0


def test_cusparse_passthrough_matches(graph):
    a, rp, ci, va, B = graph
    C = ra_spmm.spmm_csr_direct(rp, ci, va, B)
    Cc = H.spmm_cusparse(rp, ci, va, B)
    assert float((C - Cc).norm() / Cc.norm()) < 1e-5


def test_cusparse_benchmark_passthroughs_have_the_reference_dict_shape(graph):
    """benchmark_cusparse / _cold / _fp16 / _fp16_cold (bindings/ra_bindings.cpp:838-1037): keys the sweep
    driver reads (ra_real_graph_eval.py:540-560) and a sane precision-matched product."""
    a, rp, ci, va, B = graph
    warm = ra_spmm.benchmark_cusparse(rp, ci, va, B, warmup=1, iters=2)
    cold = ra_spmm.benchmark_cusparse_cold(rp, ci, va, B, 1)
    w16 = ra_spmm.benchmark_cusparse_fp16(rp, ci, va, B, warmup=1, iters=2)
    c16 = ra_spmm.benchmark_cusparse_fp16_cold(rp, ci, va, B, 1)
    for d, path in ((warm, "CUSPARSE"), (cold, "CUSPARSE"), (w16, "CUSPARSE_FP16"), (c16, "CUSPARSE_FP16")):
        assert {"plan_ms", "exec_ms", "total_ms", "gflops", "path", "preprocess_ms", "cusparse_algorithm",
                "in_main_portfolio", "legacy_baseline", "external_baseline"} <= set(d)
        assert d["path"] == path and d["exec_ms"] > 0 and d["total_ms"] >= d["exec_ms"]
    assert warm["plan_ms"] == 0 and cold["plan_ms"] > 0 and cold["in_main_portfolio"] and not w16["in_main_portfolio"]
    C = ra_spmm.spmm_csr_direct(rp, ci, va, B)
    C16 = ra_spmm.spmm_cusparse_fp16(rp, ci, va, B)
    assert C16.dtype == torch.float32 and float((C - C16).norm() / C.norm()) < 5e-3
    plan = ra_spmm.make_cusparse_plan(rp, ci, va, torch.empty_like(B))        # the callers pass a template operand
    assert float((ra_spmm.run_cusparse_plan(plan, B) - C).norm() / C.norm()) < 1e-5


def test_plan_checksums_are_reproducible_and_match_the_oracle(graph):
    a, rp, ci, va, B = graph
    p1 = ra_spmm.make_community_tc_plan(rp, ci, va, a.M, a.K, 64)
    p2 = ra_spmm.make_community_tc_plan(rp.cpu(), ci.cpu(), va.cpu(), a.M, a.K, 64)
    c1, c2 = H.plan_checksums(p1), H.plan_checksums(p2)
    assert c1 == c2 and set(c1) == {"block_offsets", "atox", "vals_f16", "win_rows"}
    wr = O.community_order(a.rowptr, a.colind, a.M)
    want = O.tile_plan(a.rowptr, a.colind, a.vals, a.M, a.K, 64, win_rows=wr)
    assert c1["atox"] == f"{H.fnv1a64(want['atox']):016x}"
    assert c1["vals_f16"] == f"{H.fnv1a64(want['vals_f16']):016x}"
    assert c1["win_rows"] == f"{H.fnv1a64(wr):016x}"


def test_lifecycle_choice_from_the_cost_model_runs(graph):
    """Kernel ranked best by the shipped model for 1 and for 1000 calls is built and run through
    the label-driven plan helpers, as the reference's lifecycle router does with its choice."""
    a, rp, ci, va, B = graph
    plan = ra_spmm.make_router_plan(rp, ci, va, a.M, a.K, 64)
    fv = plan["feature_values"]
    x = CM.design_rows(a.M, a.nnz, 64, fv["avg_nnz_per_row"], fv["degree_cv"])
    model = CM.CostModel.load()
    ref = ra_spmm.spmm_csr_direct(rp, ci, va, B)
    for calls in (1, 1000):
        est = model.lifecycle_ms(x, calls, allowed=plan["feasible_by_path"])
        best = min(est, key=est.get)
        assert best in CM.PORTFOLIO
        kp = H.build_kernel_plan(best, rp, ci, va, a.M, a.K, 64)
        C = H.run_planned_kernel(best, kp, rp, ci, va, B)
        assert float((C - ref).norm() / ref.norm()) < 5e-3
