"""Route decisions and host features: oracle, C ABI and (when built) the
reference's own compiled router against the committed golden vectors."""
import ctypes as C
import json
import sys
from pathlib import Path

import numpy as np
import pytest

from oracle import ra_oracle as O
from oracle import ref_bindings as R
from ra_spmm_b200 import _capi

GOLD = Path(__file__).parent / "golden"
sys.path.insert(0, str(GOLD))
from make_features_golden import degrees  # noqa: E402

KNOWN = json.loads((GOLD / "router_known_answers.json").read_text())
FEATS = json.loads((GOLD / "features_golden.json").read_text())


def _capi_route(lib, d, cv, M, N, nnz=0):
    f = _capi.RaFeatures()
    f.avg_nnz_per_row = float(np.float32(d)); f.degree_cv = float(np.float32(cv))
    f.matrix_M = M; f.matrix_K = M; f.output_dim_N = N; f.total_nnz = nnz
    out = _capi.RaRoute()
    assert lib.ra_route(C.byref(f), 0, C.byref(out)) == 0
    return out


def test_192_known_answers(lib):
    """Published decision == Python mirror == compiled route_dispatch == oracle == C ABI."""
    assert len(KNOWN) == 192
    for k in KNOWN:
        d, cv = np.float32(k["nnz"] / k["M"]), np.float32(k["cv_d"])
        cpp = k["cpp_path"] + ("_TF32" if k["cpp_use_tf32"] else "")
        assert k["published"] == k["python_mirror"] == cpp
        o = O.route(d, cv, k["M"], k["N"])
        assert O.route_label(o) == k["published"]
        assert o["decision_reason"] == k["cpp_reason"]
        assert float(o["estimated_risk"]) == k["cpp_risk"]
        assert [int(o["feasible_by_path"][n]) for n in O.PATH_NAMES] == k["cpp_feasible"]
        c = _capi_route(lib, d, cv, k["M"], k["N"], k["nnz"])
        assert O.PATH_NAMES[c.chosen_path] == k["cpp_path"]
        assert bool(c.use_tf32) == k["cpp_use_tf32"]
        assert c.decision_reason.decode() == k["cpp_reason"]
        assert float(c.estimated_risk) == k["cpp_risk"]
        assert [int(x) for x in c.feasible] == k["cpp_feasible"]


def test_host_features_golden(lib):
    """Two-pass host features, bit-exact with the reference (serial order)."""
    bits = lambda x: int(np.float32(x).view(np.uint32))
    for g in FEATS:
        spec = g["spec"]
        d = degrees(spec)
        rowptr = np.zeros(spec["M"] + 1, dtype=np.int64)
        np.cumsum(d, out=rowptr[1:])
        rp = rowptr.astype(np.int32)
        o = O.features_host(rp, spec["M"], spec["M"], spec["N"])
        assert (o["total_nnz"], bits(o["avg_nnz_per_row"]), bits(o["std_nnz_per_row"]),
                bits(o["degree_cv"])) == (g["total_nnz"], g["avg_bits"], g["std_bits"], g["cv_bits"])
        f = _capi.RaFeatures()
        assert lib.ra_features_from_rowptr_host(rp.ctypes.data, spec["M"], spec["M"], spec["N"], C.byref(f)) == 0
        assert (f.total_nnz, bits(f.avg_nnz_per_row), bits(f.std_nnz_per_row), bits(f.degree_cv)) == \
               (g["total_nnz"], g["avg_bits"], g["std_bits"], g["cv_bits"])
        r = O.route(o["avg_nnz_per_row"], o["degree_cv"], spec["M"], spec["N"])
        assert (r["chosen_path"], r["use_tf32"], r["decision_reason"]) == (g["path"], g["use_tf32"], g["reason"])
        assert bits(r["estimated_risk"]) == g["risk_bits"]
        rt = _capi.RaRoute()
        assert lib.ra_route(C.byref(f), 0, C.byref(rt)) == 0
        assert (O.PATH_NAMES[rt.chosen_path], bool(rt.use_tf32), rt.decision_reason.decode()) == \
               (g["path"], g["use_tf32"], g["reason"])
        assert [int(x) for x in rt.feasible] == g["feasible"]


def test_rowptr_offset_and_null(lib):
    """rowptr[0] != 0 is honoured (router/router_features.cpp:91); null / M<=0 early-outs."""
    rp = np.array([5, 8, 8, 20], dtype=np.int32)
    o = O.features_host(rp, 3, 3, 64)
    f = _capi.RaFeatures()
    assert lib.ra_features_from_rowptr_host(rp.ctypes.data, 3, 3, 64, C.byref(f)) == 0
    assert f.total_nnz == o["total_nnz"] == 15
    assert np.float32(f.degree_cv) == o["degree_cv"]
    assert lib.ra_features_from_rowptr_host(None, 3, 3, 64, C.byref(f)) == 0
    assert f.total_nnz == 0 and f.matrix_M == 3
    assert lib.ra_features_from_rowptr_host(rp.ctypes.data, 0, 3, 64, C.byref(f)) == 0
    assert f.total_nnz == 0


def test_random_sweep_against_compiled_reference(lib):
    """Oracle and C ABI against the reference's route_dispatch on random features
    concentrated around every threshold (skipped when oracle/_ref is not built)."""
    if R.router() is None:
        pytest.skip("oracle/_ref/libra_ref_router.so not built")
    rng = np.random.default_rng(7)
    thr_d = [4.5, 5.0, 7.0, 9.0, 12.0, 25.0, 40.0]
    thr_cv = [0.2, 0.7, 0.8, 1.10, 1.45, 1.5, 1.8, 3.0, 5.0]
    thr_m = [20000, 25000, 250000]
    for t in range(6000):
        d = np.float32(rng.choice(thr_d) + rng.choice([0, 0, 1e-6, -1e-6, 0.5, -0.5, rng.uniform(-5, 30)]))
        cv = np.float32(rng.choice(thr_cv) + rng.choice([0, 0, 1e-7, -1e-7, 0.05, -0.05, rng.uniform(-1, 3)]))
        d = max(d, np.float32(0)); cv = max(cv, np.float32(0))
        M = int(rng.choice(thr_m) + rng.choice([0, -1, 1, 1000, -1000, rng.integers(0, 2_000_000_000)]))
        N = int(rng.choice([8, 15, 16, 32, 47, 64, 95, 96, 128, 255, 256, 257, 512]))
        ref = R.ref_route_from_features(d, 0.0, cv, M, M, N, 0)
        o = O.route(d, cv, M, N)
        c = _capi_route(lib, d, cv, M, N)
        want = (O.PATH_NAMES[ref.chosen_path], bool(ref.use_tf32), ref.decision_reason.decode(),
                float(ref.estimated_risk), [int(x) for x in ref.feasible])
        assert (o["chosen_path"], o["use_tf32"], o["decision_reason"], float(o["estimated_risk"]),
                [int(o["feasible_by_path"][n]) for n in O.PATH_NAMES]) == want
        assert (O.PATH_NAMES[c.chosen_path], bool(c.use_tf32), c.decision_reason.decode(),
                float(c.estimated_risk), [int(x) for x in c.feasible]) == want


def test_config_routes():
    """Routes of the benchmark configurations under the reference's rules."""
    assert O.route_label(O.route(16.0, 0.0, 4096, 64)) == "TC_DIRECT"            # C1
    assert O.route_label(O.route(10.85, 6.8, 1048576, 128)) == "ZERO_OVERHEAD_CSR"  # C2
    assert O.route_label(O.route(490.0, 0.05, 232960, 256)) == "TC_DIRECT"        # C3
    assert O.route_label(O.route(30.6, 11.3, 4194304, 64)) == "ZERO_OVERHEAD_CSR"  # C4
    assert O.route_label(O.route(51.0, 0.14, 2449029, 47)) == "TC_DIRECT"          # C5


def _capi_details(lib, d, cv, M, N):
    f = _capi.RaFeatures(avg_nnz_per_row=float(d), degree_cv=float(cv), output_dim_N=N, matrix_M=M, matrix_K=M)
    r = _capi.RaRoute()
    assert lib.ra_route(C.byref(f), 0, C.byref(r)) == 0
    det = _capi.RaRouteDetails()
    assert lib.ra_route_details(C.byref(f), 0, C.byref(r), C.byref(det)) == 0
    return det


def test_scores_and_rejections_against_compiled_reference(lib):
    """scores (float bits), rejection code and text of every path, and the gate margins: the
    C ABI and the oracle against the reference's compute_router_scores + route_dispatch."""
    if R.router() is None or not hasattr(R.router(), "ref_route_details_from_features"):
        pytest.skip("oracle/_ref/libra_ref_router.so not built with the details export")
    rng = np.random.default_rng(11)
    thr_d = [4.5, 5.0, 7.0, 9.0, 12.0, 25.0, 40.0]
    thr_cv = [0.2, 0.7, 0.8, 1.10, 1.45, 1.5, 1.8, 3.0, 5.0]
    bits = lambda x: np.float32(x).tobytes()
    for t in range(3000):
        d = max(np.float32(rng.choice(thr_d) + rng.choice([0, 1e-6, -1e-6, 0.5, rng.uniform(-5, 600)])), np.float32(0))
        cv = max(np.float32(rng.choice(thr_cv) + rng.choice([0, 1e-7, -1e-7, 0.05, rng.uniform(-1, 30)])), np.float32(0))
        M = int(rng.choice([20000, 25000, 149999, 150000, 250000]) + rng.choice([0, -1, 1, rng.integers(0, 2_000_000_000)]))
        N = int(rng.choice([8, 15, 16, 32, 47, 63, 64, 95, 96, 128, 255, 256, 257, 512, 1024]))
        ref = R.ref_route_details_from_features(d, 0.0, cv, M, M, N, 0)
        o = O.route_details(d, cv, M, N)
        c = _capi_details(lib, d, cv, M, N)
        for i, k in enumerate(O.SCORE_KEYS):
            assert bits(ref.scores[i]) == bits(c.scores[i]) == bits(o["scores"][k]), (k, d, cv, M, N)
        for i, name in enumerate(O.PATH_NAMES):
            want = (O.REJECT_NAMES[ref.rejection_code[i]], ref.rejection_detail[i].value.decode())
            assert (lib.ra_reject_reason_name(c.rejection_code[i]).decode(), c.rejection_detail[i].value.decode()) == want, (name, d, cv, M, N)
            assert (o["rejection_codes"][name], o["rejection_details"][name]) == want, (name, d, cv, M, N)
        assert bits(ref.gate_margin_raw) == bits(c.gate_margin_raw) == bits(0.0)
        assert bits(ref.gate_margin_norm) == bits(c.gate_margin_norm) == bits(0.0)


def test_scores_and_rejections_against_the_golden_fixture(lib):
    """Same check against tests/golden/route_details_golden.json (written from the reference's
    compiled router by make_route_details_golden.py), for boxes without oracle/_ref."""
    cases = json.loads((Path(__file__).parent / "golden" / "route_details_golden.json").read_text())
    assert len(cases) >= 20
    for g in cases:
        c = _capi_details(lib, g["avg"], g["cv"], g["M"], g["N"])
        o = O.route_details(g["avg"], g["cv"], g["M"], g["N"])
        assert [int(np.float32(x).view(np.uint32)) for x in c.scores] == g["score_bits"], g
        assert [int(np.float32(o["scores"][k]).view(np.uint32)) for k in O.SCORE_KEYS] == g["score_bits"], g
        assert [lib.ra_reject_reason_name(x).decode() for x in c.rejection_code] == g["codes"], g
        assert [c.rejection_detail[i].value.decode() for i in range(len(O.PATH_NAMES))] == g["details"], g
        assert [o["rejection_codes"][n] for n in O.PATH_NAMES] == g["codes"]
        assert [o["rejection_details"][n] for n in O.PATH_NAMES] == g["details"]
