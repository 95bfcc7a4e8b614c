"""The 34 structural features (analyze_matrix): the numpy restatement against golden vectors
generated from the reference's own compute_router_features (router/router_features.cpp:113-432),
against the reference compiled here where it is present, and the CUDA entry point through the
C ABI against both. Every float field is compared by bit pattern."""
import importlib.util
import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
from oracle import ra_oracle as O  # noqa: E402
from oracle import ref_bindings as R  # noqa: E402
from ra_spmm_b200 import generators as G  # noqa: E402

GOLDEN = json.loads((ROOT / "tests" / "golden" / "analysis_golden.json").read_text())
_spec = importlib.util.spec_from_file_location("make_analysis_golden", ROOT / "tests" / "golden" / "make_analysis_golden.py")
_gen = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(_gen)
SPECIAL = {label: (rp, ci, M, K, N) for label, rp, ci, M, K, N in _gen.special_cases()}


def case_matrix(case):
    if "special" in case:
        rp, ci, M, K, N = SPECIAL[case["special"]]
        return rp, ci, M, K, N
    a, _, _ = G.make_config(case["config"], case["scale"])
    assert (a.M, a.K, a.nnz) == (case["M"], case["K"], case["nnz"])
    return a.rowptr, a.colind, a.M, a.K, case["N"]


def case_id(case):
    return case.get("special") or f"{case['config']}x{case['scale']}N{case['N']}"


def bits(v):
    return int(np.float32(v).view(np.uint32))


def assert_fields(got, want_bits, what):
    for k, w in want_bits.items():
        g = got[k]
        g = int(g) if k in R.ANALYSIS_INT_KEYS else bits(g)
        assert g == w, f"{what}: {k} = {got[k]!r} (bits {g}) but the reference gives bits {w}"


@pytest.mark.parametrize("case", GOLDEN, ids=case_id)
def test_oracle_matches_the_golden_vectors(case):
    rp, ci, M, K, N = case_matrix(case)
    assert_fields(O.analyze_matrix(rp, ci, M, K, N), case["fields"], "oracle")


def test_oracle_matches_the_compiled_reference_on_fresh_matrices():
    lib = R.router()
    if lib is None or not hasattr(lib, "ref_analyze_matrix"):
        pytest.skip("the reference's router is not built here")
    rng = np.random.default_rng(11)
    for trial in range(6):
        M = int(rng.integers(1, 400)); K = int(rng.integers(1, 900))
        lens = np.minimum(rng.integers(0, 60, size=M), K)
        if trial % 2:
            lens[rng.integers(0, M)] = min(K, 500)                 # one hub row
        rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
        ci = (np.concatenate([np.sort(rng.choice(K, size=int(n), replace=False)) for n in lens]).astype(np.int32)
              if lens.sum() else np.zeros(0, dtype=np.int32))
        N = int(rng.choice([16, 64, 128, 300, 512]))
        ref = R.ref_analyze_matrix(rp, ci, M, K, N)
        mine = O.analyze_matrix(rp, ci, M, K, N)
        assert_fields(mine, {k: (int(v) if k in R.ANALYSIS_INT_KEYS else bits(v)) for k, v in ref.items()},
                      f"trial {trial} (M={M}, K={K}, N={N})")


def test_degenerate_shapes_give_zeros():
    z = O.analyze_matrix(np.zeros(1, dtype=np.int32), np.zeros(0, dtype=np.int32), 0, 0, 64)
    assert all(v == 0 for v in z.values())
    e = O.analyze_matrix(np.zeros(5, dtype=np.int32), np.zeros(0, dtype=np.int32), 4, 4, 64)
    assert e["matrix_M"] == 4 and e["total_nnz"] == 0 and e["avg_nnz_per_row"] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("where", ["host", "device"])
@pytest.mark.parametrize("case", GOLDEN, ids=case_id)
def test_cuda_analysis_is_bit_exact(case, where):
    import torch
    from ra_spmm_b200 import ra_spmm
    rp, ci, M, K, N = case_matrix(case)
    trp, tci = torch.from_numpy(np.ascontiguousarray(rp, dtype=np.int32)), torch.from_numpy(np.ascontiguousarray(ci, dtype=np.int32))
    if where == "device":
        trp, tci = trp.cuda(), tci.cuda()
    d = ra_spmm.analyze_matrix(trp, tci, M, K, N)
    want = dict(case["fields"])
    assert d["nnz"] == want["total_nnz"]
    for k in ("output_dim_N", "matrix_M", "matrix_K", "total_nnz"):    # context fields are not in the dict
        want.pop(k)
    got = {k: (np.float32(v) if k != "tc_candidate_tiles" else v) for k, v in d.items() if k != "nnz"}
    assert set(got) == set(want)
    assert_fields(got, want, f"cuda ({where} CSR)")


@pytest.mark.gpu
def test_cuda_analysis_rejects_duplicates_and_handles_empty():
    import torch
    from ra_spmm_b200 import ra_spmm
    z = ra_spmm.analyze_matrix(torch.zeros(5, dtype=torch.int32), torch.zeros(0, dtype=torch.int32), 4, 4, 64)
    assert z["nnz"] == 0 and z["avg_nnz_per_row"] == 0.0
    # 300 copies of one entry: a tile with more than 256 entries cannot come from duplicate-free CSR
    rp = torch.tensor([0, 300], dtype=torch.int32)
    ci = torch.zeros(300, dtype=torch.int32)
    with pytest.raises(RuntimeError):
        ra_spmm.analyze_matrix(rp, ci, 1, 4, 64)


@pytest.mark.gpu
def test_cuda_analysis_full_size_against_the_compiled_reference():
    """Configuration 2 at full size (1,048,576 rows, 11.4 M entries, 6 M nonempty tiles): the sorted-key
    histogram and the two chained row sorts at a size where they run many tiles per pass."""
    import torch
    from ra_spmm_b200 import ra_spmm
    lib = R.router()
    if lib is None or not hasattr(lib, "ref_analyze_matrix"):
        pytest.skip("the reference's router is not built here")
    a, N, _ = G.cached_config("C2", 1.0)
    ref = R.ref_analyze_matrix(a.rowptr, a.colind, a.M, a.K, N)
    d = ra_spmm.analyze_matrix(torch.from_numpy(a.rowptr).cuda(), torch.from_numpy(a.colind).cuda(), a.M, a.K, N)
    for k in R.ANALYSIS_FLOAT_KEYS:
        assert bits(d[k]) == bits(ref[k]), f"{k}: {d[k]!r} vs reference {ref[k]!r}"
    assert d["tc_candidate_tiles"] == ref["tc_candidate_tiles"] and d["nnz"] == ref["total_nnz"]
