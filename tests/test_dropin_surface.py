"""The reference's own callers against the drop-in module `ra_spmm` (repository root).

Two levels:
  * without a GPU: every `ra_spmm.<name>` (or `spmm_next.<name>`) that the reference's
    hot-path callers touch resolves on the drop-in module, with the keyword names the callers
    use - read from the callers' source text, so the check follows the reference as it is;
  * on a GPU, when an RA-SpMM checkout is available (RA_REFERENCE_DIR): the callers' own
    functions run unmodified on the drop-in module - build_kernel_plan / run_planned_kernel
    for the eight kernel labels, the lifecycle router with the shipped cost model, and the
    GCN harness' GraphBackend with its validation.
The reference tree is never copied; both levels skip when it is absent.
"""
import ast
import importlib
import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF = Path(os.environ.get("RA_REFERENCE_DIR") or ROOT.parent / "reference")
CALLERS = ["ra_real_graph_eval.py", "ra_runtime_router.py", "ra_router_parity_test.py",
           "bench/profile_case_ra.py", "gnn_bench/router_vs_baselines_gcn.py"]
# entry points of kernels that are not part of the deployed path (retired from the router,
# legacy ablation roster): the drop-in module does not carry them
OUT_OF_SCOPE = {"make_rode_enhanced_plan", "run_rode_enhanced_plan", "make_row_split_plan", "run_row_split_plan",
                "make_tc_reordered_plan", "run_tc_reordered_plan", "make_hybrid_tc_cuda_plan",
                "run_hybrid_tc_cuda_plan"}

need_ref = pytest.mark.skipif(not (REF / "ra_real_graph_eval.py").exists(), reason="no RA-SpMM checkout available")


def _module_uses(path: Path):
    """(attribute name, keyword names) for every use of the extension module in a caller."""
    tree = ast.parse(path.read_text())
    aliases = set()
    for node in ast.walk(tree):
        if isinstance(node, ast.Import):
            for a in node.names:
                if a.name == "ra_spmm":
                    aliases.add(a.asname or a.name)
    uses = {}
    for node in ast.walk(tree):
        if isinstance(node, ast.Attribute) and isinstance(node.value, ast.Name) and node.value.id in aliases:
            uses.setdefault(node.attr, set())
        if (isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute)
                and isinstance(node.func.value, ast.Name) and node.func.value.id in aliases):
            uses.setdefault(node.func.attr, set()).update(k.arg for k in node.keywords if k.arg)
    return uses


@need_ref
def test_every_entry_point_the_callers_use_resolves():
    import inspect
    sys.path.insert(0, str(ROOT))
    mod = importlib.import_module("ra_spmm")
    seen = 0
    for rel in CALLERS:
        for name, kwargs in _module_uses(REF / rel).items():
            if name in OUT_OF_SCOPE:
                continue
            assert hasattr(mod, name), f"{rel} uses ra_spmm.{name}, which the drop-in module lacks"
            params = inspect.signature(getattr(mod, name)).parameters
            for k in kwargs:
                assert k in params, f"{rel} calls ra_spmm.{name}({k}=...), unknown keyword"
            seen += 1
    assert seen >= 25


@need_ref
@pytest.mark.gpu
def test_reference_callers_run_unmodified(cuda):
    import torch
    from ra_spmm_b200 import cost_model as CM
    from ra_spmm_b200 import generators as G
    sys.path[:0] = [str(ROOT), str(REF)]
    for m in ("ra_spmm", "ra_real_graph_eval", "ra_runtime_router"):
        sys.modules.pop(m, None)
    ev = importlib.import_module("ra_real_graph_eval")
    rr = importlib.import_module("ra_runtime_router")
    assert Path(sys.modules["ra_spmm"].__file__).parent == ROOT          # the drop-in, not a built reference
    a = G.chung_lu_power_law(n=20000, seed=3)
    rp, ci, va = a.torch(cuda)
    N = 64
    B = G.dense(a.K, N, 3).to(cuda)
    want = torch.sparse.mm(torch.sparse_csr_tensor(rp.long(), ci.long(), va, size=(a.M, a.K)), B)
    for label in ("CSR_DIRECT", "ZERO_OVERHEAD_CSR", "TC_DIRECT", "TC_DIRECT_TF32", "COMMUNITY_TC",
                  "COMMUNITY_TC_TF32", "SEGMENT_HYBRID", "SEGMENT_HYBRID_TF32", "TC_DIRECT_ZC"):
        plan = ev.build_kernel_plan(label, rp.cpu(), ci.cpu(), va.cpu(), a.M, a.K, N)
        got = ev.run_planned_kernel(label, plan, rp, ci, va, B)
        tol = 1e-5 if label in ("CSR_DIRECT", "ZERO_OVERHEAD_CSR") else 5e-3
        assert float((got - want).norm() / want.norm()) < tol, label
    got = ev.run_kernel("CUSPARSE", rp, ci, va, B, {}, "k")
    assert float((got - want).norm() / want.norm()) < 1e-5
    plan = rr.make_runtime_router_plan(rp, ci, va, a.M, a.K, N, expected_calls=100, model_path=CM.SHIPPED_MODEL)
    assert plan.chosen_path in CM.PORTFOLIO
    got = plan.run(rp, ci, va, B)
    assert float((got - want).norm() / want.norm()) < 5e-3
