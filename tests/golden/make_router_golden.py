"""Generates tests/golden/router_known_answers.json.

Usage: make_router_golden.py <RA-SpMM checkout> (or RA_REFERENCE_DIR in the environment), with
oracle/_ref built (make -C oracle REF=<checkout>). For every (graph, N) row of the reference's
published sweep (fgcs_results/revision/tf32/final_fair_v3.csv: M, nnz, cv_d;
router_quality_v8.csv: the routed kernel) it records the inputs (M, nnz, cv_d, N)
and three answers: the label the reference published, the label of the
reference's Python mirror ra_router_eval.simple_router, and the decision of the
reference's C++ route_dispatch compiled from source. Dataset names are not kept.
"""
import csv
import json
import os
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["RA_REFERENCE_DIR"])
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(REF))

from oracle import ref_bindings as R  # noqa: E402
import ra_router_eval  # the reference's Python mirror  # noqa: E402

NAMES = ["CSR_DIRECT", "CSR_ADAPTIVE", "STAGED_REUSE", "TC_SPARSE", "ROW_SPLIT_CUDA", "TC_REORDERED",
         "HYBRID_TC_CUDA", "CUSPARSE", "RODE_ENHANCED", "VECTORIZED_COARSE", "LOCALITY_TILED",
         "TC_DIRECT", "COMMUNITY_TC", "ZERO_OVERHEAD_CSR", "SEGMENT_HYBRID"]

feat = {}
for row in csv.DictReader(open(REF / "fgcs_results/revision/tf32/final_fair_v3.csv")):
    feat[(row["dataset"], int(row["N"]))] = (int(row["M"]), int(row["nnz"]), float(row["cv_d"]))
out = []
for row in csv.DictReader(open(REF / "fgcs_results/revision/tf32/router_quality_v8.csv")):
    M, nnz, cv = feat[(row["dataset"], int(row["N"]))]
    N = int(row["N"])
    d32, cv32 = np.float32(nnz / M), np.float32(cv)
    rr = R.ref_route_from_features(d32, 0.0, cv32, M, M, N, nnz)
    out.append(dict(
        M=M, nnz=nnz, cv_d=cv, N=N,
        published=row["router_kernel"],
        python_mirror=ra_router_eval.simple_router(nnz / M, cv, M, N, nnz),
        cpp_path=NAMES[rr.chosen_path], cpp_use_tf32=bool(rr.use_tf32),
        cpp_reason=rr.decision_reason.decode(), cpp_risk=float(rr.estimated_risk),
        cpp_feasible=[int(x) for x in rr.feasible]))
(ROOT / "tests/golden/router_known_answers.json").write_text(json.dumps(out, indent=0))
print(len(out), "rows")
