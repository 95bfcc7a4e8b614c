"""Generates tests/golden/analysis_golden.json from the reference's own compute_router_features
(router/router_features.cpp:113-432) compiled into oracle/_ref/libra_ref_router.so
(make -C oracle REF=<RA-SpMM checkout>): the 33 float fields as float32 bit patterns and the
integer fields, for seeded synthetic matrices that the tests regenerate.

    python tests/golden/make_analysis_golden.py
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import ref_bindings as R  # noqa: E402
from ra_spmm_b200 import generators as G  # noqa: E402

# (configuration, scale, N): shapes of the five benchmark families at test size, plus edge shapes
CASES = [("C1", 1.0, 64), ("C1", 0.05, 512), ("C2", 0.01, 128), ("C2", 0.05, 128), ("C3", 0.02, 256),
         ("C4", 2 ** -9, 64), ("C4", 2 ** -7, 64), ("C5", 0.004, 47), ("C5", 0.004, 256)]


def special_cases():
    """Hand-made shapes: empty rows, a single row, M not a multiple of 16, unsorted columns."""
    rng = np.random.default_rng(7)
    out = []
    rp = np.array([0, 0, 3, 3, 3, 7, 8], dtype=np.int32)
    ci = np.array([5, 1, 9, 0, 2, 4, 6, 3], dtype=np.int32)          # first row unsorted
    out.append(("ragged6", rp, ci, 6, 10, 32))
    out.append(("single", np.array([0, 4], dtype=np.int32), np.array([0, 1, 2, 3], dtype=np.int32), 1, 4, 16))
    lens = rng.integers(0, 40, size=1000)
    lens[::7] = 0
    rp = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    ci = np.concatenate([np.sort(rng.choice(777, size=int(n), replace=False)) for n in lens]).astype(np.int32)
    out.append(("rand1000", rp, ci, 1000, 777, 128))
    return out


def encode(d):
    return {k: (int(np.float32(v).view(np.uint32)) if isinstance(v, np.floating) else int(v)) for k, v in d.items()}


def main():
    out = []
    for name, scale, N in CASES:
        a, _, _ = G.make_config(name, scale)
        out.append({"config": name, "scale": scale, "N": N, "M": a.M, "K": a.K, "nnz": a.nnz,
                    "fields": encode(R.ref_analyze_matrix(a.rowptr, a.colind, a.M, a.K, N))})
    for label, rp, ci, M, K, N in special_cases():
        out.append({"special": label, "N": N, "M": M, "K": K,
                    "fields": encode(R.ref_analyze_matrix(rp, ci, M, K, N))})
    path = Path(__file__).with_name("analysis_golden.json")
    path.write_text(json.dumps(out, indent=1) + "\n")
    print(f"wrote {len(out)} cases to {path}")


if __name__ == "__main__":
    main()
