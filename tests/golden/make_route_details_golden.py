"""Generates tests/golden/route_details_golden.json from the reference's own router compiled
into oracle/_ref/libra_ref_router.so (make -C oracle REF=<RA-SpMM checkout>): for a fixed list
of production feature values, the eight diagnostic scores (float32 bit patterns), the
rejection code and text of every path and the gate margins that the reference's
route_dispatch leaves in its plan.

    python tests/golden/make_route_details_golden.py
"""
import json
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import ra_oracle as O  # noqa: E402
from oracle import ref_bindings as R  # noqa: E402

CASES = [  # (avg degree, degree CV, M, N)
    (16.0, 0.0, 4096, 64), (10.85, 6.81, 1048576, 128), (489.87, 0.0431, 232960, 256),
    (30.59, 11.3, 4194304, 64), (50.8, 0.14, 2449029, 47), (50.8, 0.14, 2449029, 256),
    (3.9, 0.1, 100000, 32), (3.9, 0.1, 100000, 512), (6.0, 0.3, 50000, 128), (6.0, 0.3, 50000, 256),
    (12.0, 0.79, 149999, 63), (12.0001, 0.8, 150000, 63), (30.0, 1.0, 15000, 64), (30.0, 1.0, 15000, 128),
    (30.0, 1.0, 15000, 256), (30.0, 2.0, 500000, 128), (8.0, 1.2, 300000, 128), (45.0, 2.5, 100000, 15),
    (45.0, 2.5, 100000, 8), (20.0, 3.5, 100000, 64), (20.0, 3.5, 300000, 64), (2000.0, 0.5, 50_000_000, 64),
    (0.0, 0.0, 10, 16), (24.99, 1.79, 19999, 95),
]


def main():
    out = []
    for d, cv, M, N in CASES:
        r = R.ref_route_details_from_features(d, 0.0, cv, M, M, N, 0)
        out.append({"avg": d, "cv": cv, "M": M, "N": N,
                    "score_bits": [int(np.float32(x).view(np.uint32)) for x in r.scores],
                    "codes": [O.REJECT_NAMES[c] for c in r.rejection_code],
                    "details": [r.rejection_detail[i].value.decode() for i in range(len(O.PATH_NAMES))],
                    "margin_bits": [int(np.float32(r.gate_margin_raw).view(np.uint32)),
                                    int(np.float32(r.gate_margin_norm).view(np.uint32))]})
    (Path(__file__).parent / "route_details_golden.json").write_text(json.dumps(out, indent=0))
    print(len(out), "cases")


if __name__ == "__main__":
    main()
