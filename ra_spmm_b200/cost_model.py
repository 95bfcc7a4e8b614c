"""The fitted kernel cost model that the reference's lifecycle router reads.

ra_runtime_router.py (reference project) loads `results/router/runtime_cost_model.json`
and evaluates, per kernel, two log-linear models of one seven-term design row
(ra_runtime_router.py:24-32, 73-86). The reference ships the router but not the file;
this module owns the file for B200: its schema, the shipped fit
(`runtime_cost_model.json`, produced by `fit_cost_model.py` on a B200) and a small
evaluator used by the fit script and the tests. The router itself is not restated
here: the reference's own module runs on this library unchanged with
`make_runtime_router_plan(..., model_path=cost_model.SHIPPED_MODEL)`.

Schema: {"kernels": {<kernel label>: {"setup_coefficients": [7 floats],
"warm_coefficients": [7 floats]}}, ...}; a cost in ms is exp(coefficients . row).
"""
from __future__ import annotations

import json
from pathlib import Path

import numpy as np

SHIPPED_MODEL = Path(__file__).resolve().parent / "runtime_cost_model.json"
PORTFOLIO = ("CSR_DIRECT", "ZERO_OVERHEAD_CSR", "TC_DIRECT", "COMMUNITY_TC", "SEGMENT_HYBRID")
TERMS = ("1", "log1p M", "log1p nnz", "log1p N", "log1p nnz*N", "log1p avg", "log1p cv")


def design_rows(M, nnz, N, avg_degree, degree_cv) -> np.ndarray:
    """[..., 7] design rows; arguments broadcast against each other."""
    M, nnz, N, avg, cv = np.broadcast_arrays(*(np.asarray(v, dtype=np.float64)
                                               for v in (M, nnz, N, avg_degree, degree_cv)))
    return np.stack([np.ones_like(M), np.log1p(M), np.log1p(nnz), np.log1p(N),
                     np.log1p(nnz * N), np.log1p(avg), np.log1p(cv)], axis=-1)


class CostModel:
    """Coefficient tables of a model file, evaluated with numpy."""

    def __init__(self, kernels: dict, meta: dict | None = None):
        self.meta = dict(meta or {})
        self.setup = {k: np.asarray(v["setup_coefficients"], dtype=np.float64) for k, v in kernels.items()}
        self.warm = {k: np.asarray(v["warm_coefficients"], dtype=np.float64) for k, v in kernels.items()}
        for k in self.setup:
            if self.setup[k].shape != (len(TERMS),) or self.warm[k].shape != (len(TERMS),):
                raise ValueError(f"cost model: kernel {k} needs {len(TERMS)} coefficients per table")

    @classmethod
    def load(cls, path=SHIPPED_MODEL) -> "CostModel":
        doc = json.loads(Path(path).read_text())
        return cls(doc["kernels"], {k: v for k, v in doc.items() if k != "kernels"})

    @classmethod
    def fit(cls, samples: dict, meta: dict | None = None) -> "CostModel":
        """samples: kernel -> list of (design row, setup ms, warm ms); least squares in log space."""
        kernels = {}
        for k, rows in samples.items():
            X = np.asarray([r[0] for r in rows], dtype=np.float64)
            solve = lambda y: np.linalg.lstsq(X, np.log(np.asarray(y, dtype=np.float64)), rcond=None)[0]
            kernels[k] = {"setup_coefficients": solve([r[1] for r in rows]).tolist(),
                          "warm_coefficients": solve([r[2] for r in rows]).tolist()}
        return cls(kernels, meta)

    def kernels(self):
        return list(self.setup)

    def costs_ms(self, kernel: str, rows: np.ndarray):
        """(setup ms, warm ms) of one kernel for each design row."""
        rows = np.asarray(rows, dtype=np.float64)
        return np.exp(rows @ self.setup[kernel]), np.exp(rows @ self.warm[kernel])

    def lifecycle_ms(self, row: np.ndarray, calls: int, allowed=None) -> dict:
        """Predicted set-up + calls x warm time per kernel of the model (restricted to `allowed`)."""
        out = {}
        for k in self.setup:
            if allowed is not None and not allowed.get(k, False):
                continue
            s, w = self.costs_ms(k, row)
            out[k] = float(s + max(1, int(calls)) * w)
        return out

    def save(self, path) -> None:
        doc = dict(self.meta)
        doc["features"] = ", ".join(TERMS)
        doc["kernels"] = {k: {"setup_coefficients": self.setup[k].tolist(),
                              "warm_coefficients": self.warm[k].tolist()} for k in self.setup}
        Path(path).write_text(json.dumps(doc, indent=1))
