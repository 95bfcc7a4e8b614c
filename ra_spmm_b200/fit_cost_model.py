"""Fits runtime_cost_model.json on the current GPU: log-linear setup and warm cost per
kernel over [1, log1p M, log1p nnz, log1p N, log1p nnz*N, log1p avg, log1p cv]
(the design row of ra_runtime_router.py:24-32), from timings of seeded synthetic graphs.

    python -m ra_spmm_b200.fit_cost_model [--out path]"""
from __future__ import annotations

import argparse
import time

import numpy as np
import torch

from . import generators as G
from .harness import build_kernel_plan, measure_cuda_exec_ms, run_planned_kernel
from .cost_model import PORTFOLIO as KERNELS, SHIPPED_MODEL, CostModel, design_rows


def graphs():
    yield "er16", G.erdos_renyi_fixed_degree(4096, 4096, 16, 0)
    yield "rmat13", G.rmat_graph(13, 8, seed=11)
    for n, s in ((20000, 1), (100000, 2), (400000, 3)):
        yield f"cl{n}", G.chung_lu_power_law(n=n, seed=s)
    for sc, ef, s in ((14, 16, 4), (16, 8, 5), (17, 16, 6)):
        yield f"rmat{sc}", G.rmat_graph(sc, ef, seed=s)
    for n, d, s in ((20000, 60, 7), (60000, 30, 8), (150000, 12, 9), (30000, 200, 10)):
        yield f"sbm{n}", G.sbm_graph(n=n, n_comm=20, mean_degree=d, seed=s, value_dtype="float32")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default=str(SHIPPED_MODEL))
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    rows = {k: [] for k in KERNELS}
    for name, a in graphs():
        rp, ci, va = a.torch(dev)
        deg = a.degrees().astype(np.float64)
        avg, cv = float(deg.mean()), float(deg.std() / max(deg.mean(), 1e-9))
        for N in (32, 64, 128, 256):
            B = torch.randn(a.K, N, device=dev)
            x = design_rows(a.M, a.nnz, N, avg, cv)
            for k in KERNELS:
                torch.cuda.synchronize(); t0 = time.perf_counter()
                plan = build_kernel_plan(k, rp, ci, va, a.M, a.K, N)
                torch.cuda.synchronize(); setup_ms = max((time.perf_counter() - t0) * 1e3, 1e-3)
                warm_ms = measure_cuda_exec_ms(lambda: run_planned_kernel(k, plan, rp, ci, va, B), 3, 10)
                rows[k].append((x, setup_ms, warm_ms))
                del plan
        print(name, a.M, a.nnz, flush=True)
    meta = {"device": torch.cuda.get_device_name(0), "samples_per_kernel": len(rows[KERNELS[0]])}
    CostModel.fit(rows, meta).save(args.out)
    print("wrote", args.out)


if __name__ == "__main__":
    main()
