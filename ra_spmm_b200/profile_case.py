"""One SpMM launch group inside an NVTX range, for profilers.

    ncu --nvtx --nvtx-include "SPMM_PROFILE/" --clock-control none ... \
        python -m ra_spmm_b200.profile_case --config C2 --kernel ZERO_OVERHEAD_CSR --scale 0.5

The plan is built and the kernel warmed outside the range; exactly one call runs inside it
(the protocol of bench/profile_case_ra.py:1-16, 61-71).
"""
from __future__ import annotations

import argparse

import torch

from . import generators as G
from . import harness as H


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="C2", choices=["C1", "C2", "C3", "C4", "C5"])
    ap.add_argument("--kernel", default="routed")
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--f32-b", action="store_true", help="hand B over as fp32 even when the configuration's B is fp16")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    a, N, b_dtype = G.cached_config(args.config, args.scale)
    B = G.dense(a.K, N, G.CONFIG_SEEDS[args.config], b_dtype).to(dev)
    if args.f32_b or b_dtype == "float32":
        B = B.float()
    rp, ci, va = a.torch(dev)
    kernel = args.kernel
    if kernel.endswith("_TF32") or kernel in ("CSR_DIRECT", "ZERO_OVERHEAD_CSR"):
        B = B.float()
    if kernel == "routed":
        from . import ra_spmm
        d = ra_spmm.make_router_plan(rp, ci, va, a.M, a.K, N)
        kernel = d["chosen_path"] + ("_TF32" if d["use_tf32"] else "")
    plan = H.build_kernel_plan(kernel, rp, ci, va, a.M, a.K, N)
    for _ in range(args.warmup):
        H.run_planned_kernel(kernel, plan, rp, ci, va, B)
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_push("SPMM_PROFILE")
    out = H.run_planned_kernel(kernel, plan, rp, ci, va, B)
    torch.cuda.synchronize()
    torch.cuda.nvtx.range_pop()
    print(f"{args.config} {kernel} M={a.M} nnz={a.nnz} N={N} checksum={float(out.double().sum()):.6e}")


if __name__ == "__main__":
    main()
