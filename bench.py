#!/usr/bin/env python
"""Benchmark of the SpMM hot path: warm SpMM GFLOP/s (2*nnz*N) and fraction of the
HBM roofline on 1/2/4/8 B200s of one node.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C4] [--kernel named]
    python bench.py --impl reference ...     # torch.sparse.mm on the host cores

A step is one SpMM (plan already built, as in the reference's warm protocol,
ra_real_graph_eval.py:37-38,210-221). Default workload: configuration 4 of
BASELINE.json, the largest single SpMM (R-MAT scale 22, 128 M nonzeros, N=64), through the
kernel BASELINE.json names for it (SEGMENT_HYBRID on the TF32 path); the kernel the router
picks is timed beside it, and so are configurations 2 and 3, in the `also` block of the
same JSON line (each with 50 warm-ups + 200 timed launches, the reference's WARMUP /
TIMED_ITERS). With N>1 ranks (torchrun) the rows of A are split into contiguous row blocks
whose boundaries are tuned at plan time from the measured time of each rank's block, B is
replicated, each rank writes its own slab of C and no collective runs on the data path of
the device-timed SpMM; the total work is fixed (strong scaling) and the reported time is
the max over ranks. The end-to-end path uploads each rank's K/N row slab of B from pinned
host memory, rebuilds the replica with one NCCL all-gather over NVLink, runs the SpMM and
copies the rank's slab of C back.
Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "spmm_gflops_warm"
UNIT = "GFLOP/s (2*nnz*N)"
CONFIG_KERNEL = {"C1": "CSR_DIRECT", "C2": "ZERO_OVERHEAD_CSR", "C3": "COMMUNITY_TC",
                 "C4": "SEGMENT_HYBRID_TF32", "C5": "TC_DIRECT"}
CONFIG_DESC = {
    "C1": "Erdos-Renyi 4096x4096, 16 nnz/row, N=64 fp32, seed 0",
    "C2": "Chung-Lu power-law, 1,048,576 nodes, gamma 2.1, mean degree ~10, symmetrised + self loops, "
          "vals 1/sqrt(di*dj) fp32, N=128 fp32, seed 1",
    "C3": "SBM 232,960 nodes, 50 communities, mean degree ~490, fp16 values, N=256 fp16 B, seed 2",
    "C4": "R-MAT scale 22, edge factor 16, symmetrised + dedup, N=64 fp32 on the TF32 path, seed 3",
    "C5": "GCN-normalised SBM 2,449,029 nodes, mean degree 50, N=256 fp32, seed 123 (single SpMM)",
}
DEFAULT_CONFIG = "C4"
# (configuration, kernel selector) timed beside the headline in the same run
ALSO = [("C4", "routed"), ("C2", "named"), ("C3", "named"), ("C3", "routed")]
TOL = {"fp32": 1e-5, "tile": 5e-3}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--config", default=DEFAULT_CONFIG, choices=list(CONFIG_KERNEL))
    ap.add_argument("--kernel", default="named",
                    help="named (the kernel BASELINE.json names for the config) | routed | CSR_DIRECT | ZERO_OVERHEAD_CSR | TC_DIRECT[_TF32] | COMMUNITY_TC[_TF32] | "
                         "SEGMENT_HYBRID[_TF32]")
    ap.add_argument("--scale", type=float, default=1.0, help="shrink the graph (debugging only)")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--also", default="auto", choices=["auto", "on", "off"],
                    help="time the other configurations / kernels too (auto: when the default configuration runs at full size)")
    ap.add_argument("--inner-warmup", type=int, default=50, help="warm-up launches of each `also` entry")
    ap.add_argument("--inner-iters", type=int, default=200, help="timed launches of each `also` entry")
    ap.add_argument("--row-weight", type=float, default=None,
                    help="multi-GPU row partition: nonzeros that one row is worth in the first cut of the blocks "
                         "(default: 3 for the CSR kernels, 1 for the tile kernels); the cut is then tuned from measured times")
    ap.add_argument("--balance-rounds", type=int, default=3,
                    help="multi-GPU: rounds of measuring every rank's block and moving the boundaries")
    ap.add_argument("--gcn-panels", type=int, default=1,
                    help="multi-GPU GCN step: column panels per all-gather (SpMM of a panel overlaps the next gather)")
    ap.add_argument("--emulate-ranks", type=int, default=0,
                    help="diagnostic, one GPU: cut the rows as for this many ranks, time the blocks one after the other "
                         "and report the balance (no JSON contract line)")
    return ap.parse_args()


def algorithmic_bytes(M, K, nnz, N, sA=4, sB=4):
    """rowptr + colind + values + B read once + C written once."""
    return 4 * (M + 1) + 4 * nnz + sA * nnz + sB * K * N + 4 * M * N


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock/throttle samples while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "samples": len(sm),
                "reasons": sorted(reasons)}


def load_config(name, scale, rank=0, dist_on=False):
    """Graph + dense operand of a configuration. Rank 0 generates (or loads the on-disk cache)
    first; the other ranks load what it cached."""
    from ra_spmm_b200 import generators as G
    if dist_on:
        import torch.distributed as dist
        if rank == 0:
            out = G.cached_config(name, scale)
        dist.barrier()
        if rank != 0:
            out = G.cached_config(name, scale)
    else:
        out = G.cached_config(name, scale)
    a, N, b_dtype = out
    B = G.dense(a.K, N, G.CONFIG_SEEDS[name], b_dtype)
    return a, N, B, b_dtype


def strided_row_sample(a, stride):
    """Every stride-th row of A as a CSR (same K): a representative bounded sample."""
    import numpy as np
    rows = np.arange(0, a.M, stride)
    deg = (a.rowptr[rows + 1] - a.rowptr[rows]).astype(np.int64)
    rp = np.zeros(rows.size + 1, dtype=np.int64)
    np.cumsum(deg, out=rp[1:])
    idx = np.repeat(a.rowptr[rows].astype(np.int64) - rp[:-1], deg) + np.arange(rp[-1])
    return rp, a.colind[idx].astype(np.int64), a.vals[idx]


def cpu_spmm_bench(a, B, steps, warmup, budget_s=20.0, keep_result=False):
    """torch.sparse.mm on a CPU CSR tensor (the reference harness's CPU-runnable
    operator, test_ra.py:106-172), all host threads, on a bounded strided row sample.
    Returns a dict; with keep_result the sample's rows and its product stay in it."""
    import torch
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    Bf = B.float().contiguous()
    N = Bf.shape[1]

    def make(stride):
        rp, ci, va = strided_row_sample(a, stride)
        A = torch.sparse_csr_tensor(torch.from_numpy(rp), torch.from_numpy(ci), torch.from_numpy(va),
                                    size=(rp.size - 1, a.K))
        return A, int(rp[-1])

    stride = 1
    A, nnz_s = make(stride)
    t0 = time.perf_counter(); out = torch.sparse.mm(A, Bf); t_full = time.perf_counter() - t0
    per_step_budget = budget_s / max(1, steps + warmup)
    if t_full > per_step_budget:
        stride = int(min(a.M, max(2, round(t_full / per_step_budget))))
        A, nnz_s = make(stride)
    for _ in range(warmup):
        out = torch.sparse.mm(A, Bf)
    times = []
    for _ in range(steps):
        t0 = time.perf_counter(); out = torch.sparse.mm(A, Bf); times.append(time.perf_counter() - t0)
    total = sum(times)
    res = {"gflops": 2.0 * nnz_s * N * steps / total / 1e9, "ms": total / steps * 1e3, "cores": cores,
           "stride": stride,
           "sample": (f"torch.sparse.mm CSR fp32, rows 0::{stride} of the workload ({A.shape[0]} rows, {nnz_s} nnz), "
                      f"{steps} passes after {warmup} warm-up")}
    if keep_result:
        res["result"] = out
    return res


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    a, N, B, b_dtype = load_config(args.config, args.scale)
    r = cpu_spmm_bench(a, B, args.steps, max(args.warmup, 1), budget_s=120.0)
    line = {
        "metric": METRIC, "value": r["gflops"], "unit": UNIT, "impl": "reference", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms"], "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.config}: {CONFIG_DESC[args.config]}", "kernel": "torch.sparse.mm (CPU, CSR)",
                   "note": "reference arm = the reference harness's CPU operator on the host cores; "
                           "each step is a bounded strided row sample of the workload"},
        "cpu_baseline": {"value": r["gflops"], "unit": UNIT, "cores": r["cores"], "kind": "reference", "sample": r["sample"]},
        "e2e": {"value": r["gflops"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


class Runner:
    """One rank's SpMM through the public module (ra_spmm mirror over the C ABI)."""

    def __init__(self, kernel, a_local, K, N, dev, b_dtype):
        import torch
        from ra_spmm_b200 import ra_spmm
        self.torch, self.m, self.kernel, self.dev = torch, ra_spmm, kernel, dev
        self.rp, self.ci, self.va = (torch.from_numpy(x).to(dev) for x in a_local)
        self.M = a_local[0].size - 1
        self.K, self.N = K, N
        fam = kernel.replace("_TF32", "")
        self.tf32 = kernel.endswith("_TF32")
        self.plan = None
        self.launches = 1
        builders = {
            "ZERO_OVERHEAD_CSR": lambda: ra_spmm.make_zero_overhead_plan(self.rp, self.M, K),
            "TC_DIRECT": lambda: ra_spmm.make_tc_direct_plan(self.rp, self.ci, self.va, self.M, K, N),
            "COMMUNITY_TC": lambda: ra_spmm.make_community_tc_plan(self.rp, self.ci, self.va, self.M, K, N),
            "SEGMENT_HYBRID": lambda: ra_spmm.make_segment_hybrid_plan(self.rp, self.ci, self.va, self.M, K, N),
        }
        if fam not in builders and fam != "CSR_DIRECT":
            raise SystemExit(f"unknown kernel {kernel}")
        # wall-clock time of the plan build from device-resident CSR (for COMMUNITY_TC it includes the
        # locality sort, for the tile families the window sort and the packing of the blocks): the
        # faster of two builds, since the first one of a process also loads the builder kernels
        self.plan_ms = 0.0
        if fam in builders:
            times = []
            for _ in range(2):
                self.plan = None
                torch.cuda.synchronize()
                t_plan = time.perf_counter()
                self.plan = builders[fam]()
                torch.cuda.synchronize()
                times.append((time.perf_counter() - t_plan) * 1e3)
            self.plan_ms = min(times)
        if fam == "ZERO_OVERHEAD_CSR":
            data = (self.plan.num_chunks > 0) + (self.plan.num_small > 0)
            long_rows = N >= 256 and self.plan.num_chunks >= 16 * self.plan.num_small
            if data == 2 and N in (32, 64, 128, 256, 512) and not long_rows:
                data = 1                           # chunks and small rows share one launch at these widths
            self.launches = data + (self.plan.num_zero_rows > 0)
        elif fam == "SEGMENT_HYBRID":
            self.launches = 1 + (self.plan.num_split_windows > 0)
        if fam in ("TC_DIRECT", "COMMUNITY_TC", "SEGMENT_HYBRID") and not self.tf32 and b_dtype == "float32":
            self.launches += 1                     # per-call fp32 -> fp16 conversion of B
        self.fam = fam

    def __call__(self, B):
        m = self.m
        if self.fam == "CSR_DIRECT":
            return m.spmm_csr_direct(self.rp, self.ci, self.va, B)
        if self.fam == "ZERO_OVERHEAD_CSR":
            return m.run_zero_overhead_plan(self.plan, self.rp, self.ci, self.va, B)
        if self.fam == "TC_DIRECT":
            return m.run_tc_direct_plan_tf32(self.plan, B) if self.tf32 else m.run_tc_direct_plan(self.plan, B)
        if self.fam == "COMMUNITY_TC":
            return m.run_community_tc_plan_tf32(self.plan, B) if self.tf32 else m.run_community_tc_plan(self.plan, B)
        return (m.run_segment_hybrid_plan_tf32(self.plan, self.ci, self.va, B) if self.tf32
                else m.run_segment_hybrid_plan(self.plan, self.ci, self.va, B))


def local_ms(torch, fn, warm, iters):
    """Mean device time of one call on this rank: CUDA events around back-to-back calls."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def timed_loop(torch, fn, steps, dist_on):
    """K back-to-back calls between two CUDA events on the current stream, bracketed by a
    barrier + synchronize on both sides; returns (max over ranks, per-rank list) in ms."""
    import torch.distributed as dist
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    ms = e0.elapsed_time(e1)
    every = [ms]
    if dist_on:
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        out = torch.empty(dist.get_world_size(), device="cuda", dtype=torch.float64)
        dist.all_gather_into_tensor(out, t)
        every = [float(x) for x in out.tolist()]
    return max(every), every


def zo_phase_times(torch, runner, B, iters=20):
    """Average duration of each ZERO_OVERHEAD phase timed alone (chunks, small rows, merge)
    and of the launch that a normal run uses for the two data phases together."""
    from ra_spmm_b200 import _capi
    lib = _capi.load()
    Cbuf = torch.empty((runner.M, runner.N), dtype=torch.float32, device=runner.dev)
    st = torch.cuda.current_stream().cuda_stream
    out = {}
    for name, mask in (("csr_stream_kernel<chunks>", 1), ("csr_stream_kernel<small rows>", 2),
                       ("csr_stream_kernel<chunks + small rows, one launch>", 3), ("zo_finish_kernel", 4)):
        call = lambda: lib.ra_zo_plan_run_phases(runner.plan._h, runner.rp.data_ptr(), runner.ci.data_ptr(),
                                                 runner.va.data_ptr(), B.data_ptr(), Cbuf.data_ptr(),
                                                 runner.N, mask, st)
        out[name] = local_ms(torch, call, 3, iters)
    return out


def resolve_kernel(cfg, selector, routed):
    if selector == "named":
        return CONFIG_KERNEL[cfg]
    if selector == "routed":
        return routed
    return selector


def first_row_weight(args, fam):
    if args.row_weight is not None:
        return args.row_weight
    return 3.0 if fam in ("CSR_DIRECT", "ZERO_OVERHEAD_CSR") else 1.0


def build_balanced(torch, a, kernel, K, N, dev, b_dtype, B_dev, world, rank, args, gather_times):
    """Row blocks for `world` ranks and this rank's runner. The first cut equalises nonzeros +
    row_weight x rows; then, `balance_rounds` times, every rank times its own block, the times
    are exchanged (gather_times: list of all ranks' ms given this rank's ms) and the boundaries
    move so that every block would take the same time at the measured cost per unit of weight.
    The best cut seen is kept. Returns (bounds, runner, log of rounds)."""
    from ra_spmm_b200 import partition as P
    fam = kernel.replace("_TF32", "")
    rw = first_row_weight(args, fam)
    bounds = P.nnz_balanced_row_splits(a.rowptr, world, row_weight=rw)

    def make(b):
        return Runner(kernel, P.row_block(a.rowptr, a.colind, a.vals, int(b[rank]), int(b[rank + 1])), K, N, dev, b_dtype)

    runner = make(bounds)
    log = []
    if world == 1 or args.balance_rounds <= 0:
        return bounds, runner, log
    best = None
    for rnd in range(args.balance_rounds + 1):
        # time enough launches to fill about 30 ms: a 0.1 ms block timed over 20 launches is noise
        quick = local_ms(torch, lambda: runner(B_dev), 5, 10)
        iters = int(min(400, max(20, 30.0 / max(quick, 1e-3))))
        times = gather_times(local_ms(torch, lambda: runner(B_dev), 2, iters))
        log.append({"bounds": [int(x) for x in bounds], "ms": [round(t, 4) for t in times]})
        if best is None or max(times) < best[0]:
            best = (max(times), bounds.copy())
        if rnd == args.balance_rounds or max(times) <= 1.02 * (sum(times) / len(times)):
            break
        bounds = P.rebalance_by_time(a.rowptr, bounds, times, row_weight=rw)
        del runner
        runner = make(bounds)
    if not all(int(x) == int(y) for x, y in zip(bounds, best[1])):
        bounds = best[1]
        del runner
        runner = make(bounds)
    return bounds, runner, log


def parity_check(torch, runner, B_dev, a, B, kernel, budget_s=3.0):
    """Relative Frobenius error of the kernel's C against torch.sparse.mm on the host cores,
    on a strided row sample sized to about `budget_s` of CPU time (all rows when that fits)."""
    cpu = cpu_spmm_bench(a, B, steps=1, warmup=0, budget_s=budget_s, keep_result=True)
    C = runner(B_dev)[:: cpu["stride"]].float().cpu()
    ref = cpu["result"]
    err = float(torch.linalg.vector_norm((C.double() - ref.double()).flatten()) /
                torch.linalg.vector_norm(ref.double().flatten()))
    tile = kernel.replace("_TF32", "") in ("TC_DIRECT", "COMMUNITY_TC", "SEGMENT_HYBRID")
    tol = TOL["tile"] if tile else TOL["fp32"]
    return {"rel_fro_vs_cpu_sparse_mm": err, "tolerance": tol, "ok": err < tol,
            "rows": f"0::{cpu['stride']} ({ref.shape[0]} rows)"}, cpu


def traffic_entry(cfg, kernel):
    """DRAM bytes per SpMM from the committed ncu captures (profiles/dram_traffic.json)."""
    f = ROOT / "profiles" / "dram_traffic.json"
    try:
        e = json.loads(f.read_text()).get(f"{cfg}:{kernel}")
    except Exception:
        return None, None
    if isinstance(e, dict):
        return e.get("bytes"), e.get("source")
    return (e, "profiles/dram_traffic.json") if e is not None else (None, None)


def measure_entry(torch, dist, args, cfg, selector, dev, world, rank, peak):
    """One `also` entry: a configuration through one kernel, 50 warm-ups + 200 timed launches."""
    from ra_spmm_b200 import ra_spmm
    dist_on = world > 1
    a, N, B, b_dtype = load_config(cfg, args.scale, rank, dist_on)
    feats = ra_spmm.make_router_plan(torch.from_numpy(a.rowptr).to(dev), None, None, a.M, a.K, N)
    routed = feats["chosen_path"] + ("_TF32" if feats["use_tf32"] else "")
    kernel = resolve_kernel(cfg, selector, routed)
    fam = kernel.replace("_TF32", "")
    B_dev = B.to(dev)
    if kernel.endswith("_TF32") or fam in ("CSR_DIRECT", "ZERO_OVERHEAD_CSR"):
        B_dev = B_dev.float()

    def gather_times(ms):
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        out = torch.empty(world, device=dev, dtype=torch.float64)
        dist.all_gather_into_tensor(out, t)
        return [float(x) for x in out.tolist()]

    bounds, runner, _ = build_balanced(torch, a, kernel, a.K, N, dev, b_dtype, B_dev, world, rank, args, gather_times)
    for _ in range(args.inner_warmup):
        runner(B_dev)
    ms_total, every = timed_loop(torch, lambda: runner(B_dev), args.inner_iters, dist_on)
    ms = ms_total / args.inner_iters
    sA = 2 if cfg == "C3" else 4
    sB = 2 if B_dev.dtype == torch.float16 else 4
    bytes_algo = algorithmic_bytes(a.M, a.K, a.nnz, N, sA, sB)
    entry = {"config": cfg, "kernel": kernel, "selector": selector, "routed_kernel": routed,
             "ms_per_step": ms, "gflops": 2.0 * a.nnz * N / (ms * 1e-3) / 1e9,
             "bytes_algo": bytes_algo, "nnz": a.nnz, "N": N,
             "roofline_frac": bytes_algo / (ms * 1e-3) / 1e9 / (peak * world),
             "warmup": args.inner_warmup, "iters": args.inner_iters, "plan_build_ms": runner.plan_ms}
    tb, src = traffic_entry(cfg, kernel)
    if tb is not None and world == 1 and args.scale == 1.0:
        entry["traffic"], entry["traffic_source"] = tb, src
    if world > 1:
        entry["rank_ms"] = [x / args.inner_iters for x in every]
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        entry["parity"], _ = parity_check(torch, runner, B_dev, a, B, kernel)
    del runner, B_dev
    torch.cuda.empty_cache()
    return entry


def emulate_ranks(torch, args, a, N, B, b_dtype, kernel, dev):
    """One GPU, P row blocks timed one after the other: the balance a P-rank run would see."""
    from ra_spmm_b200 import partition as P
    Pn = args.emulate_ranks
    fam = kernel.replace("_TF32", "")
    B_dev = B.to(dev)
    if kernel.endswith("_TF32") or fam in ("CSR_DIRECT", "ZERO_OVERHEAD_CSR"):
        B_dev = B_dev.float()
    rw = first_row_weight(args, fam)
    bounds = P.nnz_balanced_row_splits(a.rowptr, Pn, row_weight=rw)
    whole = Runner(kernel, (a.rowptr, a.colind, a.vals), a.K, N, dev, b_dtype)
    t1 = local_ms(torch, lambda: whole(B_dev), 5, 20)
    del whole
    rounds = []
    for rnd in range(args.balance_rounds + 1):
        times = []
        for r in range(Pn):
            run = Runner(kernel, P.row_block(a.rowptr, a.colind, a.vals, int(bounds[r]), int(bounds[r + 1])),
                         a.K, N, dev, b_dtype)
            times.append(local_ms(torch, lambda: run(B_dev), 5, 20))
            del run
        rounds.append({"round": rnd, "max_ms": max(times), "mean_ms": sum(times) / Pn,
                       "efficiency_vs_1gpu": t1 / (Pn * max(times)), "ms": [round(t, 4) for t in times],
                       "rows": [int(bounds[i + 1] - bounds[i]) for i in range(Pn)],
                       "nnz": [int(a.rowptr[int(bounds[i + 1])] - a.rowptr[int(bounds[i])]) for i in range(Pn)]})
        if rnd < args.balance_rounds:
            bounds = P.rebalance_by_time(a.rowptr, bounds, times, row_weight=rw)
    print(json.dumps({"emulated_ranks": Pn, "kernel": kernel, "ms_1gpu": t1, "rounds": rounds}))


def main():
    args = parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import numpy as np
    import torch
    import torch.distributed as dist
    from ra_spmm_b200 import ra_spmm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist_on = world > 1
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if dist_on:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"      # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=dev)
    n_gpus = world
    peak, peak_kind = measured_peak()

    a, N, B, b_dtype = load_config(args.config, args.scale, rank, dist_on)
    M, K, nnz = a.M, a.K, a.nnz

    # routing decision on the global matrix (device feature scan)
    feats = ra_spmm.make_router_plan(torch.from_numpy(a.rowptr).to(dev), None, None, M, K, N)
    routed = feats["chosen_path"] + ("_TF32" if feats["use_tf32"] else "")
    kernel = resolve_kernel(args.config, args.kernel, routed)
    if args.emulate_ranks > 1:
        return emulate_ranks(torch, args, a, N, B, b_dtype, kernel, dev)
    fam0 = kernel.replace("_TF32", "")
    f32_operand = kernel.endswith("_TF32") or fam0 in ("CSR_DIRECT", "ZERO_OVERHEAD_CSR")
    if f32_operand:
        B = B.float()
    B_dev = B.to(dev)
    torch.cuda.synchronize()

    def gather_times(ms):
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        out = torch.empty(world, device=dev, dtype=torch.float64)
        dist.all_gather_into_tensor(out, t)
        return [float(x) for x in out.tolist()]

    bounds, runner, balance_log = build_balanced(torch, a, kernel, K, N, dev, b_dtype, B_dev, world, rank,
                                                 args, gather_times)
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])

    # ---- device-resident timing ------------------------------------------------
    for _ in range(max(args.warmup, 3)):
        runner(B_dev)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_total, rank_ms = timed_loop(torch, lambda: runner(B_dev), args.steps, dist_on)
    clocks = sampler.stop() if rank == 0 else None
    ms_step = ms_total / args.steps
    rank_ms_step = [x / args.steps for x in rank_ms]
    gflops = 2.0 * nnz * N / (ms_step * 1e-3) / 1e9

    # ---- end to end: host B in, C out, every step ---------------------------------
    # Every rank owns rows [rank*Ks, (rank+1)*Ks) of B in pinned host memory. Per step it
    # uploads that slab, one NCCL all-gather rebuilds the replica of B on every GPU (the SpMM
    # reads its own GPU's memory only), the SpMM runs, and the rank's slab of C goes back to
    # pinned host memory. Three streams (copy-in + gather, compute, copy-out) and two staging
    # buffers, so the upload of step i+1 and the download of step i-1 overlap the SpMM of step i.
    Ks = (K + world - 1) // world
    slab_rows = max(0, min(K, (rank + 1) * Ks) - rank * Ks)
    slab_host = torch.zeros((Ks, N), dtype=B.dtype).pin_memory()
    slab_host[:slab_rows].copy_(B[rank * Ks: rank * Ks + slab_rows])
    C_host = [torch.empty((r1 - r0, N), dtype=torch.float32).pin_memory() for _ in range(2)]
    B_stage = [torch.empty((world * Ks, N), dtype=B.dtype, device=dev) for _ in range(2)]
    slab_dev = [torch.empty((Ks, N), dtype=B.dtype, device=dev) for _ in range(2)] if dist_on else None
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    s_main = torch.cuda.current_stream()

    def e2e_run(steps):
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_done = [None, None]            # compute finished reading B_stage[k]
        ev_out = [None, None]             # copy-out of C_host[k] finished
        keep = []
        for i in range(steps):
            k = i & 1
            with torch.cuda.stream(s_in):
                if ev_done[k] is not None:
                    s_in.wait_event(ev_done[k])
                if dist_on:
                    slab_dev[k].copy_(slab_host, non_blocking=True)
                    dist.all_gather_into_tensor(B_stage[k], slab_dev[k])
                else:
                    B_stage[k].copy_(slab_host, non_blocking=True)
                ev_in[k].record(s_in)
            s_main.wait_event(ev_in[k])
            Cd = runner(B_stage[k][:K])
            ev_done[k] = torch.cuda.Event(); ev_done[k].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_done[k])
                if ev_out[k] is not None:
                    s_out.wait_event(ev_out[k])
                C_host[k].copy_(Cd, non_blocking=True)
                ev_out[k] = torch.cuda.Event(); ev_out[k].record(s_out)
            Cd.record_stream(s_out)
            keep.append(Cd)
            if len(keep) > 4:
                keep.pop(0)
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)

    e2e_run(2)
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    ms_e2e = timed_loop(torch, lambda: e2e_run(e2e_steps), 1, dist_on)[0] / e2e_steps
    e2e_gflops = 2.0 * nnz * N / (ms_e2e * 1e-3) / 1e9
    h2d_bytes = int(slab_host.numel() * slab_host.element_size()) * n_gpus

    # ---- row-sharded B, device-resident: every rank holds only its K/P-row slab of B; a step is
    # one NCCL all-gather of the slabs followed by the rank's SpMM (the exchange a caller pays when
    # the dense operand is produced sharded, as between two GNN layers) ----
    sharded_b = None
    if dist_on:
        def sharded_step():
            dist.all_gather_into_tensor(B_stage[0], slab_dev[0])
            runner(B_stage[0][:K])
        for _ in range(3):
            sharded_step()
        ms_sh = timed_loop(torch, sharded_step, args.steps, dist_on)[0] / args.steps
        sharded_b = {"ms_per_step": ms_sh, "value": 2.0 * nnz * N / (ms_sh * 1e-3) / 1e9, "unit": UNIT,
                     "gathered_bytes_per_rank": int(slab_host.numel() * slab_host.element_size()) * (world - 1),
                     "path": "K/P-row slab of B resident per rank -> NCCL all-gather -> SpMM on the rank's row block"}
    del B_stage, slab_dev
    torch.cuda.empty_cache()

    line = None
    if rank == 0:
        sA = 2 if args.config == "C3" else 4
        sB = 2 if B.dtype == torch.float16 else 4
        bytes_algo = algorithmic_bytes(M, K, nnz, N, sA, sB)
        achieved = bytes_algo / (ms_step * 1e-3) / 1e9
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak * n_gpus, "unit": "GB/s",
                "frac": achieved / (peak * n_gpus), "peak_source": f"of {peak_kind}",
                "bytes_algo_per_step": bytes_algo, "traffic": None, "traffic_source": None,
                "launch": f"one {kernel} SpMM = {runner.launches} kernel launch(es); duration = CUDA-event "
                          f"time of the step"}
        if args.scale == 1.0 and n_gpus == 1:     # captures are of one GPU at full size (or scaled to it)
            roof["traffic"], roof["traffic_source"] = traffic_entry(args.config, kernel)
        if runner.fam == "ZERO_OVERHEAD_CSR" and n_gpus == 1:
            ph = zo_phase_times(torch, runner, B_dev)
            fused = "csr_stream_kernel<chunks + small rows, one launch>"
            used = [fused, "zo_finish_kernel"] if runner.launches <= 2 and ph.get(fused) else \
                   [k for k in ph if k != fused]
            tot = sum(ph[k] for k in used)
            # share = part of a step's launches; phases not launched on their own in a step have none
            roof["kernels"] = {k: {"ms": v, "share": (v / tot) if k in used else None} for k, v in ph.items()}
            roof["dominant_kernel"] = max(used, key=lambda k: ph[k])
        row_weight = first_row_weight(args, fam0)
        line = {
            "metric": METRIC, "value": gflops, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32" if sB == 4 else "f16",
            "data": "synthetic",
            "config": {"workload": f"{args.config}: {CONFIG_DESC[args.config]}", "kernel": kernel,
                       "routed_kernel": routed, "M": M, "K": K, "nnz": nnz, "N": N,
                       "avg_degree": feats["feature_values"]["avg_nnz_per_row"],
                       "degree_cv": feats["feature_values"]["degree_cv"],
                       "partition": f"{n_gpus} contiguous row block(s), first cut by nnz + {row_weight:g} x rows, "
                                    f"then tuned from the measured time of each rank's block; B replicated, "
                                    f"no collective in the device-timed SpMM",
                       "l2": f"inputs larger than L2: B {sB * K * N / 1e6:.0f} MB + C {4 * M * N / 1e6:.0f} MB per step",
                       "a_resident": "CSR arrays and the plan are uploaded/built once (warm protocol)",
                       "plan_build_ms": runner.plan_ms},
            "roofline": roof, "clocks": clocks,
            "e2e": {"value": e2e_gflops, "unit": UNIT, "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": int(4 * M * N), "steps": e2e_steps,
                    "path": ("pinned K/P-row slab of B per rank -> NCCL all-gather of the replica -> SpMM -> "
                             "rank's slab of C to pinned host memory") if dist_on else
                            "pinned B -> device, SpMM, C -> pinned host memory"},
            "gpu_launches": runner.launches * args.steps * n_gpus,
            "edgewise_gbs": (4 * (M + 1) + (4 + sA) * nnz + sB * nnz * N + 4 * M * N) / (ms_step * 1e-3) / 1e9,
        }
        if sharded_b is not None:
            line["sharded_b"] = sharded_b
        if n_gpus > 1:
            # balance report: per-rank step time and the nonzeros / rows of each row block
            line["ranks"] = {"ms_per_step": rank_ms_step,
                             "nnz": [int(a.rowptr[int(bounds[i + 1])] - a.rowptr[int(bounds[i])]) for i in range(n_gpus)],
                             "rows": [int(bounds[i + 1] - bounds[i]) for i in range(n_gpus)],
                             "balance_rounds": balance_log}
        if n_gpus == 1 and not args.no_cpu_baseline:
            cpu = cpu_spmm_bench(a, B, steps=5, warmup=1, budget_s=20.0, keep_result=True)
            line["cpu_baseline"] = {"value": cpu["gflops"], "unit": UNIT, "cores": cpu["cores"], "kind": "reference",
                                    "sample": cpu["sample"], "ms_per_pass": cpu["ms"]}
            # parity of the timed kernel against that leg's own product (outside every timed region)
            C = runner(B_dev)[:: cpu["stride"]].float().cpu()
            ref = cpu.pop("result")
            err = float(torch.linalg.vector_norm((C.double() - ref.double()).flatten()) /
                        torch.linalg.vector_norm(ref.double().flatten()))
            tol = TOL["tile"] if fam0 in ("TC_DIRECT", "COMMUNITY_TC", "SEGMENT_HYBRID") else TOL["fp32"]
            line["parity"] = {"rel_fro_vs_cpu_sparse_mm": err, "tolerance": tol, "ok": err < tol,
                              "rows": f"0::{cpu['stride']} ({ref.shape[0]} rows)"}
            del C, ref
    del runner, B_dev
    torch.cuda.empty_cache()

    # ---- the other configurations / kernels, same protocol, same run -------------------
    want_also = args.also == "on" or (args.also == "auto" and args.config == DEFAULT_CONFIG
                                      and args.kernel == "named" and args.scale == 1.0)
    if want_also:
        also = []
        for cfg, sel in ALSO:
            try:
                also.append(measure_entry(torch, dist, args, cfg, sel, dev, world, rank, peak))
            except Exception as exc:                # one entry failing must not lose the headline
                also.append({"config": cfg, "selector": sel, "error": f"{type(exc).__name__}: {exc}"})
        # configuration 5: the 2-layer GCN training step on the row-partitioned operator
        # (forward + backward + Adam; NCCL all-gather of each layer's row slabs at N > 1),
        # once with the routed kernels (FP16 tile path) and once all in fp32 through CSR_DIRECT
        from ra_spmm_b200 import gcn_bench
        # and once with layer 1 associated the other way, (A X) W1: the same model, but the first SpMM
        # runs at the input width and its backward needs none (reported beside, not instead of, the
        # reference harness's order)
        for gk, order in (("routed", "reference"), ("CSR_DIRECT", "reference"), ("routed", "aggregate-first")):
            try:
                gargs = gcn_bench.parse_args(["--scale", str(args.scale), "--steps", "10", "--warmup", "3",
                                              "--kernel", gk, "--order", order,
                                              "--panels", str(args.gcn_panels if dist_on else 1)])
                g = gcn_bench.measure(gargs, world, rank, dev)
                if rank == 0:
                    also.append({"config": "C5", "order": order,
                                 "kernel": f"2-layer GCN step, {gk} SpMM (" +
                                 ", ".join(f"N={k}: {v}" for k, v in sorted(g["config"]["labels"].items())) + ")",
                                 "gcn_step_ms": g["value"], "spmm_gflops": g["spmm_gflops"], "loss": g["loss"],
                                 "steps": g["steps"], "warmup": g["warmup"], "workload": g["config"]["workload"],
                                 "allgather_bytes_per_step_per_rank": g["config"]["allgather_bytes_per_step_per_rank"],
                                 "panels": g["config"]["panels"]})
            except Exception as exc:
                if rank == 0:
                    also.append({"config": "C5", "kernel": gk, "error": f"{type(exc).__name__}: {exc}"})
        if rank == 0:
            line["also"] = also
            line["gpu_launches"] += sum(e.get("iters", 0) for e in also) * n_gpus
    if rank == 0:
        print(json.dumps(line))
    if dist_on:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
