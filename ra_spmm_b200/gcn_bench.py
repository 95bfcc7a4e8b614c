"""Warm 2-layer GCN training-step time on configuration 5 (SBM graph, 2,449,029 nodes,
mean degree 50, 100 features, hidden 256, 47 classes), A row-partitioned over the ranks.

    python -m ra_spmm_b200.gcn_bench [--scale 1.0] [--kernel routed] [--steps 10] [--warmup 3]
    torchrun --nproc-per-node 8 -m ra_spmm_b200.gcn_bench ...

Protocol of the reference harness (gnn_bench/router_vs_baselines_gcn.py:482-498, 520-537):
X ~ randn, labels ~ randint, Adam lr 1e-2, seed 123; a step is zero_grad, forward, cross-entropy,
backward, Adam step. Device time between CUDA events, max over ranks. Prints one JSON line."""
from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist

from . import generators as G
from . import partition as P
from .gcn import GCN2, GraphOperator, RowSharding, train_step


def parse_args(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--scale", type=float, default=1.0)
    ap.add_argument("--kernel", default="routed")
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--cpu-baseline", action="store_true")
    ap.add_argument("--breakdown", action="store_true",
                    help="after the timed steps, run one more step with CUDA events around every SpMM call")
    ap.add_argument("--gather", default="kernel", choices=["kernel", "fp32"],
                    help="multi-GPU: all-gather the row slabs in the format the kernel reads (fp16, padded, "
                         "for the FP16 tile paths) or as fp32")
    ap.add_argument("--panels", type=int, default=1,
                    help="multi-GPU: gather wide operands in this many column panels and start each panel's "
                         "SpMM when its own gather has landed")
    ap.add_argument("--order", default="reference", choices=["reference", "aggregate-first"],
                    help="layer 1 as A (X W1), the reference harness's order, or as (A X) W1: the same layer with the "
                         "SpMM at the input width and no SpMM in its backward (X needs no gradient)")
    ap.add_argument("--chunks", type=int, default=1,
                    help="multi-GPU: gather every slab in this many runs of rows and split the operator by the "
                         "chunk that owns the column, so the SpMM of a chunk overlaps the gather of the next")
    return ap.parse_args(argv)


def measure(args, world: int, rank: int, dev):
    """Times the step on an initialised process group; returns the result line on rank 0, else None."""
    if world > 1:
        if rank == 0:
            a, _, _ = G.cached_config("C5", args.scale)
        dist.barrier()
        if rank != 0:
            a, _, _ = G.cached_config("C5", args.scale)
    else:
        a, _, _ = G.cached_config("C5", args.scale)
    bounds = P.nnz_balanced_row_splits(a.rowptr, world)
    r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
    rp, ci, va = P.row_block(a.rowptr, a.colind, a.vals, r0, r1)
    sharding = RowSharding(bounds, rank, world, chunks=args.chunks)
    # A^T = A: one operator both ways; its columns address the padded gathered operand
    op = GraphOperator(rp, sharding.remap_columns(ci), va, sharding.gathered_rows, dev, kernel=args.kernel)
    spmm = op.matmul
    if sharding.chunks > 1:
        # the routing decision is the one of the whole row block; one operator per row chunk
        for width in (256, 47, 100):
            op.operand_format(width)
        chunk_ops = [GraphOperator(crp, cci, cva, cK, dev, kernel=args.kernel, labels=op.labels)
                     for crp, cci, cva, cK in sharding.split_columns(rp, ci, va)]
        spmm = [o.matmul for o in chunk_ops]
    g = torch.Generator().manual_seed(123)
    X = torch.randn((a.M, 100), generator=g)[r0:r1].to(dev)
    y = torch.randint(0, 47, (a.M,), generator=g)[r0:r1].to(dev)
    torch.manual_seed(123)
    model = GCN2(100, 256, 47, spmm, sharding=sharding,
                 operand_format=op.operand_format if args.gather == "kernel" else None,
                 panels=args.panels, aggregate_first=args.order == "aggregate-first").to(dev)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)

    for _ in range(max(args.warmup, 1)):
        loss = train_step(model, opt, X, y, a.M)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sharding.comm_bytes = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        loss = train_step(model, opt, X, y, a.M)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    spmm_ms = None
    if args.breakdown and sharding.chunks == 1:
        calls = []
        inner = op.matmul

        def timed_matmul(B):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); out = inner(B); e1.record()
            calls.append((int(B.shape[1]), str(B.dtype).replace("torch.", ""), e0, e1))
            return out
        model.spmm = model.spmm_t = timed_matmul
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record(); train_step(model, opt, X, y, a.M); s1.record()
        torch.cuda.synchronize()
        spmm_ms = {"step_ms": s0.elapsed_time(s1),
                   "spmm_calls": [{"N": n, "dtype": dt, "ms": e0.elapsed_time(e1)} for n, dt, e0, e1 in calls]}
    line = None
    if rank == 0:
        nnz = a.nnz
        # forward + backward of the two SpMM sites; aggregate-first: width 100 forward only at site 1
        spmm_flops = 2.0 * nnz * ((256 + 47) * 2 if args.order == "reference" else (100 + 47 * 2))
        line = {"metric": "gcn_step_ms_warm", "value": ms, "unit": "ms", "higher_is_better": False,
                "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 1),
                "spmm_gflops": spmm_flops / (ms * 1e-3) / 1e9, "loss": float(loss),
                "config": {"workload": f"2-layer GCN on SBM {a.M} nodes, nnz {nnz}, 100->256->47", "kernel": args.kernel,
                           "labels": op.labels, "allgather_bytes_per_step_per_rank": sharding.comm_bytes // args.steps,
                           "partition": f"{world} nnz-balanced row blocks, all-gather before each SpMM", "gather": args.gather,
                           "panels": args.panels, "chunks": sharding.chunks, "order": args.order}}
        if spmm_ms is not None:
            line["breakdown"] = spmm_ms
        if args.cpu_baseline and world == 1:
            Ac = torch.sparse_csr_tensor(torch.from_numpy(a.rowptr.astype(np.int64)), torch.from_numpy(a.colind.astype(np.int64)),
                                         torch.from_numpy(a.vals), size=(a.M, a.K))
            torch.set_num_threads(os.cpu_count())
            cm = GCN2(100, 256, 47, lambda B: torch.sparse.mm(Ac, B), sharding=RowSharding([0, a.M]))
            co = torch.optim.Adam(cm.parameters(), lr=1e-2)
            Xc, yc = X.cpu(), y.cpu()
            train_step(cm, co, Xc, yc, a.M)
            t0 = time.perf_counter(); train_step(cm, co, Xc, yc, a.M); t_cpu = time.perf_counter() - t0
            line["cpu_baseline"] = {"value": t_cpu * 1e3, "unit": "ms", "cores": os.cpu_count(),
                                    "kind": "reference", "sample": "one full step, torch.sparse.mm CPU"}
    del model, opt, op
    torch.cuda.empty_cache()
    return line


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1")); rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
    line = measure(args, world, rank, dev)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
