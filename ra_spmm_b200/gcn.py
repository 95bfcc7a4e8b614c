"""2-layer GNN training steps (GCN, GraphSAGE-mean, GIN) on top of the SpMM kernels,
single- or multi-GPU.

Mirrors the reference harnesses (gnn_bench/router_vs_baselines_gcn.py: aggregation operators
:89-126, GraphBackend :140-410, SparseMMFunction :448-461, GCNBench :464-476, measure_step
:482-498; router_vs_baselines_sage.py:48-67; router_vs_baselines_gin.py:47-74): bias-free
Linear layers, cross-entropy, Adam; GCN h = relu(A (X W1)), out = A (h W2).

Multi-GPU (not in the reference): A is row-partitioned, every rank owns the rows
[b[r], b[r+1]) of X, H, the logits and the labels. Each SpMM needs all rows of its
dense operand, so the row slabs are all-gathered first (in place, one NCCL
all_gather_into_tensor into a padded layout that the operator's remapped column
indices address directly; when the kernel reads fp16, the slab is rounded to fp16
before the gather, not after); the backward of
an SpMM is the same operation with the transposed operator: grad_in_local =
(A^T)[rows] @ allgather(grad_out). For the symmetric GCN operator A^T = A, so
one plan serves both directions; the row-mean operator of GraphSAGE is not symmetric and
gets a second operator built from the transposed row block (`transpose_csr`). Weight
gradients are all-reduced. With `panels` > 1 a wide operand is gathered in column panels and
the SpMM of panel j runs while panel j+1 is still on NVLink.
"""
from __future__ import annotations

from typing import Callable, Optional

import numpy as np
import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F


def aggregation_operator(rowptr, colind, M: int, model: str, vals=None):
    """Per-model aggregation matrix from a raw adjacency (CSR, duplicate-free), as
    build_aggregation_operator does (gnn_bench/router_vs_baselines_gcn.py:89-126):
      gcn  : D~^-1/2 (A + I) D~^-1/2, the diagonal added only where absent;
      sage : D^-1 A (row mean; zero-degree rows stay zero, no self loop);
      gin  : A unchanged.
    Arithmetic in float64, result (rowptr int32, colind int32, vals float32) with sorted columns."""
    rowptr = np.asarray(rowptr, dtype=np.int64)
    colind = np.asarray(colind, dtype=np.int64)
    w = np.ones(colind.size, dtype=np.float64) if vals is None else np.asarray(vals, dtype=np.float64)
    rows = np.repeat(np.arange(M, dtype=np.int64), np.diff(rowptr))
    m = model.lower()
    if m == "gcn":
        has_diag = np.zeros(M, dtype=bool)
        has_diag[rows[rows == colind]] = True
        add = np.flatnonzero(~has_diag)
        rows = np.concatenate([rows, add]); colind = np.concatenate([colind, add])
        w = np.concatenate([w, np.ones(add.size)])
    order = np.lexsort((colind, rows))
    rows, colind, w = rows[order], colind[order], w[order]
    if m == "gcn":
        d = np.bincount(rows, weights=w, minlength=M)
        dis = np.divide(1.0, np.sqrt(d), out=np.zeros_like(d), where=d > 0)
        w = dis[rows] * w * dis[colind]
    elif m in ("sage", "graphsage"):
        d = np.bincount(rows, weights=w, minlength=M)
        w = w * np.divide(1.0, d, out=np.zeros_like(d), where=d > 0)[rows]
    elif m != "gin":
        raise ValueError(f"unknown model for aggregation operator: {model}")
    rp = np.zeros(M + 1, dtype=np.int64)
    np.cumsum(np.bincount(rows, minlength=M), out=rp[1:])
    return rp.astype(np.int32), colind.astype(np.int32), w.astype(np.float32)


def transpose_csr(rowptr, colind, vals, M: int, K: int):
    """CSR of A^T (K x M), columns sorted: the operator of the backward pass when A is not
    symmetric (GraphBackend builds it with scipy, gnn_bench/router_vs_baselines_gcn.py:166-168)."""
    rowptr = np.asarray(rowptr, dtype=np.int64)
    rows = np.repeat(np.arange(M, dtype=np.int64), np.diff(rowptr))
    order = np.argsort(np.asarray(colind), kind="stable")          # by column, rows stay ascending
    rp = np.zeros(K + 1, dtype=np.int64)
    np.cumsum(np.bincount(np.asarray(colind), minlength=K), out=rp[1:])
    return rp.astype(np.int32), rows[order].astype(np.int32), np.asarray(vals)[order]


class GraphOperator:
    """Rows [r0, r1) of a sparse matrix on one GPU with a cached kernel plan per
    family (the role of GraphBackend._get_executor, gnn_bench/router_vs_baselines_gcn.py:216-348).

    kernel: "routed" (router decision on this block), "CSR_DIRECT", "ZERO_OVERHEAD_CSR",
    "TC_DIRECT[_TF32]", "COMMUNITY_TC[_TF32]", "SEGMENT_HYBRID[_TF32]"."""

    def __init__(self, rowptr: np.ndarray, colind: np.ndarray, vals: np.ndarray, K: int,
                 device, kernel: str = "routed", labels=None):
        from . import ra_spmm
        self.m = ra_spmm
        self.device = torch.device(device)
        self.M, self.K = int(rowptr.size - 1), int(K)
        self.rp = torch.from_numpy(np.ascontiguousarray(rowptr, dtype=np.int32)).to(self.device)
        self.ci = torch.from_numpy(np.ascontiguousarray(colind, dtype=np.int32)).to(self.device)
        self.va = torch.from_numpy(np.ascontiguousarray(vals, dtype=np.float32)).to(self.device)
        self.kernel = kernel
        self._plans = {}
        self.labels = dict(labels or {})      # width -> kernel label; preset labels skip the router (chunk operators
                                              # take the decision made on the whole row block)

    def _resolve(self, N: int) -> str:
        if self.kernel != "routed":
            return self.kernel
        d = self.m.make_router_plan(self.rp, self.ci, self.va, self.M, self.K, N)
        label = d["chosen_path"] + ("_TF32" if d["use_tf32"] else "")
        return "CSR_DIRECT" if label == "CUSPARSE" else label

    def operand_format(self, N: int):
        """(dtype, width) in which the kernel chosen for width N reads its dense operand: the
        FP16 tile paths round B to fp16 first (and pad its rows to a multiple of 16 columns), so a
        sharded caller can round and pad its own row slab before the all-gather - half the bytes
        on NVLink, and each rank converts 1/world of the operand instead of all of it. The
        rounding is the library's own (round to nearest even), so the SpMM sees the same bits."""
        label = self.labels.get(N)
        if label is None:
            label = self.labels[N] = self._resolve(N)
        if label in ("TC_DIRECT", "COMMUNITY_TC", "SEGMENT_HYBRID"):
            width = (N + 15) // 16 * 16
            self.labels.setdefault(width, label)
            return torch.float16, width
        return torch.float32, N

    def matmul(self, B: torch.Tensor) -> torch.Tensor:
        m, N = self.m, B.shape[1]
        label = self.labels.get(N)
        if label is None:
            label = self.labels[N] = self._resolve(N)
        fam, tf32 = label.replace("_TF32", ""), label.endswith("_TF32")
        B = B.contiguous()
        if fam == "CSR_DIRECT":
            return m.spmm_csr_direct(self.rp, self.ci, self.va, B)
        plan = self._plans.get(fam)
        if plan is None:
            make = {"ZERO_OVERHEAD_CSR": lambda: m.make_zero_overhead_plan(self.rp, self.M, self.K),
                    "TC_DIRECT": lambda: m.make_tc_direct_plan(self.rp, self.ci, self.va, self.M, self.K, 64),
                    "COMMUNITY_TC": lambda: m.make_community_tc_plan(self.rp, self.ci, self.va, self.M, self.K, 64),
                    "SEGMENT_HYBRID": lambda: m.make_segment_hybrid_plan(self.rp, self.ci, self.va, self.M, self.K, 64)}
            plan = self._plans[fam] = make[fam]()
        if fam == "ZERO_OVERHEAD_CSR":
            return m.run_zero_overhead_plan(plan, self.rp, self.ci, self.va, B)
        if fam == "TC_DIRECT":
            return m.run_tc_direct_plan_tf32(plan, B) if tf32 else m.run_tc_direct_plan(plan, B)
        if fam == "COMMUNITY_TC":
            return m.run_community_tc_plan_tf32(plan, B) if tf32 else m.run_community_tc_plan(plan, B)
        return (m.run_segment_hybrid_plan_tf32(plan, self.ci, self.va, B) if tf32
                else m.run_segment_hybrid_plan(plan, self.ci, self.va, B))


class _Done:
    def wait(self):
        return True


class RowSharding:
    """Row boundaries of the partition and the collective that rebuilds a full
    dense operand from the ranks' row slabs.

    The slabs have different heights (nnz-balanced boundaries), so the gathered
    operand is kept in a padded layout: rank r's rows start at r * max_rows. One
    all_gather_into_tensor then lands every slab in place, and the sparse
    operator's column indices are remapped once (`remap_columns`) to address that
    layout, so no compaction pass is needed."""

    def __init__(self, bounds, rank: int = 0, world: int = 1, group=None, chunks: int = 1):
        self.bounds = [int(b) for b in bounds]
        self.rank, self.world, self.group = rank, world, group
        self.max_rows = max((self.bounds[i + 1] - self.bounds[i] for i in range(world)), default=0)
        self.comm_bytes = 0
        self._slabs = {}
        # Row chunks: every rank's slab is cut into `chunks` runs of rows, chunk j of all ranks is
        # gathered on its own, and the operator is split by the chunk that owns the column
        # (`split_columns`). The SpMM of chunk j then runs while chunk j+1 is still on the wire, with
        # rows of the operand at their full width.
        self.chunks = max(1, int(chunks)) if world > 1 else 1
        self.chunk_starts = [[(self.bounds[r + 1] - self.bounds[r]) * j // self.chunks for j in range(self.chunks + 1)]
                             for r in range(world)]
        self.max_chunk_rows = [max((cs[j + 1] - cs[j] for cs in self.chunk_starts), default=0)
                               for j in range(self.chunks)]

    @property
    def rows(self):
        return self.bounds[self.rank], self.bounds[self.rank + 1]

    @property
    def gathered_rows(self) -> int:
        """Row count of the gathered (padded) dense operand = K of the remapped operator."""
        return self.bounds[-1] if self.world == 1 else self.world * self.max_rows

    def remap_columns(self, colind: np.ndarray) -> np.ndarray:
        """Column index in the global matrix -> row index in the padded gathered operand."""
        if self.world == 1:
            return colind
        b = np.asarray(self.bounds, dtype=np.int64)
        owner = np.searchsorted(b, colind, side="right") - 1
        return (owner * self.max_rows + (colind - b[owner])).astype(np.int32)

    def split_columns(self, rowptr: np.ndarray, colind: np.ndarray, vals: np.ndarray):
        """The rank's row block cut by the chunk that owns each column: a list of `chunks` tuples
        (rowptr, colind, vals, K) whose columns address the gathered operand of that chunk
        (rank r's rows of chunk j start at r * max_chunk_rows[j])."""
        k = self.chunks
        starts = np.array([self.bounds[r] + self.chunk_starts[r][j] for r in range(self.world) for j in range(k)],
                          dtype=np.int64)
        idx = np.searchsorted(starts, colind, side="right") - 1
        owner, chunk = idx // k, idx % k
        local = colind.astype(np.int64) - starts[idx]
        rows = np.repeat(np.arange(rowptr.size - 1, dtype=np.int64), np.diff(rowptr))
        out = []
        for j in range(k):
            sel = np.flatnonzero(chunk == j)
            rp = np.zeros(rowptr.size, dtype=np.int64)
            np.cumsum(np.bincount(rows[sel], minlength=rowptr.size - 1), out=rp[1:])
            ci = (owner[sel] * self.max_chunk_rows[j] + local[sel]).astype(np.int32)
            out.append((rp.astype(np.int32), ci, np.ascontiguousarray(vals[sel]), self.world * self.max_chunk_rows[j]))
        return out

    def all_gather_chunk(self, local: torch.Tensor, j: int, dtype=None, width=None):
        """Starts the gather of row chunk j of every rank's slab; returns (operand, work handle)."""
        dtype = dtype or local.dtype
        width = width or local.shape[1]
        c0, c1 = self.chunk_starts[self.rank][j], self.chunk_starts[self.rank][j + 1]
        src = torch.zeros((self.max_chunk_rows[j], width), dtype=dtype, device=local.device)
        src[: c1 - c0, : local.shape[1]].copy_(local[c0:c1])
        full = torch.empty((self.world * self.max_chunk_rows[j], width), dtype=dtype, device=local.device)
        work = dist.all_gather_into_tensor(full, src, group=self.group, async_op=True)
        self.comm_bytes += full.numel() * full.element_size()
        return full, work

    def _padded_slab(self, local: torch.Tensor, dtype, width: int, keep: bool = True) -> torch.Tensor:
        """This rank's slab in the gather layout: max_rows x width in `dtype`, filled from `local`
        in one pass (conversion, column padding and row padding together). The buffer is kept per
        (dtype, width) and its padding stays zero: only the live rectangle is rewritten. keep=False
        (a gather that stays in flight while the next slab is prepared) takes a fresh buffer."""
        key = (dtype, width, local.device)
        buf = self._slabs.get(key) if keep else None
        if buf is None:
            buf = torch.zeros((self.max_rows, width), dtype=dtype, device=local.device)
            if keep:
                self._slabs[key] = buf
        buf[: local.shape[0], : local.shape[1]].copy_(local)
        return buf

    def all_gather_rows(self, local: torch.Tensor, async_op: bool = False, dtype=None, width=None):
        """Gathered operand; with async_op the pair (operand, work handle to wait on). dtype / width:
        format of the gathered operand (default: that of `local`)."""
        dtype = dtype or local.dtype
        width = width or local.shape[1]
        if self.world == 1:
            out = local if (dtype == local.dtype and width == local.shape[1]) else self._padded_slab(local, dtype, width)
            return (out, _Done()) if async_op else out
        full = torch.empty((self.world * self.max_rows, width), dtype=dtype, device=local.device)
        r0, r1 = self.rows
        if r1 - r0 == self.max_rows and dtype == local.dtype and width == local.shape[1] and local.is_contiguous():
            src = local
        else:
            src = self._padded_slab(local, dtype, width, keep=not async_op)
        work = dist.all_gather_into_tensor(full, src, group=self.group, async_op=async_op)
        self.comm_bytes += full.numel() * full.element_size()
        return (full, work) if async_op else full


def _gather_and_multiply(local, spmm: Callable, sharding: RowSharding, fmt, panels: int = 1):
    """all-gather the row slabs (in the operand format of the kernel when `fmt` is given), SpMM.
    panels > 1: the operand is cut into that many column panels (each at least 32 columns and a
    multiple of 16); all panel gathers are queued at once and the SpMM of a panel starts as soon
    as its own gather has landed, so it overlaps the gathers behind it."""
    n = local.shape[1]
    if isinstance(spmm, (list, tuple)):
        # row chunks: one operator per chunk; all gathers are queued, chunk j is multiplied as soon
        # as it has landed and the partial results are added in chunk order
        assert len(spmm) == sharding.chunks, "one operator per row chunk"
        dtype, width = fmt(n) if fmt is not None else (local.dtype, n)
        pending = [sharding.all_gather_chunk(local, j, dtype, width) for j in range(sharding.chunks)]
        out = None
        for op, (full, work) in zip(spmm, pending):
            work.wait()
            part = op(full)
            out = part if out is None else out.add_(part)
        return out[:, :n].contiguous() if width != n else out
    if sharding.world > 1 and panels > 1 and n % (16 * panels) == 0 and n // panels >= 32:
        w = n // panels
        pending = []
        for j in range(panels):
            src = local[:, j * w:(j + 1) * w]
            if fmt is not None:
                dtype, width = fmt(w)
                assert width == w
                src = src.to(dtype)
            pending.append(sharding.all_gather_rows(src.contiguous(), async_op=True))
        out = None
        for j, (full, work) in enumerate(pending):
            work.wait()
            part = spmm(full)
            if out is None:
                out = part.new_empty((part.shape[0], n))
            out[:, j * w:(j + 1) * w] = part
        return out
    if sharding.world > 1 and fmt is not None:
        dtype, width = fmt(n)
        if dtype != local.dtype or width != n:
            out = spmm(sharding.all_gather_rows(local, dtype=dtype, width=width))
            return out[:, :n].contiguous() if width != n else out
    return spmm(sharding.all_gather_rows(local))


class _ShardedSpMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, H_local, spmm: Callable, spmm_t: Callable, sharding: RowSharding, fmt, fmt_t, panels):
        ctx.spmm_t, ctx.sharding, ctx.fmt_t, ctx.panels = spmm_t, sharding, fmt_t, panels
        return _gather_and_multiply(H_local.detach(), spmm, sharding, fmt, panels)

    @staticmethod
    def backward(ctx, grad_out):
        if not ctx.needs_input_grad[0]:              # the operand is an input of the model: nothing to propagate
            return None, None, None, None, None, None, None
        g = _gather_and_multiply(grad_out.contiguous(), ctx.spmm_t, ctx.sharding, ctx.fmt_t, ctx.panels)
        return g, None, None, None, None, None, None


def sharded_spmm(H_local, spmm, spmm_t, sharding, operand_format=None, operand_format_t=None, panels=1):
    return _ShardedSpMM.apply(H_local, spmm, spmm_t, sharding, operand_format,
                              operand_format_t or operand_format, panels)


class GCN2(nn.Module):
    """h = relu(A (X W1)); out = A (h W2) with bias-free Linear layers
    (GCNBench, gnn_bench/router_vs_baselines_gcn.py:464-476)."""

    def __init__(self, in_dim: int, hidden: int, out_dim: int, spmm: Callable,
                 spmm_t: Optional[Callable] = None, sharding: Optional[RowSharding] = None,
                 operand_format: Optional[Callable] = None, operand_format_t: Optional[Callable] = None,
                 panels: int = 1, aggregate_first: bool = False):
        super().__init__()
        self.lin1 = nn.Linear(in_dim, hidden, bias=False)
        self.lin2 = nn.Linear(hidden, out_dim, bias=False)
        # aggregate_first: layer 1 as (A X) W1 instead of A (X W1) - the same layer, associated the
        # other way. With in_dim < hidden the SpMM (and its gather) runs at the narrower width, and
        # because X needs no gradient the backward of layer 1 has no SpMM at all: dW1 = (A X)^T g.
        # Off by default: the reference harness multiplies by W first.
        self.aggregate_first = aggregate_first
        _attach(self, spmm, spmm_t, sharding, operand_format, operand_format_t, panels)

    def forward(self, X_local):
        if self.aggregate_first:
            h = F.relu(self.lin1(self.aggregate(X_local)))
        else:
            h = F.relu(self.aggregate(self.lin1(X_local)))
        return self.aggregate(self.lin2(h))


def _attach(module, spmm, spmm_t, sharding, operand_format, operand_format_t, panels):
    module.spmm, module.spmm_t = spmm, spmm_t or spmm
    module.sharding = sharding or RowSharding([0, 0])
    module.operand_format = operand_format        # GraphOperator.operand_format, or None = gather as is
    module.operand_format_t = operand_format_t or operand_format
    module.panels = panels
    module.aggregate = lambda H: sharded_spmm(H, module.spmm, module.spmm_t, module.sharding,
                                              module.operand_format, module.operand_format_t, module.panels)


class SAGE2(nn.Module):
    """GraphSAGE with the mean aggregator: h = relu(W1 [x | A x]), out = W2 [h | A h], A = D^-1 Adj
    (SAGEBench, gnn_bench/router_vs_baselines_sage.py:48-67). A is not symmetric: pass the operator
    of the transposed row block as `spmm_t`."""

    def __init__(self, in_dim: int, hidden: int, out_dim: int, spmm: Callable, spmm_t: Callable,
                 sharding: Optional[RowSharding] = None, operand_format: Optional[Callable] = None,
                 operand_format_t: Optional[Callable] = None, panels: int = 1):
        super().__init__()
        self.lin1 = nn.Linear(2 * in_dim, hidden, bias=False)
        self.lin2 = nn.Linear(2 * hidden, out_dim, bias=False)
        _attach(self, spmm, spmm_t, sharding, operand_format, operand_format_t, panels)

    def forward(self, X_local):
        h = F.relu(self.lin1(torch.cat([X_local, self.aggregate(X_local)], dim=1)))
        return self.lin2(torch.cat([h, self.aggregate(h)], dim=1))


class GIN2(nn.Module):
    """GIN: h' = MLP((1 + eps) h + A h) with two-layer bias-free MLPs and learnable eps, raw
    adjacency A (GINBench, gnn_bench/router_vs_baselines_gin.py:47-74)."""

    def __init__(self, in_dim: int, hidden: int, out_dim: int, spmm: Callable,
                 spmm_t: Optional[Callable] = None, sharding: Optional[RowSharding] = None,
                 operand_format: Optional[Callable] = None, operand_format_t: Optional[Callable] = None,
                 panels: int = 1):
        super().__init__()
        self.eps1 = nn.Parameter(torch.zeros(1))
        self.eps2 = nn.Parameter(torch.zeros(1))
        self.mlp1 = nn.Sequential(nn.Linear(in_dim, hidden, bias=False), nn.ReLU(), nn.Linear(hidden, hidden, bias=False))
        self.mlp2 = nn.Sequential(nn.Linear(hidden, hidden, bias=False), nn.ReLU(), nn.Linear(hidden, out_dim, bias=False))
        _attach(self, spmm, spmm_t, sharding, operand_format, operand_format_t, panels)

    def forward(self, X_local):
        h = F.relu(self.mlp1((1.0 + self.eps1) * X_local + self.aggregate(X_local)))
        return self.mlp2((1.0 + self.eps2) * h + self.aggregate(h))


def train_step(model, opt, X_local, y_local, total_rows: int):
    """zero_grad -> forward -> cross-entropy (mean over ALL rows) -> backward ->
    all-reduce of the weight gradients -> optimizer step. Returns the global loss."""
    sh = model.sharding
    opt.zero_grad(set_to_none=True)
    out = model(X_local)
    loss = F.cross_entropy(out, y_local, reduction="sum") / total_rows
    loss.backward()
    if sh.world > 1:
        for p in model.parameters():
            dist.all_reduce(p.grad, group=sh.group)
        loss_g = loss.detach().clone()
        dist.all_reduce(loss_g, group=sh.group)
    else:
        loss_g = loss.detach()
    opt.step()
    return loss_g
