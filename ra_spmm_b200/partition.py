"""Partition of A (rows) and B (column panels) for multi-GPU SpMM (one process per GPU).

Output rows of C = A*B are independent, so A is cut into contiguous row blocks
with nnz-balanced boundaries, B is replicated, and every rank writes its own row
slab of C; a standalone SpMM needs no collective. Boundaries are multiples of
8 rows so that the 8-row tile windows of the reference format
(tc/ra_tc_direct.cu:648-660) never straddle two ranks.

Router features are additive over row blocks: every rank scans its own rowptr
slice for (sum d, sum d^2) and the host adds them, which reproduces the
single-GPU decision bit for bit.
"""
from __future__ import annotations

import numpy as np


def nnz_balanced_row_splits(rowptr: np.ndarray, parts: int, align: int = 8,
                            row_weight: float = 1.0) -> np.ndarray:
    """Boundaries b[0..parts] with b[0]=0, b[parts]=M, each a multiple of `align`
    (except M), chosen so that every block holds an equal share of the weight
    nonzeros + row_weight * rows (rows cost output bandwidth and per-row work even
    when empty; row_weight says how many nonzeros one row is worth)."""
    rowptr = np.asarray(rowptr, dtype=np.int64)
    M = rowptr.size - 1
    nnz = int(rowptr[-1] - rowptr[0])
    bounds = np.zeros(parts + 1, dtype=np.int64)
    bounds[parts] = M
    # weight of a row prefix = nonzeros + rows (one C row write per row)
    weight = (rowptr - rowptr[0]) + np.floor(np.arange(M + 1, dtype=np.float64) * row_weight).astype(np.int64)
    total = int(weight[-1])
    for p in range(1, parts):
        target = total * p // parts
        r = int(np.searchsorted(weight, target, side="left"))
        r = min(M, (r + align // 2) // align * align)
        bounds[p] = max(bounds[p - 1], r)
    return bounds


def rebalance_by_time(rowptr: np.ndarray, bounds, times_ms, row_weight: float = 1.0,
                      align: int = 8) -> np.ndarray:
    """New boundaries from the measured time of every block.

    Block i spans weight w_i (nonzeros + row_weight * rows) and took t_i: inside a block the
    cost per unit of weight is taken as constant (t_i / w_i), which makes the cumulative cost a
    piecewise-linear function of the weight coordinate. The new boundaries sit where that
    function crosses p/P of the total, mapped back to a row and rounded to a multiple of
    `align` rows. A degree-binned kernel does not cost the same per nonzero in a block of
    hub rows as in a block of short rows, so a cut by weight alone leaves the blocks unequal;
    two or three rounds of this update equalise the measured times."""
    rowptr = np.asarray(rowptr, dtype=np.int64)
    M = rowptr.size - 1
    bounds = np.asarray(bounds, dtype=np.int64)
    parts = bounds.size - 1
    t = np.maximum(np.asarray(times_ms, dtype=np.float64), 1e-9)
    assert t.size == parts
    weight = (rowptr - rowptr[0]).astype(np.float64) + np.arange(M + 1, dtype=np.float64) * row_weight
    wb = weight[bounds]                                  # weight coordinate of the old boundaries
    cum_t = np.concatenate([[0.0], np.cumsum(t)])
    new = bounds.copy()
    for p in range(1, parts):
        target = cum_t[-1] * p / parts
        j = int(min(parts - 1, np.searchsorted(cum_t, target, side="right") - 1))
        frac = (target - cum_t[j]) / t[j]
        coord = wb[j] + frac * (wb[j + 1] - wb[j])
        r = int(np.searchsorted(weight, coord, side="left"))
        r = min(M, (r + align // 2) // align * align)
        new[p] = max(new[p - 1], r)
    new[parts] = M
    return new


L2_BYTES = 126 * 1000 * 1000      # B200 L2 capacity


def choose_grid(world: int, N: int, K: int, b_elem_bytes: int = 4, min_panel: int = 32,
                column_shard: bool = True):
    """(row_blocks, col_panels) with row_blocks * col_panels == world.

    The ranks form a grid: `col_panels` column panels of B (each N / col_panels wide, at
    least `min_panel`) times `row_blocks` row blocks of A. Column panels are used only when
    the replicated B would not fit the L2 (then every rank re-reads gathered B rows from
    HBM, and a narrower panel raises the L2 hit rate far more than the extra reads of A
    cost); otherwise the partition is by rows only."""
    if world <= 1 or not column_shard or K * N * b_elem_bytes <= L2_BYTES:
        return max(world, 1), 1
    cols = 1
    while cols * 2 <= world and world % (cols * 2) == 0 and N % (cols * 2) == 0 and N // (cols * 2) >= min_panel:
        cols *= 2
    return world // cols, cols


def row_block(rowptr: np.ndarray, colind: np.ndarray, vals: np.ndarray, r0: int, r1: int):
    """Sub-CSR of rows [r0, r1) with rowptr rebased to 0 (same K)."""
    rowptr = np.asarray(rowptr)
    s, e = int(rowptr[r0]), int(rowptr[r1])
    return ((rowptr[r0 : r1 + 1] - rowptr[r0]).astype(np.int32),
            np.ascontiguousarray(colind[s:e]), np.ascontiguousarray(vals[s:e]))


def combine_moments(moments) -> tuple[int, int]:
    """Sum per-rank (sum_deg, sum_deg_sq) pairs (exact Python integers)."""
    s1 = sum(int(m[0]) for m in moments)
    s2 = sum(int(m[1]) for m in moments)
    return s1, s2


def features_from_moments(sum_deg: int, sum_deg_sq: int, M: int):
    """Host finish of the device feature scan on global moments: the one-pass
    formula of router/router_features_cuda.cu:83-90. Returns (avg, std, cv) as
    float32 values."""
    s = np.float64(sum_deg); ss = np.float64(sum_deg_sq)
    avg = s / np.float64(M)
    var = max(np.float64(0.0), ss / np.float64(M) - avg * avg)
    std = np.sqrt(var)
    cv = np.float32(std / avg) if avg > 1e-6 else np.float32(0.0)
    return np.float32(avg), np.float32(std), cv
