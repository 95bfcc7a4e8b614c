"""Synthetic configuration generators and the multi-GPU row partition (host logic)."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

from oracle import ra_oracle as O
from ra_spmm_b200 import generators as G
from ra_spmm_b200 import partition as P

ROOT = Path(__file__).resolve().parent.parent


def _check_csr(a):
    assert a.rowptr.dtype == np.int32 and a.colind.dtype == np.int32 and a.vals.dtype == np.float32
    assert a.rowptr[0] == 0 and a.rowptr[-1] == a.colind.size == a.vals.size
    rows = np.repeat(np.arange(a.M), np.diff(a.rowptr))
    key = rows.astype(np.int64) * a.K + a.colind
    assert np.all(np.diff(key) > 0)          # sorted, unique columns inside each row
    assert a.colind.min() >= 0 and a.colind.max() < a.K


def test_c1_exact_shape():
    a = G.erdos_renyi_fixed_degree()
    _check_csr(a)
    assert (a.M, a.K, a.nnz) == (4096, 4096, 65536)
    assert np.all(a.degrees() == 16)
    assert np.abs(a.vals).max() <= 1.0
    b = G.erdos_renyi_fixed_degree()
    assert np.array_equal(a.colind, b.colind) and np.array_equal(a.vals, b.vals)   # seeded


def test_reduced_configs_have_the_named_regimes():
    a = G.chung_lu_power_law(n=65536, seed=1)
    _check_csr(a)
    f = O.features_device(a.rowptr, a.M, a.K, 128)
    assert f["degree_cv"] > 3.0 and 8 < f["avg_nnz_per_row"] < 13
    assert np.all(a.colind[a.rowptr[:-1]] <= np.arange(a.M))     # self loop present => first col <= row
    s = G.sbm_graph(n=5000, n_comm=50, mean_degree=60, seed=2)
    _check_csr(s)
    assert np.array_equal(s.vals, s.vals.astype(np.float16).astype(np.float32))  # fp16-exact values
    r = G.rmat_graph(scale=12, seed=3)
    _check_csr(r)
    assert (r.degrees() == 0).mean() > 0.1 and O.features_device(r.rowptr, r.M, r.K, 64)["degree_cv"] > 1.5
    g = G.gcn_normalized_sbm(n=4000, n_comm=8, seed=123)
    _check_csr(g)
    d = g.degrees().astype(np.float64)
    rows = np.repeat(np.arange(g.M), g.degrees())
    assert np.allclose(g.vals, 1.0 / np.sqrt(d[rows] * d[g.colind]), rtol=1e-6)


def test_row_splits_balanced_and_aligned():
    a = G.rmat_graph(scale=14, seed=3)
    for parts in (1, 2, 4, 8):
        b = P.nnz_balanced_row_splits(a.rowptr, parts)
        assert b[0] == 0 and b[-1] == a.M and np.all(np.diff(b) >= 0)
        assert np.all(b[1:-1] % 8 == 0)
        w = np.diff(a.rowptr[b].astype(np.int64)) + np.diff(b)
        assert w.max() <= 1.25 * w.mean() + 8 * 64
    # a heavier row weight moves rows out of the block that holds the many light rows
    for rw in (3.0, 6.0):
        b = P.nnz_balanced_row_splits(a.rowptr, 2, row_weight=rw)
        w = np.diff(a.rowptr[b].astype(np.int64)) + rw * np.diff(b)
        assert b[0] == 0 and b[-1] == a.M and b[1] % 8 == 0
        assert abs(w[0] - w[1]) <= 0.02 * w.sum() + 8 * 64 * rw
    b1 = P.nnz_balanced_row_splits(a.rowptr, 2)[1]
    b6 = P.nnz_balanced_row_splits(a.rowptr, 2, row_weight=6.0)[1]
    assert b6 >= b1            # R-MAT: hubs first, so the first block takes more rows
    # sub-blocks reassemble the matrix
    b = P.nnz_balanced_row_splits(a.rowptr, 4)
    cols = np.concatenate([P.row_block(a.rowptr, a.colind, a.vals, b[i], b[i + 1])[1] for i in range(4)])
    assert np.array_equal(cols, a.colind)


def test_rank_grid_choice_and_reassembly():
    # B beyond the L2: column panels down to 32 columns, the rest of the ranks split rows
    assert P.choose_grid(8, 128, 1048576) == (2, 4)
    assert P.choose_grid(4, 128, 1048576) == (1, 4)
    assert P.choose_grid(2, 128, 1048576) == (1, 2)
    assert P.choose_grid(8, 64, 4194304) == (4, 2)
    assert P.choose_grid(8, 64, 4096) == (8, 1)                # B fits the L2: rows only
    assert P.choose_grid(8, 128, 1048576, column_shard=False) == (8, 1)
    assert P.choose_grid(1, 128, 1048576) == (1, 1)
    a = G.chung_lu_power_law(n=3000, seed=2)
    B = G.dense(a.K, 64, 2).numpy()
    want = O.spmm_reference(a.rowptr, a.colind, a.vals, B)
    rows, cols = 2, 2
    bounds = P.nnz_balanced_row_splits(a.rowptr, rows)
    got = np.zeros_like(want)
    for rank in range(rows * cols):
        ri, cj = rank // cols, rank % cols
        r0, r1 = int(bounds[ri]), int(bounds[ri + 1])
        rp, ci, va = P.row_block(a.rowptr, a.colind, a.vals, r0, r1)
        Nl = 64 // cols
        got[r0:r1, cj * Nl:(cj + 1) * Nl] = O.spmm_reference(rp, ci, va, B[:, cj * Nl:(cj + 1) * Nl])
    assert np.array_equal(got, want)


def test_moments_are_additive_bit_exact():
    a = G.chung_lu_power_law(n=50000, seed=5)
    whole = O.features_device(a.rowptr, a.M, a.K, 128)
    b = P.nnz_balanced_row_splits(a.rowptr, 8)
    parts = []
    for i in range(8):
        rp, _, _ = P.row_block(a.rowptr, a.colind, a.vals, b[i], b[i + 1])
        f = O.features_device(rp, rp.size - 1, a.K, 128) if rp.size > 1 else dict(sum_deg=0, sum_deg_sq=0)
        parts.append((f["sum_deg"], f["sum_deg_sq"]))
    s1, s2 = P.combine_moments(parts)
    avg, std, cv = P.features_from_moments(s1, s2, a.M)
    assert (avg.tobytes(), std.tobytes(), cv.tobytes()) == (
        whole["avg_nnz_per_row"].tobytes(), whole["std_nnz_per_row"].tobytes(), whole["degree_cv"].tobytes())


def test_two_rank_gloo_sharded_spmm():
    """world_size 2 over gloo: each rank multiplies its row block (CPU oracle as the
    per-rank compute stand-in), moments are all-gathered, C slabs match the whole."""
    script = ROOT / "tests" / "_gloo_worker.py"
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29533")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "GLOO_OK" in r.stdout


def test_rebalance_by_time_equalises_a_two_rate_cost():
    """Rows of the first half cost 3x per nonzero: a weight cut leaves 3:1 times; the time-driven
    update converges to equal times, keeps 8-row alignment and monotone boundaries."""
    rng = np.random.default_rng(0)
    M = 40000
    deg = rng.integers(1, 20, size=M)
    rowptr = np.zeros(M + 1, dtype=np.int64); np.cumsum(deg, out=rowptr[1:])
    cost_per_row = np.where(np.arange(M) < M // 2, 3.0, 1.0) * deg
    prefix = np.concatenate([[0.0], np.cumsum(cost_per_row)])
    block_times = lambda b: [prefix[b[i + 1]] - prefix[b[i]] for i in range(len(b) - 1)]
    b = P.nnz_balanced_row_splits(rowptr, 4)
    t0 = block_times(b)
    assert max(t0) / (sum(t0) / 4) > 1.4
    for _ in range(3):
        b = P.rebalance_by_time(rowptr, b, block_times(b))
        assert b[0] == 0 and b[-1] == M and all(x % 8 == 0 for x in b[:-1]) and all(np.diff(b) >= 0)
    t = block_times(b)
    assert max(t) / (sum(t) / 4) < 1.02
    # equal measured times leave the cut (almost) where it is
    same = P.rebalance_by_time(rowptr, b, [1.0, 1.0, 1.0, 1.0])
    assert np.all(np.abs(same - b) <= 8)
