"""Seeded synthetic inputs for the five benchmark configurations.

The reference measures on public graph datasets that are not redistributed with
it; these generators produce stand-ins with the same shapes, sizes and
degree/value distributions. Sparse structure comes from numpy
`default_rng(seed)`; dense operands from `torch.manual_seed(seed)` on the CPU,
so every consumer (CPU oracle, reference kernels, this library) sees the same
bits. All CSR outputs have int32 indices, sorted unique columns per row.

Every generator takes size parameters so tests can run reduced copies of the
same distribution.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass
class CSR:
    M: int
    K: int
    rowptr: np.ndarray   # int32 [M+1]
    colind: np.ndarray   # int32 [nnz]
    vals: np.ndarray     # float32 [nnz]

    @property
    def nnz(self) -> int:
        return int(self.rowptr[-1])

    def degrees(self) -> np.ndarray:
        return np.diff(self.rowptr)

    def torch(self, device="cpu"):
        import torch
        return (torch.from_numpy(self.rowptr).to(device), torch.from_numpy(self.colind).to(device),
                torch.from_numpy(self.vals).to(device))


def dense(K: int, N: int, seed: int, dtype="float32"):
    """B ~ N(0,1) generated on the CPU with torch.manual_seed(seed)."""
    import torch
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    B = torch.randn((K, N), generator=g, dtype=torch.float32)
    if dtype == "float16":
        B = B.to(torch.float16)
    return B


def _cuda():
    """The current CUDA device when torch sees one, else None. Only the sort/dedup and the
    elementwise bit work of the generators run there (seconds instead of minutes at 10^8
    edges); the random draws always come from numpy, so the graph is the same either way."""
    try:
        import torch
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None
    except (ImportError, RuntimeError):
        return None


def _sorted_unique(keys: np.ndarray) -> np.ndarray:
    """np.unique by sort + neighbour compare (numpy's hash-based unique is several times
    slower on 10^7 integer keys)."""
    keys = np.sort(keys, kind="stable")
    if keys.size == 0:
        return keys
    keep = np.empty(keys.size, dtype=bool)
    keep[0] = True
    np.not_equal(keys[1:], keys[:-1], out=keep[1:])
    return keys[keep]


def _csr_from_edges(u, v, n: int, self_loops: bool):
    """Symmetrised, deduplicated CSR structure (rowptr int32 [n+1], cols int32) of the
    undirected edge list (u, v); `self_loops` adds the diagonal. u, v: integer numpy arrays
    or torch tensors on the build device."""
    dev = _cuda()
    if dev is not None and (not isinstance(u, np.ndarray) or u.size >= (1 << 20)):
        import torch
        tu = (torch.from_numpy(u) if isinstance(u, np.ndarray) else u).to(dev).to(torch.int64)
        tv = (torch.from_numpy(v) if isinstance(v, np.ndarray) else v).to(dev).to(torch.int64)
        parts = [tu * n + tv, tv * n + tu]
        del tu, tv
        if self_loops:
            d = torch.arange(n, dtype=torch.int64, device=dev)
            parts.append(d * n + d)
        keys = torch.unique(torch.cat(parts))
        del parts
        rows = torch.div(keys, n, rounding_mode="floor")
        cols = (keys - rows * n).to(torch.int32)
        del keys
        rowptr = torch.zeros(n + 1, dtype=torch.int64, device=dev)
        torch.cumsum(torch.bincount(rows, minlength=n), 0, out=rowptr[1:])
        assert int(rowptr[-1]) < 2**31
        out = rowptr.to(torch.int32).cpu().numpy(), cols.cpu().numpy()
        del rows, cols, rowptr
        torch.cuda.empty_cache()
        return out
    u = np.asarray(u).astype(np.int64); v = np.asarray(v).astype(np.int64)
    parts = [u * n + v, v * n + u]
    if self_loops:
        d = np.arange(n, dtype=np.int64)
        parts.append(d * n + d)
    keys = _sorted_unique(np.concatenate(parts))
    rows = keys // n
    cols = (keys - rows * n).astype(np.int32)
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(rows, minlength=n), out=rowptr[1:])
    assert rowptr[-1] < 2**31
    return rowptr.astype(np.int32), cols


def _uniform_f32(rng, lo: float, hi: float, size: int, chunk: int = 1 << 24) -> np.ndarray:
    """rng.uniform(lo, hi, size).astype(float32) drawn in chunks through one reused float64
    buffer (same values: numpy's uniform is lo + (hi - lo) * next_double)."""
    out = np.empty(size, dtype=np.float32)
    buf = np.empty(min(chunk, max(size, 1)), dtype=np.float64)
    for s0 in range(0, size, chunk):
        k = min(chunk, size - s0)
        rng.random(out=buf[:k])
        np.multiply(buf[:k], hi - lo, out=buf[:k])
        np.add(buf[:k], lo, out=buf[:k])
        out[s0:s0 + k] = buf[:k]
    return out


# ---- C1 -----------------------------------------------------------------------
def erdos_renyi_fixed_degree(M=4096, K=4096, deg=16, seed=0) -> CSR:
    """Exactly `deg` distinct uniform columns per row, sorted; values U(-1,1)."""
    rng = np.random.default_rng(seed)
    # the `deg` smallest of K iid uniforms form a uniform subset without replacement
    cols = np.argpartition(rng.random((M, K), dtype=np.float32), deg - 1, axis=1)[:, :deg]
    cols = np.sort(cols, axis=1).astype(np.int32).reshape(-1)
    rowptr = (np.arange(M + 1, dtype=np.int64) * deg).astype(np.int32)
    vals = rng.uniform(-1.0, 1.0, size=cols.size).astype(np.float32)
    return CSR(M, K, rowptr, cols, vals)


# ---- C2 -----------------------------------------------------------------------
def chung_lu_power_law(n=1_048_576, gamma=2.1, mean_degree=10.0, seed=1, cap=True) -> CSR:
    """Chung-Lu graph with expected degrees w_i proportional to (i+1)^(-1/(gamma-1)).

    n*mean_degree/2 undirected edges are drawn with both endpoints sampled
    proportionally to w; with `cap`, weights are clipped at sqrt(sum w) (the
    Chung-Lu admissibility bound w_i*w_j <= sum w). The edge list is
    symmetrised, deduplicated and self loops are added; values are
    1/sqrt(d_i*d_j) with d the final row degrees (fp32).
    """
    rng = np.random.default_rng(seed)
    w = (np.arange(1, n + 1, dtype=np.float64)) ** (-1.0 / (gamma - 1.0))
    w *= (n * mean_degree) / w.sum()
    if cap:
        w = np.minimum(w, np.sqrt(n * mean_degree))
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    n_edges = int(n * mean_degree / 2)
    u = np.searchsorted(cdf, rng.random(n_edges), side="right").astype(np.int64)
    v = np.searchsorted(cdf, rng.random(n_edges), side="right").astype(np.int64)
    np.minimum(u, n - 1, out=u); np.minimum(v, n - 1, out=v)
    rowptr, cols = _csr_from_edges(u, v, n, self_loops=True)
    deg = np.diff(rowptr).astype(np.float64)
    rows = np.repeat(np.arange(n, dtype=np.int64), np.diff(rowptr))
    vals = (1.0 / np.sqrt(deg[rows] * deg[cols])).astype(np.float32)
    return CSR(n, n, rowptr, cols, vals)


# ---- C3 / C5 structure ---------------------------------------------------------
def _triu_pairs(idx: np.ndarray, n: int):
    """Map linear indices of the strict upper triangle of an n x n matrix to (i, j)."""
    # row i starts at offset i*n - i*(i+1)/2 - i ... solve with the closed form
    idx = idx.astype(np.float64)
    i = np.floor((2 * n - 1 - np.sqrt((2 * n - 1) ** 2 - 8 * idx)) / 2).astype(np.int64)
    start = i * (2 * n - i - 1) // 2
    # guard the float rounding at row boundaries
    lo = idx.astype(np.int64) < start
    i[lo] -= 1
    start = i * (2 * n - i - 1) // 2
    nxt = (i + 1) * (2 * n - i - 2) // 2
    hi = idx.astype(np.int64) >= nxt
    i[hi] += 1
    start = i * (2 * n - i - 1) // 2
    j = idx.astype(np.int64) - start + i + 1
    return i, j


def sbm_edges(n: int, n_comm: int, mean_degree: float, intra_frac: float, rng):
    """Undirected SBM edge list (u, v) with near-equal communities c = floor(n_comm*i/n)."""
    bounds = (np.arange(n_comm + 1, dtype=np.int64) * n + n_comm - 1) // n_comm  # ceil splits
    bounds[-1] = n
    us, vs = [], []
    intra_deg = mean_degree * intra_frac
    for c in range(n_comm):
        lo, hi = int(bounds[c]), int(bounds[c + 1])
        sz = hi - lo
        if sz < 2:
            continue
        pairs = sz * (sz - 1) // 2
        p_in = min(1.0, intra_deg / (sz - 1))
        if p_in > 0.02 and pairs < 60_000_000:
            hit = np.flatnonzero(rng.random(pairs, dtype=np.float32) < p_in)
        else:
            m = rng.binomial(pairs, p_in)
            hit = _sorted_unique(rng.integers(0, pairs, size=m, dtype=np.int64))
        i, j = _triu_pairs(hit, sz)
        us.append(i + lo); vs.append(j + lo)
    # inter-community edges: uniform pairs, same-community pairs rejected
    m_inter = int(n * mean_degree * (1.0 - intra_frac) / 2)
    if m_inter > 0 and n_comm > 1:
        over = int(m_inter * (1.0 + 2.0 / n_comm) + 16)
        a = rng.integers(0, n, size=over, dtype=np.int64)
        b = rng.integers(0, n, size=over, dtype=np.int64)
        ca = np.searchsorted(bounds, a, side="right")
        cb = np.searchsorted(bounds, b, side="right")
        keep = np.flatnonzero(ca != cb)[:m_inter]
        us.append(a[keep]); vs.append(b[keep])
    return np.concatenate(us), np.concatenate(vs)


def sbm_graph(n=232_960, n_comm=50, mean_degree=490.0, intra_frac=0.92, seed=2,
              value_dtype="float16", shuffle=True) -> CSR:
    """Stochastic block model, symmetric, node order shuffled; values U(0,1)
    drawn in `value_dtype` and returned as float32 (exact for fp16 draws)."""
    rng = np.random.default_rng(seed)
    u, v = sbm_edges(n, n_comm, mean_degree, intra_frac, rng)
    if shuffle:
        perm = rng.permutation(n).astype(np.int64)
        u, v = perm[u], perm[v]
    rowptr, cols = _csr_from_edges(u, v, n, self_loops=False)
    vals = rng.random(cols.size, dtype=np.float32)
    if value_dtype == "float16":
        vals = vals.astype(np.float16).astype(np.float32)
    return CSR(n, n, rowptr, cols, vals)


# ---- C4 -----------------------------------------------------------------------
def rmat_graph(scale=22, edge_factor=16, a=0.57, b=0.19, c=0.19, seed=3) -> CSR:
    """R-MAT (bit-recursive quadrant sampling), symmetrised and deduplicated,
    no added self loops; values U(-1,1)."""
    rng = np.random.default_rng(seed)
    n = 1 << scale
    m = edge_factor * n
    assert scale <= 31
    ab, abc = a + b, a + b + c
    r = np.empty(m, dtype=np.float32)
    dev = _cuda() if m >= (1 << 20) else None
    if dev is not None:                 # draws on the host, bit assembly on the device
        import torch
        u = torch.zeros(m, dtype=torch.int32, device=dev)
        v = torch.zeros(m, dtype=torch.int32, device=dev)
        # thresholds as float32, the type numpy compares a float32 array against a Python float in
        a32, ab32, abc32 = (float(np.float32(x)) for x in (a, ab, abc))
        for _ in range(scale):
            rng.random(out=r, dtype=np.float32)
            t = torch.from_numpy(r).to(dev)
            u.mul_(2).add_(t >= ab32)
            v.mul_(2).add_(((t >= a32) & (t < ab32)) | (t >= abc32))
        del t
    else:
        u = np.zeros(m, dtype=np.uint32)
        v = np.zeros(m, dtype=np.uint32)
        t1 = np.empty(m, dtype=bool)
        t2 = np.empty(m, dtype=bool)
        for _ in range(scale):
            rng.random(out=r, dtype=np.float32)
            np.left_shift(u, 1, out=u)
            np.bitwise_or(u, np.greater_equal(r, ab, out=t1), out=u)        # row bit
            np.greater_equal(r, a, out=t1)
            np.less(r, ab, out=t2)
            t1 &= t2
            t1 |= np.greater_equal(r, abc, out=t2)                           # column bit
            np.left_shift(v, 1, out=v)
            np.bitwise_or(v, t1, out=v)
    del r
    rowptr, cols = _csr_from_edges(u, v, n, self_loops=False)
    vals = _uniform_f32(rng, -1.0, 1.0, cols.size)
    return CSR(n, n, rowptr, cols, vals)


# ---- C5 -----------------------------------------------------------------------
def gcn_normalized_sbm(n=2_449_029, n_comm=500, mean_degree=50.0, intra_frac=0.9, seed=123) -> CSR:
    """D^-1/2 (A+I) D^-1/2 of a shuffled SBM graph, computed in float64 and cast
    to fp32 (the operator of gnn_bench/router_vs_baselines_gcn.py:89-126)."""
    rng = np.random.default_rng(seed)
    u, v = sbm_edges(n, n_comm, mean_degree, intra_frac, rng)
    perm = rng.permutation(n).astype(np.int64)
    u, v = perm[u], perm[v]
    rowptr, cols = _csr_from_edges(u, v, n, self_loops=True)
    deg = np.diff(rowptr).astype(np.float64)
    dinv = 1.0 / np.sqrt(deg)
    rows = np.repeat(np.arange(n, dtype=np.int64), np.diff(rowptr))
    vals = (dinv[rows] * dinv[cols]).astype(np.float32)
    return CSR(n, n, rowptr, cols, vals)


# ---- named configurations -------------------------------------------------------
CONFIG_SEEDS = {"C1": 0, "C2": 1, "C3": 2, "C4": 3, "C5": 123}


def make_config(name: str, scale: float = 1.0):
    """(CSR, N, b_dtype) for configuration C1..C5; `scale` < 1 shrinks the node
    count (degree distribution parameters unchanged) for tests."""
    if name == "C1":
        m = max(64, int(4096 * scale))
        return erdos_renyi_fixed_degree(m, m, 16, CONFIG_SEEDS[name]), 64, "float32"
    if name == "C2":
        return chung_lu_power_law(max(1024, int(1_048_576 * scale)), 2.1, 10.0,
                                  CONFIG_SEEDS[name]), 128, "float32"
    if name == "C3":
        n = max(1000, int(232_960 * scale))
        return sbm_graph(n, 50, min(490.0, n / 10), 0.92, CONFIG_SEEDS[name]), 256, "float16"
    if name == "C4":
        sc = max(10, 22 + int(np.floor(np.log2(scale))) if scale < 1 else 22)
        return rmat_graph(sc, 16, 0.57, 0.19, 0.19, CONFIG_SEEDS[name]), 64, "float32"
    if name == "C5":
        n = max(2000, int(2_449_029 * scale))
        return gcn_normalized_sbm(n, max(2, int(500 * scale)), 50.0, 0.9,
                                  CONFIG_SEEDS[name]), 256, "float32"
    raise ValueError(name)


def cached_config(name: str, scale: float = 1.0, cache_dir=None):
    """make_config through an on-disk cache: one uncompressed .npz per (configuration, seed,
    scale) under `cache_dir` (default: $RA_SPMM_GRAPH_CACHE, else <tmp>/ra_spmm_b200_graphs).
    Ranks of one job call this on rank 0 first and on the others after a barrier, so the
    10^8-edge graphs are generated once per machine instead of once per process."""
    import os
    import tempfile
    from pathlib import Path
    root = Path(cache_dir or os.environ.get("RA_SPMM_GRAPH_CACHE")
                or Path(tempfile.gettempdir()) / "ra_spmm_b200_graphs")
    path = root / f"{name}_scale{scale:g}_seed{CONFIG_SEEDS[name]}_v1.npz"
    if path.exists():
        try:
            with np.load(path) as z:
                meta = z["meta"]
                return (CSR(int(meta[0]), int(meta[1]), z["rowptr"], z["colind"], z["vals"]),
                        int(meta[2]), "float16" if int(meta[3]) else "float32")
        except Exception:
            pass                                   # unreadable file: regenerate
    a, N, b_dtype = make_config(name, scale)
    if a.nnz >= (1 << 20):
        try:
            root.mkdir(parents=True, exist_ok=True)
            tmp = path.with_suffix(f".{os.getpid()}.tmp.npz")
            np.savez(tmp, rowptr=a.rowptr, colind=a.colind, vals=a.vals,
                     meta=np.array([a.M, a.K, N, 1 if b_dtype == "float16" else 0], dtype=np.int64))
            os.replace(tmp, path)
        except OSError:
            pass                                   # read-only or full disk: run uncached
    return a, N, b_dtype
