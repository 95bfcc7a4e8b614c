"""CPU restatement of the RA-SpMM hot path. TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA library: only tests, the smoke check
and the benchmark's CPU-baseline leg may import it; the product never does.

Every function restates an algorithm of the reference and cites the file and
lines (paths inside the RA-SpMM project) it follows. Parity pins:
  * route decisions: the 192 (graph, N) known answers in the reference's
    fgcs_results/revision/tf32/{final_fair_v3,router_quality_v8}.csv and the
    reference's own route_dispatch compiled from source (oracle/_ref);
  * features: the reference's compute_production_router_features compiled from
    source (oracle/_ref);
  * plan arrays and kernel outputs: the reference's plan builders and kernels
    compiled from source for sm_100a (oracle/_ref), compared on the GPU.
Golden vectors generated from those pins live in tests/golden/.
"""
from __future__ import annotations

import numpy as np

PATH_NAMES = [
    "CSR_DIRECT", "CSR_ADAPTIVE", "STAGED_REUSE", "TC_SPARSE", "ROW_SPLIT_CUDA",
    "TC_REORDERED", "HYBRID_TC_CUDA", "CUSPARSE", "RODE_ENHANCED", "VECTORIZED_COARSE",
    "LOCALITY_TILED", "TC_DIRECT", "COMMUNITY_TC", "ZERO_OVERHEAD_CSR", "SEGMENT_HYBRID",
]

f32 = np.float32


# ---------------------------------------------------------------------------
# Router features
# ---------------------------------------------------------------------------
def features_host(rowptr, M, K, N):
    """compute_production_router_features, router/router_features.cpp:79-111.

    Two-pass formula; the squared deviations are summed serially (np.cumsum is
    a sequential float64 accumulation), which is the order the reference uses
    with one thread."""
    out = dict(avg_nnz_per_row=f32(0), std_nnz_per_row=f32(0), degree_cv=f32(0),
               total_nnz=0, matrix_M=M, matrix_K=K, output_dim_N=N)
    if rowptr is None or M <= 0 or K <= 0:
        return out
    rowptr = np.asarray(rowptr)
    nnz = int(rowptr[M]) - int(rowptr[0])
    out["total_nnz"] = nnz
    avg = np.float64(nnz) / np.float64(M)
    out["avg_nnz_per_row"] = f32(avg)
    if nnz <= 0:
        return out
    deg = np.diff(rowptr[: M + 1]).astype(np.float64)
    delta = deg - avg
    sq = np.cumsum(delta * delta)[-1]
    std = np.sqrt(sq / np.float64(M))
    out["std_nnz_per_row"] = f32(std)
    out["degree_cv"] = f32(std / avg) if avg > 1e-6 else f32(0)
    return out


def features_device(rowptr, M, K, N):
    """compute_production_router_features_gpu host finish,
    router/router_features_cuda.cu:83-90, on exact integer moments."""
    out = dict(avg_nnz_per_row=f32(0), std_nnz_per_row=f32(0), degree_cv=f32(0),
               total_nnz=0, matrix_M=M, matrix_K=K, output_dim_N=N, sum_deg=0, sum_deg_sq=0)
    if rowptr is None or M <= 0 or K <= 0:
        return out
    deg = np.diff(np.asarray(rowptr)[: M + 1]).astype(np.int64)
    s1 = int(deg.sum())
    s2 = int((deg * deg).sum())          # deg < 2^31, so each square fits int64
    s = np.float64(s1); ss = np.float64(s2)
    avg = s / np.float64(M)
    var = max(np.float64(0.0), ss / np.float64(M) - avg * avg)
    std = np.sqrt(var)
    out.update(total_nnz=int(s), avg_nnz_per_row=f32(avg), std_nnz_per_row=f32(std),
               degree_cv=f32(std / avg) if avg > 1e-6 else f32(0), sum_deg=s1, sum_deg_sq=s2)
    return out


# ---------------------------------------------------------------------------
# Router: feasibility + seven rules
# ---------------------------------------------------------------------------
def route(avg_nnz, degree_cv, M, N):
    """MAIN-portfolio decision of route_dispatch: feasibility
    (router/router_dispatch.cpp:107-464 with the production feature set, i.e.
    all diagnostic proxies zero) and the seven-rule block (:979-1110).
    Comparisons are float32 against float32 literals."""
    d = f32(avg_nnz)
    cv = f32(degree_cv)
    tile_feas = N >= 16
    feas = {n: False for n in PATH_NAMES}
    feas.update(CSR_DIRECT=True, CUSPARSE=True, ZERO_OVERHEAD_CSR=True,
                RODE_ENHANCED=not (cv < f32(0.80)), VECTORIZED_COARSE=not (d > f32(12.0)),
                LOCALITY_TILED=tile_feas, TC_DIRECT=tile_feas, COMMUNITY_TC=tile_feas,
                SEGMENT_HYBRID=tile_feas)
    est_plan_s = 2e-8 * float(d) * float(M)
    tile_ok = feas["TC_DIRECT"] and est_plan_s <= 20.0
    st = dict(choice="TC_DIRECT" if tile_feas else "CSR_DIRECT",
              reason="tc_direct_default_winner" if tile_feas else "csr_direct_tc_direct_infeasible",
              risk=f32(0.05), tf32=False)

    def pick(path, why, force=False):
        if tile_ok and feas[path]:
            st.update(choice=path, reason=why, risk=f32(0.06),
                      tf32=bool(force or d < f32(5.0) or (M <= 25000 and d < f32(9.0))))
        elif cv < f32(1.5):
            st.update(choice="CSR_DIRECT", reason="csr_direct_tile_gated", risk=f32(0.05))
        else:
            st.update(choice="ZERO_OVERHEAD_CSR", reason="zero_overhead_tile_gated", risk=f32(0.06))

    if cv >= f32(5.0):
        st.update(choice="ZERO_OVERHEAD_CSR", reason="zero_overhead_extreme_skew", risk=f32(0.06))
    elif cv < f32(0.7):
        if d < f32(4.5):
            if N <= 256:
                st.update(choice="CSR_DIRECT", reason="csr_direct_uniform_ultralow_d", risk=f32(0.05))
            else:
                pick("TC_DIRECT", "tc_direct_uniform_wideN")
        elif cv >= f32(0.2) and d < f32(7.0):
            if N <= 128:
                st.update(choice="CSR_DIRECT", reason="csr_direct_synth_community", risk=f32(0.05))
            else:
                pick("TC_DIRECT", "tc_direct_community_wideN", True)
        else:
            pick("TC_DIRECT", "tc_direct_uniform")
    elif cv >= f32(3.0):
        if M >= 250000:
            pick("COMMUNITY_TC", "community_tc_skewed_large")
        else:
            pick("SEGMENT_HYBRID", "segment_hybrid_skewed_medium")
    elif d >= f32(40.0):
        pick("COMMUNITY_TC", "community_tc_dense_rows")
    elif M < 20000 and d >= f32(25.0):
        if N < 96:
            st.update(choice="CUSPARSE", reason="cusparse_small_dense_narrowN", risk=f32(0.05))
        elif N < 256:
            pick("SEGMENT_HYBRID", "segment_hybrid_small_dense")
        else:
            pick("COMMUNITY_TC", "community_tc_small_dense_wideN")
    elif d >= f32(25.0) and cv >= f32(1.8):
        pick("COMMUNITY_TC", "community_tc_heavy_mixed")
    elif d < f32(9.0) and cv >= f32(1.10) and cv <= f32(1.45) and M >= 250000:
        pick("COMMUNITY_TC", "community_tc_web_locality", True)
    else:
        pick("TC_DIRECT", "tc_direct_default")
    is_tile = st["choice"] in ("TC_DIRECT", "COMMUNITY_TC", "SEGMENT_HYBRID")
    return dict(chosen_path=st["choice"], use_tf32=bool(is_tile and st["tf32"]),
                decision_reason=st["reason"], estimated_risk=st["risk"], feasible_by_path=feas)


REJECT_NAMES = ["CHOSEN", "NOT_FEASIBLE", "LOW_FILL", "LOW_COVERAGE", "HIGH_SKEW", "SMALL_N",
                "INSUFFICIENT_NNZ", "LOW_OCCUPANCY", "LOW_DEGREE_SKEW", "NOT_STRONG_ENOUGH",
                "MARGIN_TOO_SMALL", "NOT_IN_PORTFOLIO", "UNKNOWN"]     # reject_reason_str, ra_common.h:162-179
SCORE_KEYS = ("csr_direct", "csr_adaptive", "staged_reuse", "tc_sparse", "row_split_cuda",
              "tc_reordered", "hybrid_tc_cuda", "cusparse")


def _g(x):
    """iostream formatting of a float (operator<< with the default precision of 6)."""
    return "%g" % float(np.float32(x))


def route_details(avg_nnz, degree_cv, M, N):
    """Diagnostic half of the decision dict on the MAIN portfolio (all proxies zero):
    compute_router_scores (router/router_scores.cpp:27-86, float32 arithmetic in the
    reference's order) and the rejection code / text per path that compute_feasible
    (router/router_dispatch.cpp:107-464) and the legacy stage (:668-966) leave behind:
    the stage always settles on CUSPARSE (its only feasible candidate, suitability >= 0.34),
    which marks CSR_DIRECT "not strong enough"; the seven-rule choice is then marked CHOSEN."""
    d, cv = f32(avg_nnz), f32(degree_cv)
    one, zero = f32(1.0), f32(0.0)
    unit = lambda x: min(one, max(zero, f32(x)))
    n512 = unit(f32(N) / f32(512.0))
    uniformity = unit(one - cv / f32(2.0))
    row_split = unit(f32(0.20) * n512)
    locality = unit(f32(0.15) * uniformity + f32(0.10) * n512)
    scores = dict(
        csr_direct=unit(f32(0.40) * uniformity + f32(0.25) * (one - row_split)
                        + f32(0.20) * (one - locality) + f32(0.15) * (one - zero)),
        csr_adaptive=f32(0.60) * unit(cv / f32(2.0)),
        staged_reuse=zero,
        tc_sparse=f32(0.20) * unit(one - cv / f32(1.8)),
        row_split_cuda=row_split,
        tc_reordered=unit(f32(0.65) * locality + f32(0.15) * uniformity),
        hybrid_tc_cuda=unit(f32(0.10) * locality),
        cusparse=unit(f32(0.40) * unit(d / f32(25.0)) + f32(0.25) * uniformity
                      + f32(0.20) * (one - locality) + f32(0.15) * n512))
    codes, text = {}, {}

    def put(path, code, detail=""):
        codes[path], text[path] = code, detail

    for path in ("CSR_ADAPTIVE", "STAGED_REUSE", "TC_SPARSE"):
        put(path, "NOT_IN_PORTFOLIO", f"{path} not in selected portfolio")
    put("ROW_SPLIT_CUDA", "LOW_DEGREE_SKEW", "row_split_affinity_proxy=0 < 0.65")
    if N < 64 and M < 150000:
        put("TC_REORDERED", "SMALL_N", f"N={_g(N)} < 64")
        put("HYBRID_TC_CUDA", "SMALL_N", f"N={_g(N)} < 64")
    else:
        put("TC_REORDERED", "NOT_STRONG_ENOUGH",
            "TC_REORDERED requires either compact reorder locality or strong scramble-recovery evidence")
        put("HYBRID_TC_CUDA", "NOT_STRONG_ENOUGH", "mixedness_proxy=0 < 0.55")
    for path in ("TC_DIRECT", "COMMUNITY_TC", "LOCALITY_TILED", "SEGMENT_HYBRID"):
        put(path, *(("MARGIN_TOO_SMALL", f"N={_g(N)} < 16") if N < 16 else ("CHOSEN",)))
    put("RODE_ENHANCED", *(("NOT_STRONG_ENOUGH", f"degree_cv={_g(cv)} < 0.8") if cv < f32(0.80) else ("CHOSEN",)))
    put("VECTORIZED_COARSE", *(("NOT_STRONG_ENOUGH", f"avg_nnz={_g(d)} > 12") if d > f32(12.0) else ("CHOSEN",)))
    put("ZERO_OVERHEAD_CSR", "CHOSEN")
    put("CUSPARSE", "CHOSEN")
    put("CSR_DIRECT", "NOT_STRONG_ENOUGH",
        "specialized path has materially stronger regime evidence than explicit DIRECT suitability")
    put(route(avg_nnz, degree_cv, M, N)["chosen_path"], "CHOSEN")
    return dict(scores=scores, rejection_codes=codes, rejection_details=text,
                gate_margin_raw=zero, gate_margin_norm=zero)


def route_label(r):
    """Kernel label as the reference harness prints it: family + _TF32
    (ra_router_parity_test.py:88-103)."""
    return r["chosen_path"] + ("_TF32" if r["use_tf32"] else "")


# ---------------------------------------------------------------------------
# ZERO_OVERHEAD_CSR plan lists
# ---------------------------------------------------------------------------
def zero_overhead_plan(rowptr, M):
    """make_ra_zero_overhead_plan, csr/ra_zero_overhead.cu:331-383."""
    rowptr = np.asarray(rowptr).astype(np.int64)
    deg = np.diff(rowptr[: M + 1])
    rows = np.arange(M, dtype=np.int64)
    tiny = rows[(deg >= 1) & (deg <= 4)]
    short = rows[(deg > 4) & (deg <= 16)]
    med = rows[(deg > 16) & (deg <= 64)]
    long_rows = rows[deg > 64]
    multi = deg > 256
    zero_rows = rows[(deg == 0) | multi]
    chunk_rows, chunk_starts = [], []
    for r in long_rows:
        n = int(deg[r]); s = int(rowptr[r])
        if n <= 256:
            chunk_rows.append(np.array([r | 0x80000000], dtype=np.int64))
            chunk_starts.append(np.array([s], dtype=np.int64))
        else:
            k = (n + 255) // 256
            chunk_rows.append(np.full(k, r, dtype=np.int64))
            chunk_starts.append(s + 256 * np.arange(k, dtype=np.int64))
    cat = lambda xs: (np.concatenate(xs) if xs else np.zeros(0, dtype=np.int64))
    as_i32 = lambda a: a.astype(np.uint32).view(np.int32) if a.size else np.zeros(0, np.int32)
    max_long = int(deg[long_rows].max()) if long_rows.size else 0
    return dict(
        small_row_ids=np.concatenate([tiny, short, med]).astype(np.int32),
        chunk_rows=as_i32(cat(chunk_rows)), chunk_starts=cat(chunk_starts).astype(np.int32),
        zero_row_ids=zero_rows.astype(np.int32),
        num_tiny=int(tiny.size), num_short=int(short.size), num_medium=int(med.size),
        num_long=int(long_rows.size), num_empty=int((deg == 0).sum()),
        max_long_chunks=(max_long + 255) // 256)


# ---------------------------------------------------------------------------
# Tile format (8-row windows, 8x1 vectors, 8-vector blocks)
# ---------------------------------------------------------------------------
def float_to_half_bits(v, nan_to_inf=True):
    """fp32 -> fp16 bits, round to nearest even, overflow to inf, flush below 2^-25.
    nan_to_inf=True: host_float_to_half_bits of TC_DIRECT (tc/ra_tc_direct.cu:45-69), which
    sends every all-ones exponent - NaN included - to the infinity of its sign.
    nan_to_inf=False: float_to_half_bits of COMMUNITY_TC / SEGMENT_HYBRID
    (tc/ra_community_tc.cu:35-38, tc/ra_segment_hybrid.cu:34-37) = __float2half_rn on the
    host, whose NaN is the canonical 0x7FFF. The two agree on every other input."""
    v = np.asarray(v, dtype=np.float32)
    with np.errstate(over="ignore", invalid="ignore"):
        out = v.astype(np.float16).view(np.uint16).copy()
    nan = np.isnan(v)
    if nan.any():
        if nan_to_inf:
            sign = ((v.view(np.uint32) >> 16) & 0x8000).astype(np.uint16)
            out = np.where(nan, sign | np.uint16(0x7C00), out).astype(np.uint16)
        else:
            out = np.where(nan, np.uint16(0x7FFF), out).astype(np.uint16)
    return out


def community_order(rowptr, colind, M):
    """Locality order and window rows of make_ra_community_tc_plan,
    tc/ra_community_tc.cu:336-347: rows sorted by (first stored column, or
    INT_MAX for an empty row; row id); win_rows padded with -1 to 8*W."""
    rowptr = np.asarray(rowptr).astype(np.int64)
    first = np.full(M, np.iinfo(np.int32).max, dtype=np.int64)
    ne = rowptr[1 : M + 1] > rowptr[:M]
    first[ne] = np.asarray(colind)[rowptr[:M][ne]]
    order = np.lexsort((np.arange(M), first))
    W = (M + 7) // 8
    win_rows = np.full(W * 8, -1, dtype=np.int32)
    win_rows[:M] = order
    return win_rows


def tile_plan(rowptr, colind, vals, M, K, N, win_rows=None, nan_to_inf=None):
    """build_ra_tc_direct_plan_impl, tc/ra_tc_direct.cu:627-780 (natural order),
    or the COMMUNITY_TC variant tc/ra_community_tc.cu:355-433 when `win_rows`
    is given. Returns block_offsets [W+1], atox [8*blocks], vals_f16
    [64*blocks] (uint16 bits, fragment order: index(block, vector k, row r) =
    block*64 + (r*4 + k//2)*2 + (k&1), tc/ra_tc_direct.cu:13), or None when the
    plan is inactive (N < 16 or nnz == 0). `nan_to_inf` picks the value conversion (see
    float_to_half_bits); default: TC_DIRECT's for natural order, COMMUNITY_TC's with `win_rows`;
    pass False for SEGMENT_HYBRID."""
    rowptr = np.asarray(rowptr).astype(np.int64)
    colind = np.asarray(colind).astype(np.int64)
    vals = np.asarray(vals, dtype=np.float32)
    if nan_to_inf is None:
        nan_to_inf = win_rows is None
    if M <= 0 or K <= 0 or N < 16 or rowptr[M] <= 0:
        return None
    W = (M + 7) // 8
    deg = np.diff(rowptr[: M + 1])
    row_of = np.repeat(np.arange(M, dtype=np.int64), deg)
    if win_rows is None:
        pos = np.arange(M, dtype=np.int64)           # window position of each row
    else:
        wr = np.asarray(win_rows).astype(np.int64)
        pos = np.empty(M, dtype=np.int64)
        valid = wr >= 0
        pos[wr[valid]] = np.flatnonzero(valid)
    p = pos[row_of]
    w = p >> 3
    slot = p & 7
    order = np.lexsort((slot, colind, w))            # by window, column, row slot
    w, slot, col, val = w[order], slot[order], colind[order], vals[order]
    head = np.ones(col.size, dtype=bool)
    head[1:] = (w[1:] != w[:-1]) | (col[1:] != col[:-1])
    vec_global = np.cumsum(head) - 1                 # distinct (window, col) index
    nvec = np.bincount(w[head], minlength=W)
    blocks = (nvec + 7) // 8
    block_offsets = np.zeros(W + 1, dtype=np.int64)
    np.cumsum(blocks, out=block_offsets[1:])
    vec_base = np.zeros(W + 1, dtype=np.int64)
    np.cumsum(nvec, out=vec_base[1:])
    v_in_w = vec_global - vec_base[w]                # vector slot inside the window
    total_blocks = int(block_offsets[-1])
    atox = np.zeros(total_blocks * 8, dtype=np.int32)
    atox[(block_offsets[w[head]] * 8 + v_in_w[head])] = col[head]
    blk = block_offsets[w] + (v_in_w >> 3)
    k = v_in_w & 7
    out = np.zeros(total_blocks * 64, dtype=np.uint16)
    out[blk * 64 + (slot * 4 + (k >> 1)) * 2 + (k & 1)] = float_to_half_bits(val, nan_to_inf)
    # zero-compressed form of the same values (the zc=true branch, tc/ra_tc_direct.cu:686-735):
    # per block a mask with bit k*8+r per stored (vector k, row r), the index of the block's
    # first stored value (a window's values start at rowptr[8w]), and the stored halves in
    # (window, column, row) order
    val_masks = np.zeros(total_blocks, dtype=np.uint64)
    np.bitwise_or.at(val_masks, blk, np.uint64(1) << (k * 8 + slot).astype(np.uint64))
    first_of_block = np.ones(col.size, dtype=bool)
    first_of_block[1:] = blk[1:] != blk[:-1]
    val_base = np.zeros(total_blocks, dtype=np.int32)
    val_base[blk[first_of_block]] = np.flatnonzero(first_of_block).astype(np.int32)
    return dict(block_offsets=block_offsets.astype(np.int32), atox=atox, vals_f16=out,
                val_masks=val_masks, val_base=val_base, vals_zc=float_to_half_bits(val, True),
                num_windows=W, num_blocks=total_blocks, nnz=int(rowptr[M]))


def segment_split(block_offsets, M):
    """Balance split of make_ra_segment_hybrid_plan, tc/ra_segment_hybrid.cu:470-498:
    windows with <= 64 blocks are one sole segment (window | 0x80000000, scratch -1);
    longer windows are cut into 64-block segments with consecutive scratch slots."""
    bo = np.asarray(block_offsets).astype(np.int64)
    W = bo.size - 1
    seg_window, seg_bbegin, seg_bend, seg_scratch = [], [], [], []
    split_wins, split_off, zero_rows = [], [0], []
    slots = 0
    for w in range(W):
        b0, b1 = int(bo[w]), int(bo[w + 1])
        if b1 - b0 <= 64:
            seg_window.append(w | 0x80000000); seg_bbegin.append(b0); seg_bend.append(b1)
            seg_scratch.append(-1)
        else:
            split_wins.append(w)
            for b in range(b0, b1, 64):
                seg_window.append(w); seg_bbegin.append(b); seg_bend.append(min(b + 64, b1))
                seg_scratch.append(slots); slots += 1
            split_off.append(slots)
            zero_rows.extend(range(w * 8, min(M, (w + 1) * 8)))
    u = lambda a: np.array(a, dtype=np.int64).astype(np.uint32).view(np.int32)
    i = lambda a: np.array(a, dtype=np.int32)
    return dict(seg_window=u(seg_window), seg_bbegin=i(seg_bbegin), seg_bend=i(seg_bend),
                seg_scratch=i(seg_scratch), split_wins=i(split_wins), split_off=i(split_off),
                zero_rows=i(zero_rows), num_split_segs=slots)


# ---------------------------------------------------------------------------
# Numeric semantics
# ---------------------------------------------------------------------------
def round_fp16(x):
    """fp32 -> fp16 round-to-nearest-even -> fp32 (convert_b_to_half_kernel,
    tc/ra_tc_direct.cu:85-104)."""
    with np.errstate(over="ignore"):
        return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)


def round_tf32(x):
    """cvt.rna.tf32.f32 (tc/ra_tc_direct.cu:238-241): keep 10 mantissa bits,
    round to nearest, ties away from zero."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    return ((b + np.uint32(0x1000)) & np.uint32(0xFFFFE000)).view(np.float32)


def spmm_reference(rowptr, colind, vals, B, mode="fp32"):
    """C = A*B accumulated in float64 (error-budget reference).
    mode 'fp32': exact inputs (CSR kernels, csr/csr_direct.cu:201-224);
    mode 'fp16': A and B rounded to fp16 (FP16 tile path, tc/ra_tc_direct.cu:85-95,161-165);
    mode 'tf32': A rounded to fp16, B rounded to tf32 (tc/ra_tc_direct.cu:219-241)."""
    rowptr = np.asarray(rowptr).astype(np.int64)
    colind = np.asarray(colind).astype(np.int64)
    a = np.asarray(vals, dtype=np.float32)
    Bm = np.asarray(B, dtype=np.float32)
    if mode == "fp16":
        a, Bm = round_fp16(a), round_fp16(Bm)
    elif mode == "tf32":
        a, Bm = round_fp16(a), round_tf32(Bm)
    elif mode != "fp32":
        raise ValueError(mode)
    M = rowptr.size - 1
    C = np.zeros((M, Bm.shape[1]), dtype=np.float64)
    a64 = a.astype(np.float64)
    B64 = Bm.astype(np.float64)
    # row-blocked accumulate keeps the temporary (nnz_block x N) small
    step = max(1, 4_000_000 // max(1, Bm.shape[1]))
    for p0 in range(0, colind.size, step):
        p1 = min(colind.size, p0 + step)
        rows = np.searchsorted(rowptr, np.arange(p0, p1), side="right") - 1
        contrib = a64[p0:p1, None] * B64[colind[p0:p1]]
        _segment_add(C, rows, contrib)
    return C


def _segment_add(C, rows, contrib):
    # rows is sorted ascending: reduce runs with add.reduceat
    if rows.size == 0:
        return
    starts = np.flatnonzero(np.r_[True, rows[1:] != rows[:-1]])
    sums = np.add.reduceat(contrib, starts, axis=0)
    C[rows[starts]] += sums


def tile_spmm_from_plan(plan, B, M, mode="fp16", win_rows=None):
    """C computed from the tile arrays themselves (format-level check of
    fs_tile_spmm_kernel, tc/ra_tc_direct.cu:109-179): for each block,
    C[window row r] += vals[block, k, r] * Bq[atox[block*8 + k]]. float64."""
    Bq = round_fp16(B) if mode == "fp16" else round_tf32(B)
    Bq = Bq.astype(np.float64)
    bo = plan["block_offsets"].astype(np.int64)
    W = bo.size - 1
    nb = int(bo[-1])
    vals = plan["vals_f16"].view(np.float16).astype(np.float64).reshape(nb, 8, 4, 2)  # [b][r][k/2][k&1]
    vals = vals.reshape(nb, 8, 8)                                                   # [b][r][k]
    atox = plan["atox"].astype(np.int64).reshape(nb, 8)
    C = np.zeros((M, Bq.shape[1]), dtype=np.float64)
    win_of_block = np.repeat(np.arange(W, dtype=np.int64), np.diff(bo))
    for b in range(nb):
        w = win_of_block[b]
        part = vals[b] @ Bq[atox[b]]                 # [8 rows][N]
        for r in range(8):
            row = w * 8 + r if win_rows is None else int(win_rows[w * 8 + r])
            if 0 <= row < M:
                C[row] += part[r]
    return C


def rel_fro(x, ref):
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref)
    num = np.linalg.norm(np.asarray(x, dtype=np.float64) - ref)
    return float(num / den) if den > 0 else float(num)
