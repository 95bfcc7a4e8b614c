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


# ---- structural analysis: the 34 features of the research portfolio --------------------
_F = np.float32


def _clamp01(x):
    return _F(max(_F(0), min(_F(1), _F(x))))


def _sdiv(num, den):
    num, den = _F(num), _F(den)
    return _F(num / den) if abs(den) > _F(1e-6) else _F(0)


def _popcount(x: int) -> int:
    return bin(int(x)).count("1")


def _jaccard(a: int, b: int):
    uni = _popcount(a | b)
    return _F(0) if uni == 0 else _F(_F(_popcount(a & b)) / _F(uni))


def _mean_f(values):
    """float(sum in double, in order, / count): safe_mean, router/router_features.cpp:62-72."""
    if len(values) == 0:
        return _F(0)
    s = 0.0
    for v in values:
        s += float(v)
    return _F(s / float(len(values)))


def analyze_matrix(rowptr, colind, M, K, N):
    """compute_router_features (router/router_features.cpp:113-432) restated with the same
    arithmetic types and the same order of the floating-point additions. Python loops over rows,
    tiles and windows: for small matrices. Returns {field name: np.float32 | int}."""
    rowptr = np.asarray(rowptr, dtype=np.int64)
    colind = np.asarray(colind, dtype=np.int64)
    keys_f = ("avg_nnz_per_row", "std_nnz_per_row", "degree_cv", "max_to_mean_ratio", "frac_dense_rows", "skew_ratio",
              "long_row_fraction", "long_row_nnz_fraction", "top_1_row_nnz_fraction", "top_5_row_nnz_fraction",
              "tile_fill_mean", "tile_fill_median", "tile_fill_p90", "tile_fill_max", "tile_fill_variance",
              "tile_occupancy", "actual_nnz_coverage", "avg_nnz_per_tile", "row_window_colspan_compactness",
              "local_row_similarity_proxy", "reordered_locality_proxy", "locality_gain_proxy",
              "locality_selectivity_proxy", "road_likeness_proxy", "row_split_affinity_proxy", "mixedness_proxy",
              "tc_candidate_ratio", "tc_synergy_proxy", "estimated_tc_partition_ratio", "estimated_cuda_partition_ratio",
              "irregular_window_fraction", "tc_granularity_proxy", "redundancy_risk_proxy")
    f = {k: _F(0) for k in keys_f}
    f.update(tc_candidate_tiles=0, output_dim_N=0, matrix_M=0, matrix_K=0, total_nnz=0)
    if M <= 0 or K <= 0:
        return f
    nnz = int(rowptr[M])
    f.update(matrix_M=int(M), matrix_K=int(K), output_dim_N=int(N), total_nnz=nnz)
    if nnz <= 0:
        return f

    lens = np.diff(rowptr[:M + 1]).astype(np.int64)
    first = np.zeros(M, dtype=np.int64); last = np.zeros(M, dtype=np.int64)
    sig = [0] * M
    centroid = np.zeros(M, dtype=np.float32)
    for r in range(M):
        b, e = int(rowptr[r]), int(rowptr[r + 1])
        if e > b:
            cols = colind[b:e]
            first[r], last[r] = cols[0], cols[-1]
            s = 0
            for bucket in np.minimum(63, (cols * 64) // max(1, K)):
                s |= 1 << int(bucket)
            sig[r] = s
            centroid[r] = _F(float(int(cols.sum())) / float(e - b))

    # degree statistics
    sum_lens = 0.0
    for L in lens:
        sum_lens += float(L)
    avg = sum_lens / float(M)
    var = 0.0
    dense_rows = long_rows = long_row_nnz = 0
    thr = max(32.0, 2.0 * avg)
    for L in lens:
        d = float(L) - avg
        var += d * d
        if float(L) > 2.0 * avg:
            dense_rows += 1
        if float(L) >= thr:
            long_rows += 1; long_row_nnz += int(L)
    std = float(np.sqrt(np.float64(var / float(max(1, M)))))
    top = np.sort(lens)[::-1]
    max_len = int(top[0])
    f["avg_nnz_per_row"] = _F(avg)
    f["std_nnz_per_row"] = _F(std)
    f["degree_cv"] = _F(std / avg) if avg > 1e-6 else _F(0)
    f["max_to_mean_ratio"] = _F(float(max_len) / avg) if avg > 1e-6 else _F(0)
    f["frac_dense_rows"] = _F(_F(dense_rows) / _F(max(1, M)))
    f["skew_ratio"] = f["max_to_mean_ratio"]
    f["long_row_fraction"] = _F(_F(long_rows) / _F(max(1, M)))
    f["long_row_nnz_fraction"] = _F(_F(long_row_nnz) / _F(max(1, nnz)))
    f["top_1_row_nnz_fraction"] = _F(_F(int(top[0])) / _F(max(1, nnz)))
    f["top_5_row_nnz_fraction"] = _F(_F(int(top[:5].sum())) / _F(max(1, nnz)))

    # 16x16 tiles
    tile_rows, tile_cols = (M + 15) // 16, (K + 15) // 16
    rows_of = np.repeat(np.arange(M, dtype=np.int64), lens)
    tkeys = (rows_of // 16) * tile_cols + colind[:nnz] // 16
    _, counts = np.unique(tkeys, return_counts=True)
    fills = np.sort((counts.astype(np.float32) / _F(256)).astype(np.float32))
    nt = fills.size
    fill_mean = _mean_f(fills)
    fv = 0.0
    for x in fills:
        d = float(x) - float(fill_mean)
        fv += d * d
    fv = fv / float(nt) if nt else 0.0
    cand = fills >= _F(0.25)
    f["tile_fill_mean"] = fill_mean
    f["tile_fill_median"] = fills[nt // 2] if nt else _F(0)
    f["tile_fill_p90"] = fills[min(nt - 1, (nt * 9) // 10)] if nt else _F(0)
    f["tile_fill_max"] = fills[-1] if nt else _F(0)
    f["tile_fill_variance"] = _F(fv)
    f["tile_occupancy"] = _F(_F(nt) / _F(max(1, tile_rows * tile_cols)))
    f["actual_nnz_coverage"] = _F(_F(int(counts[counts >= 64].sum())) / _F(max(1, nnz)))
    f["avg_nnz_per_tile"] = _F(_F(nnz) / _F(nt)) if nt else _F(0)
    f["tc_candidate_tiles"] = int(cand.sum())
    f["tc_candidate_ratio"] = _F(_F(f["tc_candidate_tiles"]) / _F(nt)) if nt else _F(0)

    # similarity of neighbouring rows, stored order and proxy order
    f["local_row_similarity_proxy"] = _mean_f([_jaccard(sig[r - 1], sig[r]) for r in range(1, M)
                                                if lens[r - 1] > 0 and lens[r] > 0])
    bucket = np.array([int(_F(_F(centroid[r] * _F(16)) / _F(K))) for r in range(M)], dtype=np.int64)
    span = np.where(lens > 0, last - first + 1, K)
    order = sorted(range(M), key=lambda r: (bucket[r], span[r], -lens[r]))        # sorted() is stable
    f["reordered_locality_proxy"] = _mean_f([_jaccard(sig[a], sig[b]) for a, b in zip(order[:-1], order[1:])
                                              if lens[a] > 0 and lens[b] > 0])

    # 16-row windows
    comp_l, sim_l, irr_l = [], [], []
    tc_nnz = cuda_nnz = irregular = 0
    for base in range(0, M, 16):
        end = min(M, base + 16)
        wn = int(lens[base:end].sum()); max_row = int(lens[base:end].max())
        mn, mx = K, -1
        sim_sum, sim_cnt = _F(0), 0
        for r in range(base, end):
            if lens[r] > 0:
                mn, mx = min(mn, int(first[r])), max(mx, int(last[r]))
            if r > base and lens[r - 1] > 0 and lens[r] > 0:
                sim_sum = _F(sim_sum + _jaccard(sig[r - 1], sig[r])); sim_cnt += 1
        avg_row = _F(_F(wn) / _F(max(1, end - base)))
        wthr = max(_F(32), _F(_F(2.5) * avg_row))
        long_nnz = int(sum(int(lens[r]) for r in range(base, end) if _F(int(lens[r])) >= wthr))
        sp = (mx - mn + 1) if mx >= mn else K
        compact = _F(_F(wn) / _F(max(1, (end - base) * max(1, sp))))
        sim = _F(sim_sum / _F(sim_cnt)) if sim_cnt > 0 else _F(0)
        aligned = max(16, ((sp + 15) // 16) * 16)
        dens = _F(_F(wn) / _F(max(16, (end - base) * aligned)))
        cn = _clamp01(_F(compact * _F(6)))
        dn = _clamp01(_F(dens * _F(10)))
        un = _clamp01(_F(_F(1) - _sdiv(_F(max_row), _F(_F(_F(4) * avg_row) + _F(1)))))
        lm = _sdiv(_F(long_nnz), _F(max(1, wn)))
        comp_l.append(compact); sim_l.append(sim)
        tc_score = _F(_F(_F(_F(_F(0.35) * cn) + _F(_F(0.30) * sim)) + _F(_F(0.20) * dn)) + _F(_F(0.15) * un))
        irr = _F(_F(_F(_F(_F(0.40) * lm) +
                       _F(_F(0.25) * _clamp01(_F(_sdiv(_F(max_row), _F(avg_row + _F(1))) / _F(6))))) +
                    _F(_F(0.20) * _F(_F(1) - cn))) + _F(_F(0.15) * _F(_F(1) - sim)))
        irr_l.append(irr)
        if avg_row >= _F(8) and tc_score >= _F(0.55) and irr < _F(0.45):
            tc_nnz += wn
        if irr >= _F(0.50) or lm >= _F(0.20):
            cuda_nnz += wn; irregular += 1

    g = f
    g["row_window_colspan_compactness"] = _mean_f(comp_l)
    wsim, wirr = _mean_f(sim_l), _mean_f(irr_l)
    g["tc_synergy_proxy"] = _F(_F(_F(_F(_F(0.35) * _clamp01(_F(g["tile_fill_mean"] / _F(0.20)))) +
                                      _F(_F(0.25) * g["tc_candidate_ratio"])) +
                                   _F(_F(0.20) * g["reordered_locality_proxy"])) +
                               _F(_F(0.20) * g["row_window_colspan_compactness"]))
    g["locality_gain_proxy"] = _clamp01(_F(g["reordered_locality_proxy"] - g["local_row_similarity_proxy"]))
    ordered = _clamp01(_F(g["local_row_similarity_proxy"] * _clamp01(_F(g["row_window_colspan_compactness"] * _F(2)))))
    g["locality_selectivity_proxy"] = _clamp01(_F(g["locality_gain_proxy"] * _F(_F(1) - ordered)))
    g["road_likeness_proxy"] = _clamp01(_F(_F(_F(g["local_row_similarity_proxy"] *
                                                  _clamp01(_F(_F(1) - _F(g["degree_cv"] / _F(0.35))))) *
                                               _clamp01(_F(_F(1) - _F(g["avg_nnz_per_row"] / _F(24))))) *
                                            _clamp01(_F(g["row_window_colspan_compactness"] / _F(0.25)))))
    skew = _F(_F(_F(_F(_F(0.45) * _clamp01(_F(_F(g["skew_ratio"] - _F(2.0)) / _F(6.0)))) +
                    _F(_F(0.30) * g["long_row_nnz_fraction"])) +
                 _F(_F(0.15) * _clamp01(_F(g["top_1_row_nnz_fraction"] / _F(0.0020))))) +
              _F(_F(0.10) * _clamp01(_F(g["top_5_row_nnz_fraction"] / _F(0.0100)))))
    n_scale = _clamp01(_F(_F(_F(N) - _F(128)) / _F(384)))
    dense_reg = _F(_clamp01(_F(g["avg_nnz_per_row"] / _F(192))) * _F(_F(0.35) + _F(_F(0.65) * n_scale)))
    g["row_split_affinity_proxy"] = _clamp01(max(skew, dense_reg))
    g["estimated_tc_partition_ratio"] = _clamp01(_F(_F(tc_nnz) / _F(max(1, nnz))))
    g["estimated_cuda_partition_ratio"] = _clamp01(_F(_F(cuda_nnz) / _F(max(1, nnz))))
    g["irregular_window_fraction"] = _F(_F(irregular) / _F(max(1, (M + 15) // 16)))
    tcr, cur = g["estimated_tc_partition_ratio"], g["estimated_cuda_partition_ratio"]
    balance = _sdiv(_F(_F(2) * min(tcr, cur)), _F(_F(tcr + cur) + _F(1e-6)))
    g["mixedness_proxy"] = _clamp01(_F(balance * _clamp01(_F(_F(tcr + cur) / _F(0.60)))))
    g["tc_granularity_proxy"] = _F(_F(_F(0.55) * _clamp01(_F(g["avg_nnz_per_row"] / _F(64)))) +
                                   _F(_F(0.45) * _clamp01(_F(_F(_F(1) - g["long_row_fraction"]) +
                                                              _F(_F(0.5) * g["locality_selectivity_proxy"])))))
    g["redundancy_risk_proxy"] = _clamp01(_F(_F(_F(_F(_F(0.45) * g["long_row_nnz_fraction"]) +
                                                   _F(_F(0.30) * _F(_F(1) - g["row_window_colspan_compactness"]))) +
                                                _F(_F(0.15) * _F(_F(1) - wsim))) + _F(_F(0.10) * wirr)))
    return f
