"""Plan formats of the oracle: numpy restatement against the independent C
restatement and against hand-worked cases that follow the reference builders."""
import numpy as np
import pytest

from oracle import ra_oracle as O
from oracle import ref_bindings as R
from conftest import small_csr


def test_zero_overhead_bins_and_chunks():
    # one row at every bin edge (csr/ra_zero_overhead.cu:51-55, 331-358)
    degs = [0, 1, 4, 5, 16, 17, 64, 65, 256, 257, 600, 0, 3]
    M = len(degs)
    rowptr = np.zeros(M + 1, dtype=np.int32)
    rowptr[1:] = np.cumsum(degs)
    p = O.zero_overhead_plan(rowptr, M)
    assert p["small_row_ids"].tolist() == [1, 2, 12, 3, 4, 5, 6]
    assert p["zero_row_ids"].tolist() == [0, 9, 10, 11]
    sole = lambda r: int(np.array([r | 0x80000000], dtype=np.uint32).view(np.int32)[0])
    assert p["chunk_rows"].tolist() == [sole(7), sole(8), 9, 9, 10, 10, 10]
    s9, s10 = int(rowptr[9]), int(rowptr[10])
    assert p["chunk_starts"].tolist() == [int(rowptr[7]), int(rowptr[8]), s9, s9 + 256, s10, s10 + 256, s10 + 512]
    assert (p["num_tiny"], p["num_short"], p["num_medium"], p["num_long"], p["num_empty"]) == (3, 2, 2, 4, 2)
    assert p["max_long_chunks"] == 3


def test_tile_plan_hand_case():
    # 3 rows, one window: columns {5,9} / {9} / {2,5}; distinct sorted cols 2,5,9
    rowptr = np.array([0, 2, 3, 5], dtype=np.int32)
    colind = np.array([5, 9, 9, 2, 5], dtype=np.int32)
    vals = np.array([1.0, 2.0, 3.0, 4.0, 5.0], dtype=np.float32)
    p = O.tile_plan(rowptr, colind, vals, 3, 16, 16)
    assert p["block_offsets"].tolist() == [0, 1]
    assert p["atox"].tolist() == [2, 5, 9, 0, 0, 0, 0, 0]
    v = p["vals_f16"].view(np.float16).astype(np.float32)
    idx = lambda k, r: (r * 4 + k // 2) * 2 + (k & 1)       # tc/ra_tc_direct.cu:13
    want = np.zeros(64, dtype=np.float32)
    want[idx(1, 0)] = 1.0; want[idx(2, 0)] = 2.0; want[idx(2, 1)] = 3.0
    want[idx(0, 2)] = 4.0; want[idx(1, 2)] = 5.0
    assert v.tolist() == want.tolist()


def test_tile_plan_inactive():
    rowptr = np.array([0, 1], dtype=np.int32)
    assert O.tile_plan(rowptr, [0], [1.0], 1, 4, 8) is None              # N < 16
    assert O.tile_plan(np.zeros(5, np.int32), [], [], 4, 4, 64) is None  # nnz == 0


@pytest.mark.parametrize("M,K,seed,unsorted", [(1, 8, 0, False), (7, 40, 1, False), (8, 40, 2, True),
                                                (9, 100, 3, False), (16, 30, 4, True), (333, 500, 5, False),
                                                (1000, 64, 6, True)])
def test_tile_plan_numpy_vs_c(M, K, seed, unsorted):
    rng = np.random.default_rng(seed)
    degs = rng.integers(0, min(K, 40) + 1, size=M)
    if M > 20:
        degs[rng.integers(0, M)] = K                    # one dense row -> long window
        degs[3:6] = 0
    rowptr, colind, vals = small_csr(M, K, degs, seed, sort=not unsorted)
    if rowptr[-1] == 0:
        return
    for wr in (None, O.community_order(rowptr, colind, M)):
        a = O.tile_plan(rowptr, colind, vals, M, K, 64, win_rows=wr)
        b = R.c_tile_plan(rowptr, colind, vals, M, win_rows=wr)
        assert a["block_offsets"].tolist() == b["block_offsets"].tolist()
        assert a["atox"].tolist() == b["atox"].tolist()
        assert a["vals_f16"].tolist() == b["vals_f16"].tolist()
        # format-level product equals the CSR product on fp16-rounded inputs
        B = rng.standard_normal((K, 16)).astype(np.float32)
        got = O.tile_spmm_from_plan(a, B, M, "fp16", win_rows=wr)
        ref = O.spmm_reference(rowptr, colind, vals, B, "fp16")
        assert O.rel_fro(got, ref) < 1e-12


def test_community_order():
    # first stored column decides, ties by row id, empty rows last
    rowptr = np.array([0, 2, 2, 3, 5, 6], dtype=np.int32)
    colind = np.array([7, 1, 3, 3, 9, 0], dtype=np.int32)      # row 0 stores 7 first (unsorted row)
    wr = O.community_order(rowptr, colind, 5)
    assert wr.tolist() == [4, 2, 3, 0, 1, -1, -1, -1]


def test_segment_split_edges():
    # windows with 0, 64, 65 and 130 blocks (tc/ra_segment_hybrid.cu:31,470-498)
    bo = np.array([0, 0, 64, 129, 259], dtype=np.int32)
    s = O.segment_split(bo, M=30)
    u = lambda w: int(np.array([w | 0x80000000], dtype=np.uint32).view(np.int32)[0])
    assert s["seg_window"].tolist() == [u(0), u(1), 2, 2, 3, 3, 3]
    assert s["seg_bbegin"].tolist() == [0, 0, 64, 128, 129, 193, 257]
    assert s["seg_bend"].tolist() == [0, 64, 128, 129, 193, 257, 259]
    assert s["seg_scratch"].tolist() == [-1, -1, 0, 1, 2, 3, 4]
    assert s["split_wins"].tolist() == [2, 3]
    assert s["split_off"].tolist() == [0, 2, 5]
    assert s["zero_rows"].tolist() == list(range(16, 24)) + list(range(24, 30))


def test_half_and_tf32_rounding():
    x = np.array([0.1, 65504.0, 65520.0, 1e-8, 2.0 ** -25, 2.0 ** -25 * 1.0001, -3.3], dtype=np.float32)
    got = np.zeros(x.size, dtype=np.uint16)
    R.oracle_c().oc_f32_to_f16_bits(x.ctypes.data, got.ctypes.data, x.size)
    assert got.tolist() == O.float_to_half_bits(x).tolist()
    # special values: the bit-twiddling routine of TC_DIRECT sends NaN to the infinity of its sign,
    # the __float2half_rn of the other two families keeps the canonical NaN
    neg_nan = np.array([0xFFC00001], dtype=np.uint32).view(np.float32)[0]
    y = np.array([np.nan, neg_nan, np.inf, -np.inf, 7e4, -7e4, 1e-6, 6e-8, 2.0 ** -24, 0.0, -0.0], dtype=np.float32)
    got = np.zeros(y.size, dtype=np.uint16)
    R.oracle_c().oc_f32_to_f16_bits(y.ctypes.data, got.ctypes.data, y.size)
    assert got.tolist() == O.float_to_half_bits(y, nan_to_inf=True).tolist()
    assert got[:6].tolist() == [0x7C00, 0xFC00, 0x7C00, 0xFC00, 0x7C00, 0xFC00]
    other = O.float_to_half_bits(y, nan_to_inf=False)
    assert other[:2].tolist() == [0x7FFF, 0x7FFF] and other[2:].tolist() == got[2:].tolist()
    t = O.round_tf32(np.array([1.0 + 2.0 ** -11, 1.0 + 2.0 ** -11 + 2.0 ** -20, -(1.0 + 2.0 ** -11)], dtype=np.float32))
    assert t.tolist() == [1.0 + 2.0 ** -10, 1.0 + 2.0 ** -10, -(1.0 + 2.0 ** -10)]   # ties away from zero


def test_spmm_reference_numpy_vs_c():
    rowptr, colind, vals = small_csr(200, 300, np.random.default_rng(1).integers(0, 30, 200), 1)
    B = np.random.default_rng(2).standard_normal((300, 24)).astype(np.float32)
    for mode, m in (("fp32", 0), ("fp16", 1), ("tf32", 2)):
        a = O.spmm_reference(rowptr, colind, vals, B, mode)
        b = R.c_spmm_f64(rowptr, colind, vals, B, m)
        assert O.rel_fro(a, b) < 1e-14


def _expand_zc(p):
    """Padded fragment-order values rebuilt from the zero-compressed arrays: value of
    (vector k, row r) = vals_zc[base + popcount(mask bits below k*8+r)] when bit k*8+r is set."""
    out = np.zeros(p["num_blocks"] * 64, dtype=np.uint16)
    for b in range(p["num_blocks"]):
        m, off = int(p["val_masks"][b]), int(p["val_base"][b])
        for bit in range(64):
            if (m >> bit) & 1:
                k, r = bit >> 3, bit & 7
                out[b * 64 + (r * 4 + k // 2) * 2 + (k & 1)] = p["vals_zc"][off]
                off += 1
    return out


def test_zero_compressed_hand_case():
    # same window as test_tile_plan_hand_case: vectors (cols) 2,5,9; entries in (col,row) order:
    # (2,r2)=4, (5,r0)=1, (5,r2)=5, (9,r0)=2, (9,r1)=3
    rowptr = np.array([0, 2, 3, 5], dtype=np.int32)
    colind = np.array([5, 9, 9, 2, 5], dtype=np.int32)
    vals = np.array([1.0, 2.0, 3.0, 4.0, 5.0], dtype=np.float32)
    p = O.tile_plan(rowptr, colind, vals, 3, 16, 16)
    assert p["vals_zc"].view(np.float16).astype(np.float32).tolist() == [4.0, 1.0, 5.0, 2.0, 3.0]
    assert p["val_base"].tolist() == [0]
    want_mask = (1 << (0 * 8 + 2)) | (1 << (1 * 8 + 0)) | (1 << (1 * 8 + 2)) | (1 << (2 * 8 + 0)) | (1 << (2 * 8 + 1))
    assert [int(x) for x in p["val_masks"]] == [want_mask]


@pytest.mark.parametrize("M,K,seed", [(7, 40, 1), (9, 100, 3), (333, 500, 5), (1000, 64, 6)])
def test_zero_compressed_expands_to_padded(M, K, seed):
    rng = np.random.default_rng(seed)
    degs = rng.integers(0, min(K, 40) + 1, size=M)
    if M > 20:
        degs[rng.integers(0, M)] = K
        degs[3:6] = 0
    rowptr, colind, vals = small_csr(M, K, degs, seed)
    p = O.tile_plan(rowptr, colind, vals, M, K, 64)
    assert p["vals_zc"].size == int(rowptr[-1])
    assert np.array_equal(_expand_zc(p), p["vals_f16"])
    # a window's stored values start at rowptr[8w] (tc/ra_tc_direct.cu:727-733)
    bo = p["block_offsets"]
    for w in range(p["num_windows"]):
        if bo[w + 1] > bo[w]:
            assert p["val_base"][bo[w]] == rowptr[8 * w]
