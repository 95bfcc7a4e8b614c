"""Tile paths (TC_DIRECT, COMMUNITY_TC, SEGMENT_HYBRID; FP16 and TF32).
Plan arrays: bit-exact with the oracle and with the reference's own builders.
Outputs: within 5e-3 relative Frobenius error of the float64 oracle evaluated on
the same rounded operands, and of the reference's own kernels."""
import numpy as np
import pytest
import torch

from oracle import ra_oracle as O
from oracle import ref_bindings as R
from ra_spmm_b200 import generators as G
from ra_spmm_b200 import ra_spmm
from conftest import small_csr
from gpu_util import to_dev, RefTilePlan, rel_fro, ref_kernels

pytestmark = pytest.mark.gpu
TOL_TILE = 5e-3
KINDS = {"tc": (0, ra_spmm.make_tc_direct_plan), "ct": (1, ra_spmm.make_community_tc_plan),
         "sh": (2, ra_spmm.make_segment_hybrid_plan)}


def _run(kind, plan, B, tf32, ci=None, va=None):
    if kind == "tc":
        return ra_spmm.run_tc_direct_plan_tf32(plan, B) if tf32 else ra_spmm.run_tc_direct_plan(plan, B)
    if kind == "ct":
        return ra_spmm.run_community_tc_plan_tf32(plan, B) if tf32 else ra_spmm.run_community_tc_plan(plan, B)
    return (ra_spmm.run_segment_hybrid_plan_tf32(plan, ci, va, B) if tf32
            else ra_spmm.run_segment_hybrid_plan(plan, ci, va, B))


def _oracle_arrays(kind, rowptr, colind, vals, M, K, N):
    wr = O.community_order(rowptr, colind, M) if kind == "ct" else None
    p = O.tile_plan(rowptr, colind, vals, M, K, N, win_rows=wr)
    out = dict(block_offsets=p["block_offsets"], atox=p["atox"], vals_f16=p["vals_f16"])
    if kind == "ct":
        out["win_rows"] = wr
    if kind == "sh":
        s = O.segment_split(p["block_offsets"], M)
        s.pop("num_split_segs")
        out.update(s)
    return out


def _check_arrays(kind, plan, rowptr, colind, vals, M, K, N):
    got = {k: v.numpy() for k, v in plan.arrays().items()}
    want = _oracle_arrays(kind, rowptr, colind, vals, M, K, N)
    assert set(got) == set(want)
    for k in want:
        g = got[k].view(np.uint16) if k == "vals_f16" else got[k]
        assert np.array_equal(g, want[k]), f"{kind}: {k} differs from the oracle"
    ref = None
    if ref_kernels() is not None:
        ref = RefTilePlan(KINDS[kind][0], rowptr, colind, vals, M, K, N)
        ra = ref.arrays()
        assert set(ra) == set(got)
        for k in ra:
            g = got[k].view(np.uint16) if k == "vals_f16" else got[k]
            assert np.array_equal(g, ra[k]), f"{kind}: {k} differs from the reference builder"
    return ref


def _check_outputs(kind, plan, ref, rowptr, colind, vals, K, N, dev, seed):
    B = G.dense(K, N, seed)
    Bd = B.to(dev)
    ci, va = to_dev(colind, dev), to_dev(vals, dev)
    for tf32 in (False, True):
        C = _run(kind, plan, Bd, tf32, ci, va)
        want = R.c_spmm_f64(rowptr, colind, vals, B.numpy(), 2 if tf32 else 1)
        err = rel_fro(C, want)
        assert err < TOL_TILE, f"{kind} tf32={tf32} N={N}: {err}"
        assert err < 1e-5, f"{kind} tf32={tf32} N={N}: fp32 accumulation drifted ({err})"
        if ref is not None:
            assert rel_fro(C, ref.run(Bd, tf32)) < TOL_TILE
        assert torch.equal(C, _run(kind, plan, Bd, tf32, ci, va))       # deterministic
    # fp16 B handed over directly == fp32 B rounded by the library. At widths that are not a
    # multiple of 16 the two take different kernels (an fp16 B with unaligned rows is read
    # directly, one 8-deep MMA per block; the library's own padded copy runs on the staged
    # kernel, one 16-deep MMA per block pair), so only the rounding of the sums may differ.
    C16 = _run(kind, plan, Bd.half(), False, ci, va)
    C32 = _run(kind, plan, Bd, False, ci, va)
    if N % 16 == 0:
        assert torch.equal(C16, C32)
    else:
        assert rel_fro(C16, C32.cpu().numpy()) < 1e-6


def _mixed_matrix(M, K, seed, hub=True, unsorted=False):
    rng = np.random.default_rng(seed)
    degs = rng.integers(0, 30, size=M)
    degs[::7] = 0
    if hub and M >= 64:
        degs[40] = min(K, 900)        # window 5 gets > 64 blocks -> split segments
        degs[41] = min(K, 700)
        degs[M - 1] = min(K, 600)
    return small_csr(M, K, degs, seed, sort=not unsorted)


@pytest.mark.parametrize("kind", ["tc", "ct", "sh"])
@pytest.mark.parametrize("N", [16, 32, 64, 128, 256, 512, 47, 100])
def test_plan_and_outputs(cuda, kind, N):
    M, K = 333, 1200
    rowptr, colind, vals = _mixed_matrix(M, K, seed=N)
    rp, ci, va = torch.from_numpy(rowptr), torch.from_numpy(colind), torch.from_numpy(vals)
    plan = KINDS[kind][1](rp, ci, va, M, K, N)
    assert plan.active and plan.valid
    ref = _check_arrays(kind, plan, rowptr, colind, vals, M, K, N)
    _check_outputs(kind, plan, ref, rowptr, colind, vals, K, N, cuda, seed=N)


@pytest.mark.parametrize("kind", ["tc", "ct", "sh"])
@pytest.mark.parametrize("M", [1, 7, 8, 9, 16, 65])
def test_small_shapes(cuda, kind, M):
    rng = np.random.default_rng(M)
    degs = rng.integers(0, 12, size=M); degs[0] = max(degs[0], 1)
    rowptr, colind, vals = small_csr(M, 90, degs, seed=M)
    plan = KINDS[kind][1](to_dev(rowptr, cuda), to_dev(colind, cuda), to_dev(vals, cuda), M, 90, 64)  # device CSR
    ref = _check_arrays(kind, plan, rowptr, colind, vals, M, 90, 64)
    _check_outputs(kind, plan, ref, rowptr, colind, vals, 90, 64, cuda, seed=M)


@pytest.mark.parametrize("kind", ["tc", "ct", "sh"])
def test_unsorted_rows(cuda, kind):
    """Columns inside a row may come in any order (the builders sort per window);
    COMMUNITY_TC keys on the first *stored* column (tc/ra_community_tc.cu:339)."""
    rowptr, colind, vals = _mixed_matrix(200, 500, seed=11, unsorted=True)
    plan = KINDS[kind][1](torch.from_numpy(rowptr), torch.from_numpy(colind), torch.from_numpy(vals), 200, 500, 64)
    ref = _check_arrays(kind, plan, rowptr, colind, vals, 200, 500, 64)
    _check_outputs(kind, plan, ref, rowptr, colind, vals, 500, 64, cuda, seed=11)


@pytest.mark.parametrize("kind", ["tc", "ct", "sh"])
def test_segment_edges_64_65_blocks(cuda, kind):
    """Windows with exactly 64 and 65 blocks (512 / 513 distinct columns)."""
    K = 2000
    degs = np.zeros(24, dtype=np.int64)
    degs[0] = 512; degs[8] = 513; degs[16] = 3
    rowptr, colind, vals = small_csr(24, K, degs, seed=5)
    plan = KINDS[kind][1](torch.from_numpy(rowptr), torch.from_numpy(colind), torch.from_numpy(vals), 24, K, 128)
    ref = _check_arrays(kind, plan, rowptr, colind, vals, 24, K, 128)
    if kind == "sh":
        assert plan.num_split_windows == 1 and plan.num_segments == 4
    _check_outputs(kind, plan, ref, rowptr, colind, vals, K, 128, cuda, seed=5)


def test_inactive_plans_raise(cuda):
    rowptr, colind, vals = small_csr(16, 30, [2] * 16, seed=0)
    t = lambda a: torch.from_numpy(a)
    p = ra_spmm.make_tc_direct_plan(t(rowptr), t(colind), t(vals), 16, 30, 8)       # N < 16
    assert p.valid and not p.active and p.num_tc_tiles == 0 and p.arrays() == {}
    with pytest.raises(RuntimeError, match="inactive"):
        ra_spmm.run_tc_direct_plan(p, torch.randn(30, 8, device=cuda))
    p = ra_spmm.make_community_tc_plan(torch.zeros(17, dtype=torch.int32), torch.zeros(0, dtype=torch.int32),
                                       torch.zeros(0), 16, 30, 64)                      # nnz == 0
    assert not p.active


def test_c1_routes_to_tc_direct_and_matches(cuda):
    """Configuration 1 takes the TC_DIRECT FP16 route under the reference's rules."""
    a = G.erdos_renyi_fixed_degree()
    rp, ci, va = a.torch()
    d = ra_spmm.make_router_plan(rp, ci, va, a.M, a.K, 64)
    assert (d["chosen_path"], d["use_tf32"], d["decision_reason"]) == ("TC_DIRECT", False, "tc_direct_uniform")
    B = G.dense(a.K, 64, 0).to(cuda)
    C = ra_spmm.run_router_plan(d, rp.to(cuda), ci.to(cuda), va.to(cuda), B)
    want = R.c_spmm_f64(a.rowptr, a.colind, a.vals, B.cpu().numpy(), 1)
    assert rel_fro(C, want) < 1e-5
    assert rel_fro(C, R.c_spmm_f64(a.rowptr, a.colind, a.vals, B.cpu().numpy(), 0)) < TOL_TILE


@pytest.mark.parametrize("cfg,kind", [("C3", "ct"), ("C3", "tc"), ("C4", "sh"), ("C5", "tc")])
def test_reduced_configs(cuda, cfg, kind):
    """Configurations 3-5 at reduced size through the kernels BASELINE names."""
    scale = {"C3": 0.03, "C4": 2.0 ** -7, "C5": 0.01}[cfg]
    a, N, bdt = G.make_config(cfg, scale)
    rp, ci, va = a.torch()
    plan = KINDS[kind][1](rp, ci, va, a.M, a.K, N)
    ref = _check_arrays(kind, plan, a.rowptr, a.colind, a.vals, a.M, a.K, N)
    B = G.dense(a.K, N, G.CONFIG_SEEDS[cfg], bdt)
    Bd = B.to(cuda)
    tf32 = cfg == "C4"
    C = _run(kind, plan, Bd if not tf32 else Bd.float(), tf32, ci.to(cuda), va.to(cuda))
    want = R.c_spmm_f64(a.rowptr, a.colind, a.vals, B.float().numpy(), 2 if tf32 else 1)
    assert rel_fro(C, want) < 1e-5
    if ref is not None:
        assert rel_fro(C, ref.run(Bd.float(), tf32)) < TOL_TILE


@pytest.mark.parametrize("kind", ["tc", "ct", "sh"])
def test_bulk_copy_ring_variant(cuda, kind, monkeypatch):
    """RA_TILE_TMA=1 selects the cp.async.bulk + mbarrier ring (off by default because
    it measured slower); it must give the same results as the default ring."""
    M, K, N = 333, 1200, 128
    rowptr, colind, vals = _mixed_matrix(M, K, seed=77)
    plan = KINDS[kind][1](torch.from_numpy(rowptr), torch.from_numpy(colind), torch.from_numpy(vals), M, K, N)
    B = G.dense(K, N, 77).to(cuda)
    ci, va = to_dev(colind, cuda), to_dev(vals, cuda)
    for tf32 in (False, True):
        monkeypatch.delenv("RA_TILE_TMA", raising=False)
        want = _run(kind, plan, B, tf32, ci, va)
        monkeypatch.setenv("RA_TILE_TMA", "1")
        got = _run(kind, plan, B, tf32, ci, va)
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        assert plan.device_status() == 0
    monkeypatch.delenv("RA_TILE_TMA", raising=False)


@pytest.mark.parametrize("kind", ["tc", "ct", "sh"])
@pytest.mark.parametrize("N", [16, 64, 128, 256, 512])
def test_tcgen05_variant(cuda, kind, N, monkeypatch):
    """RA_TILE_TC5=1 runs the FP16 path on tcgen05 tensor cores with TMEM accumulators;
    same plan, same numeric contract (float64 oracle on fp16-rounded operands)."""
    M, K = 333, 1200
    rowptr, colind, vals = _mixed_matrix(M, K, seed=N + 5)
    plan = KINDS[kind][1](torch.from_numpy(rowptr), torch.from_numpy(colind), torch.from_numpy(vals), M, K, N)
    B = G.dense(K, N, N + 5)
    Bd = B.to(cuda)
    ci, va = to_dev(colind, cuda), to_dev(vals, cuda)
    want = R.c_spmm_f64(rowptr, colind, vals, B.numpy(), 1)
    monkeypatch.setenv("RA_TILE_TC5", "1")
    try:
        got = _run(kind, plan, Bd, False, ci, va)
        torch.cuda.synchronize()
        assert plan.device_status() == 0
        assert rel_fro(got, want) < 1e-5
        assert torch.equal(got, _run(kind, plan, Bd, False, ci, va))        # deterministic
        got16 = _run(kind, plan, Bd.half(), False, ci, va)
        assert torch.equal(got16, got)
    finally:
        monkeypatch.delenv("RA_TILE_TC5", raising=False)


@pytest.mark.parametrize("split", ["1", "0"])
@pytest.mark.parametrize("kind", ["tc", "ct", "sh"])
@pytest.mark.parametrize("N", [32, 64, 128, 256, 512])
def test_tma_gather_ring(cuda, kind, N, split, monkeypatch):
    """RA_TILE_G4=1 runs the TMA gather ring at sizes the engine policy would give to the cp.async
    ring; with RA_G4_SPLIT=1 the groups share windows (hub windows of 113 and 88 blocks cut across
    several groups, partial tiles merged in block order), with 0 they take whole windows. Both
    precisions against the float64 oracle on the rounded operands; reproducible; status clean."""
    M, K = 333, 1200
    rowptr, colind, vals = _mixed_matrix(M, K, seed=N + 9)
    plan = KINDS[kind][1](torch.from_numpy(rowptr), torch.from_numpy(colind), torch.from_numpy(vals), M, K, N)
    B = G.dense(K, N, N + 9)
    Bd = B.to(cuda)
    ci, va = to_dev(colind, cuda), to_dev(vals, cuda)
    monkeypatch.setenv("RA_TILE_G4", "1")
    monkeypatch.setenv("RA_G4_SPLIT", split)
    try:
        for tf32 in (False, True):
            want = R.c_spmm_f64(rowptr, colind, vals, B.numpy(), 2 if tf32 else 1)
            got = _run(kind, plan, Bd, tf32, ci, va)
            torch.cuda.synchronize()
            assert plan.device_status() == 0
            assert rel_fro(got, want) < 1e-5, f"{kind} N={N} tf32={tf32} split={split}"
            assert torch.equal(got, _run(kind, plan, Bd, tf32, ci, va))        # reproducible
    finally:
        monkeypatch.delenv("RA_TILE_G4", raising=False)
        monkeypatch.delenv("RA_G4_SPLIT", raising=False)


def test_tma_gather_ring_shares_one_long_window(cuda, monkeypatch):
    """One window of 4,000 blocks between windows of a few blocks and empty windows: most groups
    lie wholly inside the long window, so the merge walks a chain of many partial tiles."""
    M, K, N = 64, 40000, 64
    degs = np.zeros(M, dtype=np.int64)
    degs[8:16] = 4000                  # window 1: 32,000 distinct columns = 4,000 blocks
    degs[0] = 3; degs[40] = 17; degs[63] = 1
    rowptr, colind, vals = small_csr(M, K, degs, seed=3)
    B = G.dense(K, N, 3)
    Bd = B.to(cuda)
    monkeypatch.setenv("RA_TILE_G4", "1")
    try:
        for kind in ("tc", "ct"):
            plan = KINDS[kind][1](torch.from_numpy(rowptr), torch.from_numpy(colind), torch.from_numpy(vals), M, K, N)
            for tf32 in (False, True):
                got = _run(kind, plan, Bd, tf32)
                torch.cuda.synchronize()
                assert plan.device_status() == 0
                assert rel_fro(got, R.c_spmm_f64(rowptr, colind, vals, B.numpy(), 2 if tf32 else 1)) < 1e-5
    finally:
        monkeypatch.delenv("RA_TILE_G4", raising=False)


# ---- zero-compressed TC_DIRECT (make_tc_direct_zc_plan) ---------------------------------
def _zc_case(M, K, N, seed, cuda, unsorted=False):
    rowptr, colind, vals = _mixed_matrix(M, K, seed=seed, unsorted=unsorted)
    rp, ci, va = torch.from_numpy(rowptr), torch.from_numpy(colind), torch.from_numpy(vals)
    zc = ra_spmm.make_tc_direct_zc_plan(rp, ci, va, M, K, N)
    assert zc.zc and zc.valid
    return rowptr, colind, vals, zc


@pytest.mark.parametrize("M,K,unsorted", [(333, 1200, False), (8, 64, False), (1029, 300, True)])
def test_zc_plan_arrays(cuda, M, K, unsorted):
    """Masks, bases and packed values: bit-exact with the oracle and with the reference's
    own zero-compressed builder."""
    rowptr, colind, vals, zc = _zc_case(M, K, 64, M + 1, cuda, unsorted)
    got = {k: v.numpy() for k, v in zc.arrays().items()}
    want = O.tile_plan(rowptr, colind, vals, M, K, 64)
    assert set(got) == {"block_offsets", "atox", "val_masks", "val_base", "vals_zc"}
    assert np.array_equal(got["block_offsets"], want["block_offsets"])
    assert np.array_equal(got["atox"], want["atox"])
    assert np.array_equal(got["val_masks"].view(np.uint64), want["val_masks"])
    assert np.array_equal(got["val_base"], want["val_base"])
    assert np.array_equal(got["vals_zc"].view(np.uint16), want["vals_zc"])
    # plan_bytes with the reference's accounting (tc/ra_tc_direct.cu:767-773)
    nb, nnz, W = want["num_blocks"], want["nnz"], want["num_windows"]
    assert zc.plan_bytes == 4 * (W + 1) + 4 * 8 * nb + 12 * nb + 2 * nnz
    if ref_kernels() is not None:
        ra = RefTilePlan(3, rowptr, colind, vals, M, K, 64).arrays()
        assert set(ra) == set(got)
        for k in ra:
            g = got[k].view(np.uint16) if k == "vals_zc" else got[k]
            r = ra[k].view(np.uint16) if k == "vals_zc" else ra[k]
            assert np.array_equal(g, r), f"zc: {k} differs from the reference builder"


@pytest.mark.parametrize("N", [16, 47, 64, 128, 256])
def test_zc_outputs_equal_padded_plan(cuda, N):
    """The zero-compressed plan feeds the tensor cores the same operands in the same order as
    the padded plan: identical outputs on both precisions, and within tolerance of the
    reference's zero-compressed kernels."""
    M, K = 333, 1200
    rowptr, colind, vals, zc = _zc_case(M, K, N, N + 3, cuda)
    padded = ra_spmm.make_tc_direct_plan(torch.from_numpy(rowptr), torch.from_numpy(colind),
                                         torch.from_numpy(vals), M, K, N)
    B = G.dense(K, N, N + 3).to(cuda)
    ref = RefTilePlan(3, rowptr, colind, vals, M, K, N) if ref_kernels() is not None else None
    import os
    # compare against the same engine and the same order of additions: no tcgen05 path, and the TMA
    # ring with whole windows per group (shared windows add their partial tiles in another grouping)
    saved = {k: os.environ.get(k) for k in ("RA_TILE_TC5", "RA_G4_SPLIT")}
    os.environ["RA_TILE_TC5"] = "0"
    os.environ["RA_G4_SPLIT"] = "0"
    try:
        for tf32 in (False, True):
            got = _run("tc", zc, B, tf32)
            want = _run("tc", padded, B, tf32)
            torch.cuda.synchronize()
            assert torch.equal(got, want), f"N={N} tf32={tf32}"
            if ref is not None:
                assert rel_fro(got, ref.run(B, tf32)) < TOL_TILE
    finally:
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def test_zc_short_ranges_and_single_block(cuda):
    """Windows of one block and matrices smaller than the ring depth (the decode pipeline's
    start-up and drain)."""
    for M, K, deg in ((3, 40, 2), (8, 64, 1), (40, 64, 3)):
        degs = np.full(M, deg)
        rowptr, colind, vals = small_csr(M, K, degs, M)
        rp, ci, va = torch.from_numpy(rowptr), torch.from_numpy(colind), torch.from_numpy(vals)
        zc = ra_spmm.make_tc_direct_zc_plan(rp, ci, va, M, K, 64)
        B = G.dense(K, 64, M).to(cuda)
        for tf32 in (False, True):
            got = _run("tc", zc, B, tf32)
            want = R.c_spmm_f64(rowptr, colind, vals, B.cpu().numpy(), 2 if tf32 else 1)
            assert rel_fro(got, want) < 1e-5


@pytest.mark.parametrize("kind", ["tc", "ct", "sh"])
@pytest.mark.parametrize("N", [47, 64])
def test_staged_kernels_can_be_switched_off(cuda, kind, N, monkeypatch):
    """RA_TC_STAGED=0 keeps the direct-load kernels (the reference's switch,
    tc/ra_tc_direct.cu:837-838); same numeric contract."""
    M, K = 333, 1200
    rowptr, colind, vals = _mixed_matrix(M, K, seed=N + 31)
    plan = KINDS[kind][1](torch.from_numpy(rowptr), torch.from_numpy(colind), torch.from_numpy(vals), M, K, N)
    B = G.dense(K, N, N + 31)
    Bd = B.to(cuda)
    ci, va = to_dev(colind, cuda), to_dev(vals, cuda)
    monkeypatch.setenv("RA_TC_STAGED", "0")
    try:
        for tf32 in (False, True):
            got = _run(kind, plan, Bd, tf32, ci, va)
            want = R.c_spmm_f64(rowptr, colind, vals, B.numpy(), 2 if tf32 else 1)
            assert rel_fro(got, want) < 1e-5
    finally:
        monkeypatch.delenv("RA_TC_STAGED", raising=False)


def test_a_wait_that_runs_out_is_reported_and_the_plan_stays_usable(cuda, monkeypatch):
    """Bounded device waits: with a test-only poll limit of zero on the bulk-copy ring every
    consumer warp gives up on its first stage, records the status word and leaves, and the
    producer warps still collect, under the normal limit, the copies they had issued. The
    kernel returns normally, the host reads status 1 (which clears it), and the next run of
    the same plan is correct."""
    a = G.chung_lu_power_law(n=16384, seed=5)
    rp, ci, va = a.torch(cuda)
    plan = ra_spmm.make_tc_direct_plan(rp, ci, va, a.M, a.K, 64)
    B = G.dense(a.K, 64, 5).to(cuda)
    want = ra_spmm.run_tc_direct_plan(plan, B)
    assert plan.device_status() == 0
    monkeypatch.setenv("RA_TILE_TMA", "1")
    monkeypatch.setenv("RA_TILE_TC5", "0")
    monkeypatch.setenv("RA_TILE_G4", "0")
    assert rel_fro(ra_spmm.run_tc_direct_plan(plan, B), want.cpu().numpy()) < 1e-6     # the ring itself works
    assert plan.device_status() == 0
    monkeypatch.setenv("RA_TILE_TMA_POLL_LIMIT", "0")
    ra_spmm.run_tc_direct_plan(plan, B)                   # output of this run is not valid
    assert plan.device_status() == 1                      # kStatusFullTimeout, read and cleared
    assert plan.device_status() == 0
    monkeypatch.delenv("RA_TILE_TMA_POLL_LIMIT")
    assert rel_fro(ra_spmm.run_tc_direct_plan(plan, B), want.cpu().numpy()) < 1e-6
    assert plan.device_status() == 0
