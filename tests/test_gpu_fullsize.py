"""Parity at the sizes the benchmark times (configurations 2-5 at full size).

The reduced-size tests take different code paths from the full-size runs (several waves of
CTAs, weight searches over 10^6 rows, 10^7 blocks, split windows with hundreds of segments),
so every kernel the benchmark reports is checked here on the benchmark's own matrices:
  * every plan array is compared, on the device, with the array the reference's own builder
    (compiled from its sources into oracle/_ref) produces for the same CSR - bit-exact;
  * every output is compared with the reference's own kernel on the same inputs: relative
    Frobenius error <= 1e-5 for the fp32 kernels, <= 5e-3 for the FP16 / TF32 tile paths
    (the tolerances of the reference's harness, ra_real_graph_eval.py and
    gnn_bench/router_vs_baselines_gcn.py:421-445);
  * configuration 2 is also compared with the float64 C oracle, through the allocating and
    the allocation-free ZERO_OVERHEAD_CSR entry points;
  * special A values (NaN, +-Inf, 7e4, 1e-6, 6e-8) go through the three tile builders and are
    compared with the reference builders' bits.
The graphs come from the on-disk cache of the generators when the benchmark ran before.
"""
import ctypes as C
import gc

import numpy as np
import pytest
import torch

from oracle import ref_bindings as R
from ra_spmm_b200 import generators as G
from ra_spmm_b200 import ra_spmm
from gpu_util import RefTilePlan, RefZoPlan, ref_csr_direct, ref_kernels, to_dev

pytestmark = pytest.mark.gpu
TOL_FP32, TOL_TILE = 1e-5, 5e-3


class _DeviceView:
    """Zero-copy torch view of a raw device array (CUDA array interface)."""

    def __init__(self, ptr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (int(n),), "typestr": typestr,
                                         "data": (int(ptr), False), "version": 2}


def dview(ptr, n, typestr, dev):
    if n == 0 or not ptr:
        return torch.empty(0, device=dev)
    return torch.as_tensor(_DeviceView(ptr, n, typestr), device=dev)


def rel_fro_dev(x, ref):
    """Relative Frobenius error, accumulated in float64 on the device."""
    num = torch.linalg.vector_norm((x.double() - ref.double()).flatten())
    den = torch.linalg.vector_norm(ref.double().flatten())
    return float(num / den)


def _free():
    gc.collect()
    torch.cuda.empty_cache()


@pytest.fixture(scope="module")
def need_ref():
    if ref_kernels() is None:
        pytest.fail("oracle/_ref/libra_ref_kernels.so is missing: the full-size parity tests compare "
                    "with the reference's own builders and kernels")


def _load(name, dev):
    a, N, b_dtype = G.cached_config(name, 1.0)
    B = G.dense(a.K, N, G.CONFIG_SEEDS[name], b_dtype)
    rp, ci, va = a.torch(dev)
    return a, N, B, rp, ci, va


def _compare_zo_lists(plan, ref, dev):
    i, r = plan._info, ref.info
    assert (i.num_small, i.num_chunks, i.num_zero_rows) == (r.num_small, r.num_chunks, r.num_zero_rows)
    assert (i.num_tiny, i.num_short, i.num_medium, i.num_long, i.num_empty, i.max_long_chunks) == \
           (r.num_tiny, r.num_short, r.num_medium, r.num_long, r.num_empty, r.max_long_chunks)
    for name, n in (("small_row_ids", i.num_small), ("chunk_rows", i.num_chunks),
                    ("chunk_starts", i.num_chunks), ("zero_row_ids", i.num_zero_rows)):
        mine = dview(getattr(i, "d_" + name), n, "<i4", dev)
        theirs = dview(getattr(r, "d_" + name), n, "<i4", dev)
        assert torch.equal(mine, theirs), f"ZERO_OVERHEAD list {name} differs from the reference builder"


_TILE_ARRAYS = {
    # fp16 bit patterns are viewed as int16 (torch has no comparison kernels for uint16)
    "block_offsets": ("<i4", lambda i: i.num_windows + 1), "atox": ("<i4", lambda i: 8 * i.num_blocks),
    "vals_f16": ("<i2", lambda i: 64 * i.num_blocks), "win_rows": ("<i4", lambda i: 8 * i.num_windows),
    "seg_window": ("<i4", lambda i: i.num_segments), "seg_bbegin": ("<i4", lambda i: i.num_segments),
    "seg_bend": ("<i4", lambda i: i.num_segments), "seg_scratch": ("<i4", lambda i: i.num_segments),
    "split_wins": ("<i4", lambda i: i.num_split_windows), "split_off": ("<i4", lambda i: i.num_split_windows + 1),
    "zero_rows": ("<i4", lambda i: i.num_zero_rows),
}
_KIND_ARRAYS = {0: ("block_offsets", "atox", "vals_f16"),
                1: ("block_offsets", "atox", "vals_f16", "win_rows"),
                2: ("block_offsets", "atox", "vals_f16", "seg_window", "seg_bbegin", "seg_bend", "seg_scratch",
                    "split_wins", "split_off", "zero_rows")}


def _compare_tile_arrays(kind, plan, ref, dev):
    i, r = plan._info, ref.info
    assert i.active and r.active
    assert (i.num_windows, int(i.num_blocks)) == (r.num_windows, r.num_blocks)
    if kind == 2:
        assert (i.num_segments, i.num_split_segs, i.num_split_windows, i.num_zero_rows) == \
               (r.num_segments, r.num_split_segs, r.num_split_windows, r.num_zero_rows)
    for name in _KIND_ARRAYS[kind]:
        typestr, count = _TILE_ARRAYS[name]
        n = int(count(i))
        mine = dview(getattr(i, "d_" + name), n, typestr, dev)
        theirs = dview(getattr(r, "d_" + name), n, typestr, dev)
        assert torch.equal(mine, theirs), f"tile array {name} differs from the reference builder"


# ---- configuration 2: ZERO_OVERHEAD_CSR (routed and named) + CSR_DIRECT ------------------
def test_c2_zero_overhead_and_csr_direct(cuda, lib, need_ref):
    a, N, B, rp, ci, va = _load("C2", cuda)
    Bd = B.to(cuda)
    d = ra_spmm.make_router_plan(rp, ci, va, a.M, a.K, N)
    assert d["chosen_path"] == "ZERO_OVERHEAD_CSR"
    plan = ra_spmm.make_zero_overhead_plan(rp, a.M, a.K)
    ref = RefZoPlan(a.rowptr, a.M, a.K)
    _compare_zo_lists(plan, ref, cuda)
    want_ref = ref.run(rp, ci, va, Bd)
    got = ra_spmm.run_zero_overhead_plan(plan, rp, ci, va, Bd)
    assert rel_fro_dev(got, want_ref) < TOL_FP32
    assert torch.equal(got, ra_spmm.run_zero_overhead_plan(plan, rp, ci, va, Bd))      # deterministic merge
    got_cd = ra_spmm.spmm_csr_direct(rp, ci, va, Bd)
    assert rel_fro_dev(got_cd, ref_csr_direct(rp, ci, va, Bd)) < TOL_FP32
    # float64 C oracle, and the allocation-free entry point on a plan that never ran the
    # allocating one (its scratch is the array inside the library)
    want64 = torch.from_numpy(R.c_spmm_f64(a.rowptr, a.colind, a.vals, B.numpy(), 0)).to(cuda)
    assert rel_fro_dev(got, want64) < TOL_FP32 and rel_fro_dev(got_cd, want64) < TOL_FP32
    fresh = ra_spmm.make_zero_overhead_plan(rp, a.M, a.K)
    out = torch.full((a.M, N), float("nan"), dtype=torch.float32, device=cuda)
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.ra_zo_plan_run_noalloc(fresh._h, rp.data_ptr(), ci.data_ptr(), va.data_ptr(),
                                    Bd.data_ptr(), out.data_ptr(), N, st)
    assert rc == 0, lib.ra_last_error_string()
    torch.cuda.synchronize()
    assert rel_fro_dev(out, want64) < TOL_FP32 and torch.equal(out, got)
    del plan, ref, fresh
    _free()


# ---- configuration 3: COMMUNITY_TC (named) and TC_DIRECT (routed), FP16, fp16 B ----------
@pytest.mark.parametrize("kind,make,run", [
    (1, ra_spmm.make_community_tc_plan, ra_spmm.run_community_tc_plan),
    (0, ra_spmm.make_tc_direct_plan, ra_spmm.run_tc_direct_plan)])
def test_c3_fp16_tile_paths(cuda, need_ref, kind, make, run):
    a, N, B, rp, ci, va = _load("C3", cuda)
    assert B.dtype == torch.float16
    d = ra_spmm.make_router_plan(rp, ci, va, a.M, a.K, N)
    assert d["chosen_path"] == "TC_DIRECT" and not d["use_tf32"]
    plan = make(rp, ci, va, a.M, a.K, N)
    ref = RefTilePlan(kind, a.rowptr, a.colind, a.vals, a.M, a.K, N)
    _compare_tile_arrays(kind, plan, ref, cuda)
    Bh = B.to(cuda)
    got = run(plan, Bh)                                   # fp16 B handed over directly
    want = ref.run(Bh.float(), False)                     # the reference rounds the same values itself
    assert rel_fro_dev(got, want) < TOL_TILE
    assert torch.equal(got, run(plan, Bh.float()))        # == fp32 B rounded by the library
    assert plan.device_status() == 0
    del plan, ref, got, want
    _free()


# ---- configuration 4: SEGMENT_HYBRID TF32 (named) and ZERO_OVERHEAD_CSR (routed) ----------
def test_c4_segment_hybrid_tf32_and_routed(cuda, lib, need_ref):
    a, N, B, rp, ci, va = _load("C4", cuda)
    Bd = B.to(cuda)
    d = ra_spmm.make_router_plan(rp, ci, va, a.M, a.K, N)
    assert d["chosen_path"] == "ZERO_OVERHEAD_CSR" and not d["use_tf32"]
    plan = ra_spmm.make_segment_hybrid_plan(rp, ci, va, a.M, a.K, N)
    ref = RefTilePlan(2, a.rowptr, a.colind, a.vals, a.M, a.K, N)
    _compare_tile_arrays(2, plan, ref, cuda)
    assert plan.num_split_windows > 0                     # hub windows go through the merge
    got = ra_spmm.run_segment_hybrid_plan_tf32(plan, ci, va, Bd)
    assert rel_fro_dev(got, ref.run(Bd, True)) < TOL_TILE
    got16 = ra_spmm.run_segment_hybrid_plan(plan, ci, va, Bd)
    assert rel_fro_dev(got16, ref.run(Bd, False)) < TOL_TILE
    del plan, ref, got16
    _free()
    zo = ra_spmm.make_zero_overhead_plan(rp, a.M, a.K)
    rzo = RefZoPlan(a.rowptr, a.M, a.K)
    _compare_zo_lists(zo, rzo, cuda)
    want = rzo.run(rp, ci, va, Bd)
    got_zo = ra_spmm.run_zero_overhead_plan(zo, rp, ci, va, Bd)
    assert rel_fro_dev(got_zo, want) < TOL_FP32
    assert rel_fro_dev(got, want) < TOL_TILE              # the TF32 tile path against the fp32 result
    # 128 M nonzeros in 639-chunk hub rows need more scratch than the built-in array holds
    out = torch.empty((a.M, N), dtype=torch.float32, device=cuda)
    rc = lib.ra_zo_plan_run_noalloc(zo._h, rp.data_ptr(), ci.data_ptr(), va.data_ptr(), Bd.data_ptr(),
                                    out.data_ptr(), N, torch.cuda.current_stream().cuda_stream)
    assert rc == 6, "RA_ERR_TOO_LARGE expected"
    del zo, rzo
    _free()


# ---- configuration 5: the two SpMM sites of the GCN (N = 256 and N = 47) -------------------
def test_c5_gcn_spmm_sites(cuda, need_ref):
    a, N, B, rp, ci, va = _load("C5", cuda)
    d = ra_spmm.make_router_plan(rp, ci, va, a.M, a.K, N)
    assert d["chosen_path"] == "TC_DIRECT" and not d["use_tf32"]
    plan = ra_spmm.make_tc_direct_plan(rp, ci, va, a.M, a.K, N)
    ref = RefTilePlan(0, a.rowptr, a.colind, a.vals, a.M, a.K, N)
    _compare_tile_arrays(0, plan, ref, cuda)
    for width in (256, 47):
        Bw = G.dense(a.K, width, G.CONFIG_SEEDS["C5"] + width).to(cuda)
        got = ra_spmm.run_tc_direct_plan(plan, Bw)
        assert rel_fro_dev(got, ref.run(Bw, False)) < TOL_TILE, width
        got32 = ra_spmm.spmm_csr_direct(rp, ci, va, Bw)   # the all-fp32 step of the GCN harness
        assert rel_fro_dev(got32, ref_csr_direct(rp, ci, va, Bw)) < TOL_FP32, width
        assert rel_fro_dev(got, got32) < TOL_TILE, width
        del Bw, got, got32
    del plan, ref
    _free()


# ---- special values through the three tile builders ---------------------------------------
@pytest.mark.parametrize("kind,make", [(0, ra_spmm.make_tc_direct_plan), (1, ra_spmm.make_community_tc_plan),
                                       (2, ra_spmm.make_segment_hybrid_plan), (3, ra_spmm.make_tc_direct_zc_plan)])
def test_special_values_match_the_reference_builders(cuda, need_ref, kind, make):
    a = G.chung_lu_power_law(n=4096, seed=9)
    vals = a.vals.copy()
    neg_nan = np.array([0xFFC00001], dtype=np.uint32).view(np.float32)[0]
    special = np.array([np.nan, neg_nan, np.inf, -np.inf, 7e4, -7e4, 65520.0, 1e-6, 6e-8, -6e-8,
                        2.0 ** -25, 2.0 ** -25 * 1.0001, 2.0 ** -24, 0.0, -0.0], dtype=np.float32)
    idx = np.random.default_rng(4).choice(vals.size, size=special.size * 8, replace=False)
    vals[idx] = np.tile(special, 8)
    rp, ci, va = to_dev(a.rowptr, cuda), to_dev(a.colind, cuda), to_dev(vals, cuda)
    plan = make(rp, ci, va, a.M, a.K, 64)
    ref = RefTilePlan(kind, a.rowptr, a.colind, vals, a.M, a.K, 64)
    got = {k: v.numpy() for k, v in plan.arrays().items()}
    want = ref.arrays()
    assert set(got) == set(want)
    for k in want:
        g = got[k].view(np.uint16) if k in ("vals_f16", "vals_zc") else got[k]
        assert np.array_equal(g, want[k]), f"{k} differs from the reference builder for special values"
