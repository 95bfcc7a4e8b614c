"""Plan files: save -> load gives the same arrays and the same product; a damaged file is refused."""
import numpy as np
import pytest
import torch

from ra_spmm_b200 import generators as G
from ra_spmm_b200 import ra_spmm

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def graph(cuda):
    a = G.rmat_graph(scale=13, edge_factor=16, seed=8)          # hub rows: multi-chunk rows, split windows
    rp, ci, va = a.torch(cuda)
    return a, rp, ci, va, G.dense(a.K, 64, 8).to(cuda)


def _same_arrays(p, q):
    x, y = p.arrays(), q.arrays()
    assert set(x) == set(y)
    for k in x:
        assert torch.equal(x[k], y[k]), k


def test_zero_overhead_plan_round_trip(graph, tmp_path):
    a, rp, ci, va, B = graph
    plan = ra_spmm.make_zero_overhead_plan(rp, a.M, a.K)
    path = tmp_path / "zo.plan"
    ra_spmm.save_plan(plan, path)
    back = ra_spmm.load_zero_overhead_plan(path)
    _same_arrays(plan, back)
    for f in ("M", "K", "num_tiny", "num_short", "num_medium", "num_long", "num_empty", "num_chunks",
              "num_zero_rows", "max_long_chunks", "plan_bytes"):
        assert getattr(plan, f) == getattr(back, f), f
    assert torch.equal(ra_spmm.run_zero_overhead_plan(plan, rp, ci, va, B),
                       ra_spmm.run_zero_overhead_plan(back, rp, ci, va, B))


@pytest.mark.parametrize("make,run", [
    (ra_spmm.make_tc_direct_plan, lambda p, ci, va, B: ra_spmm.run_tc_direct_plan(p, B)),
    (ra_spmm.make_tc_direct_zc_plan, lambda p, ci, va, B: ra_spmm.run_tc_direct_plan_tf32(p, B)),
    (ra_spmm.make_community_tc_plan, lambda p, ci, va, B: ra_spmm.run_community_tc_plan(p, B)),
    (ra_spmm.make_segment_hybrid_plan, lambda p, ci, va, B: ra_spmm.run_segment_hybrid_plan_tf32(p, ci, va, B))])
def test_tile_plan_round_trip(graph, tmp_path, make, run):
    a, rp, ci, va, B = graph
    plan = make(rp, ci, va, a.M, a.K, 64)
    path = tmp_path / "tile.plan"
    ra_spmm.save_plan(plan, path)
    back = ra_spmm.load_tile_plan(path)
    assert type(back) is type(plan) and back.active and back.num_tc_tiles == plan.num_tc_tiles
    _same_arrays(plan, back)
    assert torch.equal(run(plan, ci, va, B), run(back, ci, va, B))
    assert back.device_status() == 0


def test_a_damaged_file_is_refused(graph, tmp_path):
    a, rp, ci, va, B = graph
    plan = ra_spmm.make_segment_hybrid_plan(rp, ci, va, a.M, a.K, 64)
    path = tmp_path / "tile.plan"
    ra_spmm.save_plan(plan, path)
    raw = bytearray(path.read_bytes())
    flipped = bytearray(raw); flipped[len(raw) // 2] ^= 0x40                 # one bit inside an array
    (tmp_path / "flip.plan").write_bytes(flipped)
    with pytest.raises(ra_spmm.RaSpmmError, match="checksum"):
        ra_spmm.load_tile_plan(tmp_path / "flip.plan")
    (tmp_path / "short.plan").write_bytes(raw[: len(raw) // 3])
    with pytest.raises(ra_spmm.RaSpmmError, match="truncated"):
        ra_spmm.load_tile_plan(tmp_path / "short.plan")
    with pytest.raises(ra_spmm.RaSpmmError, match="ZERO_OVERHEAD"):           # wrong family
        ra_spmm.load_zero_overhead_plan(path)
