"""Allocation-free ZERO_OVERHEAD_CSR run (ra_zo_plan_run_noalloc).

For hosts that may not allocate device memory once they are running - every byte
of HBM belongs to their own pool, or a cudaMalloc would stall their in-flight
streams - the library offers a run entry point whose scratch is a fixed 16 MiB
array inside the library image. This test calls it through the C ABI, with the
output buffer supplied by the caller, twice in a row, on a plan that never went
through the allocating entry point, and compares with that entry point run on a
sibling plan and with the float64 oracle (fp32 tolerance of the other tests:
1e-5 relative Frobenius error). It also checks that the device's free memory
does not change across a call, and the size limit. The file name makes pytest
collect it last."""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import ref_bindings as R
from ra_spmm_b200 import _capi
from ra_spmm_b200 import generators as G
from ra_spmm_b200 import ra_spmm

pytestmark = pytest.mark.gpu
TOL_FP32 = 1e-5


def _rel_fro(x, ref):
    return float(torch.linalg.norm(x.double() - ref.double()) / torch.linalg.norm(ref.double()))


def _noalloc(lib, plan, rp, ci, va, B, out, N):
    rc = lib.ra_zo_plan_run_noalloc(plan._h, rp.data_ptr(), ci.data_ptr(), va.data_ptr(),
                                    B.data_ptr(), out.data_ptr(), N, torch.cuda.current_stream().cuda_stream)
    assert rc == 0, lib.ra_last_error_string()


def test_noalloc_matches_allocating_run_twice(cuda, lib):
    a = G.chung_lu_power_law(n=65536, seed=21)          # has multi-chunk rows -> uses scratch
    rp, ci, va = a.torch(cuda)
    N = 128
    plan = ra_spmm.make_zero_overhead_plan(rp, a.M, a.K)          # runs through the allocating entry point
    quiet = ra_spmm.make_zero_overhead_plan(rp, a.M, a.K)         # only ever runs through the new one
    assert plan.num_chunks > 0 and plan.num_zero_rows > plan.num_empty     # multi-chunk rows exist
    out = torch.empty((a.M, N), dtype=torch.float32, device=cuda)          # caller-owned output
    for trial in range(2):
        B = G.dense(a.K, N, 100 + trial).to(cuda)
        want = ra_spmm.run_zero_overhead_plan(plan, rp, ci, va, B)
        out.fill_(float("nan"))
        if trial == 1:
            # the property the entry point exists for: the device's free memory does not move
            # across a call (the first call only looked up the address of the built-in array)
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info(cuda)[0]
        _noalloc(lib, quiet, rp, ci, va, B, out, N)
        torch.cuda.synchronize()
        if trial == 1:
            assert torch.cuda.mem_get_info(cuda)[0] == free_before
        assert not torch.isnan(out).any()
        assert _rel_fro(out, want) < TOL_FP32
        # and against the float64 oracle, not only against the sibling entry point
        want64 = torch.from_numpy(R.c_spmm_f64(a.rowptr, a.colind, a.vals, B.cpu().numpy(), 0)).to(cuda)
        assert _rel_fro(out, want64) < TOL_FP32
    # a different plan right after reuses the same built-in scratch
    b = G.rmat_graph(scale=13, seed=5)
    rp2, ci2, va2 = b.torch(cuda)
    plan2 = ra_spmm.make_zero_overhead_plan(rp2, b.M, b.K)
    quiet2 = ra_spmm.make_zero_overhead_plan(rp2, b.M, b.K)
    B2 = G.dense(b.K, N, 7).to(cuda)
    want2 = ra_spmm.run_zero_overhead_plan(plan2, rp2, ci2, va2, B2)
    out2 = torch.empty((b.M, N), dtype=torch.float32, device=cuda)
    _noalloc(lib, quiet2, rp2, ci2, va2, B2, out2, N)
    torch.cuda.synchronize()
    assert _rel_fro(out2, want2) < TOL_FP32


def test_noalloc_rejects_oversized_plans(cuda, lib):
    # one row of 300,000 nonzeros -> 1172 chunk slots; at N=4096 that is 4.8 M floats > 4 Mi
    M, K, N = 8, 300000, 4096
    rowptr = np.zeros(M + 1, dtype=np.int32)
    rowptr[1:] = 300000
    rp = torch.from_numpy(rowptr).to(cuda)
    plan = ra_spmm.make_zero_overhead_plan(rp, M, K)
    assert plan.max_long_chunks == 1172
    dummy = torch.zeros(16, device=cuda)
    rc = lib.ra_zo_plan_run_noalloc(plan._h, rp.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                    dummy.data_ptr(), dummy.data_ptr(), N, None)
    assert rc == 6                                       # RA_ERR_TOO_LARGE, nothing launched
    msg = lib.ra_last_error_string().decode()
    assert "scratch" in msg and "4194304" in msg
