"""Two-rank CPU worker: the sharded GCN step (all-gather of row slabs, transposed
operator in the backward, all-reduced weight gradients) equals the unsharded
step. The per-rank SpMM here is torch.sparse.mm on the CPU, injected by the test;
the CUDA operators are covered by the gpu-marked test."""
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
from ra_spmm_b200 import generators as G          # noqa: E402
from ra_spmm_b200 import partition as P           # noqa: E402
from ra_spmm_b200.gcn import GCN2, RowSharding, train_step   # noqa: E402

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
a = G.gcn_normalized_sbm(n=2000, n_comm=4, mean_degree=20.0, seed=123)


def cpu_op(rowptr, colind, vals, K):
    A = torch.sparse_csr_tensor(torch.from_numpy(rowptr.astype(np.int64)), torch.from_numpy(colind.astype(np.int64)),
                                torch.from_numpy(vals), size=(rowptr.size - 1, K))
    return lambda B: torch.sparse.mm(A, B)


torch.manual_seed(123)
X = torch.randn(a.M, 100)
y = torch.randint(0, 47, (a.M,))
torch.manual_seed(7)
ref_model = GCN2(100, 64, 47, cpu_op(a.rowptr, a.colind, a.vals, a.K), sharding=RowSharding([0, a.M]))
ref_opt = torch.optim.Adam(ref_model.parameters(), lr=1e-2)
ref_loss = train_step(ref_model, ref_opt, X, y, a.M)

bounds = P.nnz_balanced_row_splits(a.rowptr, world)
r0, r1 = int(bounds[rank]), int(bounds[rank + 1])
rp, ci, va = P.row_block(a.rowptr, a.colind, a.vals, r0, r1)
torch.manual_seed(7)
sh = RowSharding(bounds, rank, world)
model = GCN2(100, 64, 47, cpu_op(rp, sh.remap_columns(ci), va, sh.gathered_rows), sharding=sh)
opt = torch.optim.Adam(model.parameters(), lr=1e-2)
loss = train_step(model, opt, X[r0:r1], y[r0:r1], a.M)

assert abs(float(loss) - float(ref_loss)) < 1e-5, (float(loss), float(ref_loss))
for p, q in zip(model.parameters(), ref_model.parameters()):
    assert torch.allclose(p.grad, q.grad, rtol=1e-4, atol=1e-6)
    assert torch.allclose(p, q, rtol=1e-4, atol=1e-6)          # weights after the Adam step
# operand-format path: the slab is rounded to fp16 and padded to a multiple of 16 columns BEFORE
# the all-gather; an operator that reads fp16 must then see exactly round_fp16(operand), and the
# caller must get the unpadded width back
from ra_spmm_b200.gcn import sharded_spmm          # noqa: E402
seen = {}


def fp16_op(B):
    seen["dtype"], seen["width"] = B.dtype, B.shape[1]
    return cpu_op(rp, sh.remap_columns(ci), va, sh.gathered_rows)(B.float())


H = torch.randn(r1 - r0, 47, generator=torch.Generator().manual_seed(100 + rank))
got = sharded_spmm(H, fp16_op, fp16_op, sh, operand_format=lambda n: (torch.float16, (n + 15) // 16 * 16))
want = cpu_op(rp, sh.remap_columns(ci), va, sh.gathered_rows)(sh.all_gather_rows(H.half().float()))
assert seen["dtype"] == torch.float16 and seen["width"] == 48, seen
assert got.shape == (r1 - r0, 47) and torch.equal(got, want)

# ---- panelled gather: 4 column panels of a 128-wide operand, each gathered on its own ----
H = torch.randn(r1 - r0, 128, generator=torch.Generator().manual_seed(200 + rank))
op = cpu_op(rp, sh.remap_columns(ci), va, sh.gathered_rows)
whole = sharded_spmm(H, op, op, sh)
in_panels = sharded_spmm(H, op, op, sh, panels=4)
assert torch.allclose(whole, in_panels, rtol=1e-6, atol=1e-6)
assert torch.equal(sharded_spmm(H[:, :40].contiguous(), op, op, sh, panels=4),      # too narrow: falls back to one gather
                   sharded_spmm(H[:, :40].contiguous(), op, op, sh))

# ---- row chunks: the slab is gathered in 3 runs of rows, the operator is split by the chunk that
# owns the column, the partial products are added; with and without the fp16 operand format, and a
# whole training step ----
sh3 = RowSharding(bounds, rank, world, chunks=3)
ops3 = [cpu_op(*t) for t in sh3.split_columns(rp, ci, va)]
assert sum(int(t[0][-1]) for t in sh3.split_columns(rp, ci, va)) == int(rp[-1])
in_chunks = sharded_spmm(H, ops3, ops3, sh3)
assert torch.allclose(whole, in_chunks, rtol=1e-5, atol=1e-5)
H47 = torch.randn(r1 - r0, 47, generator=torch.Generator().manual_seed(300 + rank))
ops3_f = [(lambda B, f=f: f(B.float())) for f in ops3]
got3 = sharded_spmm(H47, ops3_f, ops3_f, sh3, operand_format=lambda n: (torch.float16, (n + 15) // 16 * 16))
want3 = cpu_op(rp, sh.remap_columns(ci), va, sh.gathered_rows)(sh.all_gather_rows(H47.half().float()))
assert got3.shape == (r1 - r0, 47) and torch.allclose(got3, want3, rtol=1e-5, atol=1e-5)
torch.manual_seed(7)
model3 = GCN2(100, 64, 47, ops3, sharding=sh3)
loss3 = train_step(model3, torch.optim.Adam(model3.parameters(), lr=1e-2), X[r0:r1], y[r0:r1], a.M)
assert abs(float(loss3) - float(loss)) < 1e-5, (float(loss3), float(loss))
for p3, q in zip(model3.parameters(), model.parameters()):
    assert torch.allclose(p3, q, rtol=1e-4, atol=1e-6)

# ---- layer 1 associated the other way, (A X) W1: same loss and weights as A (X W1), sharded or not ----
torch.manual_seed(7)
af = GCN2(100, 64, 47, cpu_op(rp, sh.remap_columns(ci), va, sh.gathered_rows), sharding=sh, aggregate_first=True)
loss_af = train_step(af, torch.optim.Adam(af.parameters(), lr=1e-2), X[r0:r1], y[r0:r1], a.M)
assert abs(float(loss_af) - float(ref_loss)) < 1e-5, (float(loss_af), float(ref_loss))
for pa, q in zip(af.parameters(), ref_model.parameters()):
    assert torch.allclose(pa.grad, q.grad, rtol=1e-3, atol=1e-5)
    assert torch.allclose(pa, q, rtol=1e-3, atol=1e-5)

# ---- GraphSAGE (row-mean operator, not symmetric: the backward needs the transposed row block)
# and GIN (raw adjacency, learnable eps) against the unsharded step ----
from ra_spmm_b200.gcn import GIN2, SAGE2, aggregation_operator, transpose_csr   # noqa: E402
raw = G.chung_lu_power_law(n=1500, seed=5)                                       # structure only
for name, cls in (("sage", SAGE2), ("gin", GIN2)):
    orp, oci, ova = aggregation_operator(raw.rowptr, raw.colind, raw.M, name)
    trp, tci, tva = transpose_csr(orp, oci, ova, raw.M, raw.K)
    torch.manual_seed(11)
    Xs = torch.randn(raw.M, 24)
    ys = torch.randint(0, 7, (raw.M,))
    torch.manual_seed(3)
    ref = cls(24, 32, 7, cpu_op(orp, oci, ova, raw.K), cpu_op(trp, tci, tva, raw.M), sharding=RowSharding([0, raw.M]))
    ref_loss = train_step(ref, torch.optim.Adam(ref.parameters(), lr=1e-2), Xs, ys, raw.M)
    b = P.nnz_balanced_row_splits(orp, world)
    q0, q1 = int(b[rank]), int(b[rank + 1])
    shs = RowSharding(b, rank, world)
    frp, fci, fva = P.row_block(orp, oci, ova, q0, q1)
    brp, bci, bva = P.row_block(trp, tci, tva, q0, q1)
    torch.manual_seed(3)
    mdl = cls(24, 32, 7, cpu_op(frp, shs.remap_columns(fci), fva, shs.gathered_rows),
              cpu_op(brp, shs.remap_columns(bci), bva, shs.gathered_rows), sharding=shs)
    loss = train_step(mdl, torch.optim.Adam(mdl.parameters(), lr=1e-2), Xs[q0:q1], ys[q0:q1], raw.M)
    assert abs(float(loss) - float(ref_loss)) < 1e-5, (name, float(loss), float(ref_loss))
    for pa, pb in zip(mdl.parameters(), ref.parameters()):
        assert torch.allclose(pa.grad, pb.grad, rtol=1e-4, atol=1e-6), name
        assert torch.allclose(pa, pb, rtol=1e-4, atol=1e-6), name

ok = torch.tensor([1]); dist.all_reduce(ok)
if rank == 0 and int(ok) == world:
    print("GCN_GLOO_OK")
dist.destroy_process_group()
