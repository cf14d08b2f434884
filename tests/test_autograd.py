"""Backward pass of the SpMM: transpose on CPU; gradients on the GPU against torch autograd."""
import pytest
import torch

from trspmm import graphs, transpose_csr


def test_transpose_csr_matches_dense_transpose():
    rp, col, val = graphs.rmat_graph(8, 6, seed=4)
    n = rp.numel() - 1
    rp, col, val = rp[: n - 40 + 1], col[: int(rp[n - 40])], val[: int(rp[n - 40])]   # rectangular: fewer rows
    m = rp.numel() - 1
    A = torch.sparse_csr_tensor(rp.long(), col.long(), val, (m, n)).to_dense()
    rp_t, col_t, val_t, perm = transpose_csr(rp, col, val, n)
    assert rp_t.dtype == rp.dtype and col_t.dtype == col.dtype and int(rp_t[-1]) == col.numel()
    At = torch.sparse_csr_tensor(rp_t.long(), col_t.long(), val_t, (n, m)).to_dense()
    assert torch.equal(At, A.t())
    for r in range(0, n, 17):   # canonical: ascending inside each row
        seg = col_t[rp_t[r]:rp_t[r + 1]]
        assert torch.all(seg[1:] > seg[:-1])
    assert torch.equal(val[perm], val_t)


@pytest.mark.gpu
def test_spmm_gradients_match_torch_autograd():
    from trspmm import DifferentiableSpmm
    rp, col, val = graphs.rmat_graph(10, 12, seed=6)
    n = rp.numel() - 1
    F = 64
    op = DifferentiableSpmm(rp.cuda(), col.cuda(), val.cuda(), n)
    assert op.stats["dropped_nnz"] == 0 and op.stats_t["dropped_nnz"] == 0
    g = torch.Generator().manual_seed(1)
    B0 = torch.randn(n, F, generator=g).half()
    G0 = torch.randn(n, F, generator=g).half()

    B = B0.cuda().requires_grad_(True)
    values = val.cuda().clone().requires_grad_(True)
    C = op(B, values=values)
    assert C.dtype == torch.float16 and C.shape == (n, F)
    C.backward(G0.cuda())

    # reference: dense fp32 autograd on the fp16-rounded operands
    v32 = val.half().float().requires_grad_(True)
    rows = torch.repeat_interleave(torch.arange(n), (rp[1:] - rp[:-1]).long())
    Bref = B0.float().requires_grad_(True)
    A = torch.sparse_coo_tensor(torch.stack([rows, col.long()]), v32, (n, n))
    Cref = torch.sparse.mm(A, Bref)
    Cref.backward(G0.float())

    def close(got, ref, tol):
        scale = ref.abs().max()
        return float((got.float().cpu() - ref).abs().max() / scale) <= tol

    assert close(C.detach(), Cref.detach(), 2e-3)
    assert close(B.grad, Bref.grad, 2e-3)
    assert close(values.grad, v32.grad, 2e-3)
    # B-only path: no gradient requested for the values
    B2 = B0.cuda().requires_grad_(True)
    op(B2).sum().backward()
    ones = torch.ones(n, F)
    assert close(B2.grad, torch.sparse.mm(A.detach().t(), ones), 2e-3)
