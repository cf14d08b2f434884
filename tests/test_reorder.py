"""Row reordering hook (the reference's apply_tca_reorder slot): permutation validity, exact CSR
row gather, effect on graphs with hidden structure, dataset wiring.  CPU only."""
import numpy as np
import pytest
import torch

from trspmm import graphs
from trspmm.reorder import METHODS, apply_tca_reorder, permute_rows, row_order, window_column_pairs


def _shuffled_clustered(n=4096, seed=3):
    rp, col, val = graphs.clustered_graph(n, community=64, intra=12, glob=1, seed=seed)
    g = torch.Generator().manual_seed(seed)
    shuffle = torch.randperm(n, generator=g)          # hide the community structure of the rows
    rp2, col2, val2 = permute_rows(rp, col, val, shuffle)
    return rp, col, val, rp2, col2, val2


@pytest.mark.parametrize("method", METHODS)
def test_order_is_a_permutation_and_rows_are_gathered_exactly(method):
    rp, col, val = graphs.rmat_graph(10, 8, seed=2)
    n = rp.numel() - 1
    rid = row_order(rp, col, method)
    assert rid.dtype == torch.int64 and sorted(rid.tolist()) == list(range(n))
    assert torch.equal(rid, row_order(rp, col, method))  # deterministic
    nrp, ncol, nval = permute_rows(rp, col, val, rid)
    assert int(nrp[-1]) == col.numel() and nrp.dtype == rp.dtype
    for i in (0, 1, n // 2, n - 1):
        o = int(rid[i])
        assert torch.equal(ncol[nrp[i]:nrp[i + 1]], col[rp[o]:rp[o + 1]])
        assert torch.equal(nval[nrp[i]:nrp[i + 1]], val[rp[o]:rp[o + 1]])
    # the matrix product is the row-permuted product
    A = torch.sparse_csr_tensor(rp.long(), col.long(), val.float(), (n, n))
    Ap = torch.sparse_csr_tensor(nrp.long(), ncol.long(), nval.float(), (n, n))
    B = torch.randn(n, 8, generator=torch.Generator().manual_seed(0))
    assert torch.allclose(torch.sparse.mm(Ap, B), torch.sparse.mm(A, B)[rid], atol=1e-5)


def test_minhash_and_hub_orders_recover_hidden_communities():
    rp, col, _, rp2, col2, _ = _shuffled_clustered()
    ordered = window_column_pairs(rp, col)
    shuffled = window_column_pairs(rp2, col2)
    assert shuffled > 2 * ordered
    for method in ("minhash", "hub"):
        rid = row_order(rp2, col2, method)
        nrp, ncol, _ = permute_rows(rp2, col2, None, rid)
        got = window_column_pairs(nrp, ncol)
        assert got < 0.6 * shuffled, (method, ordered, shuffled, got)


def test_degree_order_sorts_descending_and_keeps_empty_rows_last():
    rp = torch.tensor([0, 2, 2, 5, 6, 6], dtype=torch.int32)
    col = torch.tensor([0, 1, 0, 2, 3, 4], dtype=torch.int32)
    assert row_order(rp, col, "degree").tolist() == [2, 0, 3, 1, 4]
    assert row_order(rp, col, "minhash").tolist()[-2:] == [1, 4]
    assert row_order(rp, col, "hub").tolist()[-2:] == [1, 4]
    with pytest.raises(ValueError):
        row_order(rp, col, "rabbit")


def test_reference_call_signature():
    rp, col, _ = graphs.uniform_graph(256, 6, seed=1)
    nrp, ncol, rid = apply_tca_reorder(rp.numpy(), col.numpy(), 256, thres=16, verbose=False)
    assert nrp.dtype == np.int32 and ncol.dtype == np.int32 and rid.dtype == np.int32
    assert nrp.shape == (257,) and ncol.shape == col.shape and sorted(rid.tolist()) == list(range(256))
    import tr_tca_reorder
    assert tr_tca_reorder.apply_tca_reorder is apply_tca_reorder


@pytest.mark.gpu
@pytest.mark.parametrize("method", METHODS)
def test_orders_on_the_device_equal_the_cpu_orders_and_feed_the_spmm(method):
    """The same orders computed on CUDA tensors (the benchmark path): identical permutation, and the
    SpMM of the re-ordered matrix equals the row-permuted SpMM of the original (lossless format,
    so that the comparison does not depend on which entries each format drops)."""
    from trspmm import SpmmPlan, build_format
    rp, col, val = graphs.rmat_graph(12, 16, seed=8)
    n = rp.numel() - 1
    rid_cpu = row_order(rp, col, method, n_cols=n)
    rid = row_order(rp.cuda(), col.cuda(), method, n_cols=n)
    assert rid.is_cuda and torch.equal(rid.cpu(), rid_cpu)
    nrp, ncol, nval = permute_rows(rp.cuda(), col.cuda(), val.cuda(), rid)
    B = torch.randn(n, 64, generator=torch.Generator().manual_seed(0)).half().cuda()
    f0, _ = build_format(rp.cuda(), col.cuda(), val.cuda(), strict=True)
    f1, _ = build_format(nrp, ncol, nval, strict=True)
    c0 = SpmmPlan(f0, n, n).run(B, out_dtype=torch.float32)
    c1 = SpmmPlan(f1, n, n).run(B, out_dtype=torch.float32)
    scale = c0.abs().amax(dim=1, keepdim=True).clamp_min(1e-20)
    assert float(((c1 - c0[rid]).abs() / scale[rid]).max()) <= 2e-5
    assert window_column_pairs(nrp, ncol) <= window_column_pairs(rp.cuda(), col.cuda()) or method == "minhash"
