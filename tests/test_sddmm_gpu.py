"""SDDMM parity against the CPU restatement (no reference implementation exists: parity is
pinned only to the definition out[e] = fp16(sum_k X[row,k] * Y[col,k]) with fp32 accumulation).
Tolerance: max relative error 1e-2, mean 1e-3 on the fp16 result."""
import pytest
import torch

from oracle import oracle as O
from trspmm import graphs, sddmm

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K", [64, 128, 8, 24, 7, 200])
@pytest.mark.parametrize("gen", ["uniform", "rmat"])
def test_sddmm_matches_oracle(gen, K):
    if gen == "uniform":
        rp, col, _ = graphs.uniform_graph(1000, 9, seed=1)
    else:
        rp, col, _ = graphs.rmat_graph(11, 12, seed=1)  # hub rows span many warps' entry ranges
    n = rp.numel() - 1
    g = torch.Generator().manual_seed(K)
    X = torch.randn(n, K, generator=g).half()
    Y = torch.randn(n, K, generator=g).half()
    ref = O.sddmm_csr(rp, col, X, Y)
    out = sddmm(rp.cuda(), col.cuda(), X.cuda(), Y.cuda()).cpu()
    mx, mean = O.rel_errors(out, ref)
    assert mx <= 1e-2 and mean <= 1e-3


def test_sddmm_rectangular_and_empty_rows():
    # 300 x 500 pattern with many empty rows
    g = torch.Generator().manual_seed(0)
    rows = torch.randint(0, 300, (2000,), generator=g)
    rows[rows % 7 == 0] = 1
    cols = torch.randint(0, 500, (2000,), generator=g)
    rp, col, _ = graphs.coo_to_csr(rows, cols, 300, 500)
    X = torch.randn(300, 64, generator=g).half()
    Y = torch.randn(500, 64, generator=g).half()
    ref = O.sddmm_csr(rp, col, X, Y)
    out = sddmm(rp.cuda(), col.cuda(), X.cuda(), Y.cuda()).cpu()
    assert O.rel_errors(out, ref)[0] <= 1e-2
    # empty pattern
    rp0 = torch.zeros(301, dtype=torch.int32).cuda()
    out0 = sddmm(rp0, torch.zeros(0, dtype=torch.int32).cuda(), X.cuda(), Y.cuda())
    assert out0.numel() == 0
