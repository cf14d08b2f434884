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


@pytest.mark.parametrize("K", [64, 32, 128, 24])
@pytest.mark.parametrize("gen", ["uniform", "rmat", "clustered"])
def test_planned_sddmm_matches_oracle_and_the_unplanned_entry(gen, K):
    """trs_sddmm_plan_*: tensor-core path for K in {32, 64, 128}, fallback otherwise; every entry
    must be written (the output starts as NaN) and agree with the CPU definition."""
    from trspmm import SddmmPlan
    if gen == "uniform":
        rp, col, _ = graphs.uniform_graph(1000, 9, seed=1)        # 1000 rows: ragged last window
    elif gen == "rmat":
        rp, col, _ = graphs.rmat_graph(11, 12, seed=1)            # hub windows: hundreds of blocks
    else:
        rp, col, _ = graphs.clustered_graph(2048, community=64, intra=12, glob=2, seed=2)
    n = rp.numel() - 1
    g = torch.Generator().manual_seed(K)
    X = torch.randn(n, K, generator=g).half()
    Y = torch.randn(n, K, generator=g).half()
    ref = O.sddmm_csr(rp, col, X, Y)
    plan = SddmmPlan(rp.cuda(), col.cuda(), n)
    assert 0 < plan.n_pairs <= col.numel() and plan.n_blocks * 8 >= plan.n_pairs
    out = torch.full((col.numel(),), float("nan"), dtype=torch.float16, device="cuda")
    plan.run(X.cuda(), Y.cuda(), out=out)
    out = out.cpu()
    assert not torch.isnan(out).any()
    mx, mean = O.rel_errors(out, ref)
    assert mx <= 1e-2 and mean <= 1e-3
    again = plan.run(X.cuda(), Y.cuda()).cpu()
    assert torch.equal(again, out)                                # deterministic
    plain = sddmm(rp.cuda(), col.cuda(), X.cuda(), Y.cuda()).cpu()
    assert O.rel_errors(out, plain.float())[0] <= 1e-2


def test_planned_sddmm_rectangular_empty_rows_and_empty_pattern():
    from trspmm import SddmmPlan
    g = torch.Generator().manual_seed(0)
    rows = torch.randint(0, 300, (2000,), generator=g)
    rows[rows % 7 == 0] = 1
    cols = torch.randint(0, 500, (2000,), generator=g)
    rp, col, _ = graphs.coo_to_csr(rows, cols, 300, 500)
    X = torch.randn(300, 64, generator=g).half()
    Y = torch.randn(500, 64, generator=g).half()
    ref = O.sddmm_csr(rp, col, X, Y)
    plan = SddmmPlan(rp.cuda(), col.cuda(), 500)
    out = torch.full((col.numel(),), float("nan"), dtype=torch.float16, device="cuda")
    plan.run(X.cuda(), Y.cuda(), out=out)
    assert not torch.isnan(out).any()
    assert O.rel_errors(out.cpu(), ref)[0] <= 1e-2
    # the number of pairs is the number of distinct (window, column) keys
    r = torch.repeat_interleave(torch.arange(300), (rp[1:] - rp[:-1]).long())
    assert plan.n_pairs == torch.unique((r // 16) * 500 + col.long()).numel()
    empty = SddmmPlan(torch.zeros(301, dtype=torch.int32).cuda(), torch.zeros(0, dtype=torch.int32).cuda(), 500)
    assert empty.n_blocks == 0 and empty.run(X.cuda(), Y.cuda()).numel() == 0


def test_sddmm_plan_rejects_patterns_it_cannot_address():
    """The plan finds an entry as start + popcount, which needs ascending unique columns per row."""
    from trspmm import SddmmPlan
    from trspmm._lib import TrsError
    rp = torch.tensor([0, 3, 5], dtype=torch.int32).cuda()
    with pytest.raises(TrsError) as e:
        SddmmPlan(rp, torch.tensor([0, 2, 1, 0, 3], dtype=torch.int32).cuda(), 4)      # 2, 1 descending in row 0
    assert e.value.code == -8
    with pytest.raises(TrsError) as e:
        SddmmPlan(rp, torch.tensor([0, 1, 1, 0, 3], dtype=torch.int32).cuda(), 4)      # duplicate column
    assert e.value.code == -8
    with pytest.raises(TrsError) as e:
        SddmmPlan(rp, torch.tensor([0, 1, 2, 0, 4], dtype=torch.int32).cuda(), 4)      # column 4 of 4
    assert e.value.code == -5
    ok = SddmmPlan(rp, torch.tensor([0, 1, 2, 0, 3], dtype=torch.int32).cuda(), 4)
    assert ok.n_pairs == 4   # columns 0, 1, 2, 3 of the single window (column 0 twice)


def test_unplanned_entry_bounds_bad_columns():
    """trs_sddmm does not validate the pattern; an out-of-range column must not become an
    out-of-range gather: that entry comes back as NaN, every other entry is computed as usual."""
    rp, col, _ = graphs.uniform_graph(512, 6, seed=1)
    n = rp.numel() - 1
    g = torch.Generator().manual_seed(0)
    for K in (64, 40):
        X = torch.randn(n, K, generator=g).half().cuda()
        Y = torch.randn(n, K, generator=g).half().cuda()
        good = sddmm(rp.cuda(), col.cuda(), X, Y)
        bad_col = col.clone()
        bad_col[5] = n + 1000
        bad_col[77] = -3
        out = sddmm(rp.cuda(), bad_col.cuda(), X, Y)
        nan = torch.isnan(out)
        assert nan.nonzero().flatten().tolist() == [5, 77]
        assert torch.equal(out[~nan], good[~nan])
