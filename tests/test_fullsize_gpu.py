"""Full benchmark sizes (R-MAT scale 21, 125 M nnz; clustered N = 262 144), checked through
properties that do not need the CPU oracle to finish: entry conservation of the builder,
agreement of the lossless format's SpMM with a CSR SpMM of the same matrix (torch.sparse on the
GPU is the checker here, never the product), linearity, and run-to-run bit identity."""
import pytest
import torch

from trspmm import SpmmPlan, build_format, graphs, sddmm

pytestmark = pytest.mark.gpu


def _rel(x, ref):
    scale = ref.abs().amax(dim=1, keepdim=True).clamp_min(1e-20)
    return float(((x - ref).abs() / scale).max())


@pytest.mark.parametrize("workload", ["rmat21", "clustered"])
def test_full_size_properties(workload):
    dev = torch.device("cuda")
    if workload == "rmat21":
        rp, col, val = graphs.rmat_graph(21, 32, seed=0, device=dev)
    else:
        rp, col, val = graphs.clustered_graph(262144, 128, 24, 4, seed=0, device=dev)
    n, nnz, F = rp.numel() - 1, col.numel(), 128
    g = torch.Generator(device=dev).manual_seed(7)
    B1 = torch.randn(n, F, device=dev, generator=g).half()
    B2 = torch.randn(n, F, device=dev, generator=g).half()

    # --- reference-compatible format: every entry is routed exactly once or counted as dropped
    fmt, st = build_format(rp, col, val)
    stored = fmt.t_value.numel() + fmt.c_value.numel() + fmt.cs_value.numel() + int((fmt.s_pos >= 0).sum())
    assert stored + st["dropped_nnz"] == nnz
    assert int(fmt.s_mask.to(torch.int32).bitwise_and(1).sum() + (fmt.s_mask.to(torch.int32) >> 1).bitwise_and(1).sum()
               + (fmt.s_mask.to(torch.int32) >> 2).bitwise_and(1).sum() + (fmt.s_mask.to(torch.int32) >> 3).bitwise_and(1).sum()) \
        == int((fmt.s_pos >= 0).sum()) + st["dropped_nnz"]
    off = fmt.s_window_tile_offset
    assert int(off[0]) == 0 and bool((off[1:] >= off[:-1]).all()) and int(off[-1]) == fmt.tiles
    plan = SpmmPlan(fmt, n, n)
    a = plan.run(B1, out_dtype=torch.float32)
    b = plan.run(B1, out_dtype=torch.float32)
    assert torch.equal(a, b), "results must be bit-identical from run to run"
    # linearity: A'(B1 + B2) = A'B1 + A'B2 up to the fp16 rounding of B1 + B2
    Bs = (B1.float() + B2.float()).half()
    lhs = plan.run(Bs, out_dtype=torch.float32)
    rhs = a + plan.run(B2, out_dtype=torch.float32)
    assert _rel(lhs, rhs) <= 5e-3
    assert plan.status() == 0
    del plan, fmt, lhs, rhs, b

    # --- lossless format: equals a CSR SpMM of the same matrix everywhere
    fmt, st = build_format(rp, col, val, strict=True)
    assert st["dropped_nnz"] == 0
    out = SpmmPlan(fmt, n, n).run(B1, out_dtype=torch.float32)
    A = torch.sparse_csr_tensor(rp.long(), col.long(), val.half().float(), (n, n))
    ref = torch.sparse.mm(A, B1.float())
    assert _rel(out, ref) <= 2e-5
    # and the compatible result differs from it only on rows that lost an entry
    diff_rows = ((a - ref).abs().amax(dim=1) > 1e-4 * ref.abs().amax(dim=1).clamp_min(1e-20)).sum()
    assert 0 < int(diff_rows) < n


@pytest.mark.parametrize("workload", ["clustered", "rmat20"])
def test_planned_sddmm_full_size(workload):
    """The planned tensor-core SDDMM at bench sizes: every entry written, all entries equal to the
    entry-parallel kernel's within fp16 rounding, and 2 M sampled entries equal to fp32 dot products."""
    from trspmm import SddmmPlan
    dev = torch.device("cuda")
    if workload == "clustered":
        rp, col, _ = graphs.clustered_graph(262144, 128, 24, 4, seed=0, device=dev)
    else:
        rp, col, _ = graphs.rmat_graph(20, 16, seed=0, device=dev)
    n, K = rp.numel() - 1, 64
    g = torch.Generator(device=dev).manual_seed(3)
    X = torch.randn(n, K, device=dev, generator=g).half()
    Y = torch.randn(n, K, device=dev, generator=g).half()
    plan = SddmmPlan(rp, col, n)
    out = torch.full((col.numel(),), float("nan"), dtype=torch.float16, device=dev)
    plan.run(X, Y, out=out)
    assert not bool(torch.isnan(out).any())
    plain = sddmm(rp, col, X, Y)
    scale = float(plain.float().abs().max())
    assert float((out.float() - plain.float()).abs().max()) <= 4e-3 * scale
    rows = torch.repeat_interleave(torch.arange(n, device=dev), (rp[1:] - rp[:-1]).long())
    pick = torch.randint(0, col.numel(), (2_000_000,), device=dev, generator=g)
    ref = (X[rows[pick]].float() * Y[col[pick].long()].float()).sum(-1)
    err = (out[pick].float() - ref).abs() / ref.abs().clamp_min(1e-2 * float(ref.abs().max()))
    assert float(err.max()) <= 1e-2 and float(err.mean()) <= 1e-3
    assert torch.equal(plan.run(X, Y), out)


def test_sddmm_full_size_against_row_samples():
    dev = torch.device("cuda")
    rp, col, _ = graphs.clustered_graph(262144, 128, 24, 4, seed=0, device=dev)
    n, K = rp.numel() - 1, 64
    g = torch.Generator(device=dev).manual_seed(3)
    X = torch.randn(n, K, device=dev, generator=g).half()
    Y = torch.randn(n, K, device=dev, generator=g).half()
    out = sddmm(rp, col, X, Y)
    rows = torch.repeat_interleave(torch.arange(n, device=dev), (rp[1:] - rp[:-1]).long())
    pick = torch.randint(0, col.numel(), (2_000_000,), device=dev, generator=g)
    ref = (X[rows[pick]].float() * Y[col[pick].long()].float()).sum(-1)
    err = (out[pick].float() - ref).abs() / ref.abs().clamp_min(1e-2 * float(ref.abs().max()))
    assert float(err.max()) <= 1e-2 and float(err.mean()) <= 1e-3
