"""The allocation-free SpMM entry (trs_spmm_run_static) against the ordinary one.

Some callers of this library cannot allocate device memory, nor pass any in: a host program
that gave the whole GPU to its own pool when it started, or a serving loop in which a cudaMalloc
would stall every stream.  For them the library keeps the partial sums of split windows in a
fixed device array of its own.  This test drives that entry through the C ABI on a plan that
really needs scratch, twice in a row, and compares with trs_spmm_run; it also checks that a plan
too large for the fixed array is refused before anything is launched.

Collected last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import pytest
import torch

from oracle import oracle as O
from trspmm import Format, SpmmPlan, TrsError, graphs

pytestmark = pytest.mark.gpu

MAX_ERR_F32 = 2e-5  # max |x - ref| / rowmax |ref|, the fp32 tolerance of the other SpMM tests


def _plan(monkeypatch, scale, chunk):
    rp, col, val = graphs.rmat_graph(scale, 16, seed=21)
    n = rp.numel() - 1
    arrays, _ = O.build_format(rp, col, val)
    monkeypatch.setenv("TRS_CHUNK_STEPS", str(chunk))  # small chunks: many windows are split
    return SpmmPlan(Format(arrays).to("cuda"), n, n), n


def test_static_scratch_entry_matches_ordinary_entry(monkeypatch):
    plan, n = _plan(monkeypatch, 11, 16)
    F = 128
    need = plan.static_scratch_bytes(F)
    assert 0 < need <= 8 << 20, "the case must use scratch and fit the fixed array"
    g = torch.Generator().manual_seed(5)
    for call in range(2):  # two calls in a row share the array; the second must not see the first
        B = torch.randn(n, F, generator=g).half().cuda()
        want = plan.run(B, out_dtype=torch.float32)
        got = plan.run_static(B, torch.full((n, F), float("nan"), device="cuda"))
        assert O.scaled_max_error(got.cpu(), want.cpu()) <= MAX_ERR_F32, f"call {call}"
        want16 = plan.run(B, out_dtype=torch.float16)
        got16 = plan.run_static(B, torch.zeros((n, F), dtype=torch.float16, device="cuda"))
        mx, mean = O.rel_errors(got16.cpu(), want16.cpu())
        assert mx <= 1e-2 and mean <= 1e-3, f"call {call}"
    assert plan.status() == 0


def test_static_scratch_entry_refuses_oversized_plans(monkeypatch):
    plan, n = _plan(monkeypatch, 13, 8)
    F = 256
    assert plan.static_scratch_bytes(F) > 8 << 20
    B = torch.randn(n, F).half().cuda()
    out = torch.full((n, F), 3.0, device="cuda")
    with pytest.raises(TrsError) as e:
        plan.run_static(B, out)
    assert e.value.code == -10
    assert float(out.min()) == 3.0 and float(out.max()) == 3.0  # nothing was launched
