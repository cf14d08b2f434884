"""GPU format builder: every one of the 29 arrays bit-exact against fixtures produced by the
reference's compiled builder, against the pinned CPU restatement on larger seeded graphs, and
through the Libra5BlockOnline drop-in module."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as O
from trspmm import build_format, graphs

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden"
CASES = json.loads((GOLD / "cases.json").read_text())


def _same(fmt, want, names=O.FORMAT_NAMES):
    for n, a, b in zip(names, fmt.arrays(), want):
        a = a.cpu()
        assert a.dtype == b.dtype, (n, a.dtype, b.dtype)
        assert a.shape == b.shape, (n, a.shape, b.shape)
        assert torch.equal(a, b), n


@pytest.mark.parametrize("name", sorted(CASES["small"]))
def test_builder_matches_reference_fixtures(name, env_ctx):
    gen, gkw, bkw, env = CASES["small"][name]
    z = np.load(GOLD / f"{name}.npz")
    rp, col, val = (torch.from_numpy(z[k]).cuda() for k in ("in_rowptr", "in_col", "in_val"))
    with env_ctx(env):
        fmt, info = build_format(rp, col, val, **bkw)
    _same(fmt, [torch.from_numpy(z[n]) for n in O.FORMAT_NAMES])
    assert info["nnz"] == col.numel()


@pytest.mark.parametrize("name", sorted(CASES["digest"]))
def test_builder_matches_reference_digests(name, env_ctx):
    gen, gkw, bkw, env = CASES["digest"][name]
    want = json.loads((GOLD / "digests.json").read_text())[name]
    rp, col, val = getattr(graphs, gen)(**gkw)
    with env_ctx(env):
        fmt, _ = build_format(rp.cuda(), col.cuda(), val.cuda(), **bkw)
    for n, a in zip(O.FORMAT_NAMES, fmt.arrays()):
        a = a.cpu().contiguous()
        assert list(a.shape) == want["shapes"][n], n
        assert hashlib.sha256(a.numpy().tobytes()).hexdigest() == want["sha256"][n], n


@pytest.mark.parametrize("case", [
    ("rmat", dict(scale=15, edge_factor=16, seed=3), {}),
    ("rmat", dict(scale=13, edge_factor=32, seed=4), dict(density=4, part_t=3, part_c=1, short_size=0)),
    ("clustered", dict(n=16384, community=128, intra=24, glob=4, seed=1), {}),
    ("clustered", dict(n=4099, community=64, intra=20, glob=2, seed=2), dict(tc_min_util=0.7, density=6)),
    ("uniform", dict(n=20000, per_row=5, seed=5), dict(window=16)),
    ("uniform", dict(n=3000, per_row=7, seed=6), dict(window=8, density=4)),
    ("uniform", dict(n=1000, per_row=3, seed=7), dict(window=5, density=2)),
])
def test_builder_matches_restatement(case):
    kind, gkw, bkw = case
    rp, col, val = getattr(graphs, kind + "_graph")(**gkw)
    want, info = O.build_format(rp, col, val, **bkw)
    fmt, stats = build_format(rp.cuda(), col.cuda(), val.cuda(), **bkw)
    _same(fmt, want)
    assert stats["dropped_nnz"] == info["dropped_nnz"]


def test_builder_hub_window():
    """A window whose rows touch tens of thousands of distinct columns (the shape of a power-law
    hub): exercises the long single-window sort / matching path."""
    g = torch.Generator().manual_seed(0)
    n = 60000
    hub_rows = torch.arange(16).repeat_interleave(9000)
    hub_cols = torch.randint(0, n, (16 * 9000,), generator=g)
    rows = torch.cat([hub_rows, torch.arange(n), torch.randint(0, n, (5 * n,), generator=g)])
    cols = torch.cat([hub_cols, torch.arange(n), torch.randint(0, n, (5 * n,), generator=g)])
    rp, col, _ = graphs.coo_to_csr(rows, cols, n, n)
    val = torch.randn(col.numel(), generator=g)
    want, _ = O.build_format(rp, col, val)
    fmt, _ = build_format(rp.cuda(), col.cuda(), val.cuda())
    _same(fmt, want)


def test_builder_edge_cases():
    from trspmm import TrsError
    # empty matrix
    rp = torch.zeros(33, dtype=torch.int32)
    want, _ = O.build_format(rp, torch.zeros(0, dtype=torch.int32), torch.zeros(0))
    fmt, _ = build_format(rp.cuda(), torch.zeros(0, dtype=torch.int32).cuda(), torch.zeros(0).cuda())
    _same(fmt, want)
    # single entry, single row
    rp = torch.tensor([0, 1], dtype=torch.int32)
    col = torch.tensor([0], dtype=torch.int32)
    val = torch.tensor([2.5])
    want, _ = O.build_format(rp, col, val)
    fmt, _ = build_format(rp.cuda(), col.cuda(), val.cuda())
    _same(fmt, want)
    # non-canonical input is refused, not silently mis-built
    rp = torch.tensor([0, 2], dtype=torch.int32)
    with pytest.raises(TrsError) as e:
        build_format(rp.cuda(), torch.tensor([3, 1], dtype=torch.int32).cuda(), torch.ones(2).cuda())
    assert e.value.code == -8
    with pytest.raises(TrsError) as e:
        build_format(torch.tensor([0, 2, 1], dtype=torch.int32).cuda(), torch.tensor([0, 1], dtype=torch.int32).cuda(),
                     torch.ones(2).cuda())
    assert e.value.code == -3
    with pytest.raises(TrsError) as e:
        build_format(rp.cuda(), torch.tensor([0, 1], dtype=torch.int32).cuda(), torch.ones(2).cuda(), window=17)
    assert e.value.code == -2


def test_dropin_module_signature_and_values():
    import Libra5BlockOnline
    rp, col, val = graphs.clustered_graph(512, 64, 12, 2, 0)
    out = Libra5BlockOnline.block_sptc_2to4_online(rp, col, val, 32, 32, 3, 8, 16, 16, 0.0, 0.5, 12)
    assert len(out) == 30 and out[29].dim() == 0 and out[29].dtype == torch.float32
    assert all(not t.is_cuda for t in out)
    z = np.load(GOLD / "clustered_n512.npz")
    for n, a in zip(O.FORMAT_NAMES, out):
        assert torch.equal(a, torch.from_numpy(z[n])), n
    with pytest.raises(RuntimeError):
        Libra5BlockOnline.block_sptc_2to4_online(rp.long(), col, val, 32, 32, 3, 8, 16, 16, 0.0, 0.5, 12)
    with pytest.raises(RuntimeError):
        Libra5BlockOnline.block_sptc_2to4_online(rp, col, val, 32, 32, 3, 8, 33, 16, 0.0, 0.5, 12)


def test_built_format_feeds_spmm():
    """builder -> plan -> SpMM entirely on the device, checked against torch.sparse on the rows
    without dropped entries and against the format's own meaning everywhere."""
    from trspmm import SpmmPlan
    rp, col, val = graphs.rmat_graph(12, 16, seed=9)
    n = rp.numel() - 1
    fmt, stats = build_format(rp.cuda(), col.cuda(), val.cuda())
    B = torch.randn(n, 128, generator=torch.Generator().manual_seed(1)).half()
    plan = SpmmPlan(fmt, n, n)
    out = plan.run(B.cuda(), out_dtype=torch.float32).cpu()
    assert plan.status() == 0
    ref = O.spmm_from_format([a.cpu() for a in fmt.arrays()], B, n)
    assert O.scaled_max_error(out, ref) <= 2e-5


def test_builder_many_heavy_windows():
    """Several windows above the block-cooperative threshold (> 4096 units each) with different tie
    structures, next to light windows: the cooperative partition path must reproduce std::sort's
    order exactly like the single-thread path does."""
    g = torch.Generator().manual_seed(5)
    n = 40000
    rows, cols = [], []
    for win, (deg, lo) in enumerate([(3000, 0), (1200, 5000), (700, 100), (5000, 20000)]):
        for r in range(16):
            k = deg if r % 3 else deg // 2
            rows.append(torch.full((k,), win * 64 + r))
            cols.append(torch.randint(lo, n, (k,), generator=g))
    rows.append(torch.randint(0, n, (3 * n,), generator=g)); cols.append(torch.randint(0, n, (3 * n,), generator=g))
    rp, col, _ = graphs.coo_to_csr(torch.cat(rows), torch.cat(cols), n, n)
    val = torch.randn(col.numel(), generator=g)
    want, _ = O.build_format(rp, col, val)
    fmt, _ = build_format(rp.cuda(), col.cuda(), val.cuda())
    _same(fmt, want)


@pytest.mark.parametrize("case", [("rmat", dict(scale=12, edge_factor=16, seed=2)),
                                  ("clustered", dict(n=2048, community=128, intra=24, glob=4, seed=3))])
def test_strict_mode_is_lossless(case):
    """strict=True: the TC and SPTC arrays stay as the reference builds them, and every entry the
    reference drops re-appears in the row's CUDA-core part, so that the format encodes A exactly and
    the SpMM equals torch.sparse A.B on every row."""
    from trspmm import SpmmPlan
    kind, gkw = case
    rp, col, val = getattr(graphs, kind + "_graph")(**gkw)
    n = rp.numel() - 1
    compat, cst = build_format(rp.cuda(), col.cuda(), val.cuda())
    strict, sst = build_format(rp.cuda(), col.cuda(), val.cuda(), strict=True)
    assert cst["dropped_nnz"] > 0 and sst["dropped_nnz"] == 0
    for name in ("t_column", "t_value", "t_binary", "s_column", "s_mask", "s_value", "s_pos", "s_packed_a",
                 "s_packed_meta", "s_tile_column", "s_offset"):
        assert torch.equal(getattr(compat, name), getattr(strict, name)), name
    extra = (strict.c_value.numel() + strict.cs_value.numel()) - (compat.c_value.numel() + compat.cs_value.numel())
    assert extra == cst["dropped_nnz"]
    # decoding gives back exactly A
    r, c, v = O.decode_format([a.cpu() for a in strict.arrays()])
    rows = torch.repeat_interleave(torch.arange(n), (rp[1:] - rp[:-1]).long()).numpy()
    full = {(int(a), int(b)): float(x) for a, b, x in zip(rows, col.numpy(), val.numpy())}
    got = {(int(a), int(b)): float(x) for a, b, x in zip(r, c, v)}
    assert got == full and len(r) == len(full)
    # CSR parts keep ascending columns inside a row part
    off, cc = strict.c_row_offset.cpu(), strict.c_column.cpu()
    for p in range(min(off.numel() - 1, 200)):
        seg = cc[off[p]:off[p + 1]]
        assert bool((seg[1:] > seg[:-1]).all())
    B = torch.randn(n, 64, generator=torch.Generator().manual_seed(0)).half()
    out = SpmmPlan(strict, n, n).run(B.cuda(), out_dtype=torch.float32).cpu()
    assert O.scaled_max_error(out, O.spmm_csr(rp, col, val, B)) <= 2e-5


def test_builder_with_caller_owned_arena():
    """trs_build_query / trs_build_fill: the same 29 arrays with every device byte cut out of a
    caller-provided arena (no cudaMalloc inside the call); a short arena is refused cleanly and a
    second build reuses the same memory."""
    from trspmm import TrsError
    from trspmm.builder import arena_bytes
    for strict in (False, True):
        rp, col, val = graphs.rmat_graph(13, 16, seed=21)
        want, stats0 = build_format(rp.cuda(), col.cuda(), val.cuda(), strict=strict)
        need = arena_bytes(rp.numel() - 1, col.numel(), strict=strict)
        arena = torch.empty(need + 300, dtype=torch.uint8, device="cuda")[7:]   # deliberately unaligned start
        for _ in range(2):
            fmt, stats = build_format(rp.cuda(), col.cuda(), val.cuda(), strict=strict, arena=arena)
            for n, a, b in zip(O.FORMAT_NAMES, fmt.arrays(), want.arrays()):
                assert a.dtype == b.dtype and a.shape == b.shape and torch.equal(a, b), n
                if a.numel():
                    assert arena.data_ptr() <= a.data_ptr() < arena.data_ptr() + arena.numel(), n
            assert 0 < stats["arena_used"] <= need
            assert stats["dropped_nnz"] == stats0["dropped_nnz"]
        small = torch.empty(max(stats["arena_used"] // 3, 4096), dtype=torch.uint8, device="cuda")
        with pytest.raises(TrsError) as e:
            build_format(rp.cuda(), col.cuda(), val.cuda(), strict=strict, arena=small)
        assert e.value.code == -7
    # the empty matrix and the single entry still work
    rp = torch.zeros(33, dtype=torch.int32)
    arena = torch.empty(arena_bytes(32, 0), dtype=torch.uint8, device="cuda")
    fmt, _ = build_format(rp.cuda(), torch.zeros(0, dtype=torch.int32).cuda(), torch.zeros(0).cuda(), arena=arena)
    want, _ = O.build_format(rp, torch.zeros(0, dtype=torch.int32), torch.zeros(0))
    _same(fmt, want)
