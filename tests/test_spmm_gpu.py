"""GPU parity of the fused SpMM against the CPU oracle, through the C ABI.

Tolerances (north-star contract): fp16 output max relative error <= 1e-2 and mean relative
error <= 1e-3 against the fp32 evaluation of what the format arrays encode; fp32 output within
2e-5 of the row's largest magnitude (fp16 inputs, fp32 accumulation, different summation order).
"""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as O
from trspmm import Format, SpmmPlan, graphs

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden"
CASES = json.loads((GOLD / "cases.json").read_text())

MAX_REL_F16, MEAN_REL_F16 = 1e-2, 1e-3
MAX_ERR_F32 = 2e-5  # max |x - ref| / rowmax |ref|


def _golden(name):
    z = np.load(GOLD / f"{name}.npz")
    arrays = [torch.from_numpy(z[n]) for n in O.FORMAT_NAMES]
    return arrays, int(z["in_rowptr"].shape[0] - 1)


def _check(out_f32, out_f16, ref):
    err = O.scaled_max_error(out_f32.cpu(), ref)
    assert err <= MAX_ERR_F32, f"fp32 output scaled max error {err}"
    mx, mean = O.rel_errors(out_f16.cpu(), ref)
    assert mx <= MAX_REL_F16 and mean <= MEAN_REL_F16, f"fp16 output max rel {mx} mean rel {mean}"


@pytest.mark.parametrize("name", sorted(CASES["small"]))
@pytest.mark.parametrize("F", [32, 64, 128])
def test_spmm_matches_oracle_on_golden_formats(name, F):
    arrays, n = _golden(name)
    torch.manual_seed(1)
    B = torch.randn(n, F).half()
    ref = O.spmm_from_format(arrays, B, n)
    fmt = Format(arrays).to("cuda")
    plan = SpmmPlan(fmt, n, n)
    Bd = B.cuda()
    _check(plan.run(Bd, out_dtype=torch.float32), plan.run(Bd, out_dtype=torch.float16), ref)


@pytest.mark.parametrize("F", [8, 40, 100, 104, 256, 264, 3, 33])
def test_spmm_feature_widths(F):
    arrays, n = _golden("clustered_n512")
    torch.manual_seed(2)
    B = torch.randn(n, F).half()
    ref = O.spmm_from_format(arrays, B, n)
    plan = SpmmPlan(Format(arrays).to("cuda"), n, n)
    _check(plan.run(B.cuda(), out_dtype=torch.float32), plan.run(B.cuda(), out_dtype=torch.float16), ref)


def test_spmm_route_isolation():
    """Each route alone (the other arrays emptied) reproduces that route's share of the product."""
    arrays, n = _golden("rmat_s9_minnnz")
    named = dict(zip(O.FORMAT_NAMES, arrays))
    torch.manual_seed(3)
    B = torch.randn(n, 64).half()
    groups = {
        "tc": ["t_row_offset", "t_block_offset", "t_column", "t_value", "t_window_row", "t_atomic", "t_binary"],
        "csr": ["c_row_offset", "c_row", "c_atomic", "c_column", "c_value",
                "cs_row_offset", "cs_row", "cs_atomic", "cs_column", "cs_value"],
        "sptc": ["s_column", "s_mask", "s_value", "s_pos", "s_window", "s_tile_window", "s_tile_group",
                 "s_tile_column", "s_packed_a", "s_packed_meta"],
    }
    total = torch.zeros(n, 64)
    for keep in groups:
        sub = {}
        for k, v in named.items():
            drop = any(k in g for r, g in groups.items() if r != keep)
            sub[k] = v[:0].clone() if drop else v
        if keep != "sptc":
            sub["s_offset"] = torch.zeros_like(named["s_offset"])
            sub["s_window_tile_offset"] = torch.zeros_like(named["s_window_tile_offset"])
        else:
            sub["s_offset"] = named["s_offset"]
            sub["s_window_tile_offset"] = named["s_window_tile_offset"]
        ref = O.spmm_from_format(sub, B, n)
        got = SpmmPlan(Format(sub).to("cuda"), n, n).run(B.cuda(), out_dtype=torch.float32).cpu()
        mx = O.scaled_max_error(got, ref) if float(ref.abs().max()) > 0 else float(got.abs().max())
        assert mx <= MAX_ERR_F32, (keep, mx)
        total += got
    assert O.scaled_max_error(total, O.spmm_from_format(named, B, n)) <= 2 * MAX_ERR_F32


def test_spmm_split_windows_are_deterministic(monkeypatch):
    """Windows cut into several work items (partial sums + fixed-order reduction) give the same
    bits on every run and the same numbers as the unsplit schedule."""
    rp, col, val = graphs.rmat_graph(11, 16, seed=5)
    n = rp.numel() - 1
    arrays, _ = O.build_format(rp, col, val)
    B = torch.randn(n, 128, generator=torch.Generator().manual_seed(0)).half()
    ref = O.spmm_from_format(arrays, B, n)
    fmt = Format(arrays).to("cuda")
    base = SpmmPlan(fmt, n, n).run(B.cuda(), out_dtype=torch.float32)
    monkeypatch.setenv("TRS_CHUNK_STEPS", "8")
    plan = SpmmPlan(fmt, n, n)
    assert plan.launches >= 2 and plan.workspace_bytes(128) > 0
    a = plan.run(B.cuda(), out_dtype=torch.float32)
    b = plan.run(B.cuda(), out_dtype=torch.float32)
    assert torch.equal(a, b)
    assert O.scaled_max_error(a.cpu(), ref) <= MAX_ERR_F32
    assert O.scaled_max_error(a.cpu(), base.cpu()) <= MAX_ERR_F32
    h = plan.run(B.cuda(), out_dtype=torch.float16)
    mx, mean = O.rel_errors(h.cpu(), ref)
    assert mx <= MAX_REL_F16 and mean <= MEAN_REL_F16


def test_spmm_config0_uniform_vs_torch_sparse():
    """BASELINE config 0: uniform N=4096, F=64.  Checked against the arrays' own meaning (L1) and,
    on rows without dropped entries, against torch.sparse CSR A.B (L2)."""
    rp, col, val = graphs.uniform_graph(4096, 16, 0)
    n = 4096
    arrays, info = O.build_format(rp, col, val)
    B = torch.randn(n, 64, generator=torch.Generator().manual_seed(0)).half()
    plan = SpmmPlan(Format(arrays).to("cuda"), n, n)
    out32 = plan.run(B.cuda(), out_dtype=torch.float32).cpu()
    out16 = plan.run(B.cuda(), out_dtype=torch.float16).cpu()
    l1 = O.spmm_from_format(arrays, B, n)
    _check(out32, out16, l1)
    # rows touched by a dropped entry: mask bit set without a stored slot
    named = dict(zip(O.FORMAT_NAMES, arrays))
    cnt_mask = torch.from_numpy(np.unpackbits(named["s_mask"].numpy()[..., None], axis=-1).sum(-1).astype(np.int64))  # [G,16]
    cnt_slot = (named["s_pos"] >= 0).sum(-1)
    bad_g, bad_r = torch.nonzero(cnt_mask > cnt_slot, as_tuple=True)
    bad_rows = torch.unique(named["s_window"][bad_g].long() * 16 + bad_r)
    assert int((cnt_mask - cnt_slot).sum()) == info["dropped_nnz"]
    good = torch.ones(n, dtype=torch.bool)
    good[bad_rows] = False
    l2 = O.spmm_csr(rp, col, val, B)
    assert O.scaled_max_error(out32[good], l2[good]) <= MAX_ERR_F32
    if len(bad_rows):
        assert O.scaled_max_error(out32[~good], l2[~good]) > MAX_ERR_F32  # the drops are real


def test_spmm_rejects_bad_arrays():
    from trspmm import TrsError
    arrays, n = _golden("clustered_n512")
    named = dict(zip(O.FORMAT_NAMES, arrays))
    bad = dict(named); bad["s_tile_column"] = named["s_tile_column"].clone(); bad["s_tile_column"][0, 0] = n + 5
    with pytest.raises(TrsError) as e:
        SpmmPlan(Format(bad).to("cuda"), n, n)
    assert e.value.code == -5
    bad = dict(named); bad["s_window_tile_offset"] = named["s_window_tile_offset"].clone(); bad["s_window_tile_offset"][3] = 10 ** 6
    with pytest.raises(TrsError) as e:
        SpmmPlan(Format(bad).to("cuda"), n, n)
    assert e.value.code == -3
    bad = dict(named); bad["cs_row"] = named["cs_row"].clone(); bad["cs_row"][-1] = n
    with pytest.raises(TrsError) as e:
        SpmmPlan(Format(bad).to("cuda"), n, n)
    assert e.value.code == -6
    with pytest.raises(TrsError) as e:
        SpmmPlan(Format(named).to("cuda"), n, n, window=17)
    assert e.value.code == -2
    # a TC bitmap that names more values than the block owns would read past t_value
    assert named["t_binary"].numel() > 0
    bad = dict(named); bad["t_binary"] = named["t_binary"].clone(); bad["t_binary"][0] ^= 1
    with pytest.raises(TrsError) as e:
        SpmmPlan(Format(bad).to("cuda"), n, n)
    assert e.value.code == -4
    # array lengths that disagree are refused before anything is handed to the library
    bad = dict(named); bad["t_column"] = named["t_column"][:-8]
    with pytest.raises(ValueError):
        SpmmPlan(Format(bad).to("cuda"), n, n)
    plan = SpmmPlan(Format(named).to("cuda"), n, n)
    short_B = torch.zeros(n - 1, 32, dtype=torch.float16, device="cuda")
    out = torch.empty(n, 32, device="cuda")
    for call in (lambda: plan.run(short_B), lambda: plan.run_static(short_B, out),
                 lambda: plan.run_windows(short_B, out, 0, 1), lambda: plan.run_bcast(short_B, [out.data_ptr()], 0)):
        with pytest.raises(ValueError):
            call()


def test_ragged_last_window_and_empty_rows():
    arrays, n = _golden("uniform_n250_ragged")  # 250 rows: last window has 10
    B = torch.randn(n, 32, generator=torch.Generator().manual_seed(4)).half()
    ref = O.spmm_from_format(arrays, B, n)
    out = SpmmPlan(Format(arrays).to("cuda"), n, n).run(B.cuda(), out_dtype=torch.float32)
    assert out.shape == (250, 32)
    assert O.scaled_max_error(out.cpu(), ref) <= MAX_ERR_F32
    # an all-empty matrix still writes zeros everywhere (C needs no memset)
    rp = torch.zeros(65, dtype=torch.int32)
    empty, _ = O.build_format(rp, torch.zeros(0, dtype=torch.int32), torch.zeros(0))
    plan = SpmmPlan(Format(empty).to("cuda"), 64, 64)
    dst = torch.full((64, 16), 7.0, device="cuda")
    plan.run(torch.randn(64, 16).half().cuda(), out=dst)
    assert float(dst.abs().max()) == 0.0


def _csr_route_format(rp, col, val, keep_sptc_rows=0, part_c=32, short_size=3):
    """Format arrays that carry rows >= keep_sptc_rows entirely on the CUDA-core route, cut the way
    split_cuda_row_online does (block_online.cpp:397-439): parts of part_c entries, a tail of at
    most short_size entries (or a whole row that short) on the short list.  Rows below
    keep_sptc_rows keep the builder's own routing."""
    n = rp.numel() - 1
    head_rp = rp.clone()
    head_rp[keep_sptc_rows + 1:] = rp[keep_sptc_rows]
    e_head = int(rp[keep_sptc_rows])
    arrays, _ = O.build_format(head_rp, col[:e_head], val[:e_head])
    named = dict(zip(O.FORMAT_NAMES, arrays))
    lists = {"c": ([0], [], [], []), "cs": ([0], [], [], [])}
    for k in ("c", "cs"):   # parts the builder already made for the head rows
        off, row = named[f"{k}_row_offset"].tolist(), named[f"{k}_row"].tolist()
        lists[k] = (off if off else [0], row, named[f"{k}_column"].tolist(), named[f"{k}_value"].tolist())
    for r in range(keep_sptc_rows, n):
        e0, e1 = int(rp[r]), int(rp[r + 1])
        while e0 < e1:
            take = min(part_c, e1 - e0)
            k = "cs" if take <= short_size else "c"
            off, row, cc, vv = lists[k]
            row.append(r); cc += col[e0:e0 + take].tolist(); vv += val[e0:e0 + take].tolist()
            off.append(off[-1] + take)
            e0 += take
    for k in ("c", "cs"):
        off, row, cc, vv = lists[k]
        named[f"{k}_row_offset"] = torch.tensor(off if row else [], dtype=torch.int32)
        named[f"{k}_row"] = torch.tensor(row, dtype=torch.int32)
        named[f"{k}_atomic"] = torch.zeros(len(row), dtype=torch.int32)
        named[f"{k}_column"] = torch.tensor(cc, dtype=torch.int32)
        named[f"{k}_value"] = torch.tensor(vv, dtype=torch.float32)
    return [named[k] for k in O.FORMAT_NAMES]


@pytest.mark.parametrize("F", [32, 64, 128, 256, 40, 100])
@pytest.mark.parametrize("chunk,keep", [("256", 0), ("8", 512)])
def test_csr_remainder_dominant(F, chunk, keep, monkeypatch):
    """The CUDA-core remainder (the reference's long and short part kernels, mGCNkernel.cu:976-1042,
    1119-1171) carrying most or all of the matrix: hub rows with hundreds of parts, single-entry short
    parts, and - with 8-step items and the first 512 rows left on the tensor-core routes - the parts
    of split windows spread over the windows' items."""
    monkeypatch.setenv("TRS_CHUNK_STEPS", chunk)
    rp, col, val = graphs.rmat_graph(10, 16, seed=12)
    n = rp.numel() - 1
    arrays = _csr_route_format(rp, col, val, keep_sptc_rows=keep)
    B = torch.randn(n, F, generator=torch.Generator().manual_seed(F)).half()
    ref = O.spmm_from_format(arrays, B, n)
    if keep == 0:   # nothing is dropped on this route: the product is A.B itself
        assert O.scaled_max_error(ref, O.spmm_csr(rp, col, val, B)) <= MAX_ERR_F32
    plan = SpmmPlan(Format(arrays).to("cuda"), n, n)
    a = plan.run(B.cuda(), out_dtype=torch.float32)
    assert torch.equal(a, plan.run(B.cuda(), out_dtype=torch.float32))
    _check(a, plan.run(B.cuda(), out_dtype=torch.float16), ref)
    r = plan.run(B.cuda(), out_dtype=torch.float32, relu=True)
    assert O.scaled_max_error(r.cpu(), torch.relu(ref)) <= MAX_ERR_F32


@pytest.mark.parametrize("name", ["clustered_n512", "rmat_s9_minnnz", "uniform_n250_ragged"])
def test_runs_are_bit_identical_and_relu_epilogue(name):
    arrays, n = _golden(name)
    B = torch.randn(n, 64, generator=torch.Generator().manual_seed(11)).half()
    ref = O.spmm_from_format(arrays, B, n)
    plan = SpmmPlan(Format(arrays).to("cuda"), n, n)
    a = plan.run(B.cuda(), out_dtype=torch.float32)
    b = plan.run(B.cuda(), out_dtype=torch.float32)
    assert torch.equal(a, b)
    _check(a, plan.run(B.cuda(), out_dtype=torch.float16), ref)
    r = plan.run(B.cuda(), out_dtype=torch.float32, relu=True)
    assert O.scaled_max_error(r.cpu(), torch.relu(ref)) <= MAX_ERR_F32
    assert plan.status() == 0


def test_rectangular_matrix_and_wide_features():
    """m_rows != k_cols (the reference passes mOri and kOri separately, mGCN_online.cpp:760-800) and
    a feature width above one slab (F = 384: three slabs of 128)."""
    g = torch.Generator().manual_seed(2)
    m, k = 1000, 5000
    rows = torch.randint(0, m, (30000,), generator=g)
    cols = torch.randint(0, k, (30000,), generator=g)
    cols[:20000] = cols[:20000] % 24        # some dense columns -> TC blocks
    rp, col, _ = graphs.coo_to_csr(rows, cols, m, k)
    val = torch.randn(col.numel(), generator=g)
    arrays, _ = O.build_format(rp, col, val)
    assert arrays[2].numel() > 0, "the case should contain TC blocks"
    for F in (64, 384):
        B = torch.randn(k, F, generator=g).half()
        ref = O.spmm_from_format(arrays, B, m)
        plan = SpmmPlan(Format(arrays).to("cuda"), m, k)
        _check(plan.run(B.cuda(), out_dtype=torch.float32), plan.run(B.cuda(), out_dtype=torch.float16), ref)
    from trspmm import TrsError
    with pytest.raises(TrsError) as e:       # a column id beyond kOri is caught before any launch
        SpmmPlan(Format(arrays).to("cuda"), m, k - 4000)
    assert e.value.code == -5


def test_unaligned_feature_pointer_falls_back():
    """B whose first row does not start on a 16-byte boundary takes the generic (plain load) path."""
    arrays, n = _golden("rmat_s9")
    base = torch.randn(n * 64 + 8, generator=torch.Generator().manual_seed(9)).half().cuda()
    B = base[4:4 + n * 64].view(n, 64)      # 8-byte offset
    assert B.data_ptr() % 16 == 8
    ref = O.spmm_from_format(arrays, B.cpu(), n)
    plan = SpmmPlan(Format(arrays).to("cuda"), n, n)
    lib = plan.lib
    from trspmm import _lib
    out = torch.empty(n, 64, device="cuda")
    ws = torch.empty(max(plan.workspace_bytes(64), 16), dtype=torch.uint8, device="cuda")
    _lib.check(lib.trs_spmm_run(plan._handle, B.data_ptr(), out.data_ptr(), 64, 0, ws.data_ptr(), ws.numel(),
                                _lib.current_stream_ptr(out.device)))
    assert O.scaled_max_error(out.cpu(), ref) <= MAX_ERR_F32


def test_bcast_epilogue_single_gpu():
    """trs_spmm_run_bcast with two destination buffers on one GPU: both receive the fp16 rows (with
    ReLU) at the requested row offset, identical to the ordinary entry; rows outside stay untouched."""
    arrays, n = _golden("clustered_n512")
    B = torch.randn(n, 128, generator=torch.Generator().manual_seed(3)).half().cuda()
    plan = SpmmPlan(Format(arrays).to("cuda"), n, n)
    want = plan.run(B, out_dtype=torch.float16, relu=True)
    row0, total = 48, n + 100
    bufs = [torch.full((total, 128), -7.0, dtype=torch.float16, device="cuda") for _ in range(2)]
    plan.run_bcast(B, [b.data_ptr() for b in bufs], row0, relu=True)
    torch.cuda.synchronize()
    for b in bufs:
        assert torch.equal(b[row0:row0 + n], want)
        assert float(b[:row0].max()) == -7.0 and float(b[row0 + n:].min()) == -7.0


def test_window_range_runs_cover_the_full_run(monkeypatch):
    """trs_spmm_run_windows: disjoint window ranges write exactly their own rows and together
    reproduce the full run bit for bit, also when windows are split into several work items."""
    monkeypatch.setenv("TRS_CHUNK_STEPS", "8")  # many split windows -> the partial-sum path is cut too
    rp, col, val = graphs.rmat_graph(11, 16, seed=9)
    n = rp.numel() - 1
    arrays, _ = O.build_format(rp, col, val)
    B = torch.randn(n, 128, generator=torch.Generator().manual_seed(4)).half().cuda()
    plan = SpmmPlan(Format(arrays).to("cuda"), n, n)
    assert plan.launches >= 2
    W = plan.num_windows
    assert W == (n + 15) // 16
    for dtype in (torch.float32, torch.float16):
        want = plan.run(B, out_dtype=dtype)
        out = torch.full((n, 128), -3.0, dtype=dtype, device="cuda")
        cuts = [0, 1, W // 3, W // 3, W - 5, W]
        for w0, w1 in zip(cuts[:-1], cuts[1:]):
            before = out.clone()
            plan.run_windows(B, out, w0, w1)
            torch.cuda.synchronize()
            changed = (out != before).any(dim=1).nonzero().flatten()
            if changed.numel():
                assert int(changed.min()) >= w0 * 16 and int(changed.max()) < w1 * 16
        assert torch.equal(out, want)
    from trspmm._lib import TrsError
    with pytest.raises(TrsError):
        plan.run_windows(B, out, 5, W + 1)
    with pytest.raises(TrsError):
        plan.run_windows(B, out, 7, 3)


def test_resident_submit_wait_matches_blocking_calls(monkeypatch):
    """A stream of trs_resident_submit calls (two device slots, three streams, output copied back
    in window chunks) returns, for every call, the bits of the blocking trs_resident_forward."""
    from trspmm import ResidentSpmm
    monkeypatch.setenv("TRS_RESIDENT_CHUNKS", "5")
    arrays, n = _golden("rmat_s9_minnnz")
    fmt = Format(arrays)
    res = ResidentSpmm(fmt, n, n, 16, 128)
    g = torch.Generator().manual_seed(8)
    Bs = [torch.randn(n, F, generator=g).half().pin_memory() for F in (128, 64, 128, 128, 32, 128)]
    want = []
    for b in Bs:
        out = torch.empty((n, b.shape[1]), dtype=torch.float32).pin_memory()
        res.forward(b, out)
        want.append(out.clone())
        assert O.scaled_max_error(out, O.spmm_from_format(arrays, b, n)) <= MAX_ERR_F32
    for dtype in (torch.float32, torch.float16):
        outs = [torch.full((n, b.shape[1]), float("nan"), dtype=dtype).pin_memory() for b in Bs]
        for b, o in zip(Bs, outs):
            res.submit(b, o)
        res.wait()
        for o, w in zip(outs, want):
            assert torch.equal(o, w.to(dtype))
    res.close()
