"""The CPU restatement (oracle/) against the reference's own outputs.

Fixtures in tests/golden/ were produced by the reference's compiled builder
(tests/golden/make_golden.py); when oracle/_ref exists the compiled reference is also
run live on fresh seeds.
"""
import hashlib
import json

import numpy as np
import pytest
import torch

from oracle import oracle as O
from trspmm import graphs

CASES = json.loads((__import__("pathlib").Path(__file__).parent / "golden" / "cases.json").read_text())


def _digest(t):
    return hashlib.sha256(t.contiguous().numpy().tobytes()).hexdigest()


@pytest.mark.parametrize("name", sorted(CASES["small"]))
def test_restatement_matches_golden_arrays(name, golden_dir, env_ctx):
    gen, gkw, bkw, env = CASES["small"][name]
    z = np.load(golden_dir / f"{name}.npz")
    rp, col, val = (torch.from_numpy(z[k]) for k in ("in_rowptr", "in_col", "in_val"))
    # the generators are part of the fixture contract: same seed -> same CSR
    g_rp, g_col, g_val = getattr(graphs, gen)(**gkw)
    assert torch.equal(g_rp, rp) and torch.equal(g_col, col) and torch.equal(g_val, val)
    with env_ctx(env):
        mine, info = O.build_format(rp, col, val, **bkw)
    assert info["check_failures"] == 0
    for n, a in zip(O.FORMAT_NAMES, mine):
        want = torch.from_numpy(z[n])
        assert a.shape == want.shape, n
        assert torch.equal(a, want), n


@pytest.mark.parametrize("name", sorted(CASES["digest"]))
def test_restatement_matches_golden_digests(name, golden_dir, env_ctx):
    gen, gkw, bkw, env = CASES["digest"][name]
    want = json.loads((golden_dir / "digests.json").read_text())[name]
    rp, col, val = getattr(graphs, gen)(**gkw)
    assert _digest(rp) == want["input"]["rowptr"] and _digest(col) == want["input"]["col"]
    assert _digest(val) == want["input"]["val"]
    with env_ctx(env):
        mine, _ = O.build_format(rp, col, val, **bkw)
    for n, a in zip(O.FORMAT_NAMES, mine):
        assert list(a.shape) == want["shapes"][n], n
        assert _digest(a) == want["sha256"][n], n


def test_exhaustive_graph_is_complete(golden_dir):
    """Re-evaluates the O(1) compatibility check on every unit pair: it never fails, so the
    shortcut (complete graph, degree = U-1) is exact."""
    z = np.load(golden_dir / "clustered_n512.npz")
    rp, col, val = (torch.from_numpy(z[k]) for k in ("in_rowptr", "in_col", "in_val"))
    fast, _ = O.build_format(rp, col, val)
    slow, info = O.build_format(rp, col, val, exhaustive=True)
    assert info["check_failures"] == 0
    for a, b in zip(fast, slow):
        assert torch.equal(a, b)


@pytest.mark.parametrize("seed", [11, 12])
def test_restatement_matches_live_reference(seed):
    if O.reference_module() is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rp, col, val = graphs.rmat_graph(10, 12, seed=seed)
    ref = O.reference_builder(rp, col, val, density=6)
    mine, _ = O.build_format(rp, col, val, density=6)
    for n, a, b in zip(O.FORMAT_NAMES, ref, mine):
        assert a.shape == b.shape and torch.equal(a, b), n


@pytest.mark.parametrize("name", ["clustered_n512", "rmat_s9_minnnz", "uniform_n250_ragged"])
def test_decode_reproduces_matrix_minus_drops(name, golden_dir):
    """Decoding TC + CSR parts + SPTC slots gives back A except exactly the entries the
    reference drops (more than two non-zeros of one row inside one 4-column group)."""
    z = np.load(golden_dir / f"{name}.npz")
    rp, col, val = (torch.from_numpy(z[k]) for k in ("in_rowptr", "in_col", "in_val"))
    arrays = {n: torch.from_numpy(z[n]) for n in O.FORMAT_NAMES}
    window = 16
    r, c, v = O.decode_format(arrays, window)
    n = rp.numel() - 1
    rows = torch.repeat_interleave(torch.arange(n), (rp[1:] - rp[:-1]).long()).numpy()
    full = {(int(a), int(b)): float(x) for a, b, x in zip(rows, col.numpy(), val.numpy())}
    got = {(int(a), int(b)): float(x) for a, b, x in zip(r, c, v)}
    assert len(got) == len(r), "an entry was routed twice"
    assert set(got) <= set(full)
    assert all(full[k] == x for k, x in got.items())
    # dropped = mask bits set without a slot
    mask = arrays["s_mask"].numpy()
    pos = arrays["s_pos"].numpy()
    dropped = int(np.unpackbits(mask[..., None], axis=-1).sum() - (pos >= 0).sum())
    assert len(full) - len(got) == dropped
    # the packed tiles encode the same SPTC entries (fp16-rounded values)
    r2, c2, v2 = O.decode_format(arrays, window, use_packed=True)
    got2 = {(int(a), int(b)): float(x) for a, b, x in zip(r2, c2, v2)}
    nz = {k: x for k, x in got.items() if np.float16(x) != 0}
    assert set(got2) == set(nz)
    assert all(np.float16(full[k]) == np.float16(x) for k, x in got2.items())


def test_f16_rounding_matches_torch():
    xs = torch.cat([torch.randn(4096) * 10.0 ** torch.randint(-9, 6, (4096,)),
                    torch.tensor([0.0, -0.0, 65504.0, 65519.9, 65520.0, 1e-8, 5.96e-8, 2.98e-8, 6.1e-5])])
    want = xs.half().view(torch.int16).numpy().astype(np.uint16)
    got = np.array([O.f32_to_f16_bits(float(x)) for x in xs], dtype=np.uint16)
    assert (want == got).all()
