"""The reference-facing modules (same names and positional signatures as the reference's torch
extensions), called the way spmm/tr_csr_fp16/test_tr_csr_online.py:83-181 calls them."""
import numpy as np
import pytest
import torch

from oracle import oracle as O

GOLD = __import__("pathlib").Path(__file__).parent / "golden"


def _inputs(name="clustered_n512", F=64):
    z = np.load(GOLD / f"{name}.npz")
    a = {n: torch.from_numpy(z[n]) for n in O.FORMAT_NAMES}
    n = int(z["in_rowptr"].shape[0] - 1)
    x = torch.randn(n, F, generator=torch.Generator().manual_seed(0)).half()
    return a, n, x


def _parallel_args(a, x, n, epoches=2, window=16):
    return (a["t_row_offset"], a["t_block_offset"], a["t_column"], a["t_value"].half(), a["t_window_row"],
            a["t_atomic"], a["t_binary"],
            a["c_row_offset"], a["c_row"], a["c_atomic"], a["c_column"], a["c_value"].half(),
            a["cs_row_offset"], a["cs_row"], a["cs_atomic"], a["cs_column"], a["cs_value"].half(),
            a["s_column"], a["s_value"], a["s_pos"], a["s_offset"], a["s_tile_window"], a["s_tile_column"],
            a["s_packed_a"], a["s_packed_meta"], a["s_window_tile_offset"], x,
            a["t_atomic"].numel(), a["c_atomic"].numel(), 32, a["cs_atomic"].numel(), window, x.size(1), n, n,
            epoches)


@pytest.mark.gpu
def test_parallel_entry_matches_oracle():
    import Libra6SpMMOnline
    a, n, x = _inputs()
    res = Libra6SpMMOnline.forward_fp16_tcu_cuda_sptc_mma_parallel_online(*_parallel_args(a, x, n))
    assert len(res) == 6 and res[0].dtype == torch.float32 and res[0].shape == (n, 64) and not res[0].is_cuda
    assert all(r.dim() == 0 for r in res[1:]) and float(res[1]) > 0
    assert O.scaled_max_error(res[0], O.spmm_from_format(a, x, n)) <= 2e-5


@pytest.mark.gpu
def test_compat_sptc_entries_sum_to_full_product():
    """base (TC + CSR with emptied SPTC arrays) + SPTC-only entry == parallel entry, the identity
    test_tr_csr_online.py:146-181 relies on; all three SPTC-only entries agree."""
    import Libra6SpMMOnline as L
    a, n, x = _inputs("rmat_s9")
    full = L.forward_fp16_tcu_cuda_sptc_mma_parallel_online(*_parallel_args(a, x, n))[0]
    e = dict(a)
    for k in ("s_column", "s_value", "s_pos", "s_tile_window", "s_tile_column", "s_packed_a", "s_packed_meta"):
        e[k] = a[k][:0].contiguous()
    e["s_offset"] = torch.zeros_like(a["s_offset"])
    e["s_window_tile_offset"] = torch.zeros_like(a["s_window_tile_offset"])
    base = L.forward_fp16_tcu_cuda_sptc_mma_parallel_online(*_parallel_args(e, x, n))[0]
    packed, ms = L.forward_fp16_sptc_mma_packed_online(a["s_tile_column"], a["s_packed_a"], a["s_packed_meta"],
                                                       a["s_window_tile_offset"], x, 16, 64, n, n, 1)
    scalar, _ = L.forward_fp16_sptc_online(a["s_column"], a["s_value"], a["s_pos"], a["s_window"], x, 16, 64, n, n, 1)
    mma, _ = L.forward_fp16_sptc_mma_online(a["s_column"], a["s_value"], a["s_pos"], a["s_offset"], x, 16, 64, n, n, 1)
    assert torch.equal(packed, scalar) and torch.equal(packed, mma)
    assert O.scaled_max_error(base + packed, full) <= 2e-5


def test_argument_errors_raise_like_torch_check():
    """No GPU needed: every check fires on the host before anything is launched."""
    import Libra6SpMMOnline as L
    a, n, x = _inputs()
    args = list(_parallel_args(a, x, n))
    bad = list(args); bad[3] = a["t_value"]  # fp32 instead of fp16
    with pytest.raises(RuntimeError, match="dtype"):
        L.forward_fp16_tcu_cuda_sptc_mma_parallel_online(*bad)
    bad = list(args); bad[-1] = 0
    with pytest.raises(RuntimeError, match="epoches"):
        L.forward_fp16_tcu_cuda_sptc_mma_parallel_online(*bad)
    bad = list(args); bad[31] = 17
    with pytest.raises(RuntimeError, match="window"):
        L.forward_fp16_tcu_cuda_sptc_mma_parallel_online(*bad)
    bad = list(args); bad[20] = a["s_offset"].clone(); bad[20][-1] += 1
    with pytest.raises(RuntimeError, match="s_offsets end"):
        L.forward_fp16_tcu_cuda_sptc_mma_parallel_online(*bad)
    bad = list(args); bad[21] = a["s_tile_window"][:-1]
    with pytest.raises(RuntimeError, match="tile count"):
        L.forward_fp16_tcu_cuda_sptc_mma_parallel_online(*bad)
    bad = list(args); bad[26] = x[:, :32].contiguous()
    with pytest.raises(RuntimeError, match="kOri \\* dimN"):
        L.forward_fp16_tcu_cuda_sptc_mma_parallel_online(*bad)
