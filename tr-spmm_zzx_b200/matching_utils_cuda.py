"""Drop-in for the reference's `matching_utils_cuda` torch extension (TR-source/setup_cuda.py,
Block/block_match_cuda.cu:1216-1625): `match_2to4(row_ptr, col_ind, values, window_size=16)` on
CUDA int32 / int32 / float32 tensors, returning the same statistics dict.

The reference kernel is non-deterministic by design (its warps race for columns and pairs,
block_match_cuda.cu:40-43).  Its rules - the per-window hash table and the order in which it is
compacted, overlap of at most 12 rows, best score first, search windows chosen by the window's
size - are reproduced here (trs_match24_stats variant 4) for the schedule in which the warps of a
block run one at a time and the window's entries are inserted in ascending column order, one of
the outcomes the reference itself can produce; the numbers are deterministic and are checked
against a CPU replay of the same rules (oracle.match_cuda_emulation)."""
import torch

from trspmm.match24 import _as_int32, common_fields, match_stats

__all__ = ["match_2to4"]


def match_2to4(row_ptr, col_ind, values, window_size=16):
    for name, t, dt in (("row_ptr", row_ptr, torch.int32), ("col_ind", col_ind, torch.int32),
                        ("values", values, torch.float32)):
        if not isinstance(t, torch.Tensor) or not t.is_cuda:
            raise RuntimeError(f"{name} must be a CUDA tensor")
        if t.dtype != dt:
            raise RuntimeError(f"{name} has an unexpected dtype")
        if t.dim() != 1:
            raise RuntimeError(f"{name} must be 1-D")
    if not 1 <= window_size <= 16:
        raise RuntimeError("window_size must be in [1, 16]")
    st = match_stats("cuda", row_ptr, col_ind, window_size)
    d = common_fields(st)
    d.update({
        "num_groups": int(st.num_groups), "num_16x16_blocks": int(st.num_16x16_blocks),
        "block_padding_groups": int(st.block_padding_groups), "fine_fallback": int(st.fine_fallback),
        "coarse_fallback": int(st.coarse_fallback), "fake_zeros": _as_int32(st.fake_zeros),
    })
    return d
