"""Drop-in for the reference's `matching_utils_online` module (Block/block_matching_online.cu:554-696):
`match_2to4_online(row_ptr, col_ind, values, window_size=16, dense_threshold=8, t_max=8)`, numpy
arrays in, statistics dict out.

The reference processes a window's columns in the slot order of a 2048-entry shared-memory hash
table that 16 threads fill concurrently (block_matching_online.cu:157-197), loses the columns
beyond the 2048th distinct one of a window, ignores `window_size` (its kernel fixes 16 rows,
:37, :143) and counts padding against the constant 32.  All of that is reproduced here
(trs_match24_stats variant 3) for the schedule in which the rows of a window insert one after the
other - one of the orders the reference itself can produce - so the numbers are deterministic;
they are checked against a CPU replay of the same rules (oracle.match_online_emulation)."""
from trspmm.match24 import _as_int32, match_stats

__all__ = ["match_2to4_online"]


def match_2to4_online(row_ptr, col_ind, values, window_size=16, dense_threshold=8, t_max=8):
    if window_size < 1 or window_size > 64:
        raise RuntimeError("window_size must be in [1, 64]")
    st = match_stats("online", row_ptr, col_ind, 16, dense_threshold, t_max)
    return {
        "total_rows": st.total_rows, "total_cols": st.total_cols, "total_nnz": st.total_nnz,
        "num_sptc_groups": int(st.num_groups), "num_tc_blocks": int(st.num_tc_blocks),
        "dense_to_tc_cols": int(st.dense_to_tc_cols), "dense_to_sptc_cols": int(st.dense_to_sptc_cols),
        "fine_fb": int(st.fine_fallback), "coarse_fb_cols": int(st.coarse_fallback),
        "num_16x16_blocks": int(st.num_16x16_blocks), "block_padding_groups": int(st.block_padding_groups),
        "fake_zeros": _as_int32(st.fake_zeros),
    }
