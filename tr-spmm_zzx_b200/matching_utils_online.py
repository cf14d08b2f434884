"""Drop-in for the reference's `matching_utils_online` module (Block/block_matching_online.cu:554-696):
`match_2to4_online(row_ptr, col_ind, values, window_size=16, dense_threshold=8, t_max=8)`, numpy
arrays in, statistics dict out.

The reference processes a window's columns in the slot order of a shared-memory hash table and
silently overflows above 2048 distinct columns per window (block_matching_online.cu:164-197); its
result therefore depends on insertion races.  Here the same dual-routing rules run over the
columns in ascending id order (the order of the CPU version it was derived from), which is
deterministic and has no column limit; dict keys and the invariants the reference's driver checks
(`pad == blocks * 4 - groups`, test_24_matching.py:317-344) are kept."""
from trspmm.match24 import _as_int32, match_stats

__all__ = ["match_2to4_online"]


def match_2to4_online(row_ptr, col_ind, values, window_size=16, dense_threshold=8, t_max=8):
    st = match_stats("para_dr", row_ptr, col_ind, window_size, dense_threshold, t_max)
    pooled = int(st.fine_fallback) + int(st.coarse_fallback)
    to_tc = int(st.num_tc_blocks) * dense_threshold
    return {
        "total_rows": st.total_rows, "total_cols": st.total_cols, "total_nnz": st.total_nnz,
        "num_sptc_groups": int(st.num_groups), "num_tc_blocks": int(st.num_tc_blocks),
        "dense_to_tc_cols": to_tc, "dense_to_sptc_cols": pooled - to_tc,
        "fine_fb": int(st.fine_fallback), "coarse_fb_cols": int(st.coarse_fallback),
        "num_16x16_blocks": int(st.num_16x16_blocks), "block_padding_groups": int(st.block_padding_groups),
        "fake_zeros": _as_int32(st.fake_zeros),
    }
