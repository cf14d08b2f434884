"""Drop-in for the reference's `matching_utils` module (built by TR-source/setup_24matching.py from
Block/block_matching_window_para_dr.cpp:361-498): sliding-window pairing with dense-pool dual
routing.  Same function, arguments and dict keys; computed on the GPU, prints nothing."""
from trspmm.match24 import _as_int32, common_fields, match_stats

__all__ = ["match_2to4"]


def match_2to4(row_ptr, col_ind, values, window_size=16, dense_threshold=8, t_max=8):
    st = match_stats("para_dr", row_ptr, col_ind, window_size, dense_threshold, t_max)
    d = common_fields(st)
    d.update({
        "num_sptc_groups": int(st.num_groups), "num_tc_blocks": int(st.num_tc_blocks),
        "num_16x16_blocks": int(st.num_16x16_blocks), "block_padding_groups": int(st.block_padding_groups),
        "fine_fallback": int(st.fine_fallback), "coarse_fallback": int(st.coarse_fallback),
        "fake_zeros": _as_int32(st.fake_zeros), "tc_total_nnz": int(st.tc_total_nnz),
        "tc_block_count": int(st.tc_block_count), "tc_block_max_nnz": int(st.tc_block_max_nnz),
        "tc_block_min_nnz": int(st.tc_block_min_nnz),
    })
    return d
