"""Drop-in for the reference's `matching_utils_hash` module (Block/block_matching_hash.cpp:373-480):
complement-hash fast path, then sliding-window pairing.  Same function and dict keys."""
from trspmm.match24 import _as_int32, common_fields, match_stats

__all__ = ["match_2to4_hash"]


def _generic(variant, row_ptr, col_ind, window_size):
    st = match_stats(variant, row_ptr, col_ind, window_size)
    d = common_fields(st)
    d.update({
        "num_groups": int(st.num_groups), "num_16x16_blocks": int(st.num_16x16_blocks),
        "block_padding_groups": int(st.block_padding_groups), "fine_fallback": int(st.fine_fallback),
        "coarse_fallback": int(st.coarse_fallback), "fake_zeros": _as_int32(st.fake_zeros),
    })
    return d


def match_2to4_hash(row_ptr, col_ind, values, window_size=16):
    return _generic("hash", row_ptr, col_ind, window_size)
