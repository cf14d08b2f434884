"""Drop-in for the reference's `matching_utils_bucket` module (Block/block_matching_bucket.cpp:430-539):
top-heavy / bottom-heavy / balanced bucket pairing.  Same function and dict keys."""
from matching_utils_hash import _generic

__all__ = ["match_2to4_bucket"]


def match_2to4_bucket(row_ptr, col_ind, values, window_size=16):
    return _generic("bucket", row_ptr, col_ind, window_size)
