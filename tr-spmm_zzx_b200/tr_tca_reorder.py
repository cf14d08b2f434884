"""Drop-in for the reference module spmm/tr_csr_fp16/tr_tca_reorder.py: same function name,
arguments and return triple; the order itself is computed by trspmm.reorder (sort-based, on the
GPU when one is present), not by the reference's MinHash-LSH clustering."""
from trspmm.reorder import apply_tca_reorder  # noqa: F401
