"""The builder's emulation of libstdc++ std::sort (csrc/trs_stdsort.cuh) against the real
std::sort, on the host: the same template the matching kernel runs on the device."""
import numpy as np
import pytest

from oracle import oracle as O
from trspmm.builder import stdsort_order


def _check(keys):
    got, heaps = stdsort_order(keys)
    want = O.std_sort_order(np.asarray(keys, dtype=np.int32))
    assert (got == want).all()
    return heaps


@pytest.mark.parametrize("seed", range(6))
def test_builder_shaped_keys(seed):
    """Unit nnz sequences as the builder produces them: non-increasing, values 1..32, long ties."""
    rng = np.random.default_rng(seed)
    for _ in range(60):
        n = int(rng.integers(0, 4000))
        hi = int(rng.integers(1, 33))
        keys = np.sort(rng.integers(1, hi + 1, n))[::-1].astype(np.uint8)
        _check(keys)
    _check(np.sort(rng.integers(1, 33, 200_000))[::-1].astype(np.uint8))


def test_arbitrary_orders_and_small_sizes():
    rng = np.random.default_rng(7)
    for n in list(range(0, 40)) + [100, 1000, 33333]:
        for hi in (1, 2, 5, 32, 255):
            _check(rng.integers(0, hi + 1, n).astype(np.uint8))
    _check(np.arange(250, dtype=np.uint8))          # ascending = worst order for a descending sort
    _check(np.arange(250, dtype=np.uint8)[::-1])


def test_heap_sort_fallback_is_emulated():
    """Median-of-three killer inputs (McIlroy's adversary played against std::sort itself) drive
    the introsort past its depth limit; the emulation must follow libstdc++ through heap sort too.
    Keys are quantised to one byte, which keeps long runs of ties inside the heap-sorted ranges."""
    import ctypes
    lib = O._lib()
    if not hasattr(lib, "trs_oracle_adversary"):
        pytest.skip("oracle built without the adversary")
    lib.trs_oracle_adversary.argtypes = [ctypes.c_int, ctypes.c_void_p]
    used = 0
    for n in (300, 2000, 20000, 60000):
        raw = np.empty(n, dtype=np.int32)
        lib.trs_oracle_adversary(n, raw.ctypes.data)
        for q in (1, 3, 7):
            keys = ((raw // q) * 255 // max(1, int(raw.max()) // q)).astype(np.uint8)
            used += _check(keys)
    assert used > 0, "no input reached the heap-sort fallback"
