"""CPU checks of the plain-Python replays of the reference's two GPU matchers
(Block/block_matching_online.cu:85-431, Block/block_match_cuda.cu:822-1201), on cases small enough
to work out by hand."""
import numpy as np

from oracle import oracle as O


def _csr(rows):
    rp = np.zeros(len(rows) + 1, dtype=np.int32)
    rp[1:] = np.cumsum([len(r) for r in rows])
    col = np.array([c for r in rows for c in r], dtype=np.int32)
    return rp, col


def test_four_disjoint_columns_make_one_group():
    # 16 rows, column c holds rows 4c..4c+3: pairs (0,1) and (2,3) have cost 0 and are compatible
    rows = [[r // 4] for r in range(16)]
    d = O.match_online_emulation(*_csr(rows))
    assert d["num_sptc_groups"] == 1 and d["num_tc_blocks"] == 0
    assert d["fine_fb"] == 0 and d["coarse_fb_cols"] == 0
    assert d["fake_zeros"] == 32 - 16
    assert d["num_16x16_blocks"] == 1 and d["block_padding_groups"] == 3
    assert d["total_rows"] == 16 and d["total_cols"] == 4 and d["total_nnz"] == 16


def test_full_columns_go_to_the_dense_pool():
    # 9 full columns in one window, t_max = 0: no pair qualifies, 8 make a TC block, 1 pads a group
    rows = [list(range(9)) for _ in range(16)]
    d = O.match_online_emulation(*_csr(rows), dense_threshold=8, t_max=0)
    assert d["fine_fb"] == 9 and d["num_tc_blocks"] == 1
    assert d["dense_to_tc_cols"] == 8 and d["dense_to_sptc_cols"] == 1
    assert d["num_sptc_groups"] == 1 and d["fake_zeros"] == 32 - 16


def test_slot_order_is_column_id_modulo_table_size():
    # columns 2048 and 1 with masks that pair at cost 0; column 2048 sits in slot 0, before column 1:
    # the order does not change the counts here, but columns 0 and 2048 collide and probe linearly
    rows = [[0, 1, 2048] if r < 8 else [4096] for r in range(16)]
    d = O.match_online_emulation(*_csr(rows))
    assert d["total_cols"] == 4097 and d["total_nnz"] == 32
    # masks: three columns with the low 8 rows, one with the high 8: the first column pairs with the
    # complementary one only if it lies within the next 32 compacted positions (it does)
    assert d["num_sptc_groups"] + d["num_tc_blocks"] >= 1
    assert d["block_padding_groups"] == d["num_16x16_blocks"] * 4 - d["num_sptc_groups"]


def test_columns_beyond_the_table_are_lost():
    rows = [list(range(3000))] + [[] for _ in range(15)]
    d = O.match_online_emulation(*_csr(rows), t_max=8)
    # 2048 columns kept, every one with the single row 0: any two pair at cost 1 <= t_max; two pairs
    # conflict (the shared row), so no group forms: all 2048 columns fall to the dense pool
    assert d["fine_fb"] == 0 and d["coarse_fb_cols"] == 2048
    assert d["num_tc_blocks"] == 256 and d["dense_to_sptc_cols"] == 0
    assert d["total_nnz"] == 3000


def test_cuda_rules_four_disjoint_columns():
    rows = [[r // 4] for r in range(16)]
    d = O.match_cuda_emulation(*_csr(rows))
    # columns pair at overlap 0 (score 16 - 4), the two pairs do not conflict: one group, every row
    # holds one of the four columns and is padded by one
    assert d["num_groups"] == 1 and d["fine_fallback"] == 0 and d["coarse_fallback"] == 0
    assert d["fake_zeros"] == 16
    assert d["num_16x16_blocks"] == 1 and d["block_padding_groups"] == 3
    assert d["num_row_panels"] == 1 and d["total_cols"] == 4


def test_cuda_rules_prefer_the_denser_partner_and_allow_overlap():
    # column 0: rows 0-3; column 1: rows 0-1 (overlap 2); column 2: rows 8-15 (overlap 0, 8 non-zeros)
    rows = [[0, 1], [0, 1], [0], [0]] + [[] for _ in range(4)] + [[2] for _ in range(8)]
    d = O.match_cuda_emulation(*_csr(rows))
    # whatever the compaction order, a zero-overlap partner beats an overlapping one, and the odd
    # column stays alone: two "pairs", grouped if they do not conflict
    assert d["fine_fallback"] == 1
    assert d["num_groups"] in (1, 2)
    assert d["total_nnz"] + d["fake_zeros"] <= d["num_groups"] * 32


def test_cuda_rules_lonely_window():
    rows = [[7]] + [[] for _ in range(15)]
    d = O.match_cuda_emulation(*_csr(rows))
    assert d["num_groups"] == 1 and d["fine_fallback"] == 1 and d["coarse_fallback"] == 2
    assert d["fake_zeros"] == 1 + 2 * 15      # row 0 holds one column, the other 15 rows none
