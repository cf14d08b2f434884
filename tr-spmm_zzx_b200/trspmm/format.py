"""Container for the 29 arrays of the reference's hybrid format.

Order and meaning follow the return list of Libra5BlockOnline.block_sptc_2to4_online
(TR-source/Block/block_online.cpp:844-870); the attribute names are the short ones used
throughout this repository (the reference's Python names are in
spmm/tr_csr_fp16/mdataset2_online.py:115-144).
"""
from __future__ import annotations

import torch

from ._lib import TrsFormat

FORMAT_NAMES = [
    "t_row_offset", "t_block_offset", "t_column", "t_value", "t_window_row", "t_atomic", "t_binary",
    "c_row_offset", "c_row", "c_atomic", "c_column", "c_value",
    "cs_row_offset", "cs_row", "cs_atomic", "cs_column", "cs_value",
    "s_column", "s_mask", "s_value", "s_pos", "s_window", "s_offset",
    "s_tile_window", "s_tile_group", "s_tile_column", "s_packed_a", "s_packed_meta",
    "s_window_tile_offset",
]
_HALF_VALUES = ("t_value", "c_value", "cs_value")


class Format:
    """The arrays, all on one device.  Value arrays of the TC / CSR routes may be fp32 (as the
    builder returns them) or fp16 (as the forward pass wants them); `half_values()` converts."""

    def __init__(self, arrays, window: int = 16):
        if isinstance(arrays, dict):
            arrays = [arrays[n] for n in FORMAT_NAMES]
        arrays = list(arrays)[:len(FORMAT_NAMES)]
        if len(arrays) != len(FORMAT_NAMES):
            raise ValueError(f"expected {len(FORMAT_NAMES)} arrays, got {len(arrays)}")
        self.window = window
        for n, a in zip(FORMAT_NAMES, arrays):
            setattr(self, n, a)

    def arrays(self):
        return [getattr(self, n) for n in FORMAT_NAMES]

    @property
    def device(self):
        return self.s_window_tile_offset.device

    def to(self, device):
        return Format([a.to(device) for a in self.arrays()], self.window)

    def half_values(self):
        out = Format(self.arrays(), self.window)
        for n in _HALF_VALUES:
            setattr(out, n, getattr(self, n).to(torch.float16))
        return out

    def contiguous(self):
        return Format([a.contiguous() for a in self.arrays()], self.window)

    # counts
    @property
    def num_windows(self):
        return max(self.s_window_tile_offset.numel() - 1, 0)

    @property
    def tiles(self):
        return self.s_tile_column.shape[0] if self.s_tile_column.dim() == 2 else self.s_tile_column.numel() // 16

    @property
    def blocks(self):
        return self.t_column.numel() // 8

    def stats(self):
        return {
            "windows": self.num_windows, "tc_blocks": self.blocks, "tc_nnz": self.t_value.numel(),
            "sptc_groups": self.s_window.numel(), "sptc_tiles": self.tiles,
            "sptc_nnz": int((self.s_pos >= 0).sum()) if self.s_pos.numel() else 0,
            "csr_long_parts": self.c_row.numel(), "csr_short_parts": self.cs_row.numel(),
            "csr_nnz": self.c_value.numel() + self.cs_value.numel(),
        }

    def c_struct(self) -> TrsFormat:
        """struct trs_format over these tensors' memory (keep `self` alive while it is used)."""
        for n in _HALF_VALUES:
            if getattr(self, n).dtype != torch.float16:
                raise TypeError(f"{n} must be fp16 for the forward pass (call half_values())")

        def ptr(t):
            return t.data_ptr() if t.numel() else None

        # Lengths the library derives sizes from must agree with each other: it reads
        # t_row_offset[parts_t], 8 column ids and 2 bitmaps per block, one row id per part, 16 column
        # ids / 64 packed words / 8 metadata words per tile.
        parts_t, blocks, tiles = self.t_window_row.numel(), self.blocks, self.tiles
        checks = [
            ("t_column", self.t_column.numel() == 8 * blocks), ("t_binary", self.t_binary.numel() == 2 * blocks),
            ("t_row_offset", parts_t == 0 or self.t_row_offset.numel() == parts_t + 1),
            ("t_block_offset", blocks == 0 or self.t_block_offset.numel() == blocks + 1),
            ("c_row_offset", self.c_row.numel() == 0 or self.c_row_offset.numel() == self.c_row.numel() + 1),
            ("cs_row_offset", self.cs_row.numel() == 0 or self.cs_row_offset.numel() == self.cs_row.numel() + 1),
            ("c_value", self.c_value.numel() == self.c_column.numel()),
            ("cs_value", self.cs_value.numel() == self.cs_column.numel()),
            ("s_packed_a", self.s_packed_a.numel() == 64 * tiles), ("s_packed_meta", self.s_packed_meta.numel() == 8 * tiles),
            ("s_tile_column", self.s_tile_column.numel() == 16 * tiles),
        ]
        for n, ok in checks:
            if not ok:
                raise ValueError(f"{n} has a length inconsistent with the other arrays of its route")

        f = TrsFormat()
        for n in ("t_row_offset", "t_block_offset", "t_column", "t_value", "t_window_row", "t_binary",
                  "c_row_offset", "c_row", "c_column", "c_value",
                  "cs_row_offset", "cs_row", "cs_column", "cs_value",
                  "s_window_tile_offset", "s_tile_column", "s_packed_a", "s_packed_meta"):
            t = getattr(self, n)
            if not t.is_contiguous():
                raise ValueError(f"{n} must be contiguous")
            setattr(f, n, ptr(t))
        f.parts_t = self.t_window_row.numel()
        f.blocks = self.blocks
        f.parts_c = self.c_row.numel()
        f.parts_c_short = self.cs_row.numel()
        f.num_windows = self.num_windows
        f.tiles = self.tiles
        return f
