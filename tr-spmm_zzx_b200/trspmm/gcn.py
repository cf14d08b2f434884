"""Two-layer GCN forward over the hybrid SpMM, row-window sharded across the GPUs of one box.

The reference has no layer or multi-GPU code (its GCN_dataset_* classes only hold data,
spmm/tr_csr_fp16/mdataset2_online.py:29-56); the layer is defined by the benchmark
configuration:  H1 = ReLU(A (X W1)),  out = A (H1 W2)  with fp16 activations and fp32
accumulation.  The dense products run first because they shrink the feature width before the
SpMM; they go through torch.matmul (a plain library GEMM).  The SpMMs, the fused ReLU and the
down-conversion are this library's kernel; ranks exchange their row blocks of the hidden matrix
with NCCL broadcasts (window-aligned blocks of different sizes) between the layers.
"""
from __future__ import annotations

import torch

from . import shard
from .builder import build_format
from .spmm import SpmmPlan


class ShardedGCN2:
    def __init__(self, rowptr, col, val, rank: int = 0, world: int = 1, window: int = 16, cuts=None, group=None):
        self.n = rowptr.numel() - 1
        self.rank, self.world, self.group = rank, world, group
        self.cuts = cuts if cuts is not None else shard.balanced_window_cuts(rowptr, world, window)
        self.r0, self.r1 = self.cuts[rank], self.cuts[rank + 1]
        rp_l, col_l, val_l = shard.slice_csr(rowptr, col, val, self.r0, self.r1)
        self.fmt, self.stats = build_format(rp_l, col_l, val_l, window=window)
        self.plan = SpmmPlan(self.fmt, max(self.r1 - self.r0, 1), self.n, window)
        self.gather_bytes = 0

    def _exchange(self, full: torch.Tensor):
        """Every rank's rows [cuts[r], cuts[r+1]) of `full` become valid on all ranks."""
        if self.world == 1:
            return
        import torch.distributed as dist
        works = []
        for src in range(self.world):
            a, b = self.cuts[src], self.cuts[src + 1]
            if b > a:
                works.append(dist.broadcast(full[a:b], src=src, group=self.group, async_op=True))
                if src != self.rank:
                    self.gather_bytes += (b - a) * full.shape[1] * full.element_size()
        for w in works:
            w.wait()

    def forward(self, X: torch.Tensor, W1: torch.Tensor, W2: torch.Tensor, gather: str = "h1") -> torch.Tensor:
        """X [N, F0] fp16 (replicated), W1 [F0, F1], W2 [F1, F2] fp16.  Returns this rank's rows of
        the output, [r1 - r0, F2] fp16.  gather="h1" exchanges the hidden matrix (N x F1);
        gather="z2" multiplies the own rows by W2 first and exchanges N x F2 instead."""
        self.gather_bytes = 0
        r0, r1 = self.r0, self.r1
        z1 = torch.matmul(X, W1)                                   # [N, F1], replicated compute
        if gather == "h1":
            h1 = torch.empty((self.n, W1.shape[1]), dtype=torch.float16, device=X.device)
            if r1 > r0:
                self.plan.run(z1, out=h1[r0:r1], relu=True)        # ReLU + fp16 fused into the one write
            self._exchange(h1)
            z2 = torch.matmul(h1, W2)                              # [N, F2]
        elif gather == "z2":
            h1_local = self.plan.run(z1, relu=True) if r1 > r0 else z1[:0]
            z2 = torch.empty((self.n, W2.shape[1]), dtype=torch.float16, device=X.device)
            if r1 > r0:
                torch.matmul(h1_local[: r1 - r0], W2, out=z2[r0:r1])
            self._exchange(z2)
        else:
            raise ValueError("gather must be 'h1' or 'z2'")
        return self.plan.run(z2)[: r1 - r0] if r1 > r0 else z2[:0]
