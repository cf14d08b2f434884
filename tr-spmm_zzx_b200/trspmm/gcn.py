"""Two-layer GCN forward over the hybrid SpMM, row-window sharded across the GPUs of one box.

The reference has no layer or multi-GPU code (its GCN_dataset_* classes only hold data,
spmm/tr_csr_fp16/mdataset2_online.py:29-56); the layer is defined by the benchmark
configuration:  H1 = ReLU(A (X W1)),  out = A (H1 W2)  with fp16 activations and fp32
accumulation.  The dense products run first because they shrink the feature width before the
SpMM; they go through torch.matmul (a plain library GEMM).  The SpMMs, the fused ReLU and the
down-conversion are this library's kernel; ranks exchange their row blocks of the hidden matrix
(window-aligned, different sizes) with one grouped batch of NCCL sends / receives between the layers.
"""
from __future__ import annotations

import torch

from . import shard
from .builder import build_format
from .spmm import SpmmPlan


def rows_gemm_bcast(H: torch.Tensor, W: torch.Tensor, dst_ptrs, row0: int, multicast_ptr: int = 0):
    """trs_rows_gemm_bcast: Z[row0 + r] = H[r] @ W, the fp16 rows written by the one kernel into every
    buffer of `dst_ptrs` (device pointers of [N_total, N] fp16 matrices: this GPU's and its NVLink
    peers').  With `multicast_ptr` (the NVLink multicast mapping of those buffers) the rows are stored
    once through it instead (trs_rows_gemm_mcast).  Asynchronous on the current stream."""
    import ctypes as C
    from . import _lib
    if H.dtype != torch.float16 or W.dtype != torch.float16 or not H.is_cuda or H.device != W.device:
        raise ValueError("H and W must be fp16 CUDA tensors on one device")
    if H.dim() != 2 or W.dim() != 2 or H.shape[1] != W.shape[0] or not H.is_contiguous() or not W.is_contiguous():
        raise ValueError("H [rows, K] and W [K, N], both contiguous")
    if not 1 <= len(dst_ptrs) <= 8 or row0 < 0:
        raise ValueError("1 to 8 destination buffers and a non-negative row offset")
    lib = _lib.load()
    if multicast_ptr:
        with torch.cuda.device(H.device):
            _lib.check(lib.trs_rows_gemm_mcast(H.data_ptr(), W.data_ptr(), int(multicast_ptr), int(row0), H.shape[0],
                                               H.shape[1], W.shape[1], _lib.current_stream_ptr(H.device)))
        return
    arr = (C.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
    with torch.cuda.device(H.device):
        _lib.check(lib.trs_rows_gemm_bcast(H.data_ptr(), W.data_ptr(), arr, len(dst_ptrs), int(row0), H.shape[0],
                                           H.shape[1], W.shape[1], _lib.current_stream_ptr(H.device)))


class ShardedGCN2:
    def __init__(self, rowptr, col, val, rank: int = 0, world: int = 1, window: int = 16, cuts=None, group=None,
                 strict: bool = False):
        self.n = rowptr.numel() - 1
        self.rank, self.world, self.group = rank, world, group
        self.cuts = cuts if cuts is not None else shard.balanced_window_cuts(rowptr, world, window)
        self.r0, self.r1 = self.cuts[rank], self.cuts[rank + 1]
        rp_l, col_l, val_l = shard.slice_csr(rowptr, col, val, self.r0, self.r1)
        self.fmt, self.stats = build_format(rp_l, col_l, val_l, window=window, strict=strict)
        self.plan = SpmmPlan(self.fmt, max(self.r1 - self.r0, 1), self.n, window)
        self.gather_bytes = 0
        self.profile = False
        self.last_breakdown = {}
        self._symm = {}   # feature width -> (tensor, handle) of the peer-mapped hidden matrix
        self._copy_streams = None
        self.push_chunks = 2
        self._calls = 0
        self.multicast = True    # gemm_bcast: store through the NVLink multicast mapping when the handle has one,
        self.multicast_min_world = 3   # from this many ranks on

    def _symmetric(self, F, device):
        """A [N, F] fp16 matrix every rank of the box can store into (torch symmetric memory).  F may be
        a (width, slot) pair: one buffer per slot."""
        key, F = F, (F[0] if isinstance(F, tuple) else F)
        if key not in self._symm:
            import torch.distributed as dist
            import torch.distributed._symmetric_memory as symm_mem
            t = symm_mem.empty((self.n, F), dtype=torch.float16, device=device)
            hdl = symm_mem.rendezvous(t, group=self.group if self.group is not None else dist.group.WORLD)
            self._symm[key] = (t, hdl)
        return self._symm[key]

    def _exchange(self, full: torch.Tensor):
        """Every rank's rows [cuts[r], cuts[r+1]) of `full` become valid on all ranks.  The blocks
        are window-aligned and of different sizes, so this is an all-gather with unequal counts:
        one batch of point-to-point sends / receives that NCCL runs as a single group, every
        NVLink direction busy at once."""
        if self.world == 1:
            return
        import torch.distributed as dist
        ops = []
        a, b = self.cuts[self.rank], self.cuts[self.rank + 1]
        for peer in range(self.world):
            if peer == self.rank:
                continue
            pa, pb = self.cuts[peer], self.cuts[peer + 1]
            if pb > pa:
                ops.append(dist.P2POp(dist.irecv, full[pa:pb], peer, self.group))
                self.gather_bytes += (pb - pa) * full.shape[1] * full.element_size()
            if b > a:
                ops.append(dist.P2POp(dist.isend, full[a:b], peer, self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    def forward(self, X: torch.Tensor, W1: torch.Tensor, W2: torch.Tensor, gather: str = "h1") -> torch.Tensor:
        """X [N, F0] fp16 (replicated), W1 [F0, F1], W2 [F1, F2] fp16.  Returns this rank's rows of
        the output, [r1 - r0, F2] fp16.  gather="h1" exchanges the hidden matrix (N x F1) with NCCL;
        gather="z2" multiplies the own rows by W2 first and exchanges N x F2 instead;
        gather="fused" lets the layer-1 SpMM store its rows into every rank's H1 itself
        (peer-mapped symmetric memory, trs_spmm_run_bcast); gather="push" multiplies the own rows by W2 in
        window chunks and has the copy engines push each finished chunk into the peers' Z2 while the
        next chunk is computed; gather="gemm_bcast" multiplies the own rows by W2 and stores the product
        into every rank's Z2 in one kernel (trs_rows_gemm_bcast: no library GEMM, no collective)."""
        self.gather_bytes = 0
        r0, r1 = self.r0, self.r1
        marks = []

        def mark(name):
            if self.profile:
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append((name, e))

        mark("start")
        z1 = torch.matmul(X, W1)                                   # [N, F1], replicated compute
        mark("gemm1")
        if gather == "h1":
            h1 = torch.empty((self.n, W1.shape[1]), dtype=torch.float16, device=X.device)
            if r1 > r0:
                self.plan.run(z1, out=h1[r0:r1], relu=True)        # ReLU + fp16 fused into the one write
            mark("spmm1")
            self._exchange(h1)
            mark("exchange")
            z2 = torch.matmul(h1, W2)                              # [N, F2]
            mark("gemm2")
        elif gather == "fused":
            # layer-1 SpMM writes its rows (ReLU, fp16) into every rank's copy of H1 over NVLink from
            # the kernel's epilogue: no separate all-gather, the exchange overlaps the SpMM
            if self.world == 1:
                h1 = torch.empty((self.n, W1.shape[1]), dtype=torch.float16, device=X.device)
                self.plan.run(z1, out=h1[r0:r1], relu=True)
            else:
                h1, hdl = self._symmetric(W1.shape[1], X.device)
                hdl.barrier(channel=0)                 # everyone is done reading the previous H1
                if r1 > r0:
                    self.plan.run_bcast(z1, [int(p) for p in hdl.buffer_ptrs], r0, relu=True)
                    self.gather_bytes += (self.n - (r1 - r0)) * W1.shape[1] * 2
                hdl.barrier(channel=1)                 # all rows of all ranks have landed
            mark("spmm1+exchange")
            z2 = torch.matmul(h1, W2)
            mark("gemm2")
        elif gather == "z2":
            h1_local = self.plan.run(z1, relu=True) if r1 > r0 else z1[:0]
            z2 = torch.empty((self.n, W2.shape[1]), dtype=torch.float16, device=X.device)
            if r1 > r0:
                torch.matmul(h1_local[: r1 - r0], W2, out=z2[r0:r1])
            mark("spmm1+gemm2")
            self._exchange(z2)
            mark("exchange")
        elif gather == "push":
            # own rows -> ReLU -> x W2 in window chunks; every finished chunk is pushed into the peers'
            # copies of Z2 by the copy engines (peer-mapped symmetric memory) while the next chunk is
            # still being multiplied; exact row counts, no padding, no collective kernel on the SMs
            if self.world == 1:
                h1_local = self.plan.run(z1, relu=True)
                z2 = torch.matmul(h1_local[: r1 - r0], W2)
                mark("spmm1+gemm2")
            else:
                z2, hdl = self._symmetric(W2.shape[1], X.device)
                if self._copy_streams is None:
                    self._copy_streams = [torch.cuda.Stream(X.device) for _ in range(min(4, self.world - 1))]
                key = ("peers", W2.shape[1])
                if key not in self._symm:
                    self._symm[key] = [hdl.get_buffer(p, (self.n, W2.shape[1]), torch.float16) for p in range(self.world)]
                peers = self._symm[key]
                hdl.barrier(channel=0)                 # every rank is done reading the previous Z2
                main = torch.cuda.current_stream(X.device)
                if r1 > r0:
                    h1_local = torch.empty((r1 - r0, W1.shape[1]), dtype=torch.float16, device=X.device)
                    W = self.plan.num_windows
                    nch = max(1, min(self.push_chunks, W))
                    k = 0
                    for i in range(nch):
                        w0, w1 = W * i // nch, W * (i + 1) // nch
                        a0, a1 = w0 * self.plan.window, min(w1 * self.plan.window, r1 - r0)
                        if a1 <= a0:
                            continue
                        self.plan.run_windows(z1, h1_local, w0, w1, relu=True)
                        torch.matmul(h1_local[a0:a1], W2, out=z2[r0 + a0:r0 + a1])
                        ready = torch.cuda.Event()
                        ready.record(main)
                        for p in range(self.world):
                            if p == self.rank:
                                continue
                            cs = self._copy_streams[k % len(self._copy_streams)]
                            k += 1
                            cs.wait_event(ready)
                            with torch.cuda.stream(cs):
                                peers[p][r0 + a0:r0 + a1].copy_(z2[r0 + a0:r0 + a1], non_blocking=True)
                        self.gather_bytes += (self.world - 1) * (a1 - a0) * W2.shape[1] * 2
                    for cs in self._copy_streams:
                        main.wait_stream(cs)
                mark("spmm1+gemm2+push")
                hdl.barrier(channel=1)                 # all rows of all ranks have landed
                mark("barrier")
        elif gather == "gemm_bcast":
            if self.world == 1:
                # nothing to exchange: a plain library GEMM (0.073 ms for 2^20 rows; the fused kernel with
                # its single destination takes 0.10 ms)
                h1_local = self.plan.run(z1, relu=True)
                z2 = torch.matmul(h1_local[: r1 - r0], W2)
                mark("spmm1+gemm2")
            else:
                # two Z2 buffers used in turn: a rank that runs ahead writes the other buffer, and it cannot
                # get two calls ahead, because the barrier below needs every rank's previous call finished -
                # so one barrier per call is enough (none before the stores)
                self._calls += 1
                z2, hdl = self._symmetric((W2.shape[1], self._calls & 1), X.device)
                if r1 > r0:
                    h1_local = self.plan.run(z1, relu=True)
                    mark("spmm1")
                    # (the SpMM in window chunks with the GEMM + stores of a finished chunk on a second stream
                    # was measured on four ranks: 1.06 / 1.33 ms with two / four chunks against 0.82 ms)
                    # with one peer a plain store already sends every row once (2 ranks measured 0.99 ms
                    # with it, 1.06 ms through the multicast mapping; 4 ranks 0.83 against 0.75 ms)
                    mc = int(getattr(hdl, "multicast_ptr", 0) or 0) if (self.multicast and self.world >= self.multicast_min_world) else 0
                    rows_gemm_bcast(h1_local[: r1 - r0], W2.contiguous(), [int(p) for p in hdl.buffer_ptrs], r0, mc)
                    self.gather_bytes += (self.n - (r1 - r0)) * W2.shape[1] * 2
                mark("gemm2+exchange")
                hdl.barrier(channel=1)                 # all rows of all ranks have landed
                mark("barrier")
        else:
            raise ValueError("gather must be 'h1', 'z2', 'fused', 'push' or 'gemm_bcast'")
        out = self.plan.run(z2)[: r1 - r0] if r1 > r0 else z2[:0]
        mark("spmm2")
        if self.profile:
            torch.cuda.synchronize()
            self.last_breakdown = {n: marks[i][1].elapsed_time(e) for i, (n, e) in enumerate(marks[1:])}
        return out
