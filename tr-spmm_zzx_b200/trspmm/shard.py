"""Row-window sharding for one multi-GPU box.

Every 16-row window is an independent unit of both the builder and the SpMM
(TR-source/Block/block_online.cpp:584 loops over windows; the SPTC kernel's grid x is the
window, TR-source/SpMM/mGCNkernel_online.cu:830), so the matrix is cut into contiguous window
ranges of about equal nnz, one per rank.  Each rank builds and multiplies its own rows against
a full replica of B; no collective is needed for a single SpMM.
"""
from __future__ import annotations

import torch


def balanced_window_cuts(rowptr: torch.Tensor, parts: int, window: int = 16):
    """Row boundaries [r_0=0, r_1, ..., r_parts=n_rows], every inner boundary a multiple of
    `window`, chosen so that each range holds about nnz/parts entries."""
    n = rowptr.numel() - 1
    W = (n + window - 1) // window
    idx = torch.arange(0, W + 1, device=rowptr.device) * window
    idx[-1] = n
    prefix = rowptr[idx.clamp_max(n)].long()  # nnz before each window boundary
    total = int(prefix[-1])
    cuts = [0]
    for k in range(1, parts):
        target = total * k // parts
        w = int(torch.searchsorted(prefix, torch.tensor(target, device=prefix.device), right=False))
        # choose the boundary closest to the target among w-1, w
        if w > 0 and abs(int(prefix[w - 1]) - target) <= abs(int(prefix[min(w, W)]) - target):
            w -= 1
        w = max(w, cuts[-1] // window if cuts[-1] % window == 0 else 0)
        cuts.append(min(w, W) * window if w < W else n)
    cuts.append(n)
    for i in range(1, len(cuts)):  # monotone
        cuts[i] = max(cuts[i], cuts[i - 1])
    return cuts


def cuts_from_window_costs(cost: torch.Tensor, parts: int, n_rows: int, window: int = 16):
    """Row boundaries from a per-window cost vector (e.g. k-steps of the built format + a fixed
    per-window overhead): contiguous window ranges of about equal total cost."""
    W = cost.numel()
    prefix = torch.zeros(W + 1, dtype=torch.float64, device=cost.device)
    prefix[1:] = torch.cumsum(cost.double(), 0)
    total = float(prefix[-1])
    cuts = [0]
    for k in range(1, parts):
        w = int(torch.searchsorted(prefix, torch.tensor(total * k / parts, dtype=torch.float64, device=cost.device)))
        w = min(max(w, cuts[-1] // window), W)
        cuts.append(min(w * window, n_rows))
    cuts.append(n_rows)
    for i in range(1, len(cuts)):
        cuts[i] = max(cuts[i], cuts[i - 1])
    return cuts


def rescale_costs(cost: torch.Tensor, cuts, times, window: int = 16, damping: float = 0.8):
    """Per-window costs corrected by what the ranks measured: the windows of a rank that ran longer
    than the mean get proportionally heavier (damped), so that the next cut moves windows away
    from it.  `cuts` are the row boundaries the times were measured with."""
    cost = cost.clone()
    mean = sum(times) / len(times)
    if mean <= 0:
        return cost
    for r, t in enumerate(times):
        w0, w1 = cuts[r] // window, (cuts[r + 1] + window - 1) // window
        if w1 > w0 and t > 0:
            cost[w0:w1] *= (t / mean) ** damping
    return cost


def window_steps(fmt, n_windows: int):
    """k-steps per window of a built format: packed tiles + pairs of TC blocks."""
    off = fmt.s_window_tile_offset
    steps = (off[1:] - off[:-1]).to(torch.float32)
    if steps.numel() < n_windows:
        steps = torch.cat([steps, torch.zeros(n_windows - steps.numel(), device=steps.device)])
    if fmt.t_window_row.numel():
        blocks_per_part = (fmt.t_row_offset[1:] - fmt.t_row_offset[:-1]).to(torch.float32)
        win = (fmt.t_window_row // 16).long()
        blocks = torch.zeros(n_windows, device=steps.device).index_add_(0, win, blocks_per_part)
        steps = steps + torch.ceil(blocks / 2)
    return steps


def slice_csr(rowptr: torch.Tensor, col: torch.Tensor, val: torch.Tensor, r0: int, r1: int):
    """Rows [r0, r1) as their own CSR (row pointers rebased, global column ids kept)."""
    b, e = int(rowptr[r0]), int(rowptr[r1])
    return (rowptr[r0:r1 + 1] - rowptr[r0]).to(torch.int32).contiguous(), col[b:e].contiguous(), val[b:e].contiguous()


def shard_for_rank(rowptr, col, val, rank: int, world: int, window: int = 16):
    cuts = balanced_window_cuts(rowptr, world, window)
    r0, r1 = cuts[rank], cuts[rank + 1]
    return (r0, r1), slice_csr(rowptr, col, val, r0, r1)


def refined_cuts(rowptr, col, val, rank: int, world: int, F, strict: bool = False, rounds: int = 2,
                 window: int = 16, group=None, report: dict = None):
    """Row cuts balanced by what the ranks measure (a collective: every rank of `group` calls it with
    the whole matrix on its GPU).  First cut by nnz; re-cut by the k-steps the built format really
    has per window (hub windows share columns, so their cost per nnz is lower) plus a fixed
    per-window overhead; then up to `rounds` re-cuts from the kernel time each rank measures on its
    own shard with an [n, F] operand (hub windows and L2 behaviour are not in the step count).  F may
    be a sequence of widths - the SpMMs of the layers of a model - whose times are added.  `report`,
    when given, receives the per-rank times of every round ("times_ms": list of lists; the last
    list belongs to the cut before the returned one unless the loop stopped on balance)."""
    import torch.distributed as dist
    from .builder import build_format
    from .spmm import SpmmPlan
    n = rowptr.numel() - 1
    dev = rowptr.device
    (r0, r1), (rp_l, col_l, val_l) = shard_for_rank(rowptr, col, val, rank, world, window)
    fmt, _ = build_format(rp_l, col_l, val_l, window=window, strict=strict)
    W = (n + window - 1) // window
    cost = torch.zeros(W, device=dev)
    mine = window_steps(fmt, (r1 - r0 + window - 1) // window) + 6.0
    cost[r0 // window:r0 // window + mine.numel()] = mine
    dist.all_reduce(cost, op=dist.ReduceOp.SUM, group=group)
    cuts = cuts_from_window_costs(cost, world, n, window)
    del fmt
    widths = (int(F),) if isinstance(F, int) else tuple(int(f) for f in F)
    gen = torch.Generator(device=dev).manual_seed(1)
    Bts = [torch.randn(n, f, device=dev, generator=gen).half() for f in widths]
    for _ in range(rounds):
        r0, r1 = cuts[rank], cuts[rank + 1]
        rp_l, col_l, val_l = slice_csr(rowptr, col, val, r0, r1)
        fmt_t, _st = build_format(rp_l, col_l, val_l, window=window, strict=strict)
        plan_t = SpmmPlan(fmt_t, max(r1 - r0, 1), n, window, validate=False)
        outs_t = [torch.empty((max(r1 - r0, 1), f), dtype=torch.float16, device=dev) for f in widths]
        for _i in range(3):
            for Bt, out_t in zip(Bts, outs_t):
                plan_t.run(Bt, out=out_t)
        torch.cuda.synchronize()
        dist.barrier(group=group)
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _i in range(5):
            for Bt, out_t in zip(Bts, outs_t):
                plan_t.run(Bt, out=out_t)
        a1.record()
        torch.cuda.synchronize()
        mine_t = torch.tensor([a0.elapsed_time(a1) / 5], device=dev)
        all_t = [torch.zeros_like(mine_t) for _i in range(world)]
        dist.all_gather(all_t, mine_t, group=group)
        times = [float(t) for t in all_t]
        if report is not None:
            report.setdefault("times_ms", []).append([round(t, 4) for t in times])
        del plan_t, fmt_t, outs_t
        if max(times) <= 1.03 * (sum(times) / world):
            break
        cost = rescale_costs(cost, cuts, times, window)
        cuts = cuts_from_window_costs(cost, world, n, window)
    return cuts


def even_row_split(n_rows: int, world: int):
    """Rows per rank and padded total for an equal-sized split of a dense [n_rows, F] operand
    (the all-gather wants equal pieces; the padding rows are never read by a kernel)."""
    per = (n_rows + world - 1) // world
    return per, per * world


def bind_to_gpu_numa_node(device_index: int):
    """Pin this process to the CPUs of the NUMA node its GPU hangs off, so that pinned host buffers
    allocated afterwards (first touch) are local to that GPU's PCIe root: with one process per GPU
    on a two-socket host, copies from the other socket's memory cross the socket link and run at a
    fraction of the PCIe rate.  Returns the node id, or None when the topology cannot be read
    (nothing is changed then).  Only this process's CPU affinity is touched."""
    import os
    try:
        props = torch.cuda.get_device_properties(device_index)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        allowed = os.sched_getaffinity(0) & cpus
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


def even_output_rows(n_rows: int, world: int, rank: int):
    """[begin, end) rows of C that `rank` hands to the host when the output is split evenly."""
    per = (n_rows + world - 1) // world
    return min(rank * per, n_rows), min((rank + 1) * per, n_rows)


def output_transfers(row_cuts, rank: int):
    """Where the rows this rank computed go when every rank delivers an even share of C.

    `row_cuts` are the computed-row boundaries of all ranks (world + 1 values).  Returns a list of
    (peer, src_begin, dst_begin, count): `count` rows starting at local row `src_begin` of this rank's
    result belong at row `dst_begin` of peer's output share (peer may be this rank)."""
    world = len(row_cuts) - 1
    n_rows = row_cuts[-1]
    r0, r1 = row_cuts[rank], row_cuts[rank + 1]
    moves = []
    for peer in range(world):
        o0, o1 = even_output_rows(n_rows, world, peer)
        a, b = max(r0, o0), min(r1, o1)
        if b > a:
            moves.append((peer, a - r0, a - o0, b - a))
    return moves


class ShardedHostSpmm:
    """Host-buffer SpMM on `world` GPUs of one box, for a stream of calls over one matrix.

    Without it every rank would pull the whole dense operand B over PCIe (world copies of the same
    bytes through the host's memory system).  Here each rank copies only its 1/world slice of B
    from pinned host memory, the slices are exchanged over NVLink (one in-place NCCL all-gather, or
    copy-engine pushes into the peers' buffers with exchange="push"), each rank multiplies its own
    row windows, and the result goes back to the host.  The row windows are cut by cost, so the
    ranks compute very different numbers of rows (R-MAT at two ranks: 0.33 M against 1.77 M); with
    `row_cuts` given, the computed rows are therefore re-dealt over NVLink first (copy-engine
    pushes into peer-mapped buffers) so that every rank copies the same 1/world of C to its host
    buffer and no PCIe link carries more than its share.  Five streams (input copy, exchange of B,
    kernels, exchange of C, output copy) and two buffer slots let consecutive calls overlap.

    The reference has no multi-GPU path; the single-GPU call this extends is
    spmm_forward_fp16_tcu_cuda_sptc_mma_parallel_online (mGCN_online.cpp:760), which copies B in and
    C out on every call.
    """

    def __init__(self, fmt, m_local: int, n_cols: int, F: int, rank: int, world: int, group=None, row_cuts=None,
                 exchange: str = "nccl"):
        import torch.distributed as dist
        from .spmm import SpmmPlan
        if exchange not in ("nccl", "push"):
            raise ValueError("exchange must be 'nccl' or 'push'")
        self.dist, self.group = dist, group
        self.rank, self.world, self.F = rank, world, F
        self.m_local, self.n_cols = max(m_local, 1), n_cols
        self.dev = fmt.device
        self.plan = SpmmPlan(fmt, self.m_local, n_cols)
        self.per, padded = even_row_split(n_cols, world)
        self.exchange = exchange if world > 1 else "nccl"
        self.row_cuts = list(row_cuts) if (row_cuts is not None and world > 1) else None
        if self.row_cuts is not None and (len(self.row_cuts) != world + 1 or
                                          self.row_cuts[rank + 1] - self.row_cuts[rank] != m_local):
            raise ValueError("row_cuts do not describe this rank's rows")
        symmetric = self.exchange == "push" or self.row_cuts is not None
        if symmetric:
            import torch.distributed._symmetric_memory as symm_mem
            pg = group if group is not None else dist.group.WORLD
        if self.exchange == "push":
            self._Bsym = symm_mem.empty((2, padded, F), dtype=torch.float16, device=self.dev)
            self._Bhdl = symm_mem.rendezvous(self._Bsym, group=pg)
            self._Bsym.zero_()
            self.B = [self._Bsym[0], self._Bsym[1]]
            self._Bpeer = [self._Bhdl.get_buffer(p, (2, padded, F), torch.float16) for p in range(world)]
            # PCIe copies run between pinned host memory and plain device memory only (copies to or from
            # the peer-mapped allocations measured at half the rate): the slice lands here first
            self._Bstage = [torch.zeros((self.per, F), dtype=torch.float16, device=self.dev) for _ in range(2)]
        else:
            self.B = [torch.zeros((padded, F), dtype=torch.float16, device=self.dev) for _ in range(2)]
        self.C = [torch.empty((self.m_local, F), dtype=torch.float16, device=self.dev) for _ in range(2)]
        if self.row_cuts is not None:
            self.out0, self.out1 = even_output_rows(self.row_cuts[-1], world, rank)
            self.per_out = (self.row_cuts[-1] + world - 1) // world
            self._Csym = symm_mem.empty((2, max(self.per_out, 1), F), dtype=torch.float16, device=self.dev)
            self._Chdl = symm_mem.rendezvous(self._Csym, group=pg)
            self._Cpeer = [self._Chdl.get_buffer(p, (2, max(self.per_out, 1), F), torch.float16) for p in range(world)]
            self._moves = output_transfers(self.row_cuts, rank)
            self._Cout = [torch.empty((max(self.per_out, 1), F), dtype=torch.float16, device=self.dev) for _ in range(2)]
        hi = lambda: torch.cuda.Stream(self.dev, priority=-1)  # noqa: E731  small kernels ahead of the SpMM's queue
        self.s_in, self.s_k, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
        self.s_comm, self.s_x = hi(), hi()
        ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
        self.in_done, self.comm_done, self.k_done, self.x_done, self.out_done = ([ev(), ev()] for _ in range(5))
        self.in_start, self.comm_start, self.k_start, self.x_start, self.out_start = ([ev(), ev()] for _ in range(5))
        self.seq = 0
        self._keep = []
        if symmetric:
            torch.cuda.synchronize(self.dev)
            dist.barrier(group=group)

    def my_rows(self):
        """[begin, end) rows of B this rank is expected to provide."""
        b = self.rank * self.per
        return b, min(b + self.per, self.n_cols)

    def out_rows(self):
        """[begin, end) rows of C this rank delivers when the output is re-dealt (row_cuts given):
        an even share of all rows.  None otherwise (the rank delivers the rows it computed)."""
        if self.row_cuts is None:
            return None
        return self.out0, self.out1

    def submit(self, B_slice_host: torch.Tensor, C_host: torch.Tensor):
        """B_slice_host: pinned fp16 [rows of my_rows(), F]; C_host: pinned fp16, [m_local, F] or, with
        row_cuts, [rows of out_rows(), F]."""
        s = self.seq & 1
        b0, b1 = self.my_rows()
        c_rows = self.m_local if self.row_cuts is None else self.out1 - self.out0
        if B_slice_host.shape != (b1 - b0, self.F) or C_host.shape != (c_rows, self.F):
            raise ValueError("slice shapes do not match this rank's share")
        self._keep.append((B_slice_host, C_host))
        Bs, Cs = self.B[s], self.C[s]
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.k_done[s])           # the kernels two calls back are done with this slot
            self.in_start[s].record(self.s_in)
            if self.exchange == "push":
                self._Bstage[s][:b1 - b0].copy_(B_slice_host, non_blocking=True)
            else:
                Bs[b0:b1].copy_(B_slice_host, non_blocking=True)
            self.in_done[s].record(self.s_in)
        with torch.cuda.stream(self.s_comm):
            self.s_comm.wait_event(self.in_done[s])
            self.comm_start[s].record(self.s_comm)
            if self.world > 1 and self.exchange == "nccl":
                mine = Bs[self.rank * self.per:(self.rank + 1) * self.per]
                self.dist.all_gather_into_tensor(Bs, mine, group=self.group)   # in place: `mine` is its own piece of Bs
            elif self.world > 1:
                # every rank's kernels two calls back are done with slot s (their input copies waited
                # for them), then the copy engines put this rank's slice into every peer's B
                self._Bhdl.barrier(channel=s)
                for d in range(self.world):
                    p = (self.rank + d) % self.world
                    self._Bpeer[p][s, b0:b1].copy_(self._Bstage[s][:b1 - b0], non_blocking=True)
                self._Bhdl.barrier(channel=2 + s)
            self.comm_done[s].record(self.s_comm)
        with torch.cuda.stream(self.s_k):
            self.s_k.wait_event(self.comm_done[s])
            self.s_k.wait_event(self.x_done[s] if self.row_cuts is not None else self.out_done[s])  # slot's C drained
            self.k_start[s].record(self.s_k)
            self.plan.run(Bs[:self.n_cols], out=Cs)
            self.k_done[s].record(self.s_k)
        if self.row_cuts is not None:
            with torch.cuda.stream(self.s_x):
                self.s_x.wait_event(self.k_done[s])
                self.x_start[s].record(self.s_x)
                self._Chdl.barrier(channel=s)               # every rank has moved slot s of two calls back out of the way
                for peer, src, dst, cnt in self._moves:
                    self._Cpeer[peer][s, dst:dst + cnt].copy_(Cs[src:src + cnt], non_blocking=True)
                self._Chdl.barrier(channel=2 + s)           # every rank's rows have landed
                self.s_x.wait_event(self.out_done[s])       # the output copy two calls back has read _Cout[s]
                if c_rows > 0:
                    self._Cout[s][:c_rows].copy_(self._Csym[s, :c_rows], non_blocking=True)   # plain memory for the PCIe copy
                self.x_done[s].record(self.s_x)
        with torch.cuda.stream(self.s_out):
            if self.row_cuts is not None:
                self.s_out.wait_event(self.x_done[s])
                self.out_start[s].record(self.s_out)
                if c_rows > 0:
                    C_host.copy_(self._Cout[s][:c_rows], non_blocking=True)
            else:
                self.s_out.wait_event(self.k_done[s])
                self.out_start[s].record(self.s_out)
                C_host.copy_(Cs, non_blocking=True)
            self.out_done[s].record(self.s_out)
        self.seq += 1

    def wait(self):
        for st in (self.s_in, self.s_comm, self.s_k, self.s_x, self.s_out):
            st.synchronize()
        self._keep.clear()

    def leg_ms(self):
        """Device time of the legs of the most recent call (after wait()): input copy, exchange of B,
        kernels, re-deal of C, output copy.  Legs of consecutive calls overlap, so the step time of a
        stream of calls tends to the longest leg, not to their sum; an exchange leg includes the
        time it waits for the slowest peer."""
        if self.seq == 0:
            return {"h2d_ms": 0.0, "allgather_ms": 0.0, "kernel_ms": 0.0, "redeal_ms": 0.0, "d2h_ms": 0.0}
        s = (self.seq - 1) & 1
        return {"h2d_ms": self.in_start[s].elapsed_time(self.in_done[s]),
                "allgather_ms": self.comm_start[s].elapsed_time(self.comm_done[s]),
                "kernel_ms": self.k_start[s].elapsed_time(self.k_done[s]),
                "redeal_ms": self.x_start[s].elapsed_time(self.x_done[s]) if self.row_cuts is not None else 0.0,
                "d2h_ms": self.out_start[s].elapsed_time(self.out_done[s])}
