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


class ShardedHostSpmm:
    """Host-buffer SpMM on `world` GPUs of one box, for a stream of calls over one matrix.

    Without it every rank would pull the whole dense operand B over PCIe (world copies of the same
    bytes through the host's memory system).  Here each rank copies only its 1/world slice of B
    from pinned host memory, the slices are exchanged with one in-place NCCL all-gather over NVLink,
    each rank multiplies its own row windows, and copies its rows of C back.  Four streams (input
    copy, all-gather, kernels, output copy) and two buffer slots let consecutive calls overlap.

    The reference has no multi-GPU path; the single-GPU call this extends is
    spmm_forward_fp16_tcu_cuda_sptc_mma_parallel_online (mGCN_online.cpp:760), which copies B in and
    C out on every call.
    """

    def __init__(self, fmt, m_local: int, n_cols: int, F: int, rank: int, world: int, group=None):
        import torch.distributed as dist
        from .spmm import SpmmPlan
        self.dist, self.group = dist, group
        self.rank, self.world, self.F = rank, world, F
        self.m_local, self.n_cols = max(m_local, 1), n_cols
        self.dev = fmt.device
        self.plan = SpmmPlan(fmt, self.m_local, n_cols)
        self.per, padded = even_row_split(n_cols, world)
        self.B = [torch.zeros((padded, F), dtype=torch.float16, device=self.dev) for _ in range(2)]
        self.C = [torch.empty((self.m_local, F), dtype=torch.float16, device=self.dev) for _ in range(2)]
        self.s_in, self.s_comm, self.s_k, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(4))
        ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
        self.in_done, self.comm_done, self.k_done, self.out_done = ([ev(), ev()] for _ in range(4))
        self.in_start, self.comm_start, self.k_start, self.out_start = ([ev(), ev()] for _ in range(4))
        self.seq = 0
        self._keep = []

    def my_rows(self):
        """[begin, end) rows of B this rank is expected to provide."""
        b = self.rank * self.per
        return b, min(b + self.per, self.n_cols)

    def submit(self, B_slice_host: torch.Tensor, C_host: torch.Tensor):
        """B_slice_host: pinned fp16 [rows of my_rows(), F]; C_host: pinned fp16 [m_local, F]."""
        s = self.seq & 1
        b0, b1 = self.my_rows()
        if B_slice_host.shape != (b1 - b0, self.F) or C_host.shape != (self.m_local, self.F):
            raise ValueError("slice shapes do not match this rank's share")
        self._keep.append((B_slice_host, C_host))
        Bs, Cs = self.B[s], self.C[s]
        with torch.cuda.stream(self.s_in):
            self.s_in.wait_event(self.k_done[s])           # the kernels two calls back are done with this slot
            self.in_start[s].record(self.s_in)
            Bs[b0:b1].copy_(B_slice_host, non_blocking=True)
            self.in_done[s].record(self.s_in)
        with torch.cuda.stream(self.s_comm):
            self.s_comm.wait_event(self.in_done[s])
            self.comm_start[s].record(self.s_comm)
            if self.world > 1:
                mine = Bs[self.rank * self.per:(self.rank + 1) * self.per]
                self.dist.all_gather_into_tensor(Bs, mine, group=self.group)   # in place: `mine` is its own piece of Bs
            self.comm_done[s].record(self.s_comm)
        with torch.cuda.stream(self.s_k):
            self.s_k.wait_event(self.comm_done[s])
            self.s_k.wait_event(self.out_done[s])           # the output copy two calls back has drained this slot
            self.k_start[s].record(self.s_k)
            self.plan.run(Bs[:self.n_cols], out=Cs)
            self.k_done[s].record(self.s_k)
        with torch.cuda.stream(self.s_out):
            self.s_out.wait_event(self.k_done[s])
            self.out_start[s].record(self.s_out)
            C_host.copy_(Cs, non_blocking=True)
            self.out_done[s].record(self.s_out)
        self.seq += 1

    def wait(self):
        for st in (self.s_in, self.s_comm, self.s_k, self.s_out):
            st.synchronize()
        self._keep.clear()

    def leg_ms(self):
        """Device time of the four legs of the most recent call (after wait()): input copy,
        all-gather, kernels, output copy.  Legs of consecutive calls overlap, so the step time of a
        stream of calls tends to the longest leg, not to their sum."""
        if self.seq == 0:
            return {"h2d_ms": 0.0, "allgather_ms": 0.0, "kernel_ms": 0.0, "d2h_ms": 0.0}
        s = (self.seq - 1) & 1
        return {"h2d_ms": self.in_start[s].elapsed_time(self.in_done[s]),
                "allgather_ms": self.comm_start[s].elapsed_time(self.comm_done[s]),
                "kernel_ms": self.k_start[s].elapsed_time(self.k_done[s]),
                "d2h_ms": self.out_start[s].elapsed_time(self.out_done[s])}
