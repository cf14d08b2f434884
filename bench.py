#!/usr/bin/env python3
"""Benchmark of the hybrid sparse hot path: SpMM GFLOP/s (2*nnz*F) and HBM roofline fraction.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A "step" is one SpMM pass C = A'.B of the whole matrix through the fused window kernel, with the
hybrid format built once, on the GPU, before the timed region.  The default workload is the
power-law R-MAT matrix of scale 21 (edge factor 32, symmetrised, self loops, GCN-normalised),
F = 128 fp16 features, generated from a fixed seed on the device (synthetic stand-in for the
SuiteSparse graphs the reference is benchmarked on).  With N > 1 (launched under
torch.distributed.run) the row windows are cut into N nnz-balanced ranges, one per rank, B is
replicated and no collective runs in the data path; timing is CUDA events, max over ranks.

One JSON line is printed by rank 0:
  value ....... whole-job GFLOP/s with every input resident in HBM (kept nnz = nnz the format stores)
  e2e ......... the same metric through the host-buffer C-ABI call (trs_resident_forward): B copied
                from pinned host memory and C copied back inside the timed region, every step
  roofline .... algorithmic bytes of one step / its device time, against the measured HBM peak
  cpu_baseline  torch.sparse CSR fp32 matmul on the host cores (N = 1 only), same matrix

--impl reference times that CPU operator alone (the reference has no CPU SpMM of its own; its
tests' oracle operator is the stand-in) and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT / "tr-spmm_zzx_b200"))
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
LEG_NAMES = ("h2d_ms", "allgather_ms", "kernel_ms", "redeal_ms", "d2h_ms")

WORKLOADS = {
    # name: (generator, kwargs, F)
    "rmat21": ("rmat_graph", dict(scale=21, edge_factor=32, seed=0), 128),
    "rmat20": ("rmat_graph", dict(scale=20, edge_factor=16, seed=0), 128),
    "rmat18": ("rmat_graph", dict(scale=18, edge_factor=32, seed=0), 128),
    "rmat16": ("rmat_graph", dict(scale=16, edge_factor=32, seed=0), 128),
    "clustered": ("clustered_graph", dict(n=262144, community=128, intra=24, glob=4, seed=0), 128),
    "uniform": ("uniform_graph", dict(n=4096, per_row=16, seed=0), 64),
}
DESCRIPTIONS = {
    "rmat21": "R-MAT scale 21, edge factor 32, a=.57 b=c=.19 d=.05, symmetrised, dedup, self loops, GCN norm",
    "rmat20": "R-MAT scale 20, edge factor 16 (GCN config matrix)",
    "rmat18": "R-MAT scale 18, edge factor 32 (reduced-size probe)",
    "rmat16": "R-MAT scale 16, edge factor 32 (profiling case)",
    "clustered": "stochastic-block graph N=262144, 2048 communities of 128, 24 intra + 4 global + self",
    "uniform": "uniform N=4096, 16 distinct columns per row + self",
}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def top_up(self, step_fn, sync_fn, min_samples=3, max_seconds=0.6):
        """A timed region shorter than the sampling period leaves no samples: keep the same kernels
        running, untimed, until a few samples under that load exist."""
        self.extra = 0
        if self.proc is None:
            return
        t0 = time.perf_counter()
        while len(self.samples) < min_samples and time.perf_counter() - t0 < max_seconds:
            for _ in range(8):
                step_fn()
            sync_fn()
            self.extra += 8

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()  # our own child, by handle
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass

    def summary(self):
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                mhz.append(float(s[0])); mx.append(float(s[1]))
            except ValueError:
                continue
            for n, v in zip(names, s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not mhz:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(mhz), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(mhz), "extra_untimed_steps_for_sampling": getattr(self, "extra", 0)}


def make_matrix(workload, device):
    from trspmm import graphs
    gen, kw, F = WORKLOADS[workload]
    rp, col, val = getattr(graphs, gen)(device=device, **kw)
    return rp, col, val, F


# DRAM bytes of one launch of the window kernel on one GPU (dram__bytes_read.sum +
# dram__bytes_write.sum of single-metric, one-pass ncu captures of this very command; the
# summaries under profiles/ give the commands).  Workloads not captured report null.
MEASURED_TRAFFIC = {("rmat21", 128): 8.090e9 + 0.616e9, ("rmat20", 128): 1.647e9 + 0.2582e9}


def algorithmic_bytes(nnz, n_rows, n_cols, F, out_bytes):
    """Canonical-CSR traffic of one SpMM: fp16 value + int32 column per entry, row pointers,
    every B row once, every C element once."""
    return nnz * 6 + (n_rows + 1) * 4 + n_cols * F * 2 + n_rows * F * out_bytes


def dropped_rows(fmt):
    """Local rows that lost an entry to the reference builder's 2-per-group rule
    (block_online.cpp:683-695): a mask bit without a stored slot."""
    if fmt.s_mask.numel() == 0:
        return torch.zeros(0, dtype=torch.int64, device=fmt.device)
    m = fmt.s_mask.to(torch.int32)
    bits = (m & 1) + ((m >> 1) & 1) + ((m >> 2) & 1) + ((m >> 3) & 1)          # [G, 16]
    slots = (fmt.s_pos >= 0).sum(-1).to(torch.int32)                            # [G, 16]
    g, r = torch.nonzero(bits > slots, as_tuple=True)
    return torch.unique(fmt.s_window[g].long() * 16 + r)


def kept_entry_mask(rp_l, col_l, fmt, n_cols):
    """1 for every CSR entry of this rank's rows that the built format still holds, 0 for the
    entries the reference builder's 2-per-group rule dropped (block_online.cpp:683-695): a bit of
    a group's row mask whose position is in neither of the row's two slots."""
    dev = col_l.device
    keep = torch.ones(col_l.numel(), dtype=torch.uint8, device=dev)
    if fmt.s_mask.numel() == 0:
        return keep
    G = fmt.s_mask.numel() // 16
    m = fmt.s_mask.reshape(G, 16).to(torch.int32)
    pos = fmt.s_pos.reshape(G, 16, -1).to(torch.int32)
    cols4 = fmt.s_column.reshape(G, 4).long()
    win = fmt.s_window.reshape(G).long()
    rows_l, cols_l = [], []
    for c in range(4):
        lost = (((m >> c) & 1) == 1) & ~(pos == c).any(-1)
        g, r = torch.nonzero(lost, as_tuple=True)
        rows_l.append(win[g] * 16 + r)
        cols_l.append(cols4[g, c])
    rows_d, cols_d = torch.cat(rows_l), torch.cat(cols_l)
    if rows_d.numel() == 0:
        return keep
    cnt = (rp_l[1:] - rp_l[:-1]).long()
    row_of = torch.repeat_interleave(torch.arange(cnt.numel(), device=dev), cnt)
    keys = row_of * n_cols + col_l.long()              # ascending: canonical CSR
    idx = torch.searchsorted(keys, rows_d * n_cols + cols_d)
    idx = idx.clamp_max(keys.numel() - 1)
    hit = keys[idx] == rows_d * n_cols + cols_d
    keep[idx[hit]] = 0
    return keep


def rel_error(got, ref):
    """|x - y| / max(|y|, 1e-3 * largest |y| of the row): (max, mean) over all elements."""
    scale = torch.maximum(ref.abs(), 1e-3 * ref.abs().amax(dim=1, keepdim=True)).clamp_min(1e-30)
    rel = (got - ref).abs() / scale
    return float(rel.max()), float(rel.mean())


def parity_sample(rp_l, col_l, val_l, fmt, B, out, n_sample=4096, seed=123):
    """Checker run after the timed region, on every rank: `n_sample` of this rank's own rows that
    lost no entry, recomputed as a CSR product in fp32 by torch.sparse on the GPU (fp16-rounded
    values and B, like the kernel's inputs) and compared with the rows the kernel wrote.
    Returns (max relative error, mean relative error, rows checked); the relative error of an
    element is |x - y| / max(|y|, 1e-3 * largest |y| of its row)."""
    dev = out.device
    m = rp_l.numel() - 1
    good = torch.ones(m, dtype=torch.bool, device=dev)
    bad = dropped_rows(fmt)
    good[bad[bad < m]] = False
    pool = torch.nonzero(good).flatten()
    if pool.numel() == 0:
        return 0.0, 0.0, 0
    g = torch.Generator(device=dev).manual_seed(seed)
    rows = pool[torch.randint(0, pool.numel(), (min(n_sample, pool.numel()),), device=dev, generator=g)]
    rows = torch.unique(rows)
    cnt = (rp_l[1:] - rp_l[:-1]).long()[rows]
    sub_rp = torch.zeros(rows.numel() + 1, dtype=torch.int64, device=dev)
    sub_rp[1:] = torch.cumsum(cnt, 0)
    ent = torch.repeat_interleave(rp_l.long()[rows] - sub_rp[:-1], cnt) + torch.arange(int(sub_rp[-1]), device=dev)
    A = torch.sparse_csr_tensor(sub_rp, col_l.long()[ent], val_l[ent].half().float(), (rows.numel(), B.shape[0]))
    ref = torch.sparse.mm(A, B.float())
    got = out[rows].float()
    scale = torch.maximum(ref.abs(), 1e-3 * ref.abs().amax(dim=1, keepdim=True)).clamp_min(1e-30)
    rel = (got - ref).abs() / scale
    return float(rel.max()), float(rel.mean()), int(rows.numel())


def cpu_spmm_time(rp, col, val, B, reps):
    """torch.sparse CSR fp32 matmul on all host threads; median seconds of `reps` runs after 1 warm-up."""
    from oracle import oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    rp, col, val, B = rp.cpu(), col.cpu(), val.cpu(), B.cpu()
    A = torch.sparse_csr_tensor(rp.long(), col.long(), val.float().half().float(), (rp.numel() - 1, B.shape[0]))
    Bf = B.float()
    torch.sparse.mm(A, Bf)
    ts = []
    for _ in range(reps):
        t0 = time.perf_counter()
        torch.sparse.mm(A, Bf)
        ts.append(time.perf_counter() - t0)
    del O
    return statistics.median(ts)


def run_reference(args, rank, world):
    """CPU arm: the oracle operator (torch.sparse CSR matmul) on the host cores, whole matrix."""
    if rank != 0:
        return
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    rp, col, val, F = make_matrix(args.workload, dev)
    n = rp.numel() - 1
    nnz = col.numel()
    B = torch.randn(n, F, device=dev, generator=torch.Generator(device=dev).manual_seed(1)).half()
    rp, col, val, B = rp.cpu(), col.cpu(), val.cpu(), B.cpu()
    torch.set_num_threads(os.cpu_count() or 1)
    A = torch.sparse_csr_tensor(rp.long(), col.long(), val.float().half().float(), (n, n))
    Bf = B.float()
    t0 = time.perf_counter()
    torch.sparse.mm(A, Bf)  # untimed first touch, also sizes the sample
    t_full = time.perf_counter() - t0
    sample = "whole matrix, all nnz (no dropped entries on the CPU path)"
    budget = 150.0
    if t_full * (args.steps + args.warmup) > budget:
        # bounded sample: every s-th block of 4096 rows (all columns), so hubs and tail both appear
        s_every = int(t_full * (args.steps + args.warmup) / budget) + 1
        blocks = torch.arange(0, (n + 4095) // 4096, s_every)
        rows = (blocks[:, None] * 4096 + torch.arange(4096)[None, :]).reshape(-1)
        rows = rows[rows < n]
        cnt = (rp[1:] - rp[:-1]).long()[rows]
        starts = rp.long()[rows]
        sub_rp = torch.zeros(rows.numel() + 1, dtype=torch.int64)
        sub_rp[1:] = torch.cumsum(cnt, 0)
        ent = torch.repeat_interleave(starts - sub_rp[:-1], cnt) + torch.arange(int(sub_rp[-1]))
        A = torch.sparse_csr_tensor(sub_rp, col.long()[ent], val.float()[ent].half().float(), (rows.numel(), n))
        nnz = int(sub_rp[-1])
        sample = f"every {s_every}th block of 4096 rows ({rows.numel()} rows, {nnz} nnz), all columns"
    for _ in range(args.warmup):
        torch.sparse.mm(A, Bf)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        torch.sparse.mm(A, Bf)
    sec = (time.perf_counter() - t0) / args.steps
    gflops = 2.0 * nnz * F / sec / 1e9
    line = {
        "impl": "reference", "metric": "SpMM GFLOP/s (2*nnz*F)", "value": gflops, "unit": "GFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "description": DESCRIPTIONS[args.workload], "n_rows": n, "nnz": nnz,
                   "F": F, "operator": "torch.sparse.mm CSR fp32 x dense fp32 on the host cores"},
        "cpu_baseline": {"value": gflops, "unit": "GFLOP/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": gflops, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank, world, local_rank):
    import torch.distributed as dist
    from trspmm import ResidentSpmm, SpmmPlan, build_format, shard

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback); use --impl reference for the CPU arm")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa_node = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        numa_node = shard.bind_to_gpu_numa_node(local_rank)   # host buffers of this rank local to its GPU

    rp, col, val, F = make_matrix(args.workload, dev)
    n = rp.numel() - 1
    nnz_total = col.numel()
    reorder_note = None
    if args.reorder != "none":
        # labelled configuration: rows re-ordered (columns keep their ids), C comes out in the new row order
        from trspmm import reorder as R
        before = R.window_column_pairs(rp, col)
        rid = R.row_order(rp, col, args.reorder, n_cols=n)
        rp, col, val = R.permute_rows(rp, col, val, rid)
        reorder_note = {"method": args.reorder, "window_column_pairs_before": before,
                        "window_column_pairs_after": R.window_column_pairs(rp, col)}
        del rid
    if world > 1:
        # cut by nnz, re-cut by the k-steps of the built format, then by measured kernel time
        cut_report = {}
        cuts = shard.refined_cuts(rp, col, val, rank, world, F, strict=args.strict, rounds=3, report=cut_report)
        r0, r1 = cuts[rank], cuts[rank + 1]
        rp_l, col_l, val_l = shard.slice_csr(rp, col, val, r0, r1)
    else:
        r0, r1, rp_l, col_l, val_l = 0, n, rp, col, val
    m_local = r1 - r0
    fmt, st = build_format(rp_l, col_l, val_l, strict=args.strict)
    kept_local = st["nnz"] - st["dropped_nnz"]
    B = torch.randn(n, F, device=dev, generator=torch.Generator(device=dev).manual_seed(1)).half()
    plan = SpmmPlan(fmt, max(m_local, 1), n, validate=True)
    out = torch.empty((max(m_local, 1), F), dtype=torch.float16, device=dev)
    cpu_inputs = (rp.cpu(), col.cpu(), val.cpu()) if (world == 1 and not args.no_cpu) else None
    rp_l, col_l, val_l = rp_l.clone(), col_l.clone(), val_l.clone()   # this rank's rows, kept for the parity sample
    del rp, col, val
    torch.cuda.empty_cache()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        plan.run(B, out=out)
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        e0.record()
        for _ in range(args.steps):
            plan.run(B, out=out)
        e1.record()
        sync_all()
        clocks.top_up(lambda: plan.run(B, out=out), torch.cuda.synchronize)
    ms = e0.elapsed_time(e1) / args.steps
    status = plan.status()
    # ---- oracle inside the run: sampled rows of this rank against a CSR product of the same rows
    p_max, p_mean, p_rows = parity_sample(rp_l, col_l, val_l, fmt, B, out)
    del rp_l, col_l, val_l
    torch.cuda.empty_cache()

    # ---- e2e with HOST buffers: B from pinned host memory, C back to the host, every step
    e2e_steps = max(2, min(args.steps, 20))
    h2d = d2h = 0.0
    legs = {k: 0.0 for k in LEG_NAMES}
    if world == 1:
        # the host-buffer C-ABI entries of one GPU
        res = ResidentSpmm(fmt, max(m_local, 1), n, 16, F)
        B_host = B.cpu().pin_memory()
        C_host = torch.empty((max(m_local, 1), F), dtype=torch.float16).pin_memory()
        res.forward(B_host, C_host)
        sync_all()
        # (a) one blocking call per step
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            _, tm = res.forward(B_host, C_host)  # blocks until C is on the host
            h2d += tm.h2d_ms; d2h += tm.d2h_ms
        e2e_sync_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        # (b) the same calls as a stream (submit ... wait): every step still copies its own B in and
        # its own C out; two host buffers of each alternate, as a caller with a producer would hold
        B_hosts = [B_host, B_host.clone().pin_memory()]
        C_hosts = [C_host, torch.empty_like(C_host).pin_memory()]
        for i in range(2):
            res.submit(B_hosts[i], C_hosts[i])
        res.wait()
        sync_all()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            res.submit(B_hosts[i & 1], C_hosts[i & 1])
        res.wait()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        res.close()
        e2e_call = ("trs_resident_submit x steps + trs_resident_wait (format resident; every step copies "
                    "B host->device and C device->host; consecutive steps overlap on three streams)")
        e2e_block_call = "trs_resident_forward, one blocking call per step"
    else:
        # every rank copies its 1/N slice of B over PCIe, the slices are exchanged over NVLink, each
        # rank multiplies its windows, the computed rows are re-dealt over NVLink so that every rank
        # copies the same 1/N of C back (the cost-balanced cut gives the ranks very different row counts)
        sh = shard.ShardedHostSpmm(fmt, m_local, n, F, rank, world, row_cuts=cuts, exchange=args.exchange)
        k0, k1 = sh.my_rows()
        o0, o1 = sh.out_rows()
        B_hosts = [B[k0:k1].cpu().pin_memory() for _ in range(2)]
        C_hosts = [torch.empty((o1 - o0, F), dtype=torch.float16).pin_memory() for _ in range(2)]
        for i in range(2):
            sh.submit(B_hosts[i], C_hosts[i])
        sh.wait()
        sync_all()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            sh.submit(B_hosts[i & 1], C_hosts[i & 1])
            sh.wait()
        e2e_sync_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        sync_all()
        t0 = time.perf_counter()
        for i in range(e2e_steps):
            sh.submit(B_hosts[i & 1], C_hosts[i & 1])
        sh.wait()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        legs = sh.leg_ms()
        e2e_call = (f"ShardedHostSpmm.submit x steps + wait: each rank copies 1/{world} of B host->device, "
                    f"{'NCCL all-gather' if args.exchange == 'nccl' else 'copy-engine pushes'} over NVLink, own windows, "
                    f"computed rows re-dealt over NVLink, 1/{world} of C device->host; steps overlap on five streams")
        e2e_block_call = "ShardedHostSpmm.submit + wait per step"
    if world == 1:
        if not torch.equal(C_hosts[0], C_hosts[1]) or not torch.equal(C_hosts[0], out.cpu()):
            raise RuntimeError("host-buffer calls disagree with the device-resident result")
    else:
        # the rows this rank delivered against the device-resident results of the ranks that computed them
        full = torch.empty((n, F), dtype=torch.float16, device=dev)
        for r in range(world):
            piece = full[cuts[r]:cuts[r + 1]]
            if r == rank and m_local > 0:
                piece.copy_(out[:m_local])
            if piece.numel():
                dist.broadcast(piece, src=r)
        want = full[o0:o1].cpu()
        if not torch.equal(C_hosts[0], C_hosts[1]) or not torch.equal(C_hosts[0], want):
            raise RuntimeError("host-buffer calls disagree with the device-resident result")
        del full, want

    kept = torch.tensor([float(kept_local), ms, e2e_ms, e2e_sync_ms, p_max, p_mean, float(p_rows)], device=dev,
                        dtype=torch.float64)
    if world > 1:
        tot = kept.clone()
        dist.all_reduce(tot[0:1], op=dist.ReduceOp.SUM)
        dist.all_reduce(tot[1:6], op=dist.ReduceOp.MAX)
        dist.all_reduce(tot[6:7], op=dist.ReduceOp.SUM)
        kept_total, ms, e2e_ms, e2e_sync_ms = float(tot[0]), float(tot[1]), float(tot[2]), float(tot[3])
        p_max, p_mean, p_rows = float(tot[4]), float(tot[5]), int(tot[6])
        legs_t = torch.tensor([legs[k] for k in LEG_NAMES], device=dev, dtype=torch.float64)
        dist.all_reduce(legs_t, op=dist.ReduceOp.MAX)
        legs = {k: float(v) for k, v in zip(LEG_NAMES, legs_t)}
    else:
        kept_total = float(kept_local)
    if p_max > 1e-2 or p_mean > 1e-3:
        raise RuntimeError(f"parity sample failed: max rel {p_max}, mean rel {p_mean} (bars 1e-2 / 1e-3)")

    if rank == 0:
        peak, peak_src = peaks()
        alg = algorithmic_bytes(kept_total, n, n, F, 2)  # whole job; B counted once per GPU below
        alg_job = alg + (world - 1) * n * F * 2          # every rank streams its own replica of B
        alg_rank = algorithmic_bytes(kept_local, m_local, n, F, 2)
        achieved = alg_rank / (ms * 1e-3) / 1e9
        line = {
            "metric": "SpMM GFLOP/s (2*nnz*F)", "value": 2.0 * kept_total * F / (ms * 1e-3) / 1e9, "unit": "GFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16 in / f32 accumulate",
            "data": "synthetic",
            "config": {"workload": args.workload + ("" if reorder_note is None else "+rows:" + args.reorder)
                       + ("+strict" if args.strict else ""),
                       "format": "lossless (strict): the entries the reference's builder drops ride the CUDA-core route"
                                 if args.strict else "reference-compatible (drops reproduced)",
                       "reorder": reorder_note, "description": DESCRIPTIONS[args.workload], "n_rows": n,
                       "nnz": nnz_total, "kept_nnz": int(kept_total), "F": F, "out": "f16",
                       "parallelism": f"row-window shards x{world} balanced by k-steps and measured kernel time, B replicated, no collective",
                       "l2": "inputs larger than L2 (no flush)" if n * F * 2 > 126e6 else "B fits L2",
                       "build_ms_rank0": st["build_ms"], "tiles_rank0": st["tiles"], "tc_blocks_rank0": st["tc_blocks"],
                       "cut_refinement_kernel_ms_per_rank": cut_report.get("times_ms") if world > 1 else None},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_source": peak_src, "algorithmic_bytes_per_step_rank0": alg_rank,
                         "algorithmic_bytes_per_step_job": alg_job,
                         "traffic": MEASURED_TRAFFIC.get((args.workload, F)) if (world == 1 and reorder_note is None
                                                                                  and not args.strict) else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch (profiles/)",
                         "kernel": "k_window_spmm_warp"},
            "e2e": {"value": 2.0 * kept_total * F / (e2e_ms * 1e-3) / 1e9, "unit": "GFLOP/s",
                    "ms_per_step": e2e_ms, "h2d_bytes_per_step": n * F * 2, "d2h_bytes_per_step": n * F * 2,
                    "h2d_ms": h2d / e2e_steps if world == 1 else legs["h2d_ms"],
                    "d2h_ms": d2h / e2e_steps if world == 1 else legs["d2h_ms"],
                    "allgather_ms": legs["allgather_ms"], "kernel_ms": legs["kernel_ms"] if world > 1 else ms,
                    "redeal_ms": legs["redeal_ms"],
                    "legs": "device time of each leg of the last streamed call, max over ranks" if world > 1 else
                            "copy legs of the blocking calls (trs_timing)",
                    "steps": e2e_steps, "numa_node_rank0": numa_node,
                    "call": e2e_call,
                    "blocking_call": {"value": 2.0 * kept_total * F / (e2e_sync_ms * 1e-3) / 1e9, "unit": "GFLOP/s",
                                      "ms_per_step": e2e_sync_ms, "call": e2e_block_call}},
            "gpu_launches": plan.launches * args.steps,
            "clocks": clocks.summary(), "kernel_status": status,
            "parity_sample": {"max_rel": p_max, "mean_rel": p_mean, "rows": p_rows, "bars": [1e-2, 1e-3],
                              "checker": "torch.sparse CSR fp32 product of sampled rows without dropped entries, on every "
                                         "rank's own rows, worst rank reported"},
        }
        if cpu_inputs is not None:
            reps = 3
            sec = cpu_spmm_time(*cpu_inputs, B, reps)
            line["cpu_baseline"] = {"value": 2.0 * nnz_total * F / sec / 1e9, "unit": "GFLOP/s", "cores": os.cpu_count(),
                                    "kind": "port", "sample": f"whole matrix, median of {reps} runs of torch.sparse.mm "
                                    f"CSR fp32 ({sec * 1e3:.0f} ms each)"}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_sddmm(args):
    """SDDMM (BASELINE config 3): X, Y dense N x 64 fp16 on the pattern of the chosen workload."""
    from trspmm import sddmm
    dev = torch.device("cuda", 0)
    rp, col, val, _ = make_matrix(args.workload, dev)
    n, nnz, K = rp.numel() - 1, col.numel(), 64
    g = torch.Generator(device=dev).manual_seed(1)
    X = torch.randn(n, K, device=dev, generator=g).half()
    Y = torch.randn(n, K, device=dev, generator=g).half()
    from trspmm import SddmmPlan
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    plan = SddmmPlan(rp, col, n)   # built once per pattern, like the SpMM format; reported separately
    torch.cuda.synchronize()
    plan_ms = (time.perf_counter() - t0) * 1e3
    out = plan.run(X, Y)

    def timed(fn):
        for _ in range(args.warmup):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / args.steps

    with ClockSampler(0) as clocks:
        ms = timed(lambda: plan.run(X, Y, out=out))
    ms_unplanned = timed(lambda: sddmm(rp, col, X, Y, out=out))
    peak, src = peaks()
    alg = nnz * 4 + (n + 1) * 4 + 2 * n * K * 2 + nnz * 2
    line = {"metric": "SDDMM GFLOP/s (2*nnz*K)", "value": 2.0 * nnz * K / (ms * 1e-3) / 1e9, "unit": "GFLOP/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "dtype": "f16 in / f32 accumulate", "data": "synthetic",
            "config": {"workload": args.workload, "op": "sddmm", "n_rows": n, "nnz": nnz, "K": K,
                       "call": "trs_sddmm_plan_run (pattern planned once)", "plan_ms": plan_ms,
                       "window_column_pairs": plan.n_pairs, "ms_per_step_unplanned_trs_sddmm": ms_unplanned},
            "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / (ms * 1e-3) / 1e9 / peak, "peak_source": src, "traffic": 184.4e6 if args.workload == "clustered" else None,
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch (profiles/)",
                         "kernel": "k_sddmm_tc_pipe"},
            "gpu_launches": args.steps, "clocks": clocks.summary()}
    if not args.no_cpu:
        from oracle import oracle as O
        torch.set_num_threads(os.cpu_count() or 1)
        rpc, colc, Xc, Yc = rp.cpu(), col.cpu(), X.cpu(), Y.cpu()
        sample = min(nnz, 4_000_000)   # bounded sample: the first rows holding ~4 M entries
        rows = int(torch.searchsorted(rpc.long(), torch.tensor(sample))) or 1
        t0 = time.perf_counter()
        O.sddmm_csr(rpc[:rows + 1], colc[:int(rpc[rows])], Xc[:rows], Yc)
        sec = time.perf_counter() - t0
        line["cpu_baseline"] = {"value": 2.0 * int(rpc[rows]) * K / sec / 1e9, "unit": "GFLOP/s", "cores": os.cpu_count(),
                                "kind": "port", "sample": f"first {rows} rows ({int(rpc[rows])} entries), gathered fp32 dot products"}
    print(json.dumps(line), flush=True)


class _QuietStdout:
    """The reference's CPU modules print tables; keep them out of this program's stdout."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        self.null = os.open(os.devnull, os.O_WRONLY)
        os.dup2(self.null, 1)

    def __exit__(self, *a):
        os.dup2(self.saved, 1)
        os.close(self.saved)
        os.close(self.null)


def _row_sample(rp, col, val, r0, rows):
    """CSR of rows [r0, r0 + rows) of the matrix (columns keep their ids), on the CPU."""
    rp = rp.cpu()
    r1 = min(r0 + rows, rp.numel() - 1)
    e0, e1 = int(rp[r0]), int(rp[r1])
    return (rp[r0:r1 + 1] - e0).contiguous(), col[e0:e1].cpu().contiguous(), val[e0:e1].cpu().contiguous(), e1 - e0


def _bounded_cpu(fn, rp, col, val, budget_s=8.0, first_rows=1024):
    """Times fn(sample) on row samples that start a third of the way into the matrix and double in
    length until one run takes budget_s / 4 or the whole matrix is covered (the reference's CPU
    builder is quadratic in the columns of a window, so the hub rows of an R-MAT graph, which sit at
    ids with few set bits, are kept out of small samples).  Returns (seconds, entries, description)."""
    n = rp.numel() - 1
    rows = min(first_rows, n)
    while True:
        r0 = 0 if rows >= n else min((n // 3) // 16 * 16, (n - rows) // 16 * 16)
        sample = _row_sample(rp, col, val, r0, rows)
        with _QuietStdout():
            t0 = time.perf_counter()
            fn(*sample[:3])
            sec = time.perf_counter() - t0
        best = (sec, sample[3], f"rows [{r0}, {min(r0 + rows, n)}) of the workload: {sample[3]} entries, one run")
        if sec >= budget_s / 4 or rows >= n:
            return best
        rows = min(n, rows * 2)


def run_build(args):
    """Format builder (block_sptc_2to4_online, block_online.cpp:545-871): CSR on the device -> the 29 arrays."""
    from trspmm import build_format
    dev = torch.device("cuda", 0)
    rp, col, val, _ = make_matrix(args.workload, dev)
    n, nnz = rp.numel() - 1, col.numel()
    from trspmm.builder import arena_bytes
    steps = max(1, min(args.steps, 10))
    # headline: trs_build_fill into a caller-owned arena sized once by trs_build_query (the call allocates nothing)
    arena = torch.empty(arena_bytes(n, nnz), dtype=torch.uint8, device=dev)
    for _ in range(min(args.warmup, 3)):
        fmt, st = build_format(rp, col, val, arena=arena)
        del fmt
    torch.cuda.synchronize()
    with ClockSampler(0) as clocks:
        t0 = time.perf_counter()
        kernel_ms = 0.0
        for _ in range(steps):
            fmt, st = build_format(rp, col, val, arena=arena)
            kernel_ms += st["build_ms"]
            out_bytes = sum(a.numel() * a.element_size() for a in fmt.arrays())
            del fmt
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) * 1e3 / steps
    arena_used = st["arena_used"]
    del arena
    torch.cuda.empty_cache()
    # beside it: trs_build_create, which allocates outputs and temporaries itself on every call
    fmt, _ = build_format(rp, col, val)
    del fmt
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(min(steps, 3)):
        fmt, _ = build_format(rp, col, val)
        del fmt
    torch.cuda.synchronize()
    ms_create = (time.perf_counter() - t0) * 1e3 / min(steps, 3)
    peak, src = peaks()
    alg = nnz * 12 + (n + 1) * 4 + out_bytes   # CSR in (i32 column, f32 value, row pointers... read once) + every array written once
    line = {"metric": "format build M nnz/s", "value": nnz / (ms * 1e-3) / 1e6, "unit": "Mnnz/s", "n_gpus": 1,
            "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "dtype": "i32 / u8 / f32->f16", "data": "synthetic",
            "config": {"workload": args.workload, "op": "build", "n_rows": n, "nnz": nnz,
                       "call": "trs_build_fill into a caller-owned arena (wall time; no allocation inside the call)",
                       "device_ms_per_build": kernel_ms / steps, "output_bytes": out_bytes,
                       "arena_bytes_query": arena_bytes(n, nnz), "arena_bytes_used": arena_used,
                       "ms_per_step_trs_build_create": ms_create,
                       "groups": st["groups"], "tiles": st["tiles"], "tc_blocks": st["tc_blocks"]},
            "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / (ms * 1e-3) / 1e9 / peak, "peak_source": src, "traffic": None,
                         "kernel": "kb_* pipeline (CUB sorts dominate)"},
            "gpu_launches": None, "clocks": clocks.summary()}
    if not args.no_cpu:
        from oracle import oracle as O
        have_ref = O.reference_module("Libra5BlockOnline") is not None
        fn = (lambda a, b, c: O.reference_builder(a, b, c)) if have_ref else (lambda a, b, c: O.build_format(a, b, c))
        sec, entries, what = _bounded_cpu(fn, rp, col, val)
        line["cpu_baseline"] = {"value": entries / sec / 1e6, "unit": "Mnnz/s", "cores": 1,
                                "kind": "reference" if have_ref else "port", "sample": what}
    print(json.dumps(line), flush=True)


def run_match24(args):
    """2:4 matching statistics (the reference's match_2to4* modules) on the GPU: the three variants with a
    CPU reference (its compiled modules timed beside them on a bounded sample) and the two restated
    from the reference's GPU matchers (online, cuda: no CPU module exists for those)."""
    from trspmm import match24
    dev = torch.device("cuda", 0)
    rp, col, val, _ = make_matrix(args.workload, dev)
    n, nnz = rp.numel() - 1, col.numel()
    peak, src = peaks()
    ref_names = {"para_dr": ("matching_utils", "match_2to4"), "hash": ("matching_utils_hash", "match_2to4_hash"),
                 "bucket": ("matching_utils_bucket", "match_2to4_bucket")}
    out = {}
    for variant in ("para_dr", "hash", "bucket", "online", "cuda"):
        for _ in range(args.warmup):
            match24.match_stats(variant, rp, col)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            match24.match_stats(variant, rp, col)   # synchronous: returns the statistics
        ms = (time.perf_counter() - t0) * 1e3 / args.steps
        alg = nnz * 4 + (n + 1) * 4
        out[variant] = {"ms": ms, "Mnnz_per_s": nnz / (ms * 1e-3) / 1e6, "GBps": alg / (ms * 1e-3) / 1e9,
                        "frac": alg / (ms * 1e-3) / 1e9 / peak}
        if not args.no_cpu and variant in ref_names:
            from oracle import oracle as O
            mod = O.reference_module(ref_names[variant][0])
            if mod is not None:
                f = getattr(mod, ref_names[variant][1])
                sec, entries, what = _bounded_cpu(lambda a, b, c: f(a.numpy(), b.numpy(), c.numpy()), rp, col, val, budget_s=4.0)
                out[variant]["cpu_reference"] = {"Mnnz_per_s": entries / sec / 1e6, "cores": os.cpu_count(), "sample": what}
    best = out["para_dr"]
    line = {"metric": "2:4 matching statistics M nnz/s (para_dr variant)", "value": best["Mnnz_per_s"], "unit": "Mnnz/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": best["ms"], "higher_is_better": True,
            "dtype": "i32", "data": "synthetic",
            "config": {"workload": args.workload, "op": "match24", "n_rows": n, "nnz": nnz, "variants": out,
                       "call": "trs_match24_stats (synchronous; wall time)"},
            "roofline": {"bound": "hbm", "achieved": best["GBps"], "peak": peak, "unit": "GB/s", "frac": best["frac"],
                         "peak_source": src, "traffic": None, "kernel": "km_para_dr"},
            "gpu_launches": None}
    if "cpu_reference" in best:
        line["cpu_baseline"] = {"value": best["cpu_reference"]["Mnnz_per_s"], "unit": "Mnnz/s", "cores": os.cpu_count(),
                                "kind": "reference", "sample": best["cpu_reference"]["sample"]}
    print(json.dumps(line), flush=True)


def run_gcn(args, rank, world, local_rank):
    """Two-layer GCN forward (BASELINE config 4 shape): features 256 -> 128 -> 64, ReLU between."""
    import torch.distributed as dist
    from trspmm import ShardedGCN2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    rp, col, val, _ = make_matrix(args.workload, dev)
    n, nnz = rp.numel() - 1, col.numel()
    g = torch.Generator(device=dev).manual_seed(1)
    X = torch.randn(n, 256, device=dev, generator=g).half()
    W1 = (torch.randn(256, 128, device=dev, generator=g) * 0.02).half()
    W2 = (torch.randn(128, 64, device=dev, generator=g) * 0.02).half()
    from trspmm import shard
    cut_report = {}
    cuts = (shard.refined_cuts(rp, col, val, rank, world, (128, 64), strict=args.strict, rounds=4, report=cut_report)
            if world > 1 else None)
    model = ShardedGCN2(rp, col, val, rank, world, cuts=cuts, strict=args.strict)
    model.multicast = not args.no_multicast
    kept = model.stats["nnz"] - model.stats["dropped_nnz"]
    for _ in range(args.warmup):
        model.forward(X, W1, W2, gather=args.gather)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        model.forward(X, W1, W2, gather=args.gather)
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps, float(kept)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.barrier()
        ms = t[0:1].clone(); dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        k = t[1:2].clone(); dist.all_reduce(k, op=dist.ReduceOp.SUM)
        t = torch.cat([ms, k])
    model.profile = True
    model.forward(X, W1, W2, gather=args.gather)
    breakdown = {k: round(v, 3) for k, v in model.last_breakdown.items()}
    # checker, after the timed region, on every rank: the whole two-layer forward recomputed with
    # torch.sparse (fp32 products, fp16 at the same stage boundaries) over the entries the built
    # format holds, compared on this rank's own rows
    model.profile = False
    out = model.forward(X, W1, W2, gather=args.gather)
    r0, r1 = model.r0, model.r1
    keep = torch.ones(nnz, dtype=torch.uint8, device=dev)
    if r1 > r0 and not args.strict:     # the lossless format keeps every entry
        e_lo, e_hi = int(rp[r0]), int(rp[r1])
        rp_l = (rp[r0:r1 + 1] - rp[r0]).contiguous()
        keep[e_lo:e_hi] = kept_entry_mask(rp_l, col[e_lo:e_hi], model.fmt, n)
    if world > 1:
        dist.all_reduce(keep, op=dist.ReduceOp.MIN)
    A = torch.sparse_csr_tensor(rp.long(), col.long(), val.half().float() * keep.float(), (n, n))
    h1_ref = torch.relu(torch.sparse.mm(A, torch.matmul(X, W1).float())).half()
    ref = torch.sparse.mm(A, torch.matmul(h1_ref, W2).float())[r0:r1]
    # two fp16 roundings sit between the input and the output, and W2 has both signs: an output far
    # below its row's largest magnitude carries the rounding noise of larger terms, so the largest
    # error is taken against the row's largest |reference| and the mean against the element itself
    if r1 > r0:
        p_mean = rel_error(out.float(), ref)[1]
        p_max = float(((out.float() - ref).abs() / ref.abs().amax(dim=1, keepdim=True).clamp_min(1e-30)).max())
    else:
        p_max = p_mean = 0.0
    del A, ref, h1_ref
    pt = torch.tensor([p_max, p_mean], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(pt, op=dist.ReduceOp.MAX)
    p_max, p_mean = float(pt[0]), float(pt[1])
    if p_max > 4e-3 or p_mean > 1e-3:
        raise RuntimeError(f"parity check failed: max row-normalised error {p_max}, mean rel {p_mean} (bars 4e-3 / 1e-3)")
    if rank == 0:
        ms, kept_total = float(t[0]), float(t[1])
        flops = 2.0 * kept_total * (128 + 64) + 2.0 * n * (256 * 128 + 128 * 64)
        print(json.dumps({"metric": "GCN 2-layer forward GFLOP/s (SpMM 2*nnz*(128+64) + dense GEMMs, counted once)",
                          "value": flops / (ms * 1e-3) / 1e9, "unit": "GFLOP/s", "n_gpus": world, "steps": args.steps,
                          "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
                          "dtype": "f16 in / f32 accumulate", "data": "synthetic",
                          "config": {"workload": args.workload, "op": "gcn2", "features": [256, 128, 64], "gather": args.gather + ("+multicast" if (args.gather == "gemm_bcast" and world > 2 and not args.no_multicast) else ""),
                                     "n_rows": n, "nnz": nnz, "kept_nnz": int(kept_total),
                                     "format": "lossless (strict)" if args.strict else "reference-compatible (drops reproduced)",
                                     "gather_bytes_received_rank0": model.gather_bytes,
                                     "stage_ms_rank0": breakdown,
                                     "cut_refinement_kernel_ms_per_rank": cut_report.get("times_ms")},
                          "parity_sample": {"max_row_normalised": p_max, "mean_rel": p_mean, "rows": n, "bars": [4e-3, 1e-3],
                                            "checker": "torch.sparse CSR fp32 two-layer forward over the entries the built "
                                                       "format holds, fp16 at the stage boundaries, every rank's own rows, "
                                                       "worst rank reported"}}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="rmat21", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--reorder", default="none", choices=["none", "minhash", "hub", "degree"],
                    help="spmm: re-order the rows first (a separate, labelled configuration)")
    ap.add_argument("--strict", action="store_true",
                    help="spmm: lossless format (no dropped entries; value counts all nnz) - a separate, labelled configuration")
    ap.add_argument("--op", default="spmm", choices=["spmm", "sddmm", "gcn", "build", "match24"],
                    help="spmm (default, the headline metric); sddmm and gcn are the other benchmark configurations")
    ap.add_argument("--exchange", default="nccl", choices=["nccl", "push"],
                    help="multi-GPU host-buffer path: how the ranks exchange their slices of B")
    ap.add_argument("--no-multicast", action="store_true",
                    help="gcn, gather=gemm_bcast: one store per peer instead of one store through the NVLink multicast "
                         "mapping (multimem.st), which is the default where the box offers one")
    ap.add_argument("--gather", default="gemm_bcast", choices=["h1", "z2", "fused", "push", "gemm_bcast"], help="gcn: which matrix the ranks exchange")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif args.op == "sddmm":
        if rank == 0:
            run_sddmm(args)
    elif args.op == "gcn":
        run_gcn(args, rank, world, local_rank)
    elif args.op == "build":
        if rank == 0:
            run_build(args)
    elif args.op == "match24":
        if rank == 0:
            run_match24(args)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
