"""torchrun worker: host-buffer SpMM sharded over the ranks (ShardedHostSpmm); every rank checks
its rows against the un-sharded device result.  Launched by tests/test_shard_gpu.py."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "tr-spmm_zzx_b200"))
sys.path.insert(0, str(ROOT))

from trspmm import SpmmPlan, build_format, graphs, shard  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rp, col, val = graphs.rmat_graph(12, 16, seed=3)
    n = rp.numel() - 1 - 5                       # not a multiple of the world size or of the window
    rp, col, val = rp[: n + 1].to(dev), col[: int(rp[n])].to(dev), val[: int(rp[n])].to(dev)
    n_cols = rp.numel() - 1 + 5
    F = 64
    cuts = shard.balanced_window_cuts(rp, world)
    r0, r1 = cuts[rank], cuts[rank + 1]
    rp_l, col_l, val_l = shard.slice_csr(rp, col, val, r0, r1)
    fmt, _ = build_format(rp_l, col_l, val_l)
    full_fmt, _ = build_format(rp, col, val)
    plan = SpmmPlan(full_fmt, n, n_cols)
    ok = True
    g = torch.Generator().manual_seed(11)
    Bs = [torch.randn(n_cols, F, generator=g).half() for _ in range(5)]      # identical on every rank (same seed)
    wants = [plan.run(b.to(dev), out_dtype=torch.float16).cpu() for b in Bs]
    # the rank's computed rows / an even share of the rows re-dealt over NVLink, NCCL / copy-engine exchange of B
    for row_cuts, exchange in ((None, "nccl"), (cuts, "nccl"), (cuts, "push")):
        if world == 1 and row_cuts is not None:
            continue
        sh = shard.ShardedHostSpmm(fmt, r1 - r0, n_cols, F, rank, world, row_cuts=row_cuts, exchange=exchange)
        k0, k1 = sh.my_rows()
        o0, o1 = (r0, r1) if row_cuts is None else sh.out_rows()
        if row_cuts is not None:
            assert (o0, o1) == shard.even_output_rows(n, world, rank)
        rows = max(r1 - r0, 1) if row_cuts is None else o1 - o0
        outs = [torch.full((rows, F), float("nan"), dtype=torch.float16).pin_memory() for _ in Bs]
        slices = [b[k0:k1].clone().pin_memory() for b in Bs]
        for sl, o in zip(slices, outs):
            sh.submit(sl, o)
        sh.wait()
        for want, o in zip(wants, outs):
            ok = ok and bool(torch.equal(o[: o1 - o0], want[o0:o1]))
        legs = sh.leg_ms()
        ok = ok and all(v >= 0.0 for v in legs.values())
        del sh
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("sharded host SpMM agrees" if int(flag) == 1 else "sharded host SpMM MISMATCH")
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
