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
    (r0, r1), (rp_l, col_l, val_l) = shard.shard_for_rank(rp, col, val, rank, world)
    fmt, _ = build_format(rp_l, col_l, val_l)
    full_fmt, _ = build_format(rp, col, val)
    sh = shard.ShardedHostSpmm(fmt, r1 - r0, n_cols, F, rank, world)
    k0, k1 = sh.my_rows()
    ok = True
    g = torch.Generator().manual_seed(11)
    Bs = [torch.randn(n_cols, F, generator=g).half() for _ in range(5)]      # identical on every rank (same seed)
    outs = [torch.full((max(r1 - r0, 1), F), float("nan"), dtype=torch.float16).pin_memory() for _ in Bs]
    slices = [b[k0:k1].clone().pin_memory() for b in Bs]
    for sl, o in zip(slices, outs):
        sh.submit(sl, o)
    sh.wait()
    plan = SpmmPlan(full_fmt, n, n_cols)
    for b, o in zip(Bs, outs):
        want = plan.run(b.to(dev), out_dtype=torch.float16)[r0:r1].cpu()
        ok = ok and bool(torch.equal(o[: r1 - r0], want))
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("sharded host SpMM agrees" if int(flag) == 1 else "sharded host SpMM MISMATCH")
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
