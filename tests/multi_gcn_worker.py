"""torchrun worker: two-layer GCN on 2 ranks; rank 0 checks the gathered result against the
single-rank run.  Launched by tests/test_gcn_gpu.py (not collected by pytest itself)."""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "tr-spmm_zzx_b200"))
sys.path.insert(0, str(ROOT))

from trspmm import ShardedGCN2, graphs  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    rp, col, val = graphs.rmat_graph(13, 16, seed=6)
    n = rp.numel() - 1
    g = torch.Generator().manual_seed(0)
    X = torch.randn(n, 256, generator=g).half().to(dev)
    W1 = (torch.randn(256, 128, generator=g) * 0.02).half().to(dev)
    W2 = (torch.randn(128, 64, generator=g) * 0.02).half().to(dev)
    rp, col, val = rp.to(dev), col.to(dev), val.to(dev)
    ok = True
    for gather in ("h1", "z2", "fused", "push", "gemm_bcast"):
        model = ShardedGCN2(rp, col, val, rank, world)
        mine = model.forward(X, W1, W2, gather=gather)
        full = torch.zeros(n, 64, dtype=torch.float16, device=dev)
        full[model.r0:model.r1] = mine
        model._exchange(full)
        if rank == 0:
            single = ShardedGCN2(rp, col, val).forward(X, W1, W2, gather=gather)
            if gather in ("h1", "fused", "gemm_bcast"):   # window ownership is exclusive and every row's GEMM is the same arithmetic: bit-identical
                ok = ok and bool(torch.equal(full, single))
            else:                # the local GEMM has a different M, cuBLAS may tile it differently
                ok = ok and bool(torch.allclose(full.float(), single.float(), rtol=1e-2, atol=1e-3))
    # gemm_bcast again on later calls (its two Z2 buffers alternate): the same rows, bit for bit
    model = ShardedGCN2(rp, col, val, rank, world)
    model.multicast = False
    one = model.forward(X, W1, W2, gather="gemm_bcast").clone()
    for _ in range(3):
        ok = ok and bool(torch.equal(model.forward(X, W1, W2, gather="gemm_bcast"), one))
    # ... and with the rows stored once through the NVLink multicast mapping, where the box offers one
    model.multicast, model.multicast_min_world = True, 2      # (by default the model takes this path from three ranks on)
    for _ in range(2):
        ok = ok and bool(torch.equal(model.forward(X, W1, W2, gather="gemm_bcast"), one))
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    dist.destroy_process_group()
    if rank == 0:
        print("GCN2 ranks agree" if ok else "GCN2 MISMATCH")
    sys.exit(0 if int(flag) == 1 else 1)


if __name__ == "__main__":
    main()
