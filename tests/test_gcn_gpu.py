"""Two-layer GCN forward (BASELINE config 4 shape, reduced size) against the fp32 CPU expression
over the matrix the format encodes; single rank here, two ranks via torchrun when 2 GPUs exist."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from oracle import oracle as O
from trspmm import ShardedGCN2, graphs

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _reference(rp, col, val, X, W1, W2):
    n = rp.numel() - 1
    arrays, _ = O.build_format(rp, col, val)
    r, c, v = O.decode_format(arrays)
    A = torch.sparse_coo_tensor(torch.stack([torch.from_numpy(r), torch.from_numpy(c)]),
                                torch.from_numpy(v).half().float(), (n, n)).coalesce().to_sparse_csr()
    z1 = (X.float() @ W1.float()).half().float()
    h1 = torch.relu(torch.sparse.mm(A, z1)).half().float()
    z2 = (h1 @ W2.float()).half().float()
    return torch.sparse.mm(A, z2)


@pytest.mark.parametrize("gather", ["h1", "z2", "gemm_bcast"])
def test_gcn2_single_rank(gather):
    rp, col, val = graphs.rmat_graph(12, 16, seed=4)
    n = rp.numel() - 1
    g = torch.Generator().manual_seed(0)
    X = torch.randn(n, 256, generator=g).half()
    W1 = (torch.randn(256, 128, generator=g) * 0.02).half()
    W2 = (torch.randn(128, 64, generator=g) * 0.02).half()
    model = ShardedGCN2(rp.cuda(), col.cuda(), val.cuda())
    out = model.forward(X.cuda(), W1.cuda(), W2.cuda(), gather=gather).cpu()
    ref = _reference(rp, col, val, X, W1, W2)
    # The hidden activations are rounded to fp16 twice on both sides, after sums taken in different
    # orders, so errors are fp16-sized relative to a row's magnitude (not to each element's own):
    # bar = 1e-2 of the row maximum, and 1e-3 on average.
    err = O.scaled_max_error(out, ref)
    mean = float((out.float() - ref).abs().mean() / ref.abs().mean())
    assert err <= 1e-2 and mean <= 3e-3, (err, mean)


def test_gcn2_two_ranks_match_single_rank():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533",
                        str(ROOT / "tests" / "multi_gcn_worker.py")], capture_output=True, text=True, env=env,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "GCN2 ranks agree" in r.stdout


@pytest.mark.parametrize("rows,K,N", [(1000, 128, 64), (16, 32, 32), (4099, 256, 128), (33, 64, 64)])
def test_rows_gemm_bcast_matches_a_dense_product(rows, K, N):
    """trs_rows_gemm_bcast with two destination buffers on one GPU: both get H @ W at the row offset,
    nothing else is touched."""
    from trspmm.gcn import rows_gemm_bcast
    g = torch.Generator().manual_seed(rows)
    H = torch.randn(rows, K, generator=g).half().cuda()
    W = (torch.randn(K, N, generator=g) * 0.1).half().cuda()
    row0, total = 7, rows + 20
    dsts = [torch.full((total, N), 3.0, dtype=torch.float16, device="cuda") for _ in range(2)]
    rows_gemm_bcast(H, W, [d.data_ptr() for d in dsts], row0)
    torch.cuda.synchronize()
    ref = (H.float() @ W.float())
    for d in dsts:
        got = d[row0:row0 + rows].float()
        assert torch.allclose(got, ref, rtol=2e-3, atol=2e-3), float((got - ref).abs().max())
        assert bool((d[:row0] == 3.0).all()) and bool((d[row0 + rows:] == 3.0).all())
    assert torch.equal(dsts[0], dsts[1])
    with pytest.raises(Exception):
        rows_gemm_bcast(H, W, [], 0)
    with pytest.raises(Exception):
        rows_gemm_bcast(H[:, :K - 8].contiguous(), W[:K - 8].contiguous(), [dsts[0].data_ptr()], 0)   # K not a multiple of 16


def test_rows_gemm_bcast_rejects_shapes_it_is_not_laid_out_for():
    from trspmm.gcn import rows_gemm_bcast
    from trspmm._lib import TrsError
    H = torch.zeros(16, 16, dtype=torch.float16, device="cuda")
    W = torch.zeros(16, 32, dtype=torch.float16, device="cuda")          # N > K
    out = torch.zeros(16, 32, dtype=torch.float16, device="cuda")
    with pytest.raises(TrsError):
        rows_gemm_bcast(H, W, [out.data_ptr()], 0)
    W48 = torch.zeros(16, 48, dtype=torch.float16, device="cuda")         # N not 32 / 64 / 128
    with pytest.raises(TrsError):
        rows_gemm_bcast(H, W48, [out.data_ptr()], 0)
