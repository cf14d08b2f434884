"""Data layer (the reference's dataset class, device-resident): CSR construction equals scipy's
COO -> CSR on the host (CPU test), and the whole chain edge list -> format -> SpMM runs on the
GPU and matches the oracle (GPU test)."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from trspmm import edges_to_csr


def _edges(seed=0, n=300, m=4000):
    g = np.random.default_rng(seed)
    return g.integers(0, n, m), g.integers(0, n + 7, m), n, n + 7


def test_edges_to_csr_matches_scipy():
    from scipy.sparse import coo_matrix
    src, dst, n, k = _edges()
    rp, col = edges_to_csr(torch.from_numpy(src), torch.from_numpy(dst), n, k, window=16)
    n_pad = n + (-n) % 16
    adj = coo_matrix((np.ones(len(src)), (src, dst)), shape=(n_pad, k)).tocsr()   # mdataset2_online.py:62-70
    adj.sort_indices()
    assert rp.dtype == torch.int32 and col.dtype == torch.int32
    assert np.array_equal(rp.numpy(), adj.indptr) and np.array_equal(col.numpy(), adj.indices)


@pytest.mark.gpu
def test_dataset_object_and_forward():
    from trspmm import GCN_dataset_tcu_sptc_cuda_online, kernel_tcu_sptc_cuda_online
    src, dst, n, k = _edges(1, 500, 9000)
    info = GCN_dataset_tcu_sptc_cuda_online({"src_li": src, "dst_li": dst, "num_nodes_src": n, "num_nodes_dst": k},
                                            64, 8, 32, 32, 3, "sp_matrix", 16, 16, seed=3)
    assert info.num_nodes == 512 and info.parts_t == info.t_atomicTensor.shape[0]
    assert info.t_valueTensor.dtype == torch.float16 and info.x.shape == (k, 64)
    out, ms, _, kind = kernel_tcu_sptc_cuda_online(info, 2)
    assert kind == "parallel_mma" and float(ms) > 0 and out.shape == (n, 64)
    arrays = [a.cpu() for a in info.format.arrays()]
    ref = O.spmm_from_format(arrays, info.x.cpu(), info.num_nodes)[:n]
    assert O.scaled_max_error(out.cpu(), ref) <= 2e-5
    # the builder saw exactly the CSR the host path would have built
    want, _ = O.build_format(info.row_pointers.cpu(), info.column_index.cpu(), info.degrees.cpu())
    assert all(torch.equal(a, b) for a, b in zip(arrays, want))
