"""Matrix ingestion: the file layouts the reference's drivers read."""
import numpy as np
import scipy.sparse as sp
import torch

from trspmm import graphs
from trspmm.io import load_matrix


def _dense(rp, col, val, shape):
    return sp.csr_matrix((val.numpy(), col.numpy(), rp.numpy()), shape=shape).toarray()


def test_matrix_market_and_npz_layouts(tmp_path):
    from scipy.io import mmwrite
    rng = np.random.default_rng(0)
    a = sp.random(37, 53, density=0.1, random_state=1, format="coo", dtype=np.float32)
    mmwrite(str(tmp_path / "a.mtx"), a)
    rp, col, val, shape = load_matrix(str(tmp_path / "a.mtx"))
    assert shape == (37, 53) and rp.dtype == torch.int32 and col.dtype == torch.int32 and val.dtype == torch.float32
    assert np.allclose(_dense(rp, col, val, shape), a.toarray())
    # symmetric pattern file
    s = sp.random(20, 20, density=0.2, random_state=2, format="coo")
    s = ((s + s.T) > 0).astype(np.int8)
    mmwrite(str(tmp_path / "s.mtx"), sp.coo_matrix(s), field="pattern", symmetry="symmetric")
    rp, col, val, shape = load_matrix(str(tmp_path / "s.mtx"))
    assert np.array_equal(_dense(rp, col, val, shape) != 0, s.toarray() != 0) and float(val.max()) == 1.0
    # scipy npz
    sp.save_npz(str(tmp_path / "b.npz"), a.tocsr())
    rp, col, val, shape = load_matrix(str(tmp_path / "b.npz"))
    assert np.allclose(_dense(rp, col, val, shape), a.toarray())
    # edge-list npz, both variants, with a duplicate edge (summed like scipy's tocsr)
    src = np.array([0, 0, 3, 3, 5]); dst = np.array([1, 1, 2, 0, 4])
    np.savez(tmp_path / "e1.npz", src_li=src, dst_li=dst, num_nodes_src=6, num_nodes_dst=5)
    rp, col, val, shape = load_matrix(str(tmp_path / "e1.npz"))
    assert shape == (6, 5) and rp.tolist() == [0, 1, 1, 1, 3, 3, 4] and col.tolist() == [1, 0, 2, 4] and val.tolist() == [2, 1, 1, 1]
    np.savez(tmp_path / "e2.npz", src_li=src, dst_li=dst, data=rng.random(5).astype(np.float32), shape=np.array([6, 5]))
    assert load_matrix(str(tmp_path / "e2.npz"))[3] == (6, 5)
    # canonical CSR: ascending, duplicate-free columns per row -> what the builder requires
    rp, col, val = graphs.uniform_graph(64, 3, seed=0)
    assert all((col[rp[r]:rp[r + 1]][1:] > col[rp[r]:rp[r + 1]][:-1]).all() for r in range(64))
