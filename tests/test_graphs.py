"""Synthetic graph builders and the edge-list -> CSR step (host side, no GPU)."""
import numpy as np
import torch

from mlx_cluster_b200 import graphs


def check_csr(rowptr, col, n):
    rowptr, col = rowptr.numpy(), col.numpy()
    assert rowptr.shape == (n + 1,) and rowptr[0] == 0 and rowptr[-1] == col.size
    assert (np.diff(rowptr) >= 0).all() and col.min() >= 0 and col.max() < n
    row = np.repeat(np.arange(n), np.diff(rowptr))
    assert (row != col).all()                                # no self-loops
    key = row * n + col
    assert (np.diff(key) > 0).all()                          # sorted by (row, col), no duplicates
    assert np.array_equal(np.sort(col * n + row), key)       # symmetric
    return row


def test_small_power_law_workload_shape():
    rowptr, col = graphs.chung_lu_csr(2708, 5278, 2.5, seed=0)
    check_csr(rowptr, col, 2708)
    assert col.numel() == 10556
    deg = rowptr.diff()
    assert deg.min() >= 1 and deg.max() > 40                 # minimum degree 1, heavy tail
    again = graphs.chung_lu_csr(2708, 5278, 2.5, seed=0)
    assert torch.equal(again[0], rowptr) and torch.equal(again[1], col)


def test_isolated_nodes_keep_their_rows():
    rowptr, col = graphs.chung_lu_csr(2708, 5278, 2.5, seed=0)
    rp, cl, iso = graphs.isolate_nodes(rowptr, col, 0.005, seed=0)
    assert iso.numel() == 14
    check_csr(rp, cl, 2708)
    assert (rp.diff()[iso] == 0).all()
    assert not np.isin(cl.numpy(), iso.numpy()).any()


def test_edges_to_csr_counts_rows_without_edges():
    # nodes 1 and 4 have no edges at all: the row pointer must still have N + 1 entries
    src = torch.tensor([0, 2, 2, 3, 3, 0])
    dst = torch.tensor([2, 0, 3, 3, 2, 2])
    rowptr, col = graphs.edges_to_csr(src, dst, 5)
    assert rowptr.tolist() == [0, 1, 1, 3, 4, 4]
    assert col.tolist() == [2, 0, 3, 2]
    rowptr, col = graphs.edges_to_csr(src, dst, 5, symmetrize=False)
    assert rowptr.tolist() == [0, 1, 1, 3, 4, 4] and col.tolist() == [2, 0, 3, 2]


def test_rmat_is_skewed_and_reproducible():
    rowptr, col = graphs.rmat_csr(12, 16, seed=1)
    check_csr(rowptr, col, 4096)
    deg = rowptr.diff()
    assert deg.max() > 20 * deg.float().mean()
    assert graphs.csr_is_symmetric(rowptr, col)
    again = graphs.rmat_csr(12, 16, seed=1)
    assert torch.equal(again[1], col)
    other = graphs.rmat_csr(12, 16, seed=2)
    assert other[1].numel() != col.numel() or not torch.equal(other[1], col)
