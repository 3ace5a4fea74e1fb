"""Edge list -> CSR on the device (``walk_b200_csr_build``) against a numpy restatement of the host
recipe (sort by (row, col), unique, counts over all nodes). The result is unique, so equality is exact."""
import numpy as np
import pytest
import torch

from mlx_cluster_b200 import _lib, csr_from_edges, graphs

pytestmark = pytest.mark.gpu


def numpy_csr(src, dst, n, symmetrize, drop_self_loops, dedupe):
    src, dst = np.asarray(src, np.int64), np.asarray(dst, np.int64)
    if drop_self_loops:
        keep = src != dst
        src, dst = src[keep], dst[keep]
    if symmetrize:
        off = src != dst  # a kept self-loop is inserted once
        src, dst = np.concatenate([src, dst[off]]), np.concatenate([dst, src[off]])
    key = src * n + dst
    key = np.unique(key) if dedupe else np.sort(key)
    row, col = key // max(n, 1), key % max(n, 1)
    rowptr = np.zeros(n + 1, np.int64)
    np.cumsum(np.bincount(row, minlength=n), out=rowptr[1:])
    return rowptr, col


def build(src, dst, n, **kw):
    rp, cl = csr_from_edges(torch.from_numpy(np.asarray(src, np.int64)).cuda(),
                            torch.from_numpy(np.asarray(dst, np.int64)).cuda(), n, **kw)
    return rp.cpu().numpy(), cl.cpu().numpy()


@pytest.mark.parametrize("symmetrize", [True, False])
@pytest.mark.parametrize("drop_self_loops", [True, False])
@pytest.mark.parametrize("dedupe", [True, False])
def test_small_random_multigraph(cuda, symmetrize, drop_self_loops, dedupe):
    rng = np.random.default_rng(5)
    n, m = 300, 6000  # many repeated edges and self-loops; nodes 290.. never occur (isolated)
    src, dst = rng.integers(0, 290, m), rng.integers(0, 290, m)
    kw = dict(symmetrize=symmetrize, drop_self_loops=drop_self_loops, dedupe=dedupe)
    rp, cl = build(src, dst, n, **kw)
    want_rp, want_cl = numpy_csr(src, dst, n, **kw)
    np.testing.assert_array_equal(rp, want_rp)
    np.testing.assert_array_equal(cl, want_cl)
    assert rp.shape == (n + 1,) and (np.diff(rp)[290:] == 0).all()


def test_row_lengths_around_the_warp_and_block_limits(cuda):
    """Rows of 0, 1, 31..33, 63..65 (the one-warp limit), 255..257, 2047..2049 and 70000 raw entries,
    each with duplicates, exercise the register network, the block radix sort and its ragged pieces."""
    rng = np.random.default_rng(9)
    lengths = [0, 1, 2, 31, 32, 33, 63, 64, 65, 66, 127, 128, 255, 256, 257, 1000, 2047, 2048, 2049, 70000]
    n = 1 << 17
    src, dst = [], []
    for r, d in enumerate(lengths):
        src.append(np.full(d, r * 7, np.int64))
        dst.append(rng.integers(0, n if d > 3000 else max(4, d), d))  # small ranges force duplicates
    src, dst = np.concatenate(src), np.concatenate(dst)
    perm = rng.permutation(src.size)
    src, dst = src[perm], dst[perm]
    for dedupe in (True, False):
        rp, cl = build(src, dst, n, symmetrize=False, drop_self_loops=False, dedupe=dedupe)
        want_rp, want_cl = numpy_csr(src, dst, n, False, False, dedupe)
        np.testing.assert_array_equal(rp, want_rp)
        np.testing.assert_array_equal(cl, want_cl)


def test_rmat_matches_the_library_route(cuda):
    """A skewed graph with hub rows of tens of thousands of entries: same CSR as sort/unique."""
    src, dst = graphs.rmat_edges(16, 16, seed=4, device="cuda")
    n = 1 << 16
    rp, cl = csr_from_edges(src, dst, n)
    want_rp, want_cl = graphs.edges_to_csr(src, dst, n)
    assert torch.equal(rp, want_rp) and torch.equal(cl, want_cl)
    assert int((rp[1:] - rp[:-1]).max()) > 2000  # there is a hub


def test_degenerate_inputs(cuda):
    rp, cl = build([], [], 5)
    np.testing.assert_array_equal(rp, np.zeros(6, np.int64))
    assert cl.size == 0
    rp, cl = build([], [], 0)
    np.testing.assert_array_equal(rp, np.zeros(1, np.int64))
    rp, cl = build([2, 2, 2], [2, 2, 2], 4)  # self-loops only, dropped
    np.testing.assert_array_equal(rp, np.zeros(5, np.int64))
    rp, cl = build([2, 2, 2], [2, 2, 2], 4, drop_self_loops=False)
    np.testing.assert_array_equal(rp, [0, 0, 0, 1, 1])
    np.testing.assert_array_equal(cl, [2])
    with pytest.raises(_lib.WalkError) as ei:
        build([0, 1, 9], [1, 2, 0], 4)
    assert "outside" in str(ei.value)
    rp, cl = build([0, 1, 9], [1, 2, 0], 4, check=False)  # the bad edge is left out
    np.testing.assert_array_equal(rp, [0, 1, 3, 4, 4])
    np.testing.assert_array_equal(cl, [1, 0, 2, 1])
