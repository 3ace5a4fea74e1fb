"""Keyword-only options of the two operators beyond the reference's signature
(``bindings.cpp:12-21,35-45``): ``validate=``, ``devices=``, ``gather=``, the ``edgeset="auto"``
default that lets a plain reference-style call reach the fast node2vec kernel, the handling of
unsorted rows, and status flags read on the stream the work ran on. All through the C ABI,
checked against the CPU restatement."""
import numpy as np
import pytest
import torch

import oracle
from mlx_cluster_b200 import _lib, clear_caches, graphs, random_walk, rejection_sampling
from mlx_cluster_b200.ops import WalkGraph
from tests.test_oracle import random_csr

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _fresh_caches():
    clear_caches()
    yield
    clear_caches()


def _t(a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def test_reference_style_call_reaches_the_pooled_kernel_on_its_second_call(cuda, golden):
    g = golden
    rowptr, col, start = _t(g["rowptr2"], cuda), _t(g["col2"], cuda), _t(g["start2"], cuda)
    want = oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"], 20, 0.25, 4.0, seed=0)
    first = rejection_sampling(rowptr, col, start, 20, 0.25, 4.0)   # positional, as the reference's demo calls it
    assert _lib.last_kernel() == "node2vec_walk_kernel"              # no hash set yet: binary search, nothing built
    second = rejection_sampling(rowptr, col, start, 20, 0.25, 4.0)
    assert _lib.last_kernel() == "node2vec_pool_kernel"              # hash set + reverse positions built on this call
    third = rejection_sampling(rowptr, col, start, 20, 0.25, 4.0, edgeset=False)
    assert _lib.last_kernel() == "node2vec_pool_kernel"              # what is built stays in use
    for got in (first, second, third):
        np.testing.assert_array_equal(got.cpu().numpy(), want)
    # a graph that is only walked once never pays for the structures
    other = rowptr.clone()
    rejection_sampling(other, col, start, 20, 0.25, 4.0)
    assert _lib.last_kernel() == "node2vec_walk_kernel"
    # where almost every first candidate is accepted the per-lane kernel stays the choice
    rejection_sampling(rowptr, col, start, 20, 1.0, 1.0)
    assert _lib.last_kernel() == "node2vec_walk_kernel"


def test_a_graph_that_keeps_being_walked_gets_the_filter(cuda, golden):
    """edgeset="auto": binary search on the first call, hash set from the second, and from the 17th the triangle
    filter -- the graph is undirected, which the library finds out by itself; a directed graph never gets it."""
    from mlx_cluster_b200 import ops
    g = golden
    rowptr, col, start = _t(g["rowptr2"], cuda), _t(g["col2"], cuda), _t(g["start2"], cuda)
    want = oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"], 20, 0.25, 4.0, seed=0)
    seen = []
    for call in range(ops._FILTER_AFTER_CALLS + 2):
        got = rejection_sampling(rowptr, col, start, 20, 0.25, 4.0)
        seen.append(_lib.last_kernel())
        np.testing.assert_array_equal(got.cpu().numpy(), want)
    assert seen[0] == "node2vec_walk_kernel" and seen[1] == "node2vec_pool_kernel"
    assert seen[ops._FILTER_AFTER_CALLS - 1] == "node2vec_pool_kernel"
    assert seen[ops._FILTER_AFTER_CALLS] == "node2vec_pool_tri_kernel" and seen[-1] == "node2vec_pool_tri_kernel"
    # q <= 1: no membership test can matter, the filter is never built
    rp2 = rowptr.clone()
    for _ in range(ops._FILTER_AFTER_CALLS + 2):
        rejection_sampling(rp2, col, start, 20, 1.0, 0.5)
        assert _lib.last_kernel() != "node2vec_pool_tri_kernel"
    # a directed graph (edges without a reverse) is recognised and left alone
    rng = np.random.default_rng(4)
    rp_d, cl_d = random_csr(rng, 300, 6.0, symmetric=False)
    st_d = rng.integers(0, 300, 1500).astype(np.int64)
    want_d = oracle.node2vec_walk(rp_d, cl_d, st_d, 12, 0.25, 4.0, seed=0)
    rp_t, cl_t, st_t = _t(rp_d, cuda), _t(cl_d, cuda), _t(st_d, cuda)
    for _ in range(ops._FILTER_AFTER_CALLS + 2):
        got = rejection_sampling(rp_t, cl_t, st_t, 12, 0.25, 4.0)
        assert _lib.last_kernel() != "node2vec_pool_tri_kernel"
    np.testing.assert_array_equal(got.cpu().numpy(), want_d)


def test_trifilter_keyword(cuda, golden):
    """trifilter=True on the operator builds the triangle filter with the graph (undirected graphs only)."""
    g = golden
    rowptr, col, start = _t(g["rowptr2"], cuda), _t(g["col2"], cuda), _t(g["start2"], cuda)
    want = oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"], 20, 0.25, 4.0, seed=3)
    got = rejection_sampling(rowptr, col, start, 20, 0.25, 4.0, seed=3, symmetric=True, edgeset=True, trifilter=True)
    assert _lib.last_kernel() == "node2vec_pool_tri_kernel"
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    host = rejection_sampling(g["rowptr2"], g["col2"], g["start2"], 20, 0.25, 4.0, seed=3, symmetric=True, edgeset=True,
                              trifilter=True)
    assert _lib.last_kernel() == "node2vec_pool_tri_kernel"
    np.testing.assert_array_equal(host.numpy(), want)
    with pytest.raises(ValueError, match="symmetric"):
        rejection_sampling(rowptr.clone(), col, start, 20, 0.25, 4.0, trifilter=True)


def _shuffled_rows(rng, rowptr, col):
    col = col.copy()
    for v in range(rowptr.size - 1):
        rng.shuffle(col[rowptr[v]:rowptr[v + 1]])
    return col


def test_unsorted_rows_on_the_default_path(cuda):
    """The reference's linear is_neighbor takes rows in any order (BiasedRandomWalk.cpp:20-28). The default
    call does too (it falls back to the edge hash set); insisting on the binary search is refused."""
    rng = np.random.default_rng(8)
    rowptr, col = random_csr(rng, 300, 7.0, symmetric=True)
    col = _shuffled_rows(rng, rowptr, col)
    start = rng.integers(0, 300, 2000).astype(np.int64)
    want = oracle.node2vec_walk(rowptr, col, start, 15, 0.25, 4.0, seed=4)
    rp, cl, st = _t(rowptr, cuda), _t(col, cuda), _t(start, cuda)
    got = rejection_sampling(rp, cl, st, 15, 0.25, 4.0, seed=4, check=True)
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    with pytest.raises(ValueError, match="not sorted"):
        rejection_sampling(rp.clone(), cl, st, 15, 0.25, 4.0, seed=4, edgeset=False)
    # a prepared graph without a hash set: same rule
    prepared = WalkGraph(rp, cl, symmetric=True)
    got = rejection_sampling(None, None, st, 15, 0.25, 4.0, seed=4, graph=prepared, check=True)
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    assert prepared.edgeset is not None and prepared.colrev is None
    # host arrays
    got = rejection_sampling(rowptr, col, start, 15, 0.25, 4.0, seed=4)
    np.testing.assert_array_equal(got.numpy(), want)
    with pytest.raises(_lib.WalkError, match="ascending"):
        rejection_sampling(rowptr, col, start, 15, 0.25, 4.0, seed=4, edgeset=False)


def test_validate_keyword(cuda, golden):
    g = golden
    rowptr, col = _t(g["rowptr1"], cuda), _t(g["col1"], cuda)
    start = _t(g["start1"], cuda)
    rand = _t(g["rand1"], cuda)
    out = random_walk(rowptr, col, start, rand, 5, validate=True)
    np.testing.assert_array_equal(out.cpu().numpy(), g["uniform1_n"])
    bad_start = start.clone()
    bad_start[7] = 2708
    with pytest.raises(ValueError, match="node id out of range"):
        random_walk(rowptr, col, bad_start, rand, 5, validate=True)
    with pytest.raises(ValueError, match="node id out of range"):
        rejection_sampling(rowptr, col, bad_start, 5, 1.0, 2.0, validate=True)
    bad_col = col.clone()
    bad_col[3] = -1
    with pytest.raises(ValueError, match="node id out of range"):
        random_walk(rowptr, bad_col, start, rand, 5, validate=True)
    # without it nothing is raised (flagged and parked), as documented
    random_walk(rowptr, col, bad_start, rand, 5)
    # host arrays: the upload validates
    with pytest.raises(_lib.WalkError):
        random_walk(g["rowptr1"], bad_col.cpu().numpy(), g["start1"], g["rand1"], 5, validate=True)


def test_devices_and_gather_keywords(cuda, golden):
    """One process, several devices: contiguous blocks of start rows, replicated CSR, global walk indices."""
    g = golden
    n_dev = torch.cuda.device_count()
    devices = [0, 1, 0] if n_dev >= 2 else [0, 0, 0]
    rowptr, col = _t(g["rowptr2"], cuda), _t(g["col2"], cuda)
    start = _t(g["start2"], cuda)
    rng = np.random.default_rng(1)
    rand = rng.random((2708, 20), dtype=np.float32)
    want_b, want_be = oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"], 20, 0.5, 2.0, seed=6, return_edges=True)
    want_u = oracle.uniform_walk(g["rowptr2"], g["col2"], g["start2"], rand, 20)
    blocks = rejection_sampling(rowptr, col, start, 20, 0.5, 2.0, seed=6, devices=devices)
    assert isinstance(blocks, list) and len(blocks) == 3
    assert [b.device.index for b in blocks] == devices
    np.testing.assert_array_equal(np.concatenate([b.cpu().numpy() for b in blocks]), want_b)
    full, full_e = rejection_sampling(rowptr, col, start, 20, 0.5, 2.0, seed=6, devices=devices, gather=True,
                                      return_edges=True)
    assert full.device == cuda
    np.testing.assert_array_equal(full.cpu().numpy(), want_b)
    np.testing.assert_array_equal(full_e.cpu().numpy(), want_be)
    full_u = random_walk(rowptr, col, start, _t(rand, cuda), 20, devices=devices, gather=True)
    np.testing.assert_array_equal(full_u.cpu().numpy(), want_u)
    blocks_u = random_walk(rowptr, col, start, _t(rand, cuda), 20, devices=devices)
    np.testing.assert_array_equal(np.concatenate([b.cpu().numpy() for b in blocks_u]), want_u)
    with pytest.raises(ValueError):
        random_walk(g["rowptr2"], g["col2"], g["start2"], rand, 20, devices=[0])


def test_flags_are_read_on_the_stream_the_walk_ran_on(cuda, golden):
    """check=True with a side stream that torch's current stream knows nothing about."""
    g = golden
    rowptr, col = _t(g["rowptr2"], cuda), _t(g["col2"], cuda)
    bad_start = _t(g["start2"], cuda).clone()
    bad_start[100] = -5
    side = torch.cuda.Stream(cuda)
    torch.cuda.synchronize(cuda)
    for _ in range(3):
        with pytest.raises(RuntimeError, match="node id out of range"):
            rejection_sampling(rowptr, col, bad_start, 20, 0.25, 4.0, stream=side, check=True)
        with pytest.raises(RuntimeError, match="node id out of range"):
            rejection_sampling(rowptr, col, bad_start, 20, 0.25, 4.0, stream=int(side.cuda_stream), check=True)
    good = rejection_sampling(rowptr, col, _t(g["start2"], cuda), 20, 0.25, 4.0, stream=side, check=True)
    np.testing.assert_array_equal(good.cpu().numpy(),
                                  oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"], 20, 0.25, 4.0, seed=0))


def test_host_arrays_edited_in_place_are_not_served_from_a_stale_graph(cuda):
    rng = np.random.default_rng(3)
    rowptr, col = random_csr(rng, 200, 5.0, symmetric=False)
    start = rng.integers(0, 200, 500).astype(np.int64)
    rand = rng.random((500, 12), dtype=np.float32)
    a = random_walk(rowptr, col, start, rand, 12).numpy().copy()
    np.testing.assert_array_equal(a, oracle.uniform_walk(rowptr, col, start, rand, 12))
    col[:] = np.roll(col, 1) % 200   # same buffers, other graph
    b = random_walk(rowptr, col, start, rand, 12).numpy()
    np.testing.assert_array_equal(b, oracle.uniform_walk(rowptr, col, start, rand, 12))
