"""Host-buffer entry points of the C ABI (resident graph + slab pipeline) against the
CPU restatement, and the L2 residency hint."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from mlx_cluster_b200 import _lib, clear_caches, random_walk, rejection_sampling
from mlx_cluster_b200.ops import HostGraph, WalkGraph

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _reset():
    yield
    _lib.set_tuning("host_slab_mb", 256)
    _lib.set_tuning("host_narrow", 2)
    _lib.set_tuning("host_threads", 0)
    _lib.set_tuning("host_single_launch", 1)
    _lib.set_tuning("n2v_pool", 1)
    _lib.set_tuning("edgeset_slots_per_edge", 4)
    clear_caches()


def test_host_arrays_uniform_and_biased(cuda, golden):
    g = golden
    out = random_walk(g["rowptr1"], g["col1"], g["start1"], g["rand1"], 5)
    assert not out.is_cuda
    np.testing.assert_array_equal(out.numpy(), g["uniform1_n"])
    for fused in (False, True):
        out, e = random_walk(torch.from_numpy(g["rowptr2"]), torch.from_numpy(g["col2"]), torch.from_numpy(g["start2"]),
                             torch.from_numpy(g["rand2"]), 20, return_edges=True, fused=fused)
        np.testing.assert_array_equal(out.numpy(), g["uniform2_n"])
        np.testing.assert_array_equal(e.numpy(), g["uniform2_e"])
    want = oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"], 20, 0.5, 2.0, seed=4)
    for kw in (dict(symmetric=False), dict(symmetric=True), dict(edgeset=True)):
        out = rejection_sampling(g["rowptr2"], g["col2"], g["start2"], 20, 0.5, 2.0, seed=4, **kw)
        np.testing.assert_array_equal(out.numpy(), want)


def test_slab_pipeline_many_slabs(cuda):
    """Force several slabs per lane: results must not depend on the slab size, and node2vec
    rows keep their global walk index across slabs."""
    from mlx_cluster_b200 import graphs
    rowptr, col = graphs.rmat_csr(12, 8, seed=3)
    n_nodes = rowptr.numel() - 1
    rng = np.random.default_rng(1)
    walks, L = 50000, 24
    start = torch.from_numpy(rng.integers(0, n_nodes, walks).astype(np.int64)).pin_memory()
    rand = torch.from_numpy(rng.random((walks, L), dtype=np.float32)).pin_memory()
    want_u = oracle.uniform_walk(rowptr.numpy(), col.numpy(), start.numpy(), rand.numpy(), L)
    want_b = oracle.node2vec_walk(rowptr.numpy(), col.numpy(), start.numpy(), L, 0.25, 4.0, seed=8, walk_index_base=17)
    for slab_mb in (1, 3, 256):
        _lib.set_tuning("host_slab_mb", slab_mb)
        before = _lib.launch_count()
        out = random_walk(rowptr, col, start, rand, L)
        launches = _lib.launch_count() - before
        np.testing.assert_array_equal(out.numpy(), want_u)
        if slab_mb == 1:
            assert launches >= 8
        out = rejection_sampling(rowptr, col, start, L, 0.25, 4.0, seed=8, walk_index_base=17, symmetric=True)
        np.testing.assert_array_equal(out.numpy(), want_b)


def test_narrow_transport_is_invisible(cuda):
    """Ids that fit int32 cross the bus as int32 and are widened by host threads, and node2vec runs
    as one launch whose finished slabs are copied out behind it: the walk and edge matrices must
    equal the plain int64 slab pipeline's for any slab size, thread count and buffer kind (pinned or
    pageable), including the -1 edge entries of walks parked on isolated nodes."""
    from mlx_cluster_b200 import graphs
    rowptr, col = graphs.rmat_csr(13, 6, seed=5)
    n_nodes = rowptr.numel() - 1
    rng = np.random.default_rng(2)
    walks, L = 70001, 19
    start_np = rng.integers(0, n_nodes, walks).astype(np.int64)
    rand_np = rng.random((walks, L), dtype=np.float32)
    want_n, want_e = oracle.uniform_walk(rowptr.numpy(), col.numpy(), start_np, rand_np, L, return_edges=True)
    assert (want_e == -1).any()
    want_b, want_be = oracle.node2vec_walk(rowptr.numpy(), col.numpy(), start_np, L, 0.25, 4.0, seed=3,
                                           return_edges=True)
    # narrow: 1 int32 on the bus, 0 int64 straight into the caller's buffer, 2 whichever the graph measured
    for narrow, threads, slab_mb, pinned, single in ((0, 0, 2, True, 1), (1, 1, 2, True, 0), (1, 3, 1, False, 1),
                                                     (1, 0, 256, True, 1), (1, 5, 3, False, 0), (1, 2, 4, True, 1),
                                                     (0, 0, 2, True, 0), (0, 0, 1, False, 1), (2, 0, 2, True, 1),
                                                     (2, 2, 256, False, 1)):
        _lib.set_tuning("host_narrow", narrow)
        _lib.set_tuning("host_single_launch", single)
        _lib.set_tuning("host_threads", threads)
        _lib.set_tuning("host_slab_mb", slab_mb)
        start = torch.from_numpy(start_np)
        rand = torch.from_numpy(rand_np)
        if pinned:
            start, rand = start.pin_memory(), rand.pin_memory()
        out, e = random_walk(rowptr, col, start, rand, L, return_edges=True)
        np.testing.assert_array_equal(out.numpy(), want_n)
        np.testing.assert_array_equal(e.numpy(), want_e)
        for kw in (dict(symmetric=True), dict(symmetric=False), dict(edgeset=True)):
            out, e = rejection_sampling(rowptr, col, start, L, 0.25, 4.0, seed=3, return_edges=True, **kw)
            np.testing.assert_array_equal(out.numpy(), want_b)
            np.testing.assert_array_equal(e.numpy(), want_be)
        for pool in (2, 0):
            _lib.set_tuning("n2v_pool", pool)
            out = rejection_sampling(rowptr, col, start, L, 0.25, 4.0, seed=3, edgeset=True)
            np.testing.assert_array_equal(out.numpy(), want_b)
            out, e = rejection_sampling(rowptr, col, start, L, 0.25, 4.0, seed=3, edgeset=True, return_edges=True)
            np.testing.assert_array_equal(out.numpy(), want_b)
            np.testing.assert_array_equal(e.numpy(), want_be)


def test_resident_graph_with_triangle_filter(cuda, golden):
    """The host entry's single launch with the triangle filter (both transports) against the restatement."""
    g = golden
    start = np.concatenate([g["start2"], g["start2"][::-1]]).astype(np.int64)
    want, want_e = oracle.node2vec_walk(g["rowptr2"], g["col2"], start, 20, 0.25, 4.0, seed=21, return_edges=True)
    hg = HostGraph(g["rowptr2"], g["col2"], symmetric=True, edgeset=True, trifilter=True)
    assert hg.device_bytes() > (2709 + 2 * 10556 + 2708) * 8 + 10556 * 16
    lib = _lib.lib()
    for narrow in (1, 0):
        _lib.set_tuning("host_narrow", narrow)
        for with_edges in (False, True):
            out = np.full((start.size, 21), -3, dtype=np.int64)
            e_out = np.full((start.size, 20), -3, dtype=np.int64)
            _lib.check(lib.walk_b200_node2vec_walk_host(hg._h, start.ctypes.data, start.size, 20, 0.25, 4.0, 21, 0, 1,
                                                        out.ctypes.data, e_out.ctypes.data if with_edges else None))
            assert _lib.last_kernel() == "node2vec_pool_tri_kernel"
            np.testing.assert_array_equal(out, want)
            if with_edges:
                np.testing.assert_array_equal(e_out, want_e)
    hg.close()


def test_transport_choice_is_reported(cuda, golden):
    g = golden
    _lib.set_tuning("host_narrow", 2)
    hg = HostGraph(g["rowptr1"], g["col1"])
    d2h, widen = _lib.host_transport_rates(hg._h)
    assert d2h > 0.5 and widen > 0.5          # GB/s, measured at creation
    chosen = _lib.host_transport(hg._h)
    assert chosen in (0, 1)
    _lib.set_tuning("host_narrow", 0)
    assert _lib.host_transport(hg._h) == 0
    _lib.set_tuning("host_narrow", 1)
    assert _lib.host_transport(hg._h) == 1
    hg.close()
    assert _lib.host_widen_probe(32 << 20) > 0.5


def test_host_entry_reports_bad_input(cuda, golden):
    g = golden
    start = g["start1"].copy()
    start[5] = 99999
    with pytest.raises(_lib.WalkError) as ei:
        random_walk(g["rowptr1"], g["col1"], start, g["rand1"], 5)
    assert ei.value.code == _lib.ERR_DEVICE_FLAGS and "node id out of range" in str(ei.value)
    bad_rowptr = g["rowptr1"].copy()
    bad_rowptr[100] = bad_rowptr[99] - 1
    with pytest.raises(_lib.WalkError) as ei:
        HostGraph(bad_rowptr, g["col1"])
    assert ei.value.code == _lib.ERR_CSR_INVALID
    unsorted = g["col1"].copy()
    r = int(np.argmax(np.diff(g["rowptr1"]) >= 2))
    a = g["rowptr1"][r]
    unsorted[a], unsorted[a + 1] = unsorted[a + 1], unsorted[a]
    with pytest.raises(_lib.WalkError):
        HostGraph(g["rowptr1"], unsorted, validate=True)
    hg = HostGraph(g["rowptr1"], g["col1"], validate=True)
    assert hg.device_bytes() == (2709 + 10556 + 2708) * 8
    hg.close()
    for slots_per_edge in (2, 4):   # half full (the minimum) and the default, a quarter full
        _lib.set_tuning("edgeset_slots_per_edge", slots_per_edge)
        hg = HostGraph(g["rowptr1"], g["col1"], edgeset=True)
        table = _lib.edgeset_buckets(10556) * slots_per_edge // 2 * 32
        assert hg.device_bytes() == (2709 + 10556 + 2708) * 8 + table + 10556 * 8
        hg.close()


def test_l2_window_hint_does_not_change_results(cuda, golden):
    g = golden
    t = lambda a: torch.from_numpy(a).to(cuda)
    graph = WalkGraph(t(g["rowptr1"]), t(g["col1"]))
    s = torch.cuda.Stream(cuda)
    granted = C.c_size_t(0)
    _lib.check(_lib.lib().walk_b200_l2_window_set(graph.rowdesc.data_ptr(), graph.rowdesc.numel() * 8, 1.0,
                                                  s.cuda_stream, C.byref(granted)))
    out = random_walk(None, None, t(g["start1"]), t(g["rand1"]), 5, graph=graph, stream=s)
    s.synchronize()
    np.testing.assert_array_equal(out.cpu().numpy(), g["uniform1_n"])
    _lib.check(_lib.lib().walk_b200_l2_window_clear(s.cuda_stream))
    assert granted.value in (0, graph.rowdesc.numel() * 8)


def test_gather_probe_reports_a_plausible_rate(cuda):
    rate = _lib.gather_probe(256 << 20, 8)
    assert 1e9 < rate < 1e12
    with pytest.raises(_lib.WalkError):
        _lib.gather_probe(1024, 8)
