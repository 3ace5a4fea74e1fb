"""The allocation-free entry point of the C ABI.

Some callers cannot allocate device memory when they call a walk: a plug-in that is
handed raw pointers by a host whose own pool owns the whole GPU, or code that must not
trigger the device-wide synchronisation a driver allocation implies. For them
``walk_b200_uniform_walk_noalloc`` keeps the one piece of scratch the fast path needs
(the packed row descriptors) in a fixed array inside the library. This test calls it
through the C ABI twice in a row -- the second time on a different, smaller graph, so
that descriptors left behind by the first call would show up if they were ever read --
and requires bit-identical walks to the ordinary entry point and to the CPU restatement of the
reference loop. Collected last on purpose.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from mlx_cluster_b200 import _lib, graphs

pytestmark = pytest.mark.gpu


def _walk_both_ways(dev, rowptr, col, n_walks, L, seed):
    lib = _lib.lib()
    n_nodes = rowptr.numel() - 1
    gen = torch.Generator(device=dev).manual_seed(seed)
    start = torch.randint(0, n_nodes, (n_walks,), generator=gen, device=dev, dtype=torch.int64)
    rand = torch.rand((n_walks, L), generator=gen, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    # existing entry point, caller-allocated row descriptors
    desc = torch.empty(n_nodes, dtype=torch.int64, device=dev)
    flags = torch.zeros(1, dtype=torch.int32, device=dev)
    _lib.check(lib.walk_b200_rowdesc_pack(rowptr.data_ptr(), n_nodes, col.numel(), desc.data_ptr(),
                                          flags.data_ptr(), stream))
    csr = _lib.Csr(rowptr.data_ptr(), col.data_ptr(), n_nodes, col.numel(), desc.data_ptr(), 0, 0, None, 0)
    want_n = torch.empty((n_walks, L + 1), dtype=torch.int64, device=dev)
    want_e = torch.empty((n_walks, L), dtype=torch.int64, device=dev)
    _lib.check(lib.walk_b200_uniform_walk(C.byref(csr), start.data_ptr(), rand.data_ptr(), n_walks, L,
                                          want_n.data_ptr(), want_e.data_ptr(), flags.data_ptr(), stream))

    # new entry point: outputs exist before the call, nothing is allocated inside it
    got_n = torch.full((n_walks, L + 1), -7, dtype=torch.int64, device=dev)
    got_e = torch.full((n_walks, L), -7, dtype=torch.int64, device=dev)
    flags2 = torch.zeros(1, dtype=torch.int32, device=dev)
    torch.cuda.synchronize(dev)
    mem_before = torch.cuda.mem_get_info(dev)[0]
    _lib.check(lib.walk_b200_uniform_walk_noalloc(rowptr.data_ptr(), col.data_ptr(), n_nodes, col.numel(),
                                                  start.data_ptr(), rand.data_ptr(), n_walks, L,
                                                  got_n.data_ptr(), got_e.data_ptr(), flags2.data_ptr(), stream))
    torch.cuda.synchronize(dev)
    mem_after = torch.cuda.mem_get_info(dev)[0]
    assert int(flags.item()) == 0 and int(flags2.item()) == 0
    assert torch.equal(got_n, want_n), "walk matrix differs from the ordinary entry point"
    assert torch.equal(got_e, want_e), "edge ids differ from the ordinary entry point"
    # and against the checker itself, not only against another CUDA path
    ref_n, ref_e = oracle.uniform_walk(rowptr.cpu().numpy(), col.cpu().numpy(), start.cpu().numpy(),
                                       rand.cpu().numpy(), L, return_edges=True)
    assert np.array_equal(got_n.cpu().numpy(), ref_n), "walk matrix differs from the CPU restatement"
    assert np.array_equal(got_e.cpu().numpy(), ref_e), "edge ids differ from the CPU restatement"
    return mem_before, mem_after


def test_noalloc_entry_matches_ordinary_entry_twice_in_a_row(cuda):
    big = graphs.rmat_csr(16, 16, seed=11, device=cuda)       # 65,536 nodes
    small = graphs.rmat_csr(10, 8, seed=12, device=cuda)      # 1,024 nodes: stale descriptors lie beyond
    _walk_both_ways(cuda, *big, n_walks=50_000, L=40, seed=1)   # first call on this device does the set-up
    before, after = _walk_both_ways(cuda, *small, n_walks=3_333, L=17, seed=2)
    assert after >= before - (1 << 20), "the second call must not take device memory"
    _walk_both_ways(cuda, *big, n_walks=1_000, L=5, seed=3)


def test_noalloc_entry_rejects_graphs_beyond_its_scratch(cuda):
    lib = _lib.lib()
    n_nodes = _lib.NOALLOC_MAX_NODES + 1
    rowptr = torch.zeros(n_nodes + 1, dtype=torch.int64, device=cuda)
    col = torch.zeros(1, dtype=torch.int64, device=cuda)
    start = torch.zeros(4, dtype=torch.int64, device=cuda)
    rand = torch.zeros((4, 3), device=cuda)
    out = torch.empty((4, 4), dtype=torch.int64, device=cuda)
    before = _lib.launch_count()
    rc = lib.walk_b200_uniform_walk_noalloc(rowptr.data_ptr(), col.data_ptr(), n_nodes, 0, start.data_ptr(),
                                            rand.data_ptr(), 4, 3, out.data_ptr(), None, None, None)
    assert rc == _lib.ERR_UNSUPPORTED
    msg = lib.walk_b200_last_error().decode()
    assert str(n_nodes) in msg and str(_lib.NOALLOC_MAX_NODES) in msg
    assert _lib.launch_count() == before
    # exactly at the limit it runs (every node isolated: walks stand still)
    rc = lib.walk_b200_uniform_walk_noalloc(rowptr.data_ptr(), col.data_ptr(), n_nodes - 1, 0, start.data_ptr(),
                                            rand.data_ptr(), 4, 3, out.data_ptr(), None, None, None)
    assert rc == 0
    torch.cuda.synchronize(cuda)
    assert bool((out == 0).all())
