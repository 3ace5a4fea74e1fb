"""Sharding layer on CPU: two gloo ranks split the start rows, walk their blocks and
(optionally) gather. The walk itself is stood in for by the CPU restatement -- what is
under test is the row partition, the global walk index handed to each shard and the
point-to-point gather, none of which touches a GPU."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mlx_cluster_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n_rows, L, q):
    import oracle
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        d = np.load(os.path.join(os.path.dirname(__file__), "golden", "walk_golden.npz"))
        rowptr, col = d["rowptr2"].astype(np.int64), d["col2"].astype(np.int64)
        start = torch.arange(n_rows, dtype=torch.int64) % 2708
        seen = {}

        def biased(s, r, base, out):
            seen["base"], seen["rows"] = base, s.shape[0]
            res = torch.from_numpy(oracle.node2vec_walk(rowptr, col, s.numpy(), L, 0.5, 2.0, seed=3,
                                                        walk_index_base=base))
            if out is not None:
                out.copy_(res)
                return out
            return res

        full_expected = oracle.node2vec_walk(rowptr, col, start.numpy(), L, 0.5, 2.0, seed=3)
        shard, (b, e) = sharding.sharded_walk(biased, start, L)
        assert (b, e) == sharding.shard_range(n_rows, world, rank) and seen["base"] == b
        ok = np.array_equal(shard.numpy(), full_expected[b:e])
        gathered, _ = sharding.sharded_walk(biased, start, L, gather=True)
        if rank == 0:
            ok = ok and gathered is not None and np.array_equal(gathered.numpy(), full_expected)
        else:
            ok = ok and gathered is None
        # cyclic layout: rank r walks rows r::world with draws indexed base + i * stride
        def biased_cyclic(s, r, idx, out):
            base, stride = idx
            return torch.from_numpy(oracle.node2vec_walk(rowptr, col, s.numpy(), L, 0.5, 2.0, seed=3,
                                                         walk_index_base=base, walk_index_stride=stride))

        shard_c, rows_c = sharding.sharded_walk(biased_cyclic, start, L, layout="cyclic")
        mine = len(range(rank, n_rows, world))
        ok = ok and shard_c.shape[0] == mine and (mine == 0 or rows_c == slice(rank, rank + mine * world, world))
        ok = ok and np.array_equal(shard_c.numpy(), full_expected[rank::world])
        gathered_c, _ = sharding.sharded_walk(biased_cyclic, start, L, layout="cyclic", gather=True)
        if rank == 0:
            ok = ok and gathered_c is not None and np.array_equal(gathered_c.numpy(), full_expected)
        else:
            ok = ok and gathered_c is None
        # already-sharded inputs and a uniform op that consumes the rand block
        rng = np.random.default_rng(0)
        rand = torch.from_numpy(rng.random((n_rows, L), dtype=np.float32))

        def uniform(s, r, base, out):
            return torch.from_numpy(oracle.uniform_walk(rowptr, col, s.numpy(), r.numpy(), L))

        got, _ = sharding.sharded_walk(uniform, start[b:e].clone(), L, rand=rand[b:e].clone(),
                                       start_is_sharded=True, num_walks=n_rows, gather=True, dst=world - 1)
        if rank == world - 1:
            ok = ok and np.array_equal(got.numpy(), oracle.uniform_walk(rowptr, col, start.numpy(), rand.numpy(), L))
        # a caller-chosen row range (what a matrix too large for one device is gathered by), chunked messages
        for lo, hi in ((0, n_rows), (n_rows // 3, n_rows - n_rows // 4), sharding.shard_range(n_rows, world, 1), (0, 0)):
            part = sharding.gather_rows(shard, n_rows, row_range=(lo, hi), chunk_rows=5)
            if rank == 0:
                ok = ok and part is not None and np.array_equal(part.numpy(), full_expected[lo:hi])
            else:
                ok = ok and part is None
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("n_rows", [2708, 7, 1])
def test_two_ranks_partition_and_gather(n_rows):
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_rows, 6, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    results = dict(q.get(timeout=10) for _ in range(world))
    assert results == {0: True, 1: True}


def test_single_process_is_the_whole_range():
    calls = []

    def op(s, r, base, out):
        calls.append((s.shape[0], base))
        return torch.zeros((s.shape[0], 4), dtype=torch.int64)

    out, (b, e) = sharding.sharded_walk(op, torch.arange(10), 3, gather=True)
    assert (b, e) == (0, 10) and calls == [(10, 0)] and out.shape == (10, 4)
