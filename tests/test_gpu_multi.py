"""Two ranks on two GPUs over NCCL: sharded walks and the optional gather of the walk matrix.
Skipped on machines with fewer than two GPUs (the CPU twin of this test runs on gloo)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_DEBUG="WARN")
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import oracle
        from mlx_cluster_b200 import graphs, random_walk, rejection_sampling, sharding
        from mlx_cluster_b200.ops import WalkGraph
        rowptr, col = graphs.rmat_csr(12, 8, seed=3)
        n_nodes, L = rowptr.numel() - 1, 24
        rng = np.random.default_rng(0)
        start_h = torch.from_numpy(rng.integers(0, n_nodes, 30001).astype(np.int64))
        rand_h = torch.from_numpy(rng.random((30001, L), dtype=np.float32))
        graph = WalkGraph(rowptr.to(dev), col.to(dev), edgeset=True)
        start, rand = start_h.to(dev), rand_h.to(dev)
        want_b = oracle.node2vec_walk(rowptr.numpy(), col.numpy(), start_h.numpy(), L, 0.25, 4.0, seed=5)
        want_u = oracle.uniform_walk(rowptr.numpy(), col.numpy(), start_h.numpy(), rand_h.numpy(), L)
        ok = True

        def biased_block(s, r, base, out):
            return rejection_sampling(None, None, s, L, 0.25, 4.0, graph=graph, seed=5, walk_index_base=base, out=out)

        def biased_cyclic(s, r, idx, out):
            return rejection_sampling(None, None, s, L, 0.25, 4.0, graph=graph, seed=5, walk_index_base=idx[0],
                                      walk_index_stride=idx[1])

        def uniform_block(s, r, base, out):
            return random_walk(None, None, s, r, L, graph=graph, out=out)

        for op, layout, want in ((biased_block, "block", want_b), (biased_cyclic, "cyclic", want_b),
                                 (uniform_block, "block", want_u)):
            shard, rows = sharding.sharded_walk(op, start, L, rand=rand, layout=layout)
            mine = want[rows[0]:rows[1]] if layout == "block" else want[rows]
            ok = ok and np.array_equal(shard.cpu().numpy(), mine)
            full, _ = sharding.sharded_walk(op, start, L, rand=rand, layout=layout, gather=True)
            if rank == 0:
                ok = ok and full is not None and np.array_equal(full.cpu().numpy(), want)
            else:
                ok = ok and full is None
        # a caller-chosen row range of the block layout, received in place on rank 0
        shard, (b, e) = sharding.sharded_walk(biased_block, start, L, layout="block")
        for lo, hi in ((0, 30001), (9000, 22000), (b, e) if rank == 0 else sharding.shard_range(30001, world, 0)):
            part = sharding.gather_rows(shard, 30001, row_range=(lo, hi), chunk_rows=4096)
            if rank == 0:
                ok = ok and part is not None and np.array_equal(part.cpu().numpy(), want_b[lo:hi])
            else:
                ok = ok and part is None
        # one process driving both devices through the operator's own keywords
        if rank == 0:
            blocks = rejection_sampling(rowptr.to(dev), col.to(dev), start, L, 0.25, 4.0, seed=5, devices=[0, 1])
            ok = ok and [t.device.index for t in blocks] == [0, 1]
            ok = ok and np.array_equal(np.concatenate([t.cpu().numpy() for t in blocks]), want_b)
            full = random_walk(rowptr.to(dev), col.to(dev), start, rand, L, devices=[1, 0], gather=True)
            ok = ok and full.device == dev and np.array_equal(full.cpu().numpy(), want_u)
        dist.barrier()
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_two_gpus_shard_and_gather_over_nccl():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    assert dict(q.get(timeout=10) for _ in range(world)) == {0: True, 1: True}
