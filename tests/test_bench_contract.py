"""Host-side checks of bench.py that need no GPU: both arms describe the same workload, the start order and the
block shards are what the documentation says, and the small-case traffic table is complete."""
import importlib.util
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    sys.modules["bench_under_test"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_both_arms_describe_the_same_workload():
    """The reference arm's `config` must equal the GPU arm's key for key (the ratio of the two lines is only
    taken when it does)."""
    b = _bench()
    for name, wl in b.WORKLOADS.items():
        if wl["kind"] != "node2vec":
            continue
        for gpus in (1, 2, 8):
            ours = b.workload_config(wl, name, 1 << wl["scale"], 12345, gpus, "hash", "fused 16-byte records", None)
            ref = b.workload_config(wl, name, 1 << wl["scale"], 12345, gpus, "hash")
            assert ours == ref
            assert ours["workload"] == name and ours["p"] == wl["p"] and ours["q"] == wl["q"]


def test_start_order_is_a_seeded_permutation_and_blocks_cover_it():
    b = _bench()
    from mlx_cluster_b200.sharding import shard_rows
    order = b.start_order(1000, 3).numpy()
    assert order.shape == (3000,) and np.array_equal(np.sort(order), np.repeat(np.arange(1000), 3))
    assert np.array_equal(order, b.start_order(1000, 3).numpy())
    assert not np.array_equal(order[:1000], np.arange(1000))
    seen = []
    for world in (1, 2, 8):
        rows = []
        for rank in range(world):
            sl, (base, stride) = shard_rows(3000, world, rank, "block")
            assert stride == 1 and base == sl.start
            rows.append(np.arange(3000)[sl])
        assert np.array_equal(np.concatenate(rows), np.arange(3000))
        seen.append(max(len(r) for r in rows))
    assert seen == [3000, 1500, 375]


def test_traffic_table_names_existing_profiles():
    b = _bench()
    assert set(b.NCU_SMALL_CASE) == {"node2vec_tri", "node2vec", "uniform"}
    for case in b.NCU_SMALL_CASE.values():
        assert (ROOT / case["source"]).exists(), case["source"]
        assert case["workload"] in b.WORKLOADS
        assert 30 < case["dram_bytes"] / case["accesses"] < 130   # DRAM bytes per random access: between 32 and 128
