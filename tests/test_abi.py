"""The C-ABI library loads without a GPU, exports every symbol the header declares, and its
host-only entry points (Philox, thresholds, sharding, argument checks) behave. No kernel
is launched here."""
import ctypes as C
import json
import re
from pathlib import Path

import numpy as np
import pytest

import oracle
from mlx_cluster_b200 import _lib

ROOT = Path(__file__).resolve().parents[1]


def test_every_declared_symbol_is_exported(walklib):
    header = (ROOT / "include" / "walk_b200.h").read_text()
    declared = set(re.findall(r"\b(walk_b200_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS), declared ^ set(_lib.EXPORTS)
    for name in declared:
        assert hasattr(walklib, name), name
    assert walklib.walk_b200_abi_version() == int(re.search(r"WALK_B200_ABI_VERSION (\d+)", header).group(1))


def test_status_codes_and_flags_match_header():
    header = (ROOT / "include" / "walk_b200.h").read_text()
    defs = {k: int(v, 0) for k, v in re.findall(r"#define (WALK_B200_[A-Z_0-9]+) (0x[0-9a-f]+|\d+)u?\b", header)}
    assert defs["WALK_B200_ERR_BAD_PQ"] == _lib.ERR_BAD_PQ
    assert defs["WALK_B200_ERR_DEVICE_FLAGS"] == _lib.ERR_DEVICE_FLAGS
    assert defs["WALK_B200_FLAG_BAD_NODE"] == _lib.FLAG_BAD_NODE
    assert defs["WALK_B200_FLAG_UNSORTED_ROW"] == _lib.FLAG_UNSORTED_ROW
    assert defs["WALK_B200_CSR_SYMMETRIC"] == _lib.CSR_SYMMETRIC
    n_counters = len(re.findall(r"^\s+WALK_B200_CNT_[A-Z0-9_]+", header, flags=re.M))
    assert n_counters == len(_lib.COUNTER_NAMES)
    assert C.sizeof(_lib.Csr) == 96
    assert defs["WALK_B200_CSR_WANT_FUSED"] == _lib.CSR_WANT_FUSED
    assert defs["WALK_B200_FLAG_EDGESET_FULL"] == _lib.FLAG_EDGESET_FULL
    assert defs["WALK_B200_CSR_WANT_EDGESET"] == _lib.CSR_WANT_EDGESET


def test_host_philox_matches_independent_implementation_and_oracle(walklib):
    doc = json.loads((ROOT / "tests" / "golden" / "philox_kat.json").read_text())
    for v in doc["vectors"]:
        assert _lib.philox4x32_10(v["counter"], v["key"]).tolist() == v["out"]
    rng = np.random.default_rng(3)
    for _ in range(200):
        seed = int(rng.integers(0, 2**63)) * 2 + int(rng.integers(0, 2))
        walk = int(rng.integers(0, 2**40))
        step, attempt = int(rng.integers(0, 200)), int(rng.integers(0, 1000))
        o = oracle.philox4x32_10([walk & 0xffffffff, step, attempt, walk >> 32], [seed & 0xffffffff, seed >> 32])
        assert _lib.node2vec_draw(seed, walk, step, attempt) == (int(o[0]) >> 1, int(o[1]) >> 1)


def test_negative_draw_replays_the_documented_stream(walklib):
    """Draw k of row g: word (k & 3) of the Philox block (g lo, k >> 2, 'NEGS', g hi), scaled to [0, N)."""
    rng = np.random.default_rng(11)
    for _ in range(200):
        seed = int(rng.integers(0, 2**63)) * 2 + int(rng.integers(0, 2))
        row = int(rng.integers(0, 2**40))
        k = int(rng.integers(0, 500))
        n = int(rng.integers(1, 2**32 + 1))
        o = oracle.philox4x32_10([row & 0xffffffff, k >> 2, 0x4E454753, row >> 32], [seed & 0xffffffff, seed >> 32])
        got = _lib.negative_draw(seed, row, k, n)
        assert got == (int(o[k & 3]) * n) >> 32 and 0 <= got < n
    with pytest.raises(_lib.WalkError):
        _lib.negative_draw(1, 2, 3, 0)
    with pytest.raises(_lib.WalkError):
        _lib.negative_draw(1, 2, 3, 2**32 + 1)


def test_csr_build_scratch_size_and_argument_checks(walklib):
    """Host arithmetic of the device CSR builder: 8 bytes per slot (a directed edge before duplicates
    are dropped) plus per-node arrays; limits and unknown option bits are refused."""
    def need(m, n, options):
        v = C.c_uint64(0)
        _lib.check(walklib.walk_b200_csr_build_scratch_bytes(m, n, options, C.byref(v)))
        return int(v.value)
    sym = _lib.BUILD_SYMMETRIZE
    m, n = 1_000_000, 50_000
    one, two = need(m, n, 0), need(m, n, sym)
    assert 8 * m <= one <= 8 * m + 16 * n + (1 << 16)
    assert 16 * m <= two <= 16 * m + 16 * n + (1 << 16) and two > one
    assert need(m, n, sym | _lib.BUILD_DROP_SELF_LOOPS | _lib.BUILD_DEDUPE) == two
    assert need(0, 0, 0) > 0 and need(10, 3, sym) % 256 == 0
    for bad in ((-1, 5, 0), (5, -1, 0), (5, 5, 0x10), (1 << 31, 5, 0), (5, 1 << 31, 0)):
        with pytest.raises(_lib.WalkError):
            need(*bad)
    with pytest.raises(_lib.WalkError):
        _lib.check(walklib.walk_b200_csr_build_scratch_bytes(5, 5, 0, None))


def test_thresholds_and_cuts_match_oracle(walklib):
    for p, q in [(1, 1), (0.5, 2), (4, 0.25), (0.25, 4), (1, 2), (1, 3), (0.7, 1.3), (3.3, 0.011), (100.0, 100.0)]:
        prob, cuts = _lib.node2vec_thresholds(p, q)
        np.testing.assert_array_equal(np.array(prob), oracle.thresholds(p, q))
        assert list(cuts) == [oracle.accept_cut(x) for x in prob]


@pytest.mark.parametrize("p,q", [(0.0, 1.0), (1.0, -2.0), (float("nan"), 1.0), (1.0, float("inf")), (1e-9, 1.0), (1.0, 1e9)])
def test_bad_pq_is_rejected(walklib, p, q):
    with pytest.raises(_lib.WalkError) as ei:
        _lib.node2vec_thresholds(p, q)
    assert ei.value.code == _lib.ERR_BAD_PQ
    assert walklib.walk_b200_last_error()


def test_extreme_but_workable_pq_is_accepted(walklib):
    # a huge p only makes returning unlikely; every candidate is still accepted with prob_2 = 1
    prob, cuts = _lib.node2vec_thresholds(1e6, 1.0)
    assert prob[2] == 1.0 and prob[0] == 1e-6 and cuts[0] == oracle.accept_cut(1e-6)
    prob, _ = _lib.node2vec_thresholds(1.0, 60000.0)
    assert prob[2] >= 2.0 ** -16


def test_shard_range_partitions(walklib):
    for n in [0, 1, 7, 8, 9, 1000, 2708, 16777216]:
        for world in [1, 2, 3, 4, 8]:
            spans = [_lib.shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (b0, e0), (b1, e1) in zip(spans, spans[1:]):
                assert e0 == b1 and b0 <= e0
            per = -(-n // world)
            assert all(e - b <= per for b, e in spans)
    with pytest.raises(_lib.WalkError):
        _lib.shard_range(10, 2, 2)
    for n in [0, 1, 7, 8, 9, 2708]:
        for world in [1, 2, 3, 8]:
            counts = [_lib.shard_count_cyclic(n, world, r) for r in range(world)]
            assert counts == [len(range(r, n, world)) for r in range(world)]


def test_argument_errors_before_any_launch(walklib):
    before = _lib.launch_count()
    csr = _lib.Csr(None, None, 4, 0, None, 0, 0, None, 0)
    assert walklib.walk_b200_uniform_walk(None, None, None, 0, 0, None, None, None, None) == _lib.ERR_INVALID_ARG
    assert walklib.walk_b200_uniform_walk(C.byref(csr), None, None, 4, 3, None, None, None, None) == _lib.ERR_INVALID_ARG
    assert b"rowptr" in walklib.walk_b200_last_error()
    csr = _lib.Csr(8, 8, -1, 0, None, 0, 0, None, 0)
    assert walklib.walk_b200_node2vec_walk(C.byref(csr), None, 0, 1, 1.0, 1.0, 0, 0, 1, None, None, None, None, None) \
        == _lib.ERR_INVALID_ARG
    csr = _lib.Csr(8, 8, 4, 4, None, 0, 0, None, 0)
    assert walklib.walk_b200_node2vec_walk(C.byref(csr), 8, 4, -1, 1.0, 1.0, 0, 0, 1, 8, None, None, None, None) \
        == _lib.ERR_INVALID_ARG
    assert walklib.walk_b200_node2vec_walk(C.byref(csr), 8, 4, 2, 0.0, 1.0, 0, 0, 1, 8, None, None, None, None) \
        == _lib.ERR_BAD_PQ
    assert walklib.walk_b200_set_tuning(b"no_such_knob", 1) == _lib.ERR_INVALID_ARG
    # edge hash set: sizing is host arithmetic; a misaligned or undersized table is refused before any launch
    assert _lib.edgeset_buckets(0) == 64 and _lib.edgeset_buckets(1000) == 500 and _lib.edgeset_buckets(1001) == 501
    assert walklib.walk_b200_edgeset_build(C.byref(csr), 8, 64, None, None) == _lib.ERR_INVALID_ARG
    big = _lib.Csr(8, 8, 4, 100000, None, 0, 0, None, 0)
    assert walklib.walk_b200_edgeset_build(C.byref(big), 64, 64, None, None) == _lib.ERR_INVALID_ARG
    assert b"too small" in walklib.walk_b200_last_error()
    assert _lib.launch_count() == before
    # empty batches succeed without touching the device
    assert walklib.walk_b200_uniform_walk(C.byref(csr), None, None, 0, 5, None, None, None, None) == 0
    assert _lib.launch_count() == before


def test_no_cpu_path_without_device(walklib):
    """On a machine without a GPU a real launch must fail loudly, not compute on the host."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    rowptr = np.array([0, 1, 2], dtype=np.int64)
    col = np.array([1, 0], dtype=np.int64)
    h = C.c_void_p(None)
    rc = walklib.walk_b200_graph_create(rowptr.ctypes.data, col.ctypes.data, 2, 2, 0, 0, C.byref(h))
    assert rc == _lib.ERR_CUDA and not h.value
    from mlx_cluster_b200 import random_walk
    with pytest.raises(Exception):
        random_walk(torch.from_numpy(rowptr), torch.from_numpy(col), torch.zeros(2, dtype=torch.int64),
                    torch.zeros(2, 3), 3)
