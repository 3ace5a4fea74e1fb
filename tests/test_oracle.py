"""Pins the CPU restatement (oracle/walk_oracle.c) to the reference: against the
committed outputs of the reference's own eval_cpu loops, and live against the compiled
reference where it is available. Runs without a GPU."""
import json
from pathlib import Path

import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

import oracle
from tests import _stats

ROOT = Path(__file__).resolve().parents[1]
needs_ref = pytest.mark.skipif(not oracle.have_ref(), reason="compiled reference not available")


def random_csr(rng, n, avg_deg, frac_isolated=0.1, symmetric=True):
    m = max(1, int(n * avg_deg / 2))
    src = rng.integers(0, n, m)
    dst = rng.integers(0, n, m)
    dead = rng.random(n) < frac_isolated
    keep = (src != dst) & ~dead[src] & ~dead[dst]
    src, dst = src[keep], dst[keep]
    if symmetric:
        src, dst = np.concatenate([src, dst]), np.concatenate([dst, src])
    key = np.unique(src.astype(np.int64) * n + dst)
    row, col = key // n, key % n
    rowptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(np.bincount(row, minlength=n), out=rowptr[1:])
    return rowptr, col.astype(np.int64)


def test_philox_matches_independent_implementation():
    doc = json.loads((ROOT / "tests" / "golden" / "philox_kat.json").read_text())
    assert len(doc["vectors"]) >= 50
    for v in doc["vectors"]:
        assert oracle.philox4x32_10(v["counter"], v["key"]).tolist() == v["out"]


def test_uniform_matches_reference_fixture(golden):
    g = golden
    n, e = oracle.uniform_walk(g["rowptr1"], g["col1"], g["start1"], g["rand1"], 5, return_edges=True)
    assert n.shape == (2000, 6)
    np.testing.assert_array_equal(n, g["uniform1_n"])
    np.testing.assert_array_equal(e, g["uniform1_e"])
    n, e = oracle.uniform_walk(g["rowptr2"], g["col2"], g["start2"], g["rand2"], 20, return_edges=True)
    np.testing.assert_array_equal(n, g["uniform2_n"])
    np.testing.assert_array_equal(e, g["uniform2_e"])
    # isolated start nodes never move and record edge id -1
    iso = g["iso2"]
    assert (n[iso] == iso[:, None]).all() and (e[iso] == -1).all()


def test_biased_rand_mode_matches_reference_fixture(golden):
    g = golden
    rows = g["biased2_pq0_srand1_n"].shape[0]
    for i, (p, q) in enumerate(g["pq"]):
        for s in g["srand"]:
            oracle.libc_srand(int(s))
            n, e = oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"][:rows], 20, p, q,
                                        draw_mode=0, return_edges=True)
            np.testing.assert_array_equal(n, g[f"biased2_pq{i}_srand{s}_n"])
            if f"biased2_pq{i}_srand{s}_e" in g:
                np.testing.assert_array_equal(e, g[f"biased2_pq{i}_srand{s}_e"])


@needs_ref
def test_factory_shapes_of_reference():
    # output 0 is [n, L+1]; uniform has 4 inputs, biased 3; dtype int64
    assert oracle.ref_factory_shapes(7, 5, 0) == (7, 6, 4, 1)
    assert oracle.ref_factory_shapes(7, 5, 1) == (7, 6, 3, 1)
    assert oracle.ref_rand_max() == 2147483647


@needs_ref
@settings(max_examples=40, deadline=None)
@given(seed=st.integers(0, 2**31 - 1), n=st.integers(2, 200), avg=st.floats(0.5, 12.0),
       L=st.integers(0, 33), walks=st.integers(1, 70), sym=st.booleans())
def test_uniform_matches_compiled_reference(seed, n, avg, L, walks, sym):
    rng = np.random.default_rng(seed)
    rowptr, col = random_csr(rng, n, avg, symmetric=sym)
    start = rng.integers(0, n, walks).astype(np.int64)
    rand = rng.random((walks, L), dtype=np.float32)
    n_ref, e_ref = oracle.ref_random_walk(rowptr, col, start, rand, L, return_edges=True)
    n_o, e_o = oracle.uniform_walk(rowptr, col, start, rand, L, return_edges=True)
    np.testing.assert_array_equal(n_o, n_ref)
    np.testing.assert_array_equal(e_o, e_ref)


@needs_ref
def test_uniform_float32_rounding_matches_compiled_reference():
    # a hub whose degree is not exactly representable in float32 and draws next to 1:
    # the float32 conversion/product/truncation must agree bit for bit
    deg = (1 << 24) + 3
    rowptr = np.array([0, deg] + [deg] * deg, dtype=np.int64)[: 3]  # node 0 = hub, node 1 = leaf
    rowptr = np.concatenate([[0, deg], np.full(2, deg)]).astype(np.int64)  # nodes 0..2
    col = (np.arange(deg, dtype=np.int64) % 2) + 1  # neighbours 1,2,1,2...
    rand = np.array([np.nextafter(np.float32(1), np.float32(0)), 0.5, 0.99999, 1e-8, 0.33333334],
                    dtype=np.float32).reshape(5, 1)
    start = np.zeros(5, dtype=np.int64)
    n_ref, e_ref = oracle.ref_random_walk(rowptr, col, start, rand, 1, return_edges=True)
    n_o, e_o = oracle.uniform_walk(rowptr, col, start, rand, 1, return_edges=True)
    np.testing.assert_array_equal(e_o, e_ref)
    np.testing.assert_array_equal(n_o, n_ref)
    assert e_ref.max() < deg


@needs_ref
@settings(max_examples=30, deadline=None)
@given(seed=st.integers(0, 2**31 - 1), n=st.integers(2, 120), avg=st.floats(0.5, 10.0),
       L=st.integers(1, 25), walks=st.integers(1, 50), sym=st.booleans(),
       pq=st.sampled_from([(1.0, 1.0), (0.5, 2.0), (4.0, 0.25), (0.25, 4.0), (1.0, 3.0), (2.0, 2.0)]))
def test_biased_rand_mode_matches_compiled_reference(seed, n, avg, L, walks, sym, pq):
    rng = np.random.default_rng(seed)
    rowptr, col = random_csr(rng, n, avg, symmetric=sym)
    start = rng.integers(0, n, walks).astype(np.int64)
    n_ref, e_ref = oracle.ref_rejection_sampling(rowptr, col, start, L, *pq, srand_seed=seed % 1000,
                                                 return_edges=True)
    oracle.libc_srand(seed % 1000)
    n_o, e_o = oracle.node2vec_walk(rowptr, col, start, L, *pq, draw_mode=0, return_edges=True)
    np.testing.assert_array_equal(n_o, n_ref)
    np.testing.assert_array_equal(e_o, e_ref)


@needs_ref
def test_biased_full_start_set_matches_compiled_reference(golden):
    g = golden
    for p, q in [(1.0, 1.0), (0.5, 2.0), (4.0, 0.25)]:
        n_ref = oracle.ref_rejection_sampling(g["rowptr2"], g["col2"], g["start2"], 20, p, q, srand_seed=11)
        oracle.libc_srand(11)
        n_o = oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"], 20, p, q, draw_mode=0)
        np.testing.assert_array_equal(n_o, n_ref)


def test_thresholds_and_integer_cuts():
    table = {(1, 1): (1, 1, 1), (0.5, 2): (1, 0.5, 0.25), (4, 0.25): (0.0625, 0.25, 1),
             (0.25, 4): (1, 0.25, 0.0625), (1, 2): (1, 1, 0.5)}
    for (p, q), want in table.items():
        np.testing.assert_array_equal(oracle.thresholds(p, q), np.array(want, dtype=np.float64))
    t = oracle.thresholds(1, 3)
    assert t[0] == 1.0 and t[1] == 1.0 and t[2] == 1.0 / 3.0
    for prob in [1.0, 0.5, 0.25, 0.0625, 1.0 / 3.0, 1e-4, 0.9999999999, 2.0 ** -16]:
        cut = oracle.accept_cut(prob)
        # r(w) = w / RAND_MAX; "r < prob" holds exactly for w < cut
        assert cut == 0 or (cut - 1) / 2147483647.0 < prob
        assert cut > 2147483647 or cut / 2147483647.0 >= prob
    assert oracle.accept_cut(1.0) == 2147483647  # r == 1.0 (w == RAND_MAX) is rejected, as in the reference


def test_biased_philox_structure(golden):
    """Philox mode: deterministic, independent of batch composition, isolated nodes stay,
    degree-1 nodes move without consuming a draw, every step follows an edge."""
    g = golden
    rowptr, col, start = g["rowptr2"], g["col2"], g["start2"]
    a, ea, cnt = oracle.node2vec_walk(rowptr, col, start, 20, 0.5, 2.0, seed=5, return_edges=True,
                                      return_counters=True)
    b = oracle.node2vec_walk(rowptr, col, start[100:300], 20, 0.5, 2.0, seed=5, walk_index_base=100)
    np.testing.assert_array_equal(a[100:300], b)
    c = oracle.node2vec_walk(rowptr, col, start, 20, 0.5, 2.0, seed=6)
    assert (a != c).any()
    iso = g["iso2"]
    assert (a[iso] == iso[:, None]).all() and (ea[iso] == -1).all()
    moved = ea >= 0
    assert (col[ea[moved]] == a[:, 1:][moved]).all()
    src = a[:, :-1][moved]
    assert ((rowptr[src] <= ea[moved]) & (ea[moved] < rowptr[src + 1])).all()
    assert cnt["steps_deg0"] + cnt["steps_deg1"] + cnt["steps_sampled"] + cnt["steps_first"] == a.shape[0] * 20
    assert cnt["attempts"] >= cnt["steps_sampled"] and cnt["membership_needed"] <= cnt["membership_ref"]


@pytest.mark.parametrize("pq", [(1.0, 1.0), (0.5, 2.0), (4.0, 0.25)])
def test_philox_restatement_matches_reference_statistics(golden, pq):
    """Chi-square of second-order transition counts: Philox-driven restatement against the
    reference's own rand()-driven loop (the compiled reference when present, otherwise the
    restatement in rand() mode, which is pinned bit-for-bit to it above)."""
    g = golden
    rowptr, col, start = g["rowptr2"], g["col2"], g["start2"]
    runs = 24
    ref_walks, phi_walks = [], []
    for k in range(runs):
        if oracle.have_ref():
            ref_walks.append(oracle.ref_rejection_sampling(rowptr, col, start, 20, *pq, srand_seed=100 + k))
        else:
            oracle.libc_srand(100 + k)
            ref_walks.append(oracle.node2vec_walk(rowptr, col, start, 20, *pq, draw_mode=0))
        phi_walks.append(oracle.node2vec_walk(rowptr, col, start, 20, *pq, seed=1000 + k))
    ca = _stats.triple_counts(np.concatenate(phi_walks), 2708)
    cb = _stats.triple_counts(np.concatenate(ref_walks), 2708)
    stat, dof, pval, cells = _stats.two_sample_chi2(ca, cb)
    assert cells > 500 and dof > 1000
    assert pval > 1e-3, (stat, dof, pval)
    # the test has power: a different (p, q) is rejected. (q < 1 <= p makes prob_2 the
    # largest threshold, so the reference then accepts every candidate and (4, 0.25) walks
    # like (1, 1); (0.25, 4) differs from all three.)
    other = (0.25, 4.0)
    wrong = [oracle.node2vec_walk(rowptr, col, start, 20, *other, seed=2000 + k) for k in range(runs)]
    _, _, p_wrong, _ = _stats.two_sample_chi2(_stats.triple_counts(np.concatenate(wrong), 2708), cb)
    assert p_wrong < 1e-6


def test_attempt_cap_of_the_restatement_only_bites_when_it_runs_out(golden):
    """max_attempts = 0 is the reference's unbounded loop; a cap no step reaches changes nothing; a small cap turns
    exactly the steps that exhaust it into stand-still steps (edge id -1) and leaves the rows before them alone."""
    g = golden
    args = (g["rowptr2"], g["col2"], g["start2"], 20, 0.25, 4.0)
    n0, e0, c0 = oracle.node2vec_walk(*args, seed=5, return_edges=True, return_counters=True)
    n1, e1, c1 = oracle.node2vec_walk(*args, seed=5, return_edges=True, return_counters=True, max_attempts=1 << 22)
    np.testing.assert_array_equal(n0, n1)
    np.testing.assert_array_equal(e0, e1)
    assert c0["steps_capped"] == 0 and c1["steps_capped"] == 0
    n2, e2, c2 = oracle.node2vec_walk(*args, seed=5, return_edges=True, return_counters=True, max_attempts=2)
    assert c2["steps_capped"] > 0
    deg = np.diff(g["rowptr2"])
    capped = (e2 == -1) & (deg[n2[:, :-1]] > 0)
    assert capped.sum() == c2["steps_capped"]
    assert (n2[:, 1:][capped] == n2[:, :-1][capped]).all()
    # up to its first capped step a walk is the uncapped walk (same draws, same decisions)
    first = np.where(capped.any(axis=1), capped.argmax(axis=1), 20)
    for w in range(0, n2.shape[0], 37):
        k = first[w]
        np.testing.assert_array_equal(n2[w, :k + 1], n0[w, :k + 1])
