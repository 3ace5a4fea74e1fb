"""Parity of the CUDA node2vec walk, through the C ABI: stream-exact versus the CPU
restatement of the reference loop fed with the same Philox stream, and statistically
matched (chi-square of second-order transitions) to the reference's own rand()-driven
output."""
import numpy as np
import pytest
import torch

import oracle
from mlx_cluster_b200 import _lib, graphs, rejection_sampling
from mlx_cluster_b200.ops import WalkGraph
from tests import _stats
from tests.test_oracle import random_csr

pytestmark = pytest.mark.gpu

PQS = [(1.0, 1.0), (0.5, 2.0), (4.0, 0.25), (0.25, 4.0), (1.0, 3.0)]


@pytest.fixture(autouse=True)
def _reset_tuning():
    yield
    _lib.set_tuning("n2v_idx", 0)
    _lib.set_tuning("n2v_rev", 1)
    _lib.set_tuning("n2v_pool", 1)
    _lib.set_tuning("l2_hints", 3)
    _lib.set_tuning("n2v_max_attempts", 1 << 22)
    _lib.set_tuning("n2v_tri", 1)


def run_gpu(dev, rowptr, col, start, L, p, q, *, seed=0, base=0, symmetric=False, rowdesc=True,
            idx64=False, edges=True, counters=False, edgeset=False, rev=True, pool=False):
    _lib.set_tuning("n2v_idx", 1 if idx64 else 0)
    _lib.set_tuning("n2v_rev", 2 if rev else 0)
    _lib.set_tuning("n2v_pool", 2 if pool else 0)
    g = WalkGraph(torch.from_numpy(rowptr).to(dev), torch.from_numpy(col).to(dev), symmetric=symmetric,
                  use_rowdesc=rowdesc, edgeset=edgeset)
    assert (g.edgeset is not None) == (edgeset and col.size > 0)
    res = rejection_sampling(None, None, torch.from_numpy(start).to(dev), L, p, q, graph=g, seed=seed,
                             walk_index_base=base, return_edges=edges, return_counters=counters, check=True)
    if not isinstance(res, tuple):
        return res.cpu().numpy()
    return tuple(r.cpu().numpy() if isinstance(r, torch.Tensor) else r for r in res)


MEMBERSHIP = {"search_candidate_row": dict(symmetric=False), "search_previous_row": dict(symmetric=True),
              "edge_hash_set": dict(edgeset=True, rev=False), "edge_hash_set_and_reverse_positions": dict(edgeset=True),
              "pooled_kernel": dict(edgeset=True, pool=True)}


@pytest.mark.parametrize("pq", PQS)
@pytest.mark.parametrize("member", list(MEMBERSHIP))
def test_small_workload_stream_exact(cuda, golden, pq, member):
    g = golden
    n_o, e_o, cnt = oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"], 20, *pq, seed=42,
                                         return_edges=True, return_counters=True)
    for rowdesc in (True, False):
        for idx64 in (False, True):
            n, e, c = run_gpu(cuda, g["rowptr2"], g["col2"], g["start2"], 20, *pq, seed=42,
                              rowdesc=rowdesc, idx64=idx64, counters=True, **MEMBERSHIP[member])
            # the uninstrumented kernel is a different instantiation: check it too
            n_plain = run_gpu(cuda, g["rowptr2"], g["col2"], g["start2"], 20, *pq, seed=42,
                              rowdesc=rowdesc, idx64=idx64, edges=False, **MEMBERSHIP[member])
            np.testing.assert_array_equal(n_plain, n_o)
            assert c["formula_probes"] == cnt["bsearch_probes"]
            assert n.shape == (2708, 21) and n.dtype == np.int64
            np.testing.assert_array_equal(n, n_o)
            np.testing.assert_array_equal(e, e_o)
            assert c["attempts"] == cnt["attempts"]
            assert c["membership"] == cnt["membership_needed"]
            assert c["steps_deg0"] == cnt["steps_deg0"] and c["steps_deg1"] == cnt["steps_deg1"]
            assert c["steps_sampled"] == cnt["steps_sampled"] and c["steps_first"] == cnt["steps_first"]
            assert c["probes"] >= c["membership"] or c["membership"] == 0
    iso = g["iso2"]
    assert (n_o[iso] == iso[:, None]).all()


def test_reference_api_signature(cuda, golden):
    g = golden
    t = lambda a: torch.from_numpy(a).to(cuda)
    s = torch.cuda.Stream(cuda)
    out = rejection_sampling(t(g["rowptr2"]), t(g["col2"]), t(g["start2"]), 5, 1.0, 3.0, stream=s)
    s.synchronize()
    assert out.shape == (2708, 6) and out.dtype == torch.int64
    np.testing.assert_array_equal(out.cpu().numpy(),
                                  oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"], 5, 1.0, 3.0, seed=0))
    with pytest.raises(TypeError):
        rejection_sampling(t(g["rowptr2"]), t(g["col2"]), t(g["start2"]), 5, 1.0, 3.0, s)
    for p, q in [(0.0, 1.0), (1.0, float("nan")), (-1.0, 1.0)]:
        with pytest.raises(_lib.WalkError):
            rejection_sampling(t(g["rowptr2"]), t(g["col2"]), t(g["start2"]), 5, p, q)


@pytest.mark.parametrize("cap", [1, 2, 4])
@pytest.mark.parametrize("member", list(MEMBERSHIP))
def test_attempt_cap_stands_still_and_raises_the_flag(cuda, golden, member, cap):
    """The reference's rejection loop is unbounded (BiasedRandomWalk.cpp:80); the CUDA path gives a step up
    after a fixed number of rejections. With the cap lowered to a handful the limit runs out on many steps:
    those stand still with edge id -1, the flag is raised, and everything else is the restatement's walk
    under the same cap."""
    g = golden
    from mlx_cluster_b200 import read_status
    _lib.set_tuning("n2v_max_attempts", cap)
    n_o, e_o, cnt = oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"], 20, 0.25, 4.0, seed=11,
                                         return_edges=True, return_counters=True, max_attempts=cap)
    assert cnt["steps_capped"] > 100
    kw = dict(MEMBERSHIP[member])
    _lib.set_tuning("n2v_rev", 2 if kw.pop("rev", True) else 0)
    _lib.set_tuning("n2v_pool", 2 if kw.pop("pool", False) else 0)
    graph = WalkGraph(torch.from_numpy(g["rowptr2"]).to(cuda), torch.from_numpy(g["col2"]).to(cuda), **kw)
    st = torch.from_numpy(g["start2"]).to(cuda)
    for edges in (True, False):
        res = rejection_sampling(None, None, st, 20, 0.25, 4.0, graph=graph, seed=11, return_edges=edges)
        flags = read_status(graph)
        assert flags == _lib.FLAG_ATTEMPT_CAP
        n = (res[0] if edges else res).cpu().numpy()
        np.testing.assert_array_equal(n, n_o)
        if edges:
            e = res[1].cpu().numpy()
            np.testing.assert_array_equal(e, e_o)
            capped = (e == -1) & (np.diff(g["rowptr2"])[n[:, :-1]] > 0)
            assert capped.sum() == cnt["steps_capped"]
            assert (n[:, 1:][capped] == n[:, :-1][capped]).all()
    with pytest.raises(RuntimeError, match="attempt cap"):
        rejection_sampling(None, None, st, 20, 0.25, 4.0, graph=graph, seed=11, check=True)
    # with the default cap nothing is given up and no flag is raised
    _lib.set_tuning("n2v_max_attempts", 1 << 22)
    rejection_sampling(None, None, st, 20, 0.25, 4.0, graph=graph, seed=11, check=True)


def test_shard_invariance_and_seed(cuda, golden):
    """Rows computed in any batch split carry the same draws (global walk index)."""
    g = golden
    full = run_gpu(cuda, g["rowptr2"], g["col2"], g["start2"], 20, 0.5, 2.0, seed=9, edges=False)
    parts = []
    for world in (2, 3, 8):
        parts = [run_gpu(cuda, g["rowptr2"], g["col2"], g["start2"][b:e], 20, 0.5, 2.0, seed=9, base=b, edges=False)
                 for b, e in (_lib.shard_range(2708, world, r) for r in range(world))]
        np.testing.assert_array_equal(np.concatenate(parts), full)
    for world in (2, 8):  # cyclic shards: rank r holds rows r::world, draws indexed base + i * stride
        for r in range(world):
            gq = WalkGraph(torch.from_numpy(g["rowptr2"]).to(cuda), torch.from_numpy(g["col2"]).to(cuda), edgeset=True)
            part = rejection_sampling(None, None, torch.from_numpy(g["start2"][r::world].copy()).to(cuda), 20, 0.5, 2.0,
                                      graph=gq, seed=9, walk_index_base=r, walk_index_stride=world, check=True)
            np.testing.assert_array_equal(part.cpu().numpy(), full[r::world])
    other = run_gpu(cuda, g["rowptr2"], g["col2"], g["start2"], 20, 0.5, 2.0, seed=10, edges=False)
    assert (other != full).any()
    big_base = (1 << 33) + 5
    a = run_gpu(cuda, g["rowptr2"], g["col2"], g["start2"][:64], 20, 0.5, 2.0, seed=9, base=big_base, edges=False)
    np.testing.assert_array_equal(a, oracle.node2vec_walk(g["rowptr2"], g["col2"], g["start2"][:64], 20, 0.5, 2.0,
                                                          seed=9, walk_index_base=big_base))


@pytest.mark.parametrize("edgeset", [False, True])
@pytest.mark.parametrize("symmetric", [False, True])
def test_ragged_shapes_and_directed_graphs(cuda, symmetric, edgeset):
    rng = np.random.default_rng(21)
    for trial, (n_nodes, walks, L, avg) in enumerate([
            (40, 1, 1, 3.0), (40, 31, 2, 3.0), (40, 33, 7, 6.0), (200, 255, 9, 2.0), (200, 257, 16, 8.0),
            (500, 1000, 33, 5.0), (64, 5, 0, 3.0), (64, 0, 5, 3.0), (2, 40, 12, 2.0), (3000, 4097, 40, 12.0)]):
        # the symmetric fast path is only valid on undirected graphs; the general path takes any CSR
        rowptr, col = random_csr(rng, n_nodes, avg, frac_isolated=0.15, symmetric=symmetric or trial % 2 == 0)
        start = rng.integers(0, n_nodes, walks).astype(np.int64)
        for pq in [(0.25, 4.0), (2.0, 0.5), (1.0, 1.0)]:
            if L == 0:
                n = run_gpu(cuda, rowptr, col, start, L, *pq, seed=trial, symmetric=symmetric, edges=False,
                            edgeset=edgeset)
                np.testing.assert_array_equal(n[:, 0], start)
                continue
            n_o, e_o = oracle.node2vec_walk(rowptr, col, start, L, *pq, seed=trial, return_edges=True)
            for pool in ((False, True) if edgeset else (False,)):
                n, e = run_gpu(cuda, rowptr, col, start, L, *pq, seed=trial, symmetric=symmetric, edgeset=edgeset,
                               pool=pool)
                np.testing.assert_array_equal(n, n_o, err_msg=f"trial {trial} pq {pq} pool {pool}")
                np.testing.assert_array_equal(e, e_o, err_msg=f"trial {trial} pq {pq} pool {pool}")


def test_self_loops_and_degree_one_chains(cuda):
    """Self-loops make 'x == t' and 't in N(x)' overlap; a path graph is all degree-1/2 nodes."""
    rowptr = np.array([0, 3, 5, 8, 9], dtype=np.int64)
    col = np.array([0, 1, 2, 0, 2, 0, 1, 2, 2], dtype=np.int64)   # 0:{0,1,2} 1:{0,2} 2:{0,1,2} 3:{2}
    start = np.array([0, 1, 2, 3] * 40, dtype=np.int64)
    for pq in PQS:
        n_o, e_o = oracle.node2vec_walk(rowptr, col, start, 30, *pq, seed=3, return_edges=True)
        for edgeset, pool in ((False, False), (True, False), (True, True)):
            n, e = run_gpu(cuda, rowptr, col, start, 30, *pq, seed=3, symmetric=False, edgeset=edgeset, pool=pool)
            np.testing.assert_array_equal(n, n_o)
            np.testing.assert_array_equal(e, e_o)
            n = run_gpu(cuda, rowptr, col, start, 30, *pq, seed=3, symmetric=False, edgeset=edgeset, pool=pool,
                        edges=False)
            np.testing.assert_array_equal(n, n_o)
    m = 50
    src = np.arange(m - 1)
    rp, cl = graphs.edges_to_csr(torch.from_numpy(src), torch.from_numpy(src + 1), m)
    rp, cl = rp.numpy(), cl.numpy()
    start = np.arange(m, dtype=np.int64)
    for sym in (False, True):
        n_o = oracle.node2vec_walk(rp, cl, start, 25, 0.25, 4.0, seed=1)
        np.testing.assert_array_equal(run_gpu(cuda, rp, cl, start, 25, 0.25, 4.0, seed=1, symmetric=sym, edges=False), n_o)


def test_unsorted_rows_fall_back_to_the_hash_set_alone(cuda):
    """Rows in arbitrary order: no binary search and no reverse positions, but the edge hash set
    still answers membership exactly."""
    rng = np.random.default_rng(5)
    rowptr, col = random_csr(rng, 400, 6.0, symmetric=True)
    col = col.copy()
    for v in range(400):
        rng.shuffle(col[rowptr[v]:rowptr[v + 1]])
    start = rng.integers(0, 400, 3000).astype(np.int64)
    g = WalkGraph(torch.from_numpy(rowptr).to(cuda), torch.from_numpy(col).to(cuda), edgeset=True)
    assert g.edgeset is not None and g.colrev is None
    for pq in [(0.25, 4.0), (2.0, 0.5)]:
        want = oracle.node2vec_walk(rowptr, col, start, 25, *pq, seed=2)
        got = rejection_sampling(None, None, torch.from_numpy(start).to(cuda), 25, *pq, graph=g, seed=2, check=True)
        np.testing.assert_array_equal(got.cpu().numpy(), want)
    sorted_graph = WalkGraph(torch.from_numpy(rowptr).to(cuda),
                             torch.from_numpy(np.concatenate([np.sort(col[rowptr[v]:rowptr[v + 1]]) for v in range(400)])).to(cuda),
                             edgeset=True)
    assert sorted_graph.colrev is not None


def test_medium_rmat_stream_exact(cuda):
    rowptr, col = graphs.rmat_csr(14, 16, seed=6, device=cuda)
    n_nodes = rowptr.numel() - 1
    start = torch.arange(n_nodes, dtype=torch.int64, device=cuda)
    rp, cl, st = rowptr.cpu().numpy(), col.cpu().numpy(), start.cpu().numpy()
    for pq in [(0.25, 4.0), (1.0, 2.0)]:
        n_o, cnt = oracle.node2vec_walk(rp, cl, st, 40, *pq, seed=77, return_counters=True)
        for sym in (True, False):
            out, c = rejection_sampling(rowptr, col, start, 40, *pq, seed=77, symmetric=sym,
                                        return_counters=True, check=True)
            np.testing.assert_array_equal(out.cpu().numpy(), n_o)
            assert c["attempts"] == cnt["attempts"] and c["membership"] == cnt["membership_needed"]
            assert c["formula_probes"] == cnt["bsearch_probes"]
        hashed = WalkGraph(rowptr, col, edgeset=True)
        assert hashed.colrev is not None
        _lib.set_tuning("n2v_pool", 2)
        out = rejection_sampling(None, None, start, 40, *pq, graph=hashed, seed=77, check=True)
        np.testing.assert_array_equal(out.cpu().numpy(), n_o)
        _lib.set_tuning("n2v_pool", 0)
        loads = {}
        for rev in (1, 0):
            _lib.set_tuning("n2v_rev", 2 if rev else 0)
            out, c = rejection_sampling(None, None, start, 40, *pq, graph=hashed, seed=77, check=True,
                                        return_counters=True)
            np.testing.assert_array_equal(out.cpu().numpy(), n_o)
            assert c["attempts"] == cnt["attempts"] and c["membership"] == cnt["membership_needed"]
            assert c["formula_probes"] == cnt["bsearch_probes"]
            loads[rev] = c["loads"]
        if pq == (0.25, 4.0):
            assert loads[1] < 0.75 * loads[0]  # three attempts in four need no gather


@pytest.mark.parametrize("pq", [(1.0, 1.0), (0.5, 2.0), (4.0, 0.25)])
def test_chi_square_against_reference_output(cuda, golden, pq):
    """Second-order transition frequencies of the CUDA walk (Philox) versus the reference's
    own rejection_sampling output (libc rand()): compiled reference when its library is
    present, else the restatement in rand() mode that is pinned bit-for-bit to it."""
    g = golden
    rowptr, col, start = g["rowptr2"], g["col2"], g["start2"]
    runs = 24
    ref_walks = []
    for k in range(runs):
        if oracle.have_ref():
            ref_walks.append(oracle.ref_rejection_sampling(rowptr, col, start, 20, *pq, srand_seed=100 + k))
        else:
            oracle.libc_srand(100 + k)
            ref_walks.append(oracle.node2vec_walk(rowptr, col, start, 20, *pq, draw_mode=0))
    graph = WalkGraph(torch.from_numpy(rowptr).to(cuda), torch.from_numpy(col).to(cuda), symmetric=True)
    st = torch.from_numpy(start).to(cuda)
    gpu_walks = [rejection_sampling(None, None, st, 20, *pq, graph=graph, seed=5000 + k, check=True).cpu().numpy()
                 for k in range(runs)]
    cb = _stats.triple_counts(np.concatenate(ref_walks), 2708)
    stat, dof, pval, cells = _stats.two_sample_chi2(_stats.triple_counts(np.concatenate(gpu_walks), 2708), cb)
    assert cells > 500 and dof > 1000
    assert pval > 1e-3, (stat, dof, pval)
    wrong = [rejection_sampling(None, None, st, 20, 0.25, 4.0, graph=graph, seed=6000 + k).cpu().numpy()
             for k in range(runs)]
    _, _, p_wrong, _ = _stats.two_sample_chi2(_stats.triple_counts(np.concatenate(wrong), 2708), cb)
    assert p_wrong < 1e-6


def test_properties_at_scale(cuda):
    """Graph larger than L2, all nodes start: steps follow edges, runs repeat exactly, the
    symmetric and general membership searches agree, 32- and 64-bit index kernels agree."""
    rowptr, col = graphs.rmat_csr(20, 16, seed=2, device=cuda)
    n_nodes = rowptr.numel() - 1
    start = torch.arange(n_nodes, dtype=torch.int64, device=cuda)
    L = 40
    out, e = rejection_sampling(rowptr, col, start, L, 0.25, 4.0, seed=3, symmetric=True,
                                return_edges=True, check=True)
    assert torch.equal(out[:, 0], start)
    src, dst = out[:, :-1], out[:, 1:]
    moved = e >= 0
    assert torch.equal(col[e[moved]], dst[moved])
    assert bool(((rowptr[src[moved]] <= e[moved]) & (e[moved] < rowptr[src[moved] + 1])).all())
    assert bool((rowptr.diff()[src[~moved]] == 0).all())
    general = rejection_sampling(rowptr, col, start, L, 0.25, 4.0, seed=3, symmetric=False, check=True)
    assert torch.equal(out, general)
    hashed = WalkGraph(rowptr, col, edgeset=True)
    assert torch.equal(out, rejection_sampling(None, None, start, L, 0.25, 4.0, graph=hashed, seed=3, check=True))
    for hints in (0, 1, 3):
        _lib.set_tuning("l2_hints", hints)
        assert torch.equal(out, rejection_sampling(None, None, start, L, 0.25, 4.0, graph=hashed, seed=3))
    _lib.set_tuning("n2v_rev", 0)
    assert torch.equal(out, rejection_sampling(None, None, start, L, 0.25, 4.0, graph=hashed, seed=3))
    _lib.set_tuning("n2v_rev", 1)
    _lib.set_tuning("n2v_idx", 1)
    assert torch.equal(out, rejection_sampling(rowptr, col, start, L, 0.25, 4.0, seed=3, symmetric=True))
    assert torch.equal(out, rejection_sampling(None, None, start, L, 0.25, 4.0, graph=hashed, seed=3))
    # every 997th row of the pooled kernel's matrix and of the per-lane kernel's against the CPU restatement,
    # which is handed the same global walk indices 0, 997, ...
    rp_h, cl_h = rowptr.cpu().numpy(), col.cpu().numpy()
    picked = torch.arange(0, n_nodes, 997, device=cuda)
    want = oracle.node2vec_walk(rp_h, cl_h, picked.cpu().numpy(), L, 0.25, 4.0, seed=3, walk_index_stride=997)
    _lib.set_tuning("n2v_idx", 0)
    for pool in (2, 0):
        _lib.set_tuning("n2v_pool", pool)
        got = rejection_sampling(None, None, start, L, 0.25, 4.0, graph=hashed, seed=3, check=True)
        assert torch.equal(got, out), pool
        np.testing.assert_array_equal(got[picked].cpu().numpy(), want)
    # a sub-sample of rows against the CPU restatement
    rows = torch.arange(0, n_nodes, 997, device=cuda)
    n_o = oracle.node2vec_walk(rowptr.cpu().numpy(), col.cpu().numpy(), rows.cpu().numpy(), L, 0.25, 4.0, seed=3,
                               walk_index_base=0)
    # walk index = row position, so recompute those rows with their own global indices
    sub = torch.stack([rejection_sampling(rowptr, col, rows[i:i + 1], L, 0.25, 4.0, seed=3, symmetric=True,
                                          walk_index_base=i)[0] for i in range(0, 64)])
    np.testing.assert_array_equal(sub.cpu().numpy(), n_o[:64])


def _filter_words_by_definition(rowptr, col):
    """Bit k of the word of edge e = (a -> b): some common neighbour of a and b sits at a position p of b's row
    with p % 64 == k. Plain numpy, small graphs only."""
    n = rowptr.size - 1
    rows = [col[rowptr[v]:rowptr[v + 1]] for v in range(n)]
    src = np.repeat(np.arange(n), np.diff(rowptr))
    words = np.zeros(col.size, dtype=np.uint64)
    for e in range(col.size):
        a, b = int(src[e]), int(col[e])
        if a == b:
            words[e] = np.uint64(0xffffffffffffffff)   # self-loops go unfiltered
            continue
        common = np.intersect1d(rows[a], rows[b], assume_unique=True)
        pos = np.searchsorted(rows[b], common)
        w = 0
        for p in pos:
            w |= 1 << (int(p) & 63)
        words[e] = np.uint64(w)
    return words


def test_triangle_filter_words_and_walks(cuda, golden):
    """The filter words equal their definition, and walks that use them are the restatement's walks."""
    g = golden
    rng = np.random.default_rng(31)
    graphs_small = [(g["rowptr2"], g["col2"]), random_csr(rng, 300, 9.0, frac_isolated=0.1, symmetric=True),
                    random_csr(rng, 200, 160.0, frac_isolated=0.0, symmetric=True)]   # the last one: rows longer than 64
    for rowptr, col in graphs_small:
        graph = WalkGraph(torch.from_numpy(rowptr).to(cuda), torch.from_numpy(col).to(cuda), symmetric=True,
                          edgeset=True, trifilter=True)
        rec = graph.colrev16.cpu().numpy()
        np.testing.assert_array_equal(rec[:, 0], graph.colrev.cpu().numpy())
        np.testing.assert_array_equal(rec[:, 1].view(np.uint64), _filter_words_by_definition(rowptr, col))
        n_nodes = rowptr.size - 1
        start = np.concatenate([np.arange(n_nodes), rng.integers(0, n_nodes, 3000)]).astype(np.int64)
        st = torch.from_numpy(start).to(cuda)
        for pq in PQS:
            n_o, e_o = oracle.node2vec_walk(rowptr, col, start, 30, *pq, seed=17, return_edges=True)
            _lib.set_tuning("n2v_pool", 2)
            for edges in (True, False):
                res = rejection_sampling(None, None, st, 30, *pq, graph=graph, seed=17, return_edges=edges, check=True)
                assert _lib.last_kernel() == "node2vec_pool_tri_kernel"
                np.testing.assert_array_equal((res[0] if edges else res).cpu().numpy(), n_o)
                if edges:
                    np.testing.assert_array_equal(res[1].cpu().numpy(), e_o)
            _lib.set_tuning("n2v_tri", 0)
            rejection_sampling(None, None, st, 30, *pq, graph=graph, seed=17)
            assert _lib.last_kernel() == "node2vec_pool_kernel"
            _lib.set_tuning("n2v_tri", 1)
        # the attempt cap runs out in the filtered kernel as in the others
        _lib.set_tuning("n2v_max_attempts", 3)
        n_o, e_o = oracle.node2vec_walk(rowptr, col, start, 30, 0.25, 4.0, seed=17, return_edges=True, max_attempts=3)
        n, e = rejection_sampling(None, None, st, 30, 0.25, 4.0, graph=graph, seed=17, return_edges=True)
        np.testing.assert_array_equal(n.cpu().numpy(), n_o)
        np.testing.assert_array_equal(e.cpu().numpy(), e_o)
        from mlx_cluster_b200 import read_status
        assert read_status(graph) == _lib.FLAG_ATTEMPT_CAP
        _lib.set_tuning("n2v_max_attempts", 1 << 22)
    # a limit on the row length leaves long rows unfiltered (all ones), never wrong
    rowptr, col = graphs_small[2]
    capped = WalkGraph(torch.from_numpy(rowptr).to(cuda), torch.from_numpy(col).to(cuda), symmetric=True, edgeset=True,
                       trifilter=True, trifilter_max_row=30)
    words = capped.colrev16.cpu().numpy()[:, 1].view(np.uint64)
    want = _filter_words_by_definition(rowptr, col)
    assert ((words == want) | (words == np.uint64(0xffffffffffffffff))).all() and (words != want).any()
    with pytest.raises(ValueError, match="undirected"):
        WalkGraph(torch.from_numpy(rowptr).to(cuda), torch.from_numpy(col).to(cuda), edgeset=True, trifilter=True)


def test_triangle_filter_at_scale(cuda):
    """Graph larger than L2: the filtered kernel reproduces the unfiltered matrix and every 997th row of the restatement."""
    rowptr, col = graphs.rmat_csr(20, 16, seed=2, device=cuda)
    n_nodes = rowptr.numel() - 1
    start = torch.arange(n_nodes, dtype=torch.int64, device=cuda)
    L = 40
    graph = WalkGraph(rowptr, col, symmetric=True, edgeset=True, trifilter=True)
    _lib.set_tuning("n2v_tri", 0)
    plain = rejection_sampling(None, None, start, L, 0.25, 4.0, graph=graph, seed=3, check=True)
    assert _lib.last_kernel() == "node2vec_pool_kernel"
    _lib.set_tuning("n2v_tri", 1)
    for pq in ((0.25, 4.0), (0.5, 2.0)):
        got = rejection_sampling(None, None, start, L, *pq, graph=graph, seed=3, check=True)
        assert _lib.last_kernel() == "node2vec_pool_tri_kernel"
        if pq == (0.25, 4.0):
            assert torch.equal(got, plain)
        picked = torch.arange(0, n_nodes, 997, device=cuda)
        want = oracle.node2vec_walk(rowptr.cpu().numpy(), col.cpu().numpy(), picked.cpu().numpy(), L, *pq, seed=3,
                                    walk_index_stride=997)
        np.testing.assert_array_equal(got[picked].cpu().numpy(), want)
