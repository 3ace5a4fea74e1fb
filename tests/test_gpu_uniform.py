"""Parity of the CUDA uniform walk against the reference, through the C ABI:
bit-exact versus the reference's committed outputs, the CPU restatement and (when its
library is present) the compiled reference itself."""
import numpy as np
import pytest
import torch

import oracle
from mlx_cluster_b200 import _lib, graphs, random_walk
from mlx_cluster_b200.ops import WalkGraph
from tests.test_oracle import random_csr

pytestmark = pytest.mark.gpu

VARIANTS = {"direct": 1, "staged8": 2, "staged16": 3, "staged4": 4, "staged16_40regs": 5, "staged8_32regs": 6,
            "staged16_64regs": 7, "staged16_48regs": 8, "staged8_40regs": 9}


@pytest.fixture(autouse=True)
def _reset_tuning():
    yield
    _lib.set_tuning("uniform_variant", 0)
    _lib.set_tuning("uniform_fused", 1)


def run_gpu(dev, rowptr, col, start, rand, L, *, variant="staged8", rowdesc=True, edges=True, check=True,
            fused=False):
    _lib.set_tuning("uniform_variant", VARIANTS[variant])
    g = WalkGraph(torch.from_numpy(rowptr).to(dev), torch.from_numpy(col).to(dev), use_rowdesc=rowdesc, fused=fused)
    assert (g.rowdesc is not None) == (rowdesc and g.num_nodes > 0)
    assert (g.fused is not None) == (fused and rowdesc and col.size > 0)
    before = _lib.launch_count()
    res = random_walk(None, None, torch.from_numpy(start).to(dev), torch.from_numpy(rand).to(dev), L,
                      graph=g, return_edges=edges, check=check)
    if start.size:
        assert _lib.launch_count() == before + 1
    if edges:
        return res[0].cpu().numpy(), res[1].cpu().numpy()
    return res.cpu().numpy()


@pytest.mark.parametrize("variant", list(VARIANTS))
@pytest.mark.parametrize("rowdesc", [True, False])
def test_fixture_workloads_bit_exact(cuda, golden, variant, rowdesc):
    g = golden
    n, e = run_gpu(cuda, g["rowptr1"], g["col1"], g["start1"], g["rand1"], 5, variant=variant, rowdesc=rowdesc)
    assert n.shape == (2000, 6) and n.dtype == np.int64
    np.testing.assert_array_equal(n, g["uniform1_n"])
    np.testing.assert_array_equal(e, g["uniform1_e"])
    n, e = run_gpu(cuda, g["rowptr2"], g["col2"], g["start2"], g["rand2"], 20, variant=variant, rowdesc=rowdesc)
    np.testing.assert_array_equal(n, g["uniform2_n"])
    np.testing.assert_array_equal(e, g["uniform2_e"])
    # fused edge records (one gather per step): same walks
    n, e = run_gpu(cuda, g["rowptr2"], g["col2"], g["start2"], g["rand2"], 20, variant=variant, rowdesc=rowdesc, fused=True)
    np.testing.assert_array_equal(n, g["uniform2_n"])
    np.testing.assert_array_equal(e, g["uniform2_e"])


def test_reference_api_signature(cuda, golden):
    """Positional call exactly as the reference's demo makes it; stream keyword-only."""
    g = golden
    t = lambda a: torch.from_numpy(a).to(cuda)
    s = torch.cuda.Stream(cuda)
    out = random_walk(t(g["rowptr1"]), t(g["col1"]), t(g["start1"]), t(g["rand1"]), 5, stream=s)
    s.synchronize()
    assert out.shape == (2000, 6) and out.dtype == torch.int64 and out.device == cuda
    np.testing.assert_array_equal(out.cpu().numpy(), g["uniform1_n"])
    with pytest.raises(TypeError):
        random_walk(t(g["rowptr1"]), t(g["col1"]), t(g["start1"]), t(g["rand1"]), 5, s)
    with pytest.raises(TypeError):
        random_walk(t(g["rowptr1"]).int(), t(g["col1"]), t(g["start1"]), t(g["rand1"]), 5)
    with pytest.raises(ValueError):
        random_walk(t(g["rowptr1"]), t(g["col1"]), t(g["start1"]), t(g["rand1"])[:, :4].contiguous(), 5)


@pytest.mark.parametrize("variant", list(VARIANTS))
def test_ragged_shapes_against_restatement(cuda, variant):
    """Walk counts that do not fill a warp or a block, walk lengths that do not fill a
    chunk, empty batches, zero-length walks, directed graphs with sink nodes."""
    rng = np.random.default_rng(11)
    for trial, (n_nodes, walks, L, sym) in enumerate([
            (50, 1, 1, True), (50, 31, 7, True), (50, 33, 8, False), (300, 255, 9, True),
            (300, 257, 16, False), (300, 513, 17, True), (1000, 1000, 33, False),
            (64, 5, 0, True), (64, 0, 5, True), (2, 40, 12, True), (5000, 4097, 40, True)]):
        rowptr, col = random_csr(rng, n_nodes, 4.0, frac_isolated=0.15, symmetric=sym)
        start = rng.integers(0, n_nodes, walks).astype(np.int64)
        rand = rng.random((walks, L), dtype=np.float32)
        n_o, e_o = oracle.uniform_walk(rowptr, col, start, rand, L, return_edges=True)
        for rowdesc in (True, False):
            n, e = run_gpu(cuda, rowptr, col, start, rand, L, variant=variant, rowdesc=rowdesc)
            np.testing.assert_array_equal(n, n_o, err_msg=f"trial {trial}")
            np.testing.assert_array_equal(e, e_o, err_msg=f"trial {trial}")
            n_only = run_gpu(cuda, rowptr, col, start, rand, L, variant=variant, rowdesc=rowdesc, edges=False)
            np.testing.assert_array_equal(n_only, n_o)
        n, e = run_gpu(cuda, rowptr, col, start, rand, L, variant=variant, fused=True)
        np.testing.assert_array_equal(n, n_o, err_msg=f"trial {trial} fused")
        np.testing.assert_array_equal(e, e_o, err_msg=f"trial {trial} fused")


def test_hub_degree_float32_rounding(cuda):
    """Degrees beyond 2^24 are not exact in float32; draws next to 1 must still land inside
    the row exactly where the reference puts them."""
    deg = (1 << 24) + 3
    rowptr = np.array([0, deg, deg, deg], dtype=np.int64)
    col = (np.arange(deg, dtype=np.int64) % 2) + 1
    rand = np.array([np.nextafter(np.float32(1), np.float32(0)), 0.5, 0.99999, 1e-8, 0.33333334, 0.0],
                    dtype=np.float32).reshape(6, 1)
    start = np.zeros(6, dtype=np.int64)
    n_o, e_o = oracle.uniform_walk(rowptr, col, start, rand, 1, return_edges=True)
    for variant in ("direct", "staged8"):
        for fused in (False, True):
            n, e = run_gpu(cuda, rowptr, col, start, rand, 1, variant=variant, fused=fused)
            np.testing.assert_array_equal(e, e_o)
            np.testing.assert_array_equal(n, n_o)


def test_medium_rmat_against_restatement_and_reference(cuda):
    rowptr, col = graphs.rmat_csr(15, 16, seed=5, device=cuda)
    n_nodes = rowptr.numel() - 1
    g = torch.Generator(device=cuda).manual_seed(9)
    L = 80
    start = torch.arange(n_nodes, dtype=torch.int64, device=cuda)
    rand = torch.rand((n_nodes, L), generator=g, device=cuda)
    out = random_walk(rowptr, col, start, rand, L, check=True).cpu().numpy()
    args = (rowptr.cpu().numpy(), col.cpu().numpy(), start.cpu().numpy(), rand.cpu().numpy(), L)
    np.testing.assert_array_equal(out, oracle.uniform_walk(*args))
    np.testing.assert_array_equal(random_walk(rowptr, col, start, rand, L, check=True, fused=True).cpu().numpy(), out)
    if oracle.have_ref():
        np.testing.assert_array_equal(out, oracle.ref_random_walk(*args))


def test_malformed_input_is_flagged_not_faulted(cuda, golden):
    g = golden
    t = lambda a: torch.from_numpy(a).to(cuda)
    rowptr, col = t(g["rowptr1"]), t(g["col1"])
    start = t(g["start1"]).clone()
    rand = t(g["rand1"]).clone()
    # a draw of exactly 1.0 indexes one past the row (undefined in the reference): flagged
    rand[3, 2] = 1.0
    start[7] = 2708          # out of range
    start[8] = -5
    start[9] = 1 << 40
    for variant in ("staged16_64regs", "direct"):
        _lib.set_tuning("uniform_variant", VARIANTS[variant])
        with pytest.raises(RuntimeError, match="status flags"):
            random_walk(rowptr, col, start, rand, 5, check=True)
        out, e = random_walk(rowptr, col, start, rand, 5, return_edges=True)
        torch.cuda.synchronize()
        assert (out[7] == 2708).all() and (out[8] == -5).all() and (out[9] == 1 << 40).all()   # parked on the bad id
        assert (e[[7, 8, 9]] == -1).all()
        good = np.ones(2000, dtype=bool)
        good[[3, 7, 8, 9]] = False
        np.testing.assert_array_equal(out.cpu().numpy()[good], g["uniform1_n"][good])
        np.testing.assert_array_equal(e.cpu().numpy()[good], g["uniform1_e"][good])
        from mlx_cluster_b200 import clear_caches
        clear_caches()   # the cached graph keeps the raised flags
    _lib.set_tuning("uniform_variant", 0)
    graph = WalkGraph(rowptr, col)
    with pytest.raises(ValueError, match="node id out of range"):
        graph.validate(start)
    graph.validate(t(g["start1"]))
    bad_col = col.clone()
    bad_col[10], bad_col[11] = bad_col[11].item(), bad_col[10].item()
    if bad_col[10] != bad_col[11]:
        with pytest.raises(ValueError, match="ascending"):
            WalkGraph(rowptr, bad_col).validate()


def test_every_step_follows_an_edge_at_full_length(cuda):
    """Size-independent property on a graph larger than L2: each consecutive pair is an
    edge of the CSR (or a repeat on an isolated node), and the run is deterministic."""
    rowptr, col = graphs.rmat_csr(20, 16, seed=1, device=cuda)
    n_nodes = rowptr.numel() - 1
    L = 80
    gen = torch.Generator(device=cuda).manual_seed(2)
    start = torch.arange(n_nodes, dtype=torch.int64, device=cuda)
    rand = torch.rand((n_nodes, L), generator=gen, device=cuda)
    out, e = random_walk(rowptr, col, start, rand, L, return_edges=True, check=True)
    assert torch.equal(out[:, 0], start)
    src, dst = out[:, :-1], out[:, 1:]
    moved = e >= 0
    assert torch.equal(col[e[moved]], dst[moved])
    assert bool(((rowptr[src[moved]] <= e[moved]) & (e[moved] < rowptr[src[moved] + 1])).all())
    deg = rowptr.diff()
    assert bool((deg[src[~moved]] == 0).all()) and torch.equal(src[~moved], dst[~moved])
    # the edge index is the reference's formula evaluated in float32
    want = rowptr[src] + (rand * deg[src].to(torch.float32)).to(torch.int64)
    assert torch.equal(e[moved], want[moved])
    out2 = random_walk(rowptr, col, start, rand, L)
    assert torch.equal(out, out2)
    fused_graph = WalkGraph(rowptr, col, fused=True)
    out3, e3 = random_walk(None, None, start, rand, L, graph=fused_graph, return_edges=True, check=True)
    assert torch.equal(out, out3) and torch.equal(e, e3)
    for v in ("direct", "staged16"):
        _lib.set_tuning("uniform_variant", VARIANTS[v])
        assert torch.equal(out, random_walk(rowptr, col, start, rand, L))
        o4, e4 = random_walk(None, None, start, rand, L, graph=fused_graph, return_edges=True, check=True)
        assert torch.equal(out, o4) and torch.equal(e, e4)


def test_draws_generated_in_the_kernel_match_their_host_replay(cuda):
    """rand=None: the kernel draws from its own Philox stream; replaying that stream on the host
    and feeding it to the reference loop must give the same walks, for any sharding of the rows."""
    rng = np.random.default_rng(3)
    for n_nodes, walks, L in [(300, 1000, 37), (50, 33, 3), (2000, 4097, 80), (64, 5, 0)]:
        rowptr, col = random_csr(rng, n_nodes, 5.0, frac_isolated=0.1)
        start = rng.integers(0, n_nodes, walks).astype(np.int64)
        rand = _lib.uniform_draws(77, walks, L)
        assert rand.shape == (walks, L) and (rand >= 0).all() and (rand < 1).all()
        want_n, want_e = oracle.uniform_walk(rowptr, col, start, rand, L, return_edges=True)
        for fused in (False, True):
            g = WalkGraph(torch.from_numpy(rowptr).to(cuda), torch.from_numpy(col).to(cuda), fused=fused)
            for variant in (0, 1):
                _lib.set_tuning("uniform_variant", variant)
                got_n, got_e = random_walk(None, None, torch.from_numpy(start).to(cuda), None, L, graph=g, seed=77,
                                           return_edges=True, check=True)
                np.testing.assert_array_equal(got_n.cpu().numpy(), want_n)
                np.testing.assert_array_equal(got_e.cpu().numpy(), want_e)
            _lib.set_tuning("uniform_variant", 0)
        for world in (2, 3):
            for r in range(world):
                part = random_walk(None, None, torch.from_numpy(start[r::world].copy()).to(cuda), None, L, graph=g,
                                   seed=77, walk_index_base=r, walk_index_stride=world)
                np.testing.assert_array_equal(part.cpu().numpy(), want_n[r::world])
    # the host replay of single draws agrees with the bulk one
    import ctypes as C
    one = C.c_float(0)
    bulk = _lib.uniform_draws(5, 3, 9, walk_index_base=10, walk_index_stride=4)
    for w in range(3):
        for l in range(9):
            _lib.lib().walk_b200_uniform_draw(5, 10 + 4 * w, l, C.byref(one))
            assert one.value == bulk[w, l]
