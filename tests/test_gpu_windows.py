"""Context windows of the walk matrix (the consumer that follows the walks in a node2vec pipeline):
bit-exact against a numpy sliding window, through the C ABI."""
import numpy as np
import pytest
import torch

from mlx_cluster_b200 import _lib, context_windows

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,L,cs", [(1, 0, 1), (1, 5, 6), (7, 5, 1), (33, 20, 10), (1000, 80, 10), (257, 41, 7),
                                    (0, 8, 3), (5000, 9, 2), (3, 2000, 64)])
def test_windows_match_numpy_sliding_window(cuda, n, L, cs):
    rng = np.random.default_rng(n * 1000 + L)
    walks = rng.integers(0, 1 << 40, (n, L + 1)).astype(np.int64)
    want = np.lib.stride_tricks.sliding_window_view(walks, cs, axis=1).reshape(-1, cs) if n else \
        np.zeros((0, cs), dtype=np.int64)
    before = _lib.launch_count()
    got = context_windows(torch.from_numpy(walks).to(cuda), cs)
    assert got.shape == (n * (L + 2 - cs), cs) and got.dtype == torch.int64
    np.testing.assert_array_equal(got.cpu().numpy(), want)
    assert _lib.launch_count() == before + (1 if n else 0)


@pytest.mark.parametrize("n,L,cs", [(33, 20, 10), (257, 41, 7), (64, 9, 2), (5, 12, 13)])
def test_windows_into_a_view_that_starts_at_an_odd_element(cuda, n, L, cs):
    """``out`` may be a view that begins 8 bytes into a larger buffer: the pairs the kernel writes with one
    16-byte store are then the other ones, and nothing else of the buffer is touched."""
    rng = np.random.default_rng(n + L + cs)
    walks = rng.integers(0, 1 << 40, (n, L + 1)).astype(np.int64)
    want = np.lib.stride_tricks.sliding_window_view(walks, cs, axis=1).reshape(-1, cs)
    buf = torch.full((want.size + 2,), -9, dtype=torch.int64, device=cuda)
    assert buf.data_ptr() % 16 == 0
    view = buf[1:-1]
    got = context_windows(torch.from_numpy(walks).to(cuda), cs, out=view)
    np.testing.assert_array_equal(got.cpu().numpy().reshape(-1, cs), want)
    assert int(buf[0]) == -9 and int(buf[-1]) == -9
    # and the walks themselves may be such a view
    wbuf = torch.zeros(walks.size + 1, dtype=torch.int64, device=cuda)
    wbuf[1:] = torch.from_numpy(walks.reshape(-1)).to(cuda)
    got2 = context_windows(wbuf[1:].view(n, L + 1), cs)
    np.testing.assert_array_equal(got2.cpu().numpy(), want)


def test_windows_argument_errors(cuda):
    walks = torch.zeros((4, 6), dtype=torch.int64, device=cuda)
    with pytest.raises(ValueError):
        context_windows(walks, 7)
    with pytest.raises(ValueError):
        context_windows(walks, 0)
    with pytest.raises(TypeError):
        context_windows(walks.int(), 3)
    assert _lib.lib().walk_b200_context_windows(walks.data_ptr(), 4, 5, 9, walks.data_ptr(), None) == _lib.ERR_INVALID_ARG


@pytest.mark.parametrize("n,L,num_nodes", [(1, 1, 7), (33, 5, 1000), (257, 20, 1 << 24), (1000, 0, 5), (64, 7, 1 << 32)])
def test_negative_walks_match_host_replay(cuda, n, L, num_nodes):
    """Column 0 is the start node, the rest the documented Philox draws (replayed on the host through
    walk_b200_negative_draw, itself checked against an independent Philox in the CPU suite)."""
    from mlx_cluster_b200 import _lib, negative_walks
    rng = np.random.default_rng(n + L)
    start = torch.from_numpy(rng.integers(0, min(num_nodes, 2**62), n).astype(np.int64)).cuda()
    seed, base, stride = 0xfeedbeef12345678, 2**33 + 3, 5
    out = negative_walks(start, L, num_nodes, seed=seed, row_index_base=base, row_index_stride=stride).cpu().numpy()
    assert out.shape == (n, L + 1)
    np.testing.assert_array_equal(out[:, 0], start.cpu().numpy())
    rows = sorted(set([0, n - 1, n // 2] + list(rng.integers(0, n, 8))))
    for r in rows:
        want = [_lib.negative_draw(seed, base + int(r) * stride, k, num_nodes) for k in range(L)]
        assert out[r, 1:].tolist() == want
    if L:
        assert out[:, 1:].min() >= 0 and out[:, 1:].max() < num_nodes


def test_negative_walks_shards_and_spread(cuda):
    """Rows dealt cyclically to two 'ranks' reproduce the unsharded matrix, and the draws cover the
    node range evenly (chi-square over 64 bins at p > 1e-6)."""
    from scipy import stats
    from mlx_cluster_b200 import negative_walks
    n, L, num_nodes = 4096, 40, 100000
    start = torch.arange(n, dtype=torch.int64, device="cuda")
    full = negative_walks(start, L, num_nodes, seed=9)
    for r in range(2):
        part = negative_walks(start[r::2].contiguous(), L, num_nodes, seed=9, row_index_base=r, row_index_stride=2)
        assert torch.equal(part, full[r::2])
    draws = full[:, 1:].reshape(-1).cpu().numpy()
    counts = np.bincount(draws * 64 // num_nodes, minlength=64).astype(np.float64)
    expect = np.bincount(np.arange(num_nodes) * 64 // num_nodes, minlength=64) * (draws.size / num_nodes)
    chi2 = float(((counts - expect) ** 2 / expect).sum())
    assert float(stats.chi2.sf(chi2, 63)) > 1e-6


def test_negative_windows_pipeline(cuda):
    """Negative rows go through the same window kernel as walks."""
    from mlx_cluster_b200 import negative_walks
    start = torch.arange(100, dtype=torch.int64, device="cuda")
    neg = negative_walks(start, 12, 5000, seed=1)
    win = context_windows(neg, 5)
    want = neg.unfold(1, 5, 1).reshape(-1, 5)
    assert torch.equal(win, want)
