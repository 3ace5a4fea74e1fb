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


def test_windows_argument_errors(cuda):
    walks = torch.zeros((4, 6), dtype=torch.int64, device=cuda)
    with pytest.raises(ValueError):
        context_windows(walks, 7)
    with pytest.raises(ValueError):
        context_windows(walks, 0)
    with pytest.raises(TypeError):
        context_windows(walks.int(), 3)
    assert _lib.lib().walk_b200_context_windows(walks.data_ptr(), 4, 5, 9, walks.data_ptr(), None) == _lib.ERR_INVALID_ARG
