"""B200-native CSR walk generators: ``random_walk`` (uniform) and ``rejection_sampling``
(node2vec), the two operators of the reference package (``mlx_cluster/__init__.py:3-4``),
computed by hand-written sm_100a CUDA kernels behind a C ABI (``include/walk_b200.h``).
"""
from .ops import (HostGraph, WalkGraph, clear_caches, context_windows, csr_from_edges, negative_walks, prepare_graph, random_walk,
                  read_status, rejection_sampling)
from .sharding import shard_range, shard_rows, sharded_walk

__all__ = ["random_walk", "rejection_sampling", "context_windows", "csr_from_edges", "negative_walks", "prepare_graph", "WalkGraph", "HostGraph",
           "read_status", "clear_caches", "shard_range", "shard_rows", "sharded_walk"]
__version__ = "0.1.0"
