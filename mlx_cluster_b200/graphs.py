"""Seeded synthetic graphs and the edge-list -> CSR step that precedes the walk path.

The reference's demo scripts build their CSR on the host with ``numpy.unique`` and a
cumulative sum (``tests/test_random_walk.py:22-28``), which silently drops nodes that
have no out-edge. ``edges_to_csr`` here counts rows over all ``num_nodes`` and runs on
whatever device the edge tensors are on (the large graphs are built on the GPU).

Generators (all return int64 ``rowptr [N+1]``, ``col [nnz]``; rows sorted ascending,
symmetric, no self-loops, no duplicate edges):

* ``chung_lu_csr``  -- power-law expected-degree graph with an exact undirected edge
  count and minimum degree 1 (the small parity/statistics workloads);
* ``rmat_csr``      -- R-MAT (recursive matrix) graph of 2**scale nodes (the
  throughput workloads);
* ``isolate_nodes`` -- removes every edge of a random share of nodes, to exercise the
  stay-in-place rule for nodes without out-edges.
"""
from __future__ import annotations

import numpy as np
import torch


def edges_to_csr(src: torch.Tensor, dst: torch.Tensor, num_nodes: int, *, symmetrize: bool = True):
    """(src, dst) int64 edge list -> CSR sorted by (row, col), duplicates and self-loops
    removed, isolated nodes kept as empty rows."""
    if symmetrize:
        src, dst = torch.cat([src, dst]), torch.cat([dst, src])
    keep = src != dst
    key = src[keep] * num_nodes + dst[keep]
    del src, dst, keep
    key = torch.unique(key, sorted=True)
    row = torch.div(key, num_nodes, rounding_mode="floor")
    col = key - row * num_nodes
    del key
    counts = torch.bincount(row, minlength=num_nodes)
    rowptr = torch.zeros(num_nodes + 1, dtype=torch.int64, device=col.device)
    torch.cumsum(counts, 0, out=rowptr[1:])
    return rowptr, col.contiguous()


def chung_lu_csr(num_nodes: int = 2708, num_undirected_edges: int = 5278, exponent: float = 2.5,
                 seed: int = 0):
    """Chung-Lu style graph: node i has weight (i+1)^(-1/(exponent-1)); edges are drawn with
    probability proportional to the product of the end weights until exactly
    ``num_undirected_edges`` distinct non-loop edges exist. Every node first gets one edge
    to a weight-sampled partner so that the minimum degree is 1. numpy, deterministic."""
    rng = np.random.default_rng(seed)
    w = (np.arange(num_nodes) + 1.0) ** (-1.0 / (exponent - 1.0))
    pw = w / w.sum()
    edges = set()
    for u in rng.permutation(num_nodes):
        if len(edges) >= num_undirected_edges:
            break
        while True:
            v = int(rng.choice(num_nodes, p=pw))
            if v != u:
                break
        edges.add((min(int(u), v), max(int(u), v)))
    deg = np.zeros(num_nodes, dtype=np.int64)
    for a, b in edges:
        deg[a] += 1
        deg[b] += 1
    assert (deg > 0).all() or len(edges) >= num_undirected_edges
    while len(edges) < num_undirected_edges:
        m = num_undirected_edges - len(edges)
        us = rng.choice(num_nodes, size=2 * m, p=pw)
        vs = rng.choice(num_nodes, size=2 * m, p=pw)
        for u, v in zip(us.tolist(), vs.tolist()):
            if u != v:
                edges.add((min(u, v), max(u, v)))
                if len(edges) >= num_undirected_edges:
                    break
    e = np.array(sorted(edges), dtype=np.int64)
    rowptr, col = edges_to_csr(torch.from_numpy(e[:, 0].copy()), torch.from_numpy(e[:, 1].copy()), num_nodes)
    return rowptr, col


def isolate_nodes(rowptr: torch.Tensor, col: torch.Tensor, fraction: float = 0.005, seed: int = 0):
    """Remove all edges (both directions) of ``round(fraction * N)`` randomly chosen nodes.
    Returns ``rowptr, col, isolated_ids``."""
    n = rowptr.numel() - 1
    k = max(1, int(round(fraction * n)))
    g = torch.Generator().manual_seed(seed)
    iso = torch.randperm(n, generator=g)[:k].sort().values
    row = torch.repeat_interleave(torch.arange(n, dtype=torch.int64), rowptr.cpu().diff())
    c = col.cpu()
    dead = torch.zeros(n, dtype=torch.bool)
    dead[iso] = True
    keep = ~(dead[row] | dead[c])
    rp, cl = edges_to_csr(row[keep], c[keep], n, symmetrize=False)
    return rp.to(rowptr.device), cl.to(col.device), iso


def rmat_edges(scale: int, edge_factor: int = 16, a: float = 0.57, b: float = 0.19, c: float = 0.19,
               d: float = 0.05, seed: int = 1, device="cpu", chunk: int = 1 << 26):
    """Raw R-MAT edge list: 2**scale nodes, edge_factor * 2**scale directed edges. Each of the
    ``scale`` bit levels picks a quadrant with probabilities (a, b, c, d)."""
    assert abs(a + b + c + d - 1.0) < 1e-9
    n_edges = edge_factor << scale
    dev = torch.device(device)
    g = torch.Generator(device=dev).manual_seed(seed)
    src = torch.empty(n_edges, dtype=torch.int64, device=dev)
    dst = torch.empty(n_edges, dtype=torch.int64, device=dev)
    for c0 in range(0, n_edges, chunk):
        m = min(chunk, n_edges - c0)
        s = torch.zeros(m, dtype=torch.int64, device=dev)
        t = torch.zeros(m, dtype=torch.int64, device=dev)
        for _ in range(scale):
            r = torch.rand(m, generator=g, device=dev)
            s_bit = r >= (a + b)
            t_bit = ((r >= a) & (r < a + b)) | (r >= a + b + c)
            s = (s << 1) | s_bit.to(torch.int64)
            t = (t << 1) | t_bit.to(torch.int64)
        src[c0:c0 + m] = s
        dst[c0:c0 + m] = t
    return src, dst


def rmat_csr(scale: int, edge_factor: int = 16, a: float = 0.57, b: float = 0.19, c: float = 0.19,
             d: float = 0.05, seed: int = 1, device="cpu"):
    """Symmetrised, deduplicated, loop-free R-MAT graph as int64 CSR on ``device``."""
    src, dst = rmat_edges(scale, edge_factor, a, b, c, d, seed, device)
    return edges_to_csr(src, dst, 1 << scale)


def csr_is_symmetric(rowptr: torch.Tensor, col: torch.Tensor) -> bool:
    n = rowptr.numel() - 1
    row = torch.repeat_interleave(torch.arange(n, dtype=torch.int64, device=col.device), rowptr.diff())
    fwd = torch.sort(row * n + col).values
    bwd = torch.sort(col * n + row).values
    return bool(torch.equal(fwd, bwd))
