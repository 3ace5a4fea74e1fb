"""Second-order transition statistics for comparing two sets of walks."""
from collections import defaultdict

import numpy as np
from scipy import stats


def triple_counts(walks: np.ndarray, num_nodes: int):
    """Counts of (t, v, x) = (walk[l-1], walk[l], walk[l+1]) over all walks and l >= 1,
    as a dict keyed by t * N + v holding {x: count}."""
    t = walks[:, :-2].reshape(-1)
    v = walks[:, 1:-1].reshape(-1)
    x = walks[:, 2:].reshape(-1)
    key = (t * num_nodes + v) * num_nodes + x
    uniq, cnt = np.unique(key, return_counts=True)
    cells = defaultdict(dict)
    for k, c in zip(uniq.tolist(), cnt.tolist()):
        cells[k // num_nodes][k % num_nodes] = c
    return cells


def two_sample_chi2(cells_a, cells_b, min_expected: float = 5.0):
    """Pooled two-sample chi-square over all (t, v) cells present in both samples.
    Categories with a pooled expectation below ``min_expected`` in either sample are
    lumped into one 'other' category per cell. Returns (statistic, dof, p_value, n_cells)."""
    stat, dof, used = 0.0, 0, 0
    for cell, ca in cells_a.items():
        cb = cells_b.get(cell)
        if not cb:
            continue
        na, nb = sum(ca.values()), sum(cb.values())
        xs = sorted(set(ca) | set(cb))
        a = np.array([ca.get(x, 0) for x in xs], dtype=np.float64)
        b = np.array([cb.get(x, 0) for x in xs], dtype=np.float64)
        pooled = (a + b) / (na + nb)
        ok = (pooled * na >= min_expected) & (pooled * nb >= min_expected)
        if ok.sum() < 1:
            continue
        a2 = np.append(a[ok], a[~ok].sum())
        b2 = np.append(b[ok], b[~ok].sum())
        keep = (a2 + b2) > 0
        a2, b2 = a2[keep], b2[keep]
        if len(a2) < 2:
            continue
        ka, kb = np.sqrt(nb / na), np.sqrt(na / nb)
        stat += float((((ka * a2 - kb * b2) ** 2) / (a2 + b2)).sum())
        dof += len(a2) - 1
        used += 1
    p = float(stats.chi2.sf(stat, dof)) if dof > 0 else 1.0
    return stat, dof, p, used
