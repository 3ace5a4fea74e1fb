"""Generates ``walk_golden.npz``: inputs of the two small workloads and the outputs of the
reference's own ``eval_cpu`` loops on them.

Needs the compiled reference (``oracle/_ref``), i.e. a machine that has the reference
checkout; the fixture is what lets machines without it still check against reference
output. The biased walk is run after ``srand(k)``: its fixtures pin the reference's
control flow on this C library's ``rand()`` sequence. Node ids are stored as int16/int32
to keep the file small. Run: ``python tests/golden/make_golden.py``.
"""
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import oracle  # noqa: E402
from mlx_cluster_b200 import graphs  # noqa: E402

HERE = Path(__file__).resolve().parent
PQ = [(1.0, 1.0), (0.5, 2.0), (4.0, 0.25), (0.25, 4.0), (1.0, 3.0)]
SRAND = [1, 2]
BIASED_ROWS = 1024


def small_workloads():
    """Inputs of the two small workloads (shared with the tests through this module)."""
    rowptr, col = graphs.chung_lu_csr(2708, 5278, 2.5, seed=0)
    rng = np.random.default_rng(0)
    start1 = rng.choice(2708, size=2000, replace=False).astype(np.int64)
    rand1 = rng.random((2000, 5), dtype=np.float32)
    rowptr2, col2, iso = graphs.isolate_nodes(rowptr, col, 0.005, seed=0)
    return dict(rowptr1=rowptr.numpy(), col1=col.numpy(), start1=start1, rand1=rand1,
                rowptr2=rowptr2.numpy(), col2=col2.numpy(), iso2=iso.numpy(),
                start2=np.arange(2708, dtype=np.int64))


def main():
    assert oracle.have_ref(), "compiled reference missing: run python oracle/build.py where the reference checkout is"
    w = small_workloads()
    assert w["col1"].size == 10556 and w["rowptr1"].size == 2709
    out = {
        "rowptr1": w["rowptr1"].astype(np.int32), "col1": w["col1"].astype(np.int16),
        "start1": w["start1"].astype(np.int16), "rand1": w["rand1"],
        "rowptr2": w["rowptr2"].astype(np.int32), "col2": w["col2"].astype(np.int16),
        "iso2": w["iso2"].astype(np.int16),
    }
    n1, e1 = oracle.ref_random_walk(w["rowptr1"], w["col1"], w["start1"], w["rand1"], 5, return_edges=True)
    out["uniform1_n"] = n1.astype(np.int16)
    out["uniform1_e"] = e1.astype(np.int16)
    # edge case: the isolated-node graph under the uniform walk (stay in place, rand unread)
    rng = np.random.default_rng(7)
    rand2 = rng.random((2708, 20), dtype=np.float32)
    n2, e2 = oracle.ref_random_walk(w["rowptr2"], w["col2"], w["start2"], rand2, 20, return_edges=True)
    out["rand2"] = rand2
    out["uniform2_n"] = n2.astype(np.int16)
    out["uniform2_e"] = e2.astype(np.int16)
    # biased walk: the first BIASED_ROWS start nodes keep the fixture small; the full start set
    # is compared live wherever the compiled reference is present
    for i, (p, q) in enumerate(PQ):
        for s in SRAND:
            n, e = oracle.ref_rejection_sampling(w["rowptr2"], w["col2"], w["start2"][:BIASED_ROWS], 20, p, q,
                                                 srand_seed=s, return_edges=True)
            out[f"biased2_pq{i}_srand{s}_n"] = n.astype(np.int16)
            if s == SRAND[0]:
                out[f"biased2_pq{i}_srand{s}_e"] = e.astype(np.int16)
    out["pq"] = np.array(PQ)
    out["srand"] = np.array(SRAND)
    np.savez_compressed(HERE / "walk_golden.npz", **out)
    print("wrote", HERE / "walk_golden.npz", (HERE / "walk_golden.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    main()
