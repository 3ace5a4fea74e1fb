"""Command-line front end of the random-gather probe (``walk_b200_gather_probe_ex``).

    python -m mlx_cluster_b200.probe [--mib 2048] [--iters 32] [--chains 1] [--bytes 8]
                                     [--fetch 64] [--threads-per-sm 0] [--sweep]

Prints one JSON line per measurement: dependent random gathers per second out of an array
far larger than L2. ``--sweep`` runs the grid that tells a limit of the memory system from
a limit of the probe itself: 1/2/4 chains per thread, 8/16/32-byte gathers, 64- and
128-byte DRAM fetches, and 256..2048 resident threads per SM. Needs a CUDA device.
"""
from __future__ import annotations

import argparse
import json

from . import _lib


def measure(mib, iters, chains, gather_bytes, fetch, tpsm):
    rate = _lib.gather_probe(mib << 20, iters, chains=chains, gather_bytes=gather_bytes, fetch_bytes=fetch,
                             threads_per_sm=tpsm)
    return {"array_mib": mib, "iters": iters, "chains": chains, "gather_bytes": gather_bytes, "fetch_bytes": fetch,
            "threads_per_sm": tpsm or "2^22 threads in waves", "gathers_per_s": rate,
            "useful_gbs": rate * gather_bytes / 1e9, "fetched_gbs": rate * fetch / 1e9}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mib", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=32)
    ap.add_argument("--chains", type=int, default=1, choices=[1, 2, 4])
    ap.add_argument("--bytes", type=int, default=8, choices=[8, 16, 32])
    ap.add_argument("--fetch", type=int, default=64, choices=[64, 128])
    ap.add_argument("--threads-per-sm", type=int, default=0)
    ap.add_argument("--sweep", action="store_true")
    a = ap.parse_args()
    if not a.sweep:
        print(json.dumps(measure(a.mib, a.iters, a.chains, a.bytes, a.fetch, a.threads_per_sm)), flush=True)
        return 0
    for fetch in (64, 128):
        for gb in (8, 16, 32):
            for chains in (1, 2, 4):
                print(json.dumps(measure(a.mib, a.iters, chains, gb, fetch, 0)), flush=True)
    for tpsm in (256, 512, 1024, 2048):
        for chains in (1, 2, 4):
            print(json.dumps(measure(a.mib, a.iters * 4, chains, 8, 64, tpsm)), flush=True)
    for mib in (512, 8192, 32768):
        print(json.dumps(measure(mib, a.iters, 1, 8, 64, 0)), flush=True)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
