#!/usr/bin/env python
"""Throughput bench of the walk path: walk steps per second on seeded synthetic graphs.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

A "step" is one pass of the walk generator over one batch of start nodes. The default
workload is the node2vec one the headline metric is quoted on (R-MAT scale 24, edge
factor 16, every node a start, walk_length 80, p=0.25, q=4, Philox draws); start rows
are sharded over the ranks, the CSR is replicated per GPU. One JSON line is printed by
rank 0. With ``--impl reference`` the reference's own CPU loops are timed instead, on
the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: kind, scale, edge_factor, graph seed, walk_length, p, q
    "node2vec_rmat24": dict(kind="node2vec", scale=24, edge_factor=16, seed=2, L=80, p=0.25, q=4.0),
    "uniform_rmat22": dict(kind="uniform", scale=22, edge_factor=16, seed=1, L=80),
    "node2vec_rmat20": dict(kind="node2vec", scale=20, edge_factor=16, seed=2, L=80, p=0.25, q=4.0),
    "uniform_rmat20": dict(kind="uniform", scale=20, edge_factor=16, seed=1, L=80),
    "node2vec_rmat22_p1q2": dict(kind="node2vec", scale=22, edge_factor=16, seed=3, L=40, p=1.0, q=2.0),
    # the largest configuration: 2^26 nodes, ~2e9 directed edges, 10 walks per node, for 8 GPUs
    # (or one rank's share of it on one GPU with --shard-of 8)
    "uniform_rmat26": dict(kind="uniform", scale=26, edge_factor=16, seed=3, L=40, walks_per_node=10),
    "node2vec_rmat26_p1q2": dict(kind="node2vec", scale=26, edge_factor=16, seed=3, L=40, p=1.0, q=2.0,
                                 walks_per_node=10),
}
RMAT = dict(a=0.57, b=0.19, c=0.19, d=0.05)
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one launch of the dominant kernel on the small
# (scale-20) case of each kind of walk, from the ncu captures summarised under profiles/, and the random
# accesses that same launch issued. A run's `roofline.traffic` is that ratio (DRAM bytes per random access,
# which does not depend on the graph's size: every access misses to DRAM in both cases) times the random
# accesses one launch of this run issues, counted in this run.
NCU_SMALL_CASE = {
    "node2vec_tri": dict(workload="node2vec_rmat20", dram_bytes=11.11e9, accesses=208205614,
                         source="profiles/node2vec_pool_tri_kernel__node2vec_rmat20.md"),
    "node2vec": dict(workload="node2vec_rmat20", dram_bytes=19.60e9, accesses=346134263,
                     source="profiles/node2vec_pool_kernel__node2vec_rmat20.md"),
    "uniform": dict(workload="uniform_rmat20", dram_bytes=4.70e9, accesses=53816512,
                    source="profiles/uniform_walk_staged_kernel__uniform_rmat20.md"),
}
PHILOX_SEED = 20240607


def env_rank():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


def measured_peak_gbs():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock, power and throttle reasons of one GPU with nvidia-smi while the
    timed region runs (reading only; no setting is touched)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.rows, self.proc, self.t0, self.t1 = [], None, None, None
        try:
            uuid = str(torch.cuda.get_device_properties(device).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", uuid, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.06)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        inside = [r for t, r in self.rows if self.t0 is not None and self.t0 <= t <= (self.t1 or t) + 0.05]
        use = inside or [r for _, r in self.rows]
        sm, mx, pw, reasons = [], [], [], set()
        for r in use:
            p = [x.strip() for x in r.split(",")]
            if len(p) < 7:
                continue
            try:
                sm.append(float(p[0])); mx.append(float(p[1])); pw.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(pw) if pw else None, "reasons": sorted(reasons),
                "samples": len(use), "samples_in_timed_region": len(inside)}


# ------------------------------------------------------------------------------ graph
def build_graph(wl, device, world, rank):
    """Rank 0 draws the seeded R-MAT edge list on its GPU and builds the CSR with the library's
    device builder (symmetrised, loop-free, duplicate-free); other ranks receive a replica."""
    from mlx_cluster_b200 import csr_from_edges, graphs
    import torch.distributed as dist
    t0 = time.time()
    if rank == 0:
        src, dst = graphs.rmat_edges(wl["scale"], wl["edge_factor"], seed=wl["seed"], device=device, **RMAT)
        rowptr, col = csr_from_edges(src, dst, 1 << wl["scale"])
        col = col.clone()  # drop the builder's spare capacity
        del src, dst
        torch.cuda.synchronize(device)
    if world > 1:
        meta = torch.tensor([rowptr.numel(), col.numel()] if rank == 0 else [0, 0], dtype=torch.int64, device=device)
        dist.broadcast(meta, 0)
        if rank != 0:
            rowptr = torch.empty(int(meta[0]), dtype=torch.int64, device=device)
            col = torch.empty(int(meta[1]), dtype=torch.int64, device=device)
        dist.broadcast(rowptr, 0)
        dist.broadcast(col, 0)
        torch.cuda.synchronize(device)
    torch.cuda.empty_cache()
    return rowptr, col, time.time() - t0


# ------------------------------------------------------------------------------ CPU reference legs
_CPU_CTX = {}  # arrays the forked CPU workers read (inherited by fork, never pickled)


def _cpu_worker(job):
    import oracle
    kind_impl, b, e, seed = job
    c = _CPU_CTX
    start = c["start"][b:e]
    rand = None if c["rand"] is None else c["rand"][b:e]
    t = time.perf_counter()
    if kind_impl == "reference":
        if c["kind"] == "uniform":
            oracle.ref_random_walk(c["rowptr"], c["col"], start, rand, c["L"])
        else:
            oracle.ref_rejection_sampling(c["rowptr"], c["col"], start, c["L"], c["p"], c["q"], srand_seed=seed)
    else:
        if c["kind"] == "uniform":
            oracle.uniform_walk(c["rowptr"], c["col"], start, rand, c["L"])
        else:
            oracle.node2vec_walk(c["rowptr"], c["col"], start, c["L"], c["p"], c["q"], seed=seed)
    return time.perf_counter() - t


def cpu_walk_seconds(wl, rowptr, col, start, rand, procs):
    """Wall seconds for the reference CPU loop over `start`, split over `procs` processes
    (the reference loop is serial and draws from the global rand(), so processes, not threads)."""
    import oracle
    kind_impl = "reference" if oracle.have_ref() else "port"
    _CPU_CTX.update(rowptr=rowptr, col=col, start=start, rand=rand, kind=wl["kind"], L=wl["L"],
                    p=wl.get("p", 1.0), q=wl.get("q", 1.0))
    n = start.shape[0]
    per = -(-n // procs)
    jobs = [(kind_impl, i * per, min(n, (i + 1) * per), 1 + i) for i in range(procs) if i * per < n]
    t = time.perf_counter()
    if len(jobs) == 1:
        _cpu_worker(jobs[0])
    else:
        import multiprocessing as mp
        with mp.get_context("fork").Pool(len(jobs)) as pool:
            pool.map(_cpu_worker, jobs, chunksize=1)
    return time.perf_counter() - t, kind_impl, len(jobs)


def start_order(n_nodes, walks_per_node=1, device=None):
    """The workload's start list: every node `walks_per_node` times, in a seeded random order (a
    tensor on `device`). Lists of up to 2^26 rows are drawn with the CPU generator, larger ones on
    the device (same result on every rank of one machine type)."""
    total = n_nodes * walks_per_node
    if total <= (1 << 26) or device is None or torch.device(device).type != "cuda":
        order = torch.randperm(total, generator=torch.Generator().manual_seed(PHILOX_SEED))
        if device is not None:
            order = order.to(device)
    else:
        order = torch.randperm(total, generator=torch.Generator(device=device).manual_seed(PHILOX_SEED), device=device)
    return order % n_nodes if walks_per_node > 1 else order


def size_cpu_sample(wl, rowptr, col, n_total, target_s, procs, rng):
    """Pick how many of the workload's first start rows give about target_s of CPU work."""
    pilot = min(n_total, 2048 * procs)
    start = start_order(n_total, wl.get("walks_per_node", 1))[:pilot].numpy()
    rand = rng.random((pilot, wl["L"]), dtype=np.float32) if wl["kind"] == "uniform" else None
    secs, _, _ = cpu_walk_seconds(wl, rowptr, col, start, rand, procs)
    rows = int(min(n_total, max(pilot, pilot * target_s / max(secs, 1e-6))))
    return rows


def run_reference_arm(args, wl):
    rank, local_rank, world = env_rank()
    if rank != 0:
        return 0
    from mlx_cluster_b200 import graphs
    dev = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    rowptr, col = graphs.rmat_csr(wl["scale"], wl["edge_factor"], seed=wl["seed"], device=dev, **RMAT)
    rowptr, col = rowptr.cpu().numpy(), col.cpu().numpy()
    n_total, L = rowptr.size - 1, wl["L"]
    procs = len(os.sched_getaffinity(0))
    rng = np.random.default_rng(0)
    budget_s = 150.0
    per_step = budget_s / max(1, args.steps + args.warmup)
    rows = size_cpu_sample(wl, rowptr, col, n_total, per_step, procs, rng)
    start = start_order(n_total, wl.get("walks_per_node", 1))[:rows].numpy()
    rand = rng.random((rows, L), dtype=np.float32) if wl["kind"] == "uniform" else None
    kind, used = "port", procs
    for _ in range(args.warmup):
        cpu_walk_seconds(wl, rowptr, col, start, rand, procs)
    t = time.perf_counter()
    for _ in range(args.steps):
        _, kind, used = cpu_walk_seconds(wl, rowptr, col, start, rand, procs)
    total = time.perf_counter() - t
    value = rows * L * args.steps / total
    sample = f"first {rows} of {n_total} start rows per step, {used} processes, process start-up included"
    line = {
        "impl": "reference", "metric": "walk_steps_per_sec", "value": value, "unit": "steps/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
        "config": workload_config(wl, args.workload, n_total, int(col.size), args.gpus, "hash"),
        "cpu_baseline": {"value": value, "unit": "steps/s", "cores": used, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def workload_config(wl, name, n_nodes, n_edges, gpus, membership=None, edge_records=None, rand_source=None):
    c = {"workload": name, "graph": f"R-MAT scale {wl['scale']} edge factor {wl['edge_factor']} "
         f"(a,b,c,d)=(0.57,0.19,0.19,0.05) seed {wl['seed']}, symmetrised, deduplicated, no self-loops, int64 CSR",
         "num_nodes": n_nodes, "num_directed_edges": n_edges, "starts": f"every node {wl.get('walks_per_node', 1)}x, in a seeded random order", "walk_length": wl["L"],
         "sharding": f"start rows (a seeded random order) cut into {gpus} contiguous block(s), one per GPU; CSR replicated",
         "l2": "no flush between steps: col (8 B x edges) is far larger than the 126 MB L2"}
    if wl["kind"] == "node2vec":
        c.update(p=wl["p"], q=wl["q"], draws="Philox4x32-10, key=seed, counter=(walk,step,attempt)",
                 membership=membership)
    else:
        c.update(rand=rand_source or "float32 uniform [0,1) [n, walk_length], caller-supplied", edge_records=edge_records)
    return c


# ------------------------------------------------------------------------------ GPU arm
def time_launches(fn, steps, warmup, stream, sampler=None, barrier=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    if sampler:
        sampler.mark_start()
    from mlx_cluster_b200 import _lib
    launches = _lib.launch_count()
    evs[0].record(stream)
    for i in range(steps):
        fn()
        evs[i + 1].record(stream)
    torch.cuda.synchronize()
    launches = _lib.launch_count() - launches
    if sampler:
        sampler.mark_end()
    if barrier:
        barrier()
    per = [evs[i].elapsed_time(evs[i + 1]) for i in range(steps)]
    return evs[0].elapsed_time(evs[steps]), per, launches


def parity_rows(wl, rowptr_h, col_h, start_rows, rand_rows, got_rows, base, stride):
    """Untimed check of the first rows of a timed walk matrix against the CPU restatement of the reference
    loop, fed with the same draws and the same global walk indices. Returns the number of rows compared."""
    import oracle
    L = wl["L"]
    if wl["kind"] == "node2vec":
        want = oracle.node2vec_walk(rowptr_h, col_h, start_rows, L, wl["p"], wl["q"], seed=PHILOX_SEED,
                                    walk_index_base=base, walk_index_stride=stride)
    else:
        want = oracle.uniform_walk(rowptr_h, col_h, start_rows, rand_rows, L)
    if not np.array_equal(want, got_rows):
        bad = int(np.argmax((want != got_rows).any(axis=1)))
        raise SystemExit(f"bench: the timed walk matrix differs from the CPU restatement at row {bad}")
    return int(want.shape[0])


def host_ceiling(dev, world, barrier, narrow):
    """What the host side of the end-to-end leg can deliver on this box: pinned device-to-host copy rate of
    this rank alone and with every rank copying at once, and the rate at which the library's host threads widen
    int32 staging into an int64 buffer (output bytes per second)."""
    from mlx_cluster_b200 import _lib
    nbytes = 1 << 30
    d = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    h = torch.empty(nbytes, dtype=torch.uint8, pin_memory=True)
    s = torch.cuda.current_stream(dev)

    def d2h(reps=3):
        h.copy_(d, non_blocking=True)
        s.synchronize()
        t = time.perf_counter()
        for _ in range(reps):
            h.copy_(d, non_blocking=True)
        s.synchronize()
        return reps * nbytes / (time.perf_counter() - t) / 1e9

    rank = env_rank()[0]
    alone = None
    if world == 1:
        alone = together = d2h()
    else:
        import torch.distributed as dist
        for r in range(min(world, 2)):  # rank 0, then rank 1, each alone (the others wait)
            barrier()
            if rank == r:
                alone = d2h()
        barrier()
        together = d2h()
        t = torch.tensor([together, alone if alone is not None else 0.0], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        together_sum = float(t[0])
        alone = float(t[1]) / min(world, 2)
    del d, h
    out = {"d2h_pinned_gbs_one_rank_alone": alone,
           "d2h_pinned_gbs_all_ranks_at_once_sum": together if world == 1 else together_sum}
    if barrier:
        barrier()
    # every rank widens at once, as in a step: what one rank's threads deliver while the others do the same
    out["widen_int64_out_gbs_per_rank"] = _lib.host_widen_probe(256 << 20)
    out["transport_in_use"] = "int32 + widening" if narrow else "int64"
    return out


def run_workload(args, name, wl, dev, world, rank, barrier, allmax, allsum, light=False):
    """Times one workload on this process group; rank 0 gets the result line (a dict), the others None.
    `light`: the compact pass that rides along with the default run (fewer steps, no CPU baseline)."""
    import torch.distributed as dist
    from mlx_cluster_b200 import _lib, random_walk, rejection_sampling
    from mlx_cluster_b200.ops import WalkGraph, HostGraph
    from mlx_cluster_b200.sharding import gather_rows, shard_rows

    steps = min(args.steps, 10) if light else args.steps
    rowptr, col, build_s = build_graph(wl, dev, world, rank)
    n_nodes, n_edges, L = rowptr.numel() - 1, col.numel(), wl["L"]
    # Every node starts `walks_per_node` walks; the start list is a seeded random order of them and each rank
    # walks one contiguous block of it (rank r of G: rows shard_range(n, G, r)). On R-MAT every bit of a node id
    # is correlated with its degree, so shards cut by id differ by up to 3x in work; in a random order any split
    # is even, and contiguous blocks are what a gather receives in place. Draws are indexed by the global row,
    # so the walks do not depend on the GPU count.
    wpn = wl.get("walks_per_node", 1)
    n_walks = n_nodes * wpn
    shard_world, shard_rank = (args.shard_of, 0) if (world == 1 and args.shard_of > 1) else (world, rank)
    row_slice, (b, stride) = shard_rows(n_walks, shard_world, shard_rank, "block")
    order = start_order(n_nodes, wpn, dev)
    start = order[row_slice].contiguous().to(dev)
    del order
    torch.cuda.empty_cache()
    rows = start.numel()
    walks_timed = n_walks if shard_world == world else rows  # a lone rank's share counts only its own rows
    t_prep = time.perf_counter()
    graph = WalkGraph(rowptr, col, symmetric=True, edgeset=(wl["kind"] == "node2vec" and args.membership == "hash"),
                      fused=(wl["kind"] == "uniform" and not args.no_fused),
                      edgeset_slots_per_edge=args.edgeset_slots_per_edge,
                      trifilter=(wl["kind"] == "node2vec" and args.membership == "hash" and not args.no_trifilter),
                      trifilter_max_row=args.trifilter_max_row)
    torch.cuda.synchronize(dev)
    prep_s = time.perf_counter() - t_prep

    # ---- the gather leg's destination (N > 1): rank 0 holds the gathered matrix, or a window of it when the
    # whole matrix does not fit beside the graph, and its own kernel writes its block straight into it
    row_bytes = (L + 1) * 8
    gather_plan = None
    full = None
    if world > 1 and not args.no_gather:
        free_b = torch.cuda.mem_get_info(dev)[0]
        need_rest = rows * row_bytes * 2  # every rank's own block, plus slack
        budget = int(min(max(free_b - need_rest, 0) * 0.8, args.gather_window_gb * 1e9))
        # the window is rank 0's to hold, and every rank must cut the same windows: rank 0's figure goes to all
        agreed = torch.tensor([int(min(n_walks, budget // row_bytes))], dtype=torch.int64, device=dev)
        dist.broadcast(agreed, 0)
        window_rows = int(agreed.item())
        if window_rows >= min(n_walks, 1 << 16):
            whole = window_rows >= n_walks
            gather_plan = {"window_rows": window_rows, "whole": whole}
            if rank == 0:
                full = torch.empty((window_rows, L + 1), dtype=torch.int64, device=dev)
    if full is not None and gather_plan["whole"]:
        out = full[b:b + rows]
    else:
        out = torch.empty((rows, L + 1), dtype=torch.int64, device=dev)
    stream = torch.cuda.current_stream(dev)

    if wl["kind"] == "node2vec":
        # untimed instrumented pass: counts the 8-byte gathers this batch needs
        _, cnt = rejection_sampling(None, None, start, L, wl["p"], wl["q"], graph=graph, seed=PHILOX_SEED,
                                    walk_index_base=b, walk_index_stride=stride, out=out, return_counters=True,
                                    check=True)
        # algorithmic bytes of the reference's algorithm with a log-time membership test: per walk
        # 16; first step 32 (24 if isolated); stay-in-place step 24; degree-1 step 32; sampled step
        # 16 + 8 plus 8 per attempt plus, per membership test that can change the outcome,
        # 16 + 8 * ceil(log2(deg(candidate) + 1))
        alg_bytes = (16 * rows + 32 * cnt["steps_first"] + 24 * cnt["steps_deg0"] + 32 * cnt["steps_deg1"]
                     + 24 * cnt["steps_sampled"] + 8 * cnt["attempts"] + 16 * cnt["membership"]
                     + 8 * cnt["formula_probes"])
        # what this implementation actually gathers and writes (8 B per gather issued)
        gathered_bytes = 8 * cnt["loads"] + 8 * rows * (L + 1) + 8 * rows
        sampled_steps = cnt["steps_sampled"] + cnt["steps_deg1"] + cnt["steps_first"]
        rand = None
        cnt_kernel = None
        if graph.colrev16 is not None:
            # the triangle-filter kernel reads less than the algorithm's counts say: count what it reads itself
            _lib.set_tuning("n2v_count_kernel", 1)
            _, cnt_kernel = rejection_sampling(None, None, start, L, wl["p"], wl["q"], graph=graph, seed=PHILOX_SEED,
                                               walk_index_base=b, walk_index_stride=stride, out=out,
                                               return_counters=True, check=True)
            _lib.set_tuning("n2v_count_kernel", 0)
            if _lib.last_kernel() != "node2vec_pool_tri_kernel":
                cnt_kernel = None
            else:
                gathered_bytes = 8 * cnt_kernel["loads"] + 8 * rows * (L + 1)

        def step():
            rejection_sampling(None, None, start, L, wl["p"], wl["q"], graph=graph, seed=PHILOX_SEED,
                               walk_index_base=b, walk_index_stride=stride, out=out)
    else:
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        rand = torch.rand((rows, L), generator=gen, device=dev)
        deg = rowptr.diff()
        cnt = {}
        cnt_kernel = None
        random_walk(None, None, start, rand, L, graph=graph, out=out, check=True)
        moved = 0
        for c0 in range(0, rows, 1 << 22):  # in slices: the index tensor of the whole matrix would not fit beside it
            moved += int((deg[out[c0:c0 + (1 << 22), :-1].reshape(-1)] > 0).sum().item())
        stay = rows * L - moved
        sampled_steps = moved
        # per step: row bounds 16 (8 via the packed descriptor, counted as the CSR's 16) + rand 4 + col 8 + out 8
        alg_bytes = rows * 16 + moved * 36 + stay * 24
        # 8-byte descriptor instead of the 16-byte row pair; fused records: one 16-byte gather per moving step
        gathered_bytes = rows * 24 + moved * 28 if not args.no_fused else rows * 16 + moved * 28 + stay * 12
        rand_timed = rand
        if args.device_rand:
            # draws generated in the kernel (same walks as feeding the replayed stream; tests check that)
            rand_timed = None
            alg_bytes -= 4 * moved
            gathered_bytes -= 4 * moved

        def step():
            random_walk(None, None, start, rand_timed, L, graph=graph, out=out, seed=PHILOX_SEED, walk_index_base=b,
                        walk_index_stride=stride)

    sampler = ClockSampler(dev) if rank == 0 else None
    total_ms, per, timed_launches = time_launches(step, steps, args.warmup, stream, sampler, barrier)
    clocks = sampler.stop() if sampler else None
    ms_per_step = allmax(total_ms / steps)
    kernel_ms = statistics.mean(per)
    value = walks_timed * L / (ms_per_step * 1e-3)
    peak, peak_kind = measured_peak_gbs()
    achieved = allsum(alg_bytes / (kernel_ms * 1e-3) / 1e9) / world  # mean per-GPU GB/s
    # random accesses one launch issues: every gather is one; a hash bucket (counted as four 8-byte loads) is one too
    if wl["kind"] == "node2vec" and cnt_kernel is not None:
        accesses = cnt_kernel["loads"] - 3 * cnt_kernel["probes"] - cnt_kernel["gathers16"]
    elif wl["kind"] == "node2vec":
        accesses = cnt["loads"] - (3 * cnt["probes"] if args.membership == "hash" else 0)
    else:
        accesses = (moved + 2 * rows) if not args.no_fused else (2 * moved + rows)
    small = NCU_SMALL_CASE["node2vec_tri" if cnt_kernel is not None else wl["kind"]]
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": f"of {peak_kind}",
                "traffic": small["dram_bytes"] / small["accesses"] * allsum(float(accesses)) / world,
                "traffic_source": f"{small['dram_bytes'] / small['accesses']:.1f} DRAM bytes per random access (ncu on "
                                  f"{small['workload']}, {small['source']}) x the random accesses one launch of this run "
                                  "issues per GPU, counted in this run",
                "kernel": ("node2vec_pool_tri_kernel" if cnt_kernel is not None else
                           "node2vec_pool_kernel (node2vec_walk_kernel where the pooled form does not apply)") if
                wl["kind"] == "node2vec" else "uniform_walk_staged_kernel", "kernel_ms": kernel_ms,
                "kernel_launched": _lib.last_kernel(), "random_accesses_per_launch": int(accesses),
                "algorithmic_bytes_per_launch": alg_bytes, "gathered_bytes_per_launch": gathered_bytes,
                "gathered_gbs": allsum(gathered_bytes / (kernel_ms * 1e-3) / 1e9) / world,
                "algorithmic_bytes_per_walk_step": alg_bytes / max(1, rows * L)}
    if cnt:
        roofline["counters"] = cnt
    if cnt_kernel is not None:
        roofline["kernel_counters"] = {k: cnt_kernel[k] for k in ("loads", "attempts", "membership", "probes", "gathers16", "filtered")}
    # second ceiling: the device's rate of dependent random gathers that miss L2 (measured now)
    if rank == 0 and not args.no_probe:
        ceiling = _lib.gather_probe(2 << 30, 32)
        roofline["random_access"] = {"ceiling_gathers_per_s": ceiling, "gathers_per_launch": int(accesses),
                                     "achieved_gathers_per_s": accesses / (kernel_ms * 1e-3),
                                     "frac": accesses / (kernel_ms * 1e-3) / ceiling,
                                     "note": "gathers issued, an upper bound on DRAM-missing ones"}

    # ---- the same launches without the triangle filter (a structure that takes seconds to build per graph)
    plain = None
    if cnt_kernel is not None and not light:
        _lib.set_tuning("n2v_tri", 0)
        p_ms, p_per, _ = time_launches(step, min(steps, 10), args.warmup, stream, None, barrier)
        plain_kernel = _lib.last_kernel()
        _lib.set_tuning("n2v_tri", 1)
        p_ms = allmax(p_ms / min(steps, 10))
        plain = {"ms_per_step": p_ms, "value": walks_timed * L / (p_ms * 1e-3), "unit": "steps/s",
                 "kernel": plain_kernel, "steps": min(steps, 10),
                 "roofline_frac": allsum(alg_bytes / (statistics.mean(p_per) * 1e-3) / 1e9) / world / peak}
        step()  # leave the filtered kernel's matrix in `out` for the checks below

    # ---- parity of what was just timed: the first rows of the matrix against the CPU restatement (untimed)
    parity = {}
    rowptr_h = col_h = None
    if rank == 0 and not args.no_parity:
        rowptr_h, col_h = rowptr.cpu().numpy(), col.cpu().numpy()
        k = min(rows, args.parity_rows)
        # the device-rand arm is checked by feeding the host replay of its draws to the restatement
        if wl["kind"] == "uniform" and args.device_rand:
            rand_rows = _lib.uniform_draws(PHILOX_SEED, k, L, b, stride)
        else:
            rand_rows = None if rand is None else rand[:k].cpu().numpy()
        parity["parity_rows_checked"] = parity_rows(wl, rowptr_h, col_h, start[:k].cpu().numpy(), rand_rows,
                                                    out[:k].cpu().numpy(), b, stride)

    # ---- optional gather of the walk matrix to rank 0 over NVLink (N > 1), timed apart from the walks
    gather = None
    if gather_plan is not None:
        wrows = gather_plan["window_rows"]
        windows = [(lo, min(n_walks, lo + wrows)) for lo in range(0, n_walks, wrows)]
        if not gather_plan["whole"] and args.gather_windows > 0:
            windows = windows[:args.gather_windows]

        def do_gather():
            for lo, hi in windows:
                gather_rows(out, n_walks, dst=0, out=None if full is None else full[:hi - lo], row_range=(lo, hi))

        do_gather()  # warm-up: NCCL sets up its point-to-point channels on first use
        torch.cuda.synchronize(dev)
        barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        do_gather()
        ev1.record(stream)
        torch.cuda.synchronize(dev)
        gather_ms = allmax(ev0.elapsed_time(ev1))
        gathered_rows = sum(hi - lo for lo, hi in windows)
        mine = sum(max(0, min(hi, b + rows) - max(lo, b)) for lo, hi in windows) if rank == 0 else 0
        inbound = allsum(float((gathered_rows - mine) * row_bytes if rank == 0 else 0))
        scale = n_walks / gathered_rows  # windows left out are charged at the measured rate
        gather = {"ms": gather_ms, "rows_gathered": gathered_rows, "bytes_into_rank0": inbound,
                  "gbs_into_rank0": inbound / (gather_ms * 1e-3) / 1e9,
                  "windows": len(windows), "window_rows": wrows,
                  "layout": "whole matrix resident on rank 0; rank 0's kernel wrote its block in place, the other "
                            "blocks were received at their row offsets in one batch of point-to-point messages"
                  if gather_plan["whole"] else
                  "matrix larger than rank 0's free memory: gathered window by window (caller-chosen row ranges) "
                  "into one reused buffer",
                  "walk_plus_gather_steps_per_s": n_walks * L / ((ms_per_step + gather_ms * scale) * 1e-3),
                  "walk_only_steps_per_s": value}
        if rank == 0 and parity and gather_plan["whole"]:
            # rows that came over the wire: the first block of the last rank
            from mlx_cluster_b200.sharding import shard_range
            rb, _ = shard_range(n_walks, world, world - 1)
            k = min(256, n_walks - rb)
            order_h = start_order(n_nodes, wpn)[rb:rb + k].numpy()
            parity["gathered_rows_checked"] = parity_rows(wl, rowptr_h, col_h, order_h, None, full[rb:rb + k].cpu().numpy(),
                                                          rb, 1) if wl["kind"] == "node2vec" else 0

    # ---- end to end: host buffers through the public API, copies inside the timed region
    e2e = None
    if not args.no_e2e and not (wl["kind"] == "uniform" and args.device_rand):
        e2e_steps = max(1, min(steps, args.e2e_steps))
        h_rowptr, h_col = rowptr.cpu(), col.cpu()
        h_start = start.cpu().pin_memory()
        h_rand = rand.cpu().pin_memory() if rand is not None else None
        del graph, out, full, rand
        torch.cuda.empty_cache()
        h_out = torch.empty((rows, L + 1), dtype=torch.int64, pin_memory=True)
        if world > 1 and _lib.get_tuning("host_threads") == 0:  # the ranks of one box share its cores
            _lib.set_tuning("host_threads", max(2, min(16, len(os.sched_getaffinity(0)) // world)))
        if barrier:
            barrier()  # all ranks create their graphs at once: the transport choice is measured under that load
        t_up = time.perf_counter()
        hg = HostGraph(h_rowptr, h_col, symmetric=True, device=dev,
                       edgeset=(wl["kind"] == "node2vec" and args.membership == "hash"),
                       fused=(wl["kind"] == "uniform" and not args.no_fused),
                       trifilter=(wl["kind"] == "node2vec" and args.membership == "hash" and not args.no_trifilter))
        upload_s = time.perf_counter() - t_up

        def host_step():
            if wl["kind"] == "node2vec":
                _lib.check(_lib.lib().walk_b200_node2vec_walk_host(
                    hg._h, h_start.data_ptr(), rows, L, wl["p"], wl["q"], PHILOX_SEED, b, stride, h_out.data_ptr(), None))
            else:
                _lib.check(_lib.lib().walk_b200_uniform_walk_host(
                    hg._h, h_start.data_ptr(), h_rand.data_ptr(), rows, L, h_out.data_ptr(), None))

        host_step()
        if barrier:
            barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host_step()
        dt = time.perf_counter() - t0
        e2e_ms = allmax(1e3 * dt / e2e_steps)
        narrow = _lib.host_transport(hg._h) == 1
        e2e = {"value": walks_timed * L / (e2e_ms * 1e-3), "unit": "steps/s",
               "h2d_bytes_per_step": int(allsum(rows * 8 + (rows * L * 4 if h_rand is not None else 0))),
               "d2h_bytes_per_step": int(allsum(rows * (L + 1) * (4 if narrow else 8))),
               "ms_per_step": e2e_ms, "steps": e2e_steps, "host_threads_per_rank": _lib.get_tuning("host_threads") or
               min(16, len(os.sched_getaffinity(0))),
               "transport": "int32 on the bus, widened to the caller's int64 buffer by host threads" if narrow
               else "int64 straight into the caller's pinned buffer",
               "transport_ranks_narrow": int(allsum(1.0 if narrow else 0.0)),
               "api": "walk_b200_*_walk_host (C ABI, pinned host buffers, graph resident)",
               "graph_upload_s_once": upload_s}
        if rank == 0 and parity:
            k = min(rows, args.parity_rows)
            rand_rows = None if h_rand is None else h_rand[:k].numpy()
            e2e["parity_rows_checked"] = parity_rows(wl, rowptr_h, col_h, h_start[:k].numpy(), rand_rows,
                                                     h_out[:k].numpy(), b, stride)
        hg.close()
        del h_out
        if not light and not args.no_ceiling:
            e2e["ceiling"] = host_ceiling(dev, world, barrier, narrow)
            c = e2e["ceiling"]
            d2h_total = e2e["d2h_bytes_per_step"]
            e2e["ceiling"]["copy_bound_ms_per_step"] = d2h_total / max(1e-9, c["d2h_pinned_gbs_all_ranks_at_once_sum"]) / 1e6
    else:
        del graph, out, full

    # ---- CPU baseline beside it (rank 0, single GPU runs only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu and not light:
        rp = rowptr_h if rowptr_h is not None else rowptr.cpu().numpy()
        cl = col_h if col_h is not None else col.cpu().numpy()
        rng = np.random.default_rng(0)
        n_rows = size_cpu_sample(wl, rp, cl, n_nodes, args.cpu_seconds, 1, rng)
        s = start_order(n_nodes, wpn)[:n_rows].numpy()
        r = rng.random((n_rows, L), dtype=np.float32) if wl["kind"] == "uniform" else None
        secs, kind, used = cpu_walk_seconds(wl, rp, cl, s, r, 1)
        cpu = {"value": n_rows * L / secs, "unit": "steps/s", "cores": used, "kind": kind,
               "sample": f"first {n_rows} of {n_nodes} start rows, one pass, {secs:.1f} s",
               "host_cores_available": len(os.sched_getaffinity(0))}

    sampled_total = allsum(float(sampled_steps))
    del rowptr, col, start
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    line = {
        "metric": "walk_steps_per_sec", "value": value, "unit": "steps/s", "n_gpus": world,
        "steps": steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
        "config": workload_config(wl, name, n_nodes, n_edges, shard_world, args.membership,
                                  "col + row descriptors" if args.no_fused else "fused 16-byte records",
                                  "generated in the kernel (Philox4x32-10)" if args.device_rand else None),
        # steps that draw and move (the rest stand still on a node without edges: 47 % of the R-MAT-24 nodes are isolated)
        "sampled_steps_per_sec": sampled_total / (ms_per_step * 1e-3),
        "roofline": roofline, "cpu_baseline": cpu,
        "e2e": e2e, "gpu_launches": int(timed_launches), "clocks": clocks, "graph_build_s": build_s,
        "graph_prepare_s_once": prep_s,
    }
    line.update(parity)
    if plain is not None:
        line["without_trifilter"] = plain
    if gather is not None:
        line["gather"] = gather
    return line


def run_ours(args, wl):
    import torch.distributed as dist
    from mlx_cluster_b200 import _lib

    rank, local_rank, world = env_rank()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this package has no CPU path")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        # NCCL writes its log lines (the version banner included) to stdout unless told otherwise; stdout is for
        # the JSON line. The log level itself is the caller's business and is left alone.
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        # a collective that does not complete within minutes is a bug of this script, not a slow step
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=args.collective_timeout_s))
    barrier = (lambda: dist.barrier()) if world > 1 else None

    def allmax(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def allsum(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    _lib.lib()  # fail now if the CUDA library is missing
    line = run_workload(args, args.workload, wl, dev, world, rank, barrier, allmax, allsum)
    # The uniform walk rides along with the default run (config 3: R-MAT scale 22, one GPU), so that both of the
    # reference's operators are measured by the one command the driver runs.
    if args.workload == "node2vec_rmat24" and world == 1 and args.shard_of == 1 and not args.no_extra:
        extra = run_workload(args, "uniform_rmat22", WORKLOADS["uniform_rmat22"], dev, world, rank, barrier, allmax,
                             allsum, light=True)
        keep = ("value", "unit", "steps", "ms_per_step", "sampled_steps_per_sec", "parity_rows_checked", "gpu_launches")
        line["extra"] = {"uniform_rmat22": {**{k: extra[k] for k in keep if k in extra},
                                            "config": extra["config"],
                                            "roofline": {k: extra["roofline"].get(k) for k in
                                                         ("achieved", "peak", "frac", "traffic", "kernel", "kernel_ms",
                                                          "algorithmic_bytes_per_launch", "random_access")},
                                            "e2e": extra["e2e"]}}
    if rank == 0:
        # stdout carries the one JSON line; whatever libraries printed there before it went out earlier
        sys.stdout.flush()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="node2vec_rmat24", choices=list(WORKLOADS))
    ap.add_argument("--e2e-steps", type=int, default=3, help="end-to-end passes (each moves the whole walk matrix to the host)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0, help="target CPU time of the cpu_baseline sample")
    ap.add_argument("--membership", default="hash", choices=["hash", "search"],
                    help="node2vec membership test: edge hash set (built once per graph) or binary search over col")
    ap.add_argument("--shard-of", type=int, default=1,
                    help="single process only: walk rank 0's share of this many ranks (sizes the largest workload "
                         "for one GPU); value then counts this share alone")
    ap.add_argument("--device-rand", action="store_true",
                    help="uniform walk: generate the draws in the kernel instead of reading a rand array")
    ap.add_argument("--no-fused", action="store_true", help="uniform walk: do not build fused edge records")
    ap.add_argument("--edgeset-slots-per-edge", type=float, default=None,
                    help="node2vec: size of the edge hash set (2 = half full, the library's minimum; 4 = a quarter full; "
                         "default: the library's tuning, 4 when it fits)")
    ap.add_argument("--no-trifilter", action="store_true",
                    help="node2vec: do not build the triangle filter (seconds per graph; the walks then run the plain pooled kernel)")
    ap.add_argument("--trifilter-max-row", type=int, default=None,
                    help="node2vec triangle filter: leave edges whose shorter row is longer than this unfiltered "
                         "(0: none; default: the library's tuning, 1024)")
    ap.add_argument("--no-probe", action="store_true", help="skip the random-gather ceiling probe")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="default workload: skip the uniform walk that rides along")
    ap.add_argument("--no-parity", action="store_true", help="skip the untimed check against the CPU restatement")
    ap.add_argument("--parity-rows", type=int, default=1024)
    ap.add_argument("--no-gather", action="store_true", help="N > 1: skip the gather of the walk matrix to rank 0")
    ap.add_argument("--gather-window-gb", type=float, default=48.0,
                    help="N > 1: largest buffer rank 0 sets aside for the gathered matrix (or a window of it)")
    ap.add_argument("--gather-windows", type=int, default=4,
                    help="N > 1, matrix larger than the window: how many windows to gather and time (0 = all)")
    ap.add_argument("--no-ceiling", action="store_true", help="skip the host-side ceiling probes of the e2e leg")
    ap.add_argument("--collective-timeout-s", type=int, default=150, help="N > 1: process-group timeout")
    ap.add_argument("--tune", action="append", default=[], help="key=value passed to walk_b200_set_tuning")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 0)
    wl = WORKLOADS[args.workload]
    if args.impl == "reference":
        return run_reference_arm(args, wl)
    if args.tune:
        from mlx_cluster_b200 import _lib
        for kv in args.tune:
            k, v = kv.split("=")
            _lib.set_tuning(k, int(v))
    return run_ours(args, wl)


if __name__ == "__main__":
    raise SystemExit(main())
