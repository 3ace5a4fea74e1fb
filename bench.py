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
# DRAM bytes (read + write) per launch of the dominant kernel, from the ncu captures summarised under
# profiles/: measured on the scale-20 case of each workload; the full-size figures are that measurement
# scaled by the number of gathers issued (traffic is proportional to gathers; see the profile notes).
NCU_TRAFFIC = {
    "node2vec_rmat20": (19.60e9, "ncu, measured"),
    "node2vec_rmat24": (19.60e9 * 14.90, "ncu on node2vec_rmat20 scaled by gathers issued (x14.90)"),
    "uniform_rmat20": (4.70e9, "ncu, measured"),
    "uniform_rmat22": (4.70e9 * 3.72, "ncu on uniform_rmat20 scaled by gathers issued (x3.72)"),
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
        "config": workload_config(wl, n_total, int(col.size), args.gpus),
        "cpu_baseline": {"value": value, "unit": "steps/s", "cores": used, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


def workload_config(wl, n_nodes, n_edges, gpus, membership=None, edge_records=None, rand_source=None):
    c = {"workload": args_workload_name(wl), "graph": f"R-MAT scale {wl['scale']} edge factor {wl['edge_factor']} "
         f"(a,b,c,d)=(0.57,0.19,0.19,0.05) seed {wl['seed']}, symmetrised, deduplicated, no self-loops, int64 CSR",
         "num_nodes": n_nodes, "num_directed_edges": n_edges, "starts": f"every node {wl.get('walks_per_node', 1)}x, in a seeded random order", "walk_length": wl["L"],
         "sharding": f"start rows dealt cyclically over {gpus} GPU(s), CSR replicated",
         "l2": "no flush between steps: col (8 B x edges) is far larger than the 126 MB L2"}
    if wl["kind"] == "node2vec":
        c.update(p=wl["p"], q=wl["q"], draws="Philox4x32-10, key=seed, counter=(walk,step,attempt)",
                 membership=membership)
    else:
        c.update(rand=rand_source or "float32 uniform [0,1) [n, walk_length], caller-supplied", edge_records=edge_records)
    return c


def args_workload_name(wl):
    for k, v in WORKLOADS.items():
        if v is wl:
            return k
    return "custom"


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


def run_ours(args, wl):
    import torch.distributed as dist
    from mlx_cluster_b200 import _lib, random_walk, rejection_sampling
    from mlx_cluster_b200.ops import WalkGraph, HostGraph
    from mlx_cluster_b200.sharding import shard_rows

    rank, local_rank, world = env_rank()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this package has no CPU path")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        # NCCL prints its version banner on stdout at the VERSION log level; stdout is for the JSON line
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=dev)
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
    rowptr, col, build_s = build_graph(wl, dev, world, rank)
    n_nodes, n_edges, L = rowptr.numel() - 1, col.numel(), wl["L"]
    # Every node starts one walk; the start list is a seeded random order of the nodes and is dealt
    # cyclically (rank r walks rows r, r + G, ...). On R-MAT every bit of a node id is correlated with
    # its degree, so shards cut by id -- blocks or strides of the natural order -- differ by up to 3x
    # in work; a random order makes any split even. Draws are indexed by the row, so the walks do
    # not depend on the GPU count.
    wpn = wl.get("walks_per_node", 1)
    n_walks = n_nodes * wpn
    shard_world, shard_rank = (args.shard_of, 0) if (world == 1 and args.shard_of > 1) else (world, rank)
    row_slice, (b, stride) = shard_rows(n_walks, shard_world, shard_rank, "cyclic")
    order = start_order(n_nodes, wpn, dev)
    start = order[row_slice].contiguous().to(dev)
    del order
    torch.cuda.empty_cache()
    rows = start.numel()
    walks_timed = n_walks if shard_world == world else rows  # a lone rank's share counts only its own rows
    t_prep = time.perf_counter()
    graph = WalkGraph(rowptr, col, symmetric=True, edgeset=(wl["kind"] == "node2vec" and args.membership == "hash"),
                      fused=(wl["kind"] == "uniform" and not args.no_fused))
    torch.cuda.synchronize(dev)
    prep_s = time.perf_counter() - t_prep
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
        rand = None

        def step():
            rejection_sampling(None, None, start, L, wl["p"], wl["q"], graph=graph, seed=PHILOX_SEED,
                               walk_index_base=b, walk_index_stride=stride, out=out)
    else:
        gen = torch.Generator(device=dev).manual_seed(1234 + rank)
        rand = torch.rand((rows, L), generator=gen, device=dev)
        deg = rowptr.diff()
        cnt = {}
        random_walk(None, None, start, rand, L, graph=graph, out=out, check=True)
        moved = 0
        for c0 in range(0, rows, 1 << 22):  # in slices: the index tensor of the whole matrix would not fit beside it
            moved += int((deg[out[c0:c0 + (1 << 22), :-1].reshape(-1)] > 0).sum().item())
        stay = rows * L - moved
        # per step: row bounds 16 (8 via the packed descriptor, counted as the CSR's 16) + rand 4 + col 8 + out 8
        alg_bytes = rows * 16 + moved * 36 + stay * 24
        # 8-byte descriptor instead of the 16-byte row pair; fused records: one 16-byte gather per moving step
        gathered_bytes = rows * 24 + moved * 28 if not args.no_fused else rows * 16 + moved * 28 + stay * 12

        if args.device_rand:
            # draws generated in the kernel (same walks as feeding the replayed stream; tests check that)
            rand = None
            alg_bytes -= 4 * moved
            gathered_bytes -= 4 * moved

        def step():
            random_walk(None, None, start, rand, L, graph=graph, out=out, seed=PHILOX_SEED, walk_index_base=b,
                        walk_index_stride=stride)

    sampler = ClockSampler(dev) if rank == 0 else None
    total_ms, per, timed_launches = time_launches(step, args.steps, args.warmup, stream, sampler, barrier)
    clocks = sampler.stop() if sampler else None
    ms_per_step = allmax(total_ms / args.steps)
    kernel_ms = statistics.mean(per)
    value = walks_timed * L / (ms_per_step * 1e-3)
    peak, peak_kind = measured_peak_gbs()
    achieved = allsum(alg_bytes / (kernel_ms * 1e-3) / 1e9) / world  # mean per-GPU GB/s
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": f"of {peak_kind}",
                "traffic": NCU_TRAFFIC.get(args.workload, (None, None))[0] if world == 1 else None,
                "traffic_source": NCU_TRAFFIC.get(args.workload, (None, None))[1], "kernel": "node2vec_pool_kernel (node2vec_walk_kernel where the pooled form does not apply)" if
                wl["kind"] == "node2vec" else "uniform_walk_staged_kernel", "kernel_ms": kernel_ms,
                "algorithmic_bytes_per_launch": alg_bytes, "gathered_bytes_per_launch": gathered_bytes,
                "gathered_gbs": allsum(gathered_bytes / (kernel_ms * 1e-3) / 1e9) / world,
                "algorithmic_bytes_per_walk_step": alg_bytes / max(1, rows * L)}
    if cnt:
        roofline["counters"] = cnt
    # second ceiling: the device's rate of dependent random gathers that miss L2 (measured now)
    if rank == 0 and not args.no_probe:
        ceiling = _lib.gather_probe(2 << 30, 32)
        if wl["kind"] == "node2vec":
            # every gather the kernel issued is one random access; a hash bucket (counted as four 8-byte
            # loads) is one access too (upper bound on DRAM misses)
            accesses = cnt["loads"] - (3 * cnt["probes"] if args.membership == "hash" else 0)
        else:
            accesses = (moved + 2 * rows) if not args.no_fused else (2 * moved + rows)
        roofline["random_access"] = {"ceiling_gathers_per_s": ceiling, "gathers_per_launch": int(accesses),
                                     "achieved_gathers_per_s": accesses / (kernel_ms * 1e-3),
                                     "frac": accesses / (kernel_ms * 1e-3) / ceiling,
                                     "note": "gathers issued, an upper bound on DRAM-missing ones"}

    # ---- end to end: host buffers through the public API, copies inside the timed region
    e2e = None
    if not args.no_e2e and not (wl["kind"] == "uniform" and args.device_rand):
        e2e_steps = max(1, min(args.steps, args.e2e_steps))
        h_rowptr, h_col = rowptr.cpu(), col.cpu()
        h_start = start.cpu().pin_memory()
        h_out = torch.empty((rows, L + 1), dtype=torch.int64, pin_memory=True)
        h_rand = rand.cpu().pin_memory() if rand is not None else None
        t_up = time.perf_counter()
        hg = HostGraph(h_rowptr, h_col, symmetric=True, device=dev,
                       edgeset=(wl["kind"] == "node2vec" and args.membership == "hash"),
                       fused=(wl["kind"] == "uniform" and not args.no_fused))
        upload_s = time.perf_counter() - t_up
        del graph, out
        torch.cuda.empty_cache()

        def host_step():
            if wl["kind"] == "node2vec":
                _lib.check(_lib.lib().walk_b200_node2vec_walk_host(
                    hg._h, h_start.data_ptr(), rows, L, wl["p"], wl["q"], PHILOX_SEED, b, stride, h_out.data_ptr(), None))
            else:
                _lib.check(_lib.lib().walk_b200_uniform_walk_host(
                    hg._h, h_start.data_ptr(), h_rand.data_ptr(), rows, L, h_out.data_ptr(), None))

        narrow = n_nodes < 2 ** 31 and _lib.get_tuning("host_narrow") != 0
        if world > 1 and _lib.get_tuning("host_threads") == 0:  # the ranks of one box share its cores
            _lib.set_tuning("host_threads", max(2, min(16, len(os.sched_getaffinity(0)) // world)))
        host_step()
        if barrier:
            barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            host_step()
        dt = time.perf_counter() - t0
        e2e_ms = allmax(1e3 * dt / e2e_steps)
        e2e = {"value": walks_timed * L / (e2e_ms * 1e-3), "unit": "steps/s",
               "h2d_bytes_per_step": int(allsum(rows * 8 + (rows * L * 4 if rand is not None else 0))),
               "d2h_bytes_per_step": int(allsum(rows * (L + 1) * (4 if narrow else 8))),
               "ms_per_step": e2e_ms, "steps": e2e_steps, "host_threads_per_rank": _lib.get_tuning("host_threads") or
               min(16, len(os.sched_getaffinity(0))),
               "transport": "int32 on the bus, widened to the caller's int64 buffer by host threads" if narrow
               else "int64",
               "api": "walk_b200_*_walk_host (C ABI, pinned host buffers, graph resident)",
               "graph_upload_s_once": upload_s}
        hg.close()

    # ---- CPU baseline beside it (rank 0, single GPU runs only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        rp, cl = rowptr.cpu().numpy(), col.cpu().numpy()
        rng = np.random.default_rng(0)
        n_rows = size_cpu_sample(wl, rp, cl, n_nodes, args.cpu_seconds, 1, rng)
        s = start_order(n_nodes, wpn)[:n_rows].numpy()
        r = rng.random((n_rows, L), dtype=np.float32) if wl["kind"] == "uniform" else None
        secs, kind, used = cpu_walk_seconds(wl, rp, cl, s, r, 1)
        cpu = {"value": n_rows * L / secs, "unit": "steps/s", "cores": used, "kind": kind,
               "sample": f"first {n_rows} of {n_nodes} start rows, one pass, {secs:.1f} s",
               "host_cores_available": len(os.sched_getaffinity(0))}

    if rank == 0:
        line = {
            "metric": "walk_steps_per_sec", "value": value, "unit": "steps/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int64", "data": "synthetic",
            "config": workload_config(wl, n_nodes, n_edges, shard_world, args.membership,
                                      "col + row descriptors" if args.no_fused else "fused 16-byte records",
                                      "generated in the kernel (Philox4x32-10)" if args.device_rand else None),
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": e2e, "gpu_launches": int(timed_launches), "clocks": clocks, "graph_build_s": build_s,
            "graph_prepare_s_once": prep_s,
        }
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
    ap.add_argument("--no-probe", action="store_true", help="skip the random-gather ceiling probe")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
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
