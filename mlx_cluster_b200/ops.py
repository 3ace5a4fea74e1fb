"""Host-side mirror of the reference's operator interface for the walk path.

``random_walk`` and ``rejection_sampling`` keep the names, positional order and
keyword-only ``stream`` of the reference's Python API (``bindings.cpp:12-21`` and
``bindings.cpp:35-45``; re-exported at ``mlx_cluster/__init__.py:3-4``) and return the
node sequence ``[n_start, walk_length + 1]`` as the reference's factories do
(``random_walks/RandomWalk.cpp:138-148``, ``random_walks/BiasedRandomWalk.cpp:183-193``).
Arrays are ``torch`` tensors: CUDA tensors run in place on their device, stream-ordered
and asynchronous like any torch CUDA op; CPU tensors / numpy arrays go through the
resident-graph host entry points (graph uploaded once, per-call batch copied in slabs).
Everything computes in the CUDA library behind the C ABI; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from collections import OrderedDict
from typing import Optional

import numpy as np
import torch

from . import _lib

__all__ = ["random_walk", "rejection_sampling", "context_windows", "prepare_graph", "WalkGraph", "HostGraph",
           "read_status", "clear_caches"]


def _stream_handle(stream, device) -> int:
    if stream is None:
        return int(torch.cuda.current_stream(device).cuda_stream)
    if isinstance(stream, torch.cuda.Stream):
        return int(stream.cuda_stream)
    if isinstance(stream, int):
        return stream
    raise TypeError(f"stream must be None, a torch.cuda.Stream or a raw handle, not {type(stream).__name__}")


def _sync_stream(stream, device) -> None:
    """Wait for the stream the kernels were launched on (``None``: torch's current stream)."""
    if stream is None:
        torch.cuda.current_stream(device).synchronize()
    elif isinstance(stream, torch.cuda.Stream):
        stream.synchronize()
    else:
        torch.cuda.ExternalStream(int(stream), device=device).synchronize()


def _take_flags(flags: torch.Tensor, stream, device) -> int:
    """Read and clear a status word that kernels on ``stream`` may have written. The read waits for that
    stream first: ``Tensor.item()`` alone only orders itself after torch's *current* stream."""
    _sync_stream(stream, device)
    f = int(flags.item())
    if f:
        flags.zero_()
        torch.cuda.current_stream(device).synchronize()  # the clear lands before a later launch on another stream
    return f


def _require(t, name, dtype, device=None):
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if t.dtype != dtype:
        # the reference reinterprets the bytes of whatever dtype it is given
        # (random_walks/RandomWalk.cpp:33-38); here that is an error instead
        raise TypeError(f"{name} must have dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    if device is not None and t.device != device:
        raise ValueError(f"{name} is on {t.device}, expected {device}")
    return t


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None or t.numel() == 0 else t.data_ptr()


class WalkGraph:
    """A CSR graph on one CUDA device plus its packed row descriptors (8 bytes per node:
    row start | degree << 36) so that a walk step fetches row bounds with one load."""

    def __init__(self, rowptr: torch.Tensor, col: torch.Tensor, *, symmetric: bool = False,
                 use_rowdesc: bool = True, edgeset: bool = False, fused: bool = False, validate: bool = False,
                 stream=None, edgeset_slots_per_edge: Optional[float] = None, trifilter: bool = False,
                 trifilter_max_row: Optional[int] = None):
        if not rowptr.is_cuda:
            raise ValueError("WalkGraph needs CUDA tensors (use HostGraph for host arrays)")
        dev = rowptr.device
        self.rowptr = _require(rowptr, "rowptr", torch.int64)
        self.col = _require(col, "col", torch.int64, dev)
        if rowptr.dim() != 1 or rowptr.numel() < 1 or col.dim() != 1:
            raise ValueError("rowptr must be 1-D with num_nodes + 1 entries and col 1-D")
        self.device = dev
        self.num_nodes = rowptr.numel() - 1
        self.num_edges = col.numel()
        self.symmetric = bool(symmetric)
        self.rowdesc = None
        self.edgeset = None
        self.edgeset_buckets = 0
        self.colrev = None
        self.colrev16 = None
        self.fused = None
        # size of the edge hash set in 8-byte slots per edge: 2 = half full (the minimum), 4 = a quarter full;
        # None = the library's tuning (default 4), taken when the table fits half of the free device memory
        self.edgeset_slots_per_edge = None if edgeset_slots_per_edge is None else max(2.0, float(edgeset_slots_per_edge))
        if trifilter and edgeset_slots_per_edge is None:
            # behind the triangle filter few tests reach the hash set: a sparser table buys nothing there (88.1 against
            # 88.2 ms on the headline workload) and costs its memory
            self.edgeset_slots_per_edge = 2.0
        self.filter_declined = False  # edgeset="auto" looked at this graph for a triangle filter and left it
        self.rows_sorted = None   # None: not checked yet (see check_rows_sorted)
        self.n2v_calls = 0        # node2vec calls served: edgeset="auto" builds the hash set on the second
        self._version = (rowptr._version, col._version)
        with torch.cuda.device(dev):
            self.flags = torch.zeros(1, dtype=torch.int32, device=dev)
            torch.cuda.current_stream(dev).synchronize()  # the zero fill lands before a launch on another stream
            sh = _stream_handle(stream, dev)
            if validate:
                self.validate(stream=stream)
                self.rows_sorted = True
            if use_rowdesc and self.num_nodes > 0:
                desc = torch.empty(self.num_nodes, dtype=torch.int64, device=dev)
                _lib.check(_lib.lib().walk_b200_rowdesc_pack(
                    rowptr.data_ptr(), self.num_nodes, self.num_edges, desc.data_ptr(),
                    self.flags.data_ptr(), sh))
                f = _take_flags(self.flags, stream, dev)
                if f & _lib.FLAG_BAD_ROWPTR:
                    raise ValueError("rowptr is not a monotone prefix array ending at col.numel()")
                if not (f & _lib.FLAG_DESC_OVERFLOW):
                    self.rowdesc = desc
            if edgeset and self.num_edges > 0:
                self.build_edgeset(stream=stream)
            if fused and self.num_edges > 0:
                self.build_fused(stream=stream)
            if trifilter and self.num_edges > 0:
                self.build_trifilter(stream=stream, max_row=trifilter_max_row)

    def build_fused(self, stream=None):
        """Build the fused edge records (16 bytes per edge: target node + its row descriptor) that
        make a uniform walk step one gather instead of two."""
        if self.fused is not None or self.rowdesc is None:
            return
        with torch.cuda.device(self.device):
            rec = torch.empty((self.num_edges, 2), dtype=torch.int64, device=self.device)
            csr = self.csr()
            _lib.check(_lib.lib().walk_b200_fused_build(C.byref(csr), rec.data_ptr(), self.flags.data_ptr(),
                                                        _stream_handle(stream, self.device)))
            f = _take_flags(self.flags, stream, self.device)
            if f:
                raise ValueError(f"fused record build failed, status flags 0x{f:x}: {describe_flags(f)}")
            self.fused = rec

    def build_trifilter(self, stream=None, max_row: Optional[int] = None):
        """Build the triangle filter of an undirected graph (16 bytes per edge; needs ``symmetric=True``, builds the
        edge hash set and reverse positions first if they are missing): per directed edge, which positions of the
        target's row hold common neighbours of its two ends. A node2vec walk then knows from the position it drew,
        before gathering the candidate, that the previous node is not a neighbour of it, which is the usual answer
        of that test. One edge-set look-up per entry of the shorter row of every undirected edge (``max_row`` > 0
        leaves edges whose shorter row is longer unfiltered; None = the library's tuning, 1024; 0 = no limit):
        seconds on a graph of 5e8 edges, so this is for graphs that are walked many times. Results do not change."""
        if self.colrev16 is not None:
            return
        if max_row is None:
            max_row = _lib.get_tuning("trifilter_max_row")
        if not self.symmetric:
            raise ValueError("the triangle filter needs a graph declared undirected (symmetric=True)")
        self.build_edgeset(stream=stream)
        if self.colrev is None:
            raise ValueError("the triangle filter needs the reverse positions (rows strictly ascending, row descriptors)")
        with torch.cuda.device(self.device):
            rec = torch.empty((self.num_edges, 2), dtype=torch.int64, device=self.device)
            csr = self.csr()
            _lib.check(_lib.lib().walk_b200_trifilter_build(C.byref(csr), rec.data_ptr(), int(max_row),
                                                            self.flags.data_ptr(), _stream_handle(stream, self.device)))
            f = _take_flags(self.flags, stream, self.device)
            if f:
                raise ValueError(f"triangle filter build failed, status flags 0x{f:x}: {describe_flags(f)}")
            self.colrev16 = rec

    def build_edgeset(self, stream=None):
        """Build the edge hash set (16 bytes per edge) that turns node2vec's membership test
        into about one 32-byte read. Any CSR: directed or not, rows sorted or not."""
        if self.edgeset is not None:
            return
        with torch.cuda.device(self.device):
            # the library's size is the smallest it accepts (half full); a sparser table answers more tests
            # from their first bucket at the price of its memory
            buckets = _lib.edgeset_buckets(self.num_edges)
            if self.edgeset_slots_per_edge is not None:
                buckets = int(buckets * self.edgeset_slots_per_edge / 2.0)
            else:
                want = int(buckets * max(2, min(16, _lib.get_tuning("edgeset_slots_per_edge"))) / 2.0)
                free, _ = torch.cuda.mem_get_info(self.device)
                cached = torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
                if want * 32 + 12 * self.num_edges < (free + cached) // 2:
                    buckets = want
            table = torch.empty(buckets * 4, dtype=torch.int64, device=self.device)
            csr = self.csr()
            _lib.check(_lib.lib().walk_b200_edgeset_build(C.byref(csr), table.data_ptr(), buckets,
                                                          self.flags.data_ptr(), _stream_handle(stream, self.device)))
            f = _take_flags(self.flags, stream, self.device)
            if f:
                raise ValueError(f"edge set build failed, status flags 0x{f:x}: {describe_flags(f)}")
            self.edgeset, self.edgeset_buckets = table, buckets
            # reverse positions ride along when they can be built (rows strictly ascending, < 2^32 - 2
            # edges); they are joined with col into the one array the kernel gathers candidates from
            if self.num_edges < 2**32 - 2 and self.rowdesc is not None and self.num_nodes < 2**32 - 1:
                rev = torch.empty(self.num_edges, dtype=torch.int32, device=self.device)
                sh = _stream_handle(stream, self.device)
                _lib.check(_lib.lib().walk_b200_revpos_build(C.byref(csr), rev.data_ptr(), self.flags.data_ptr(), sh))
                f = _take_flags(self.flags, stream, self.device)
                if self.rows_sorted is None:  # the build checks every row on its way
                    self.rows_sorted = not (f & _lib.FLAG_UNSORTED_ROW)
                if not f:
                    csr.revpos = rev.data_ptr()
                    joined = torch.empty(self.num_edges, dtype=torch.int64, device=self.device)
                    _lib.check(_lib.lib().walk_b200_colrev_build(C.byref(csr), joined.data_ptr(), self.flags.data_ptr(), sh))
                    f = _take_flags(self.flags, stream, self.device)
                    if f:
                        raise ValueError(f"colrev build failed, status flags 0x{f:x}: {describe_flags(f)}")
                    self.colrev = joined

    def csr(self) -> _lib.Csr:
        return _lib.Csr(self.rowptr.data_ptr(), _ptr(self.col), self.num_nodes, self.num_edges,
                        _ptr(self.rowdesc), _lib.CSR_SYMMETRIC if self.symmetric else 0, 0,
                        _ptr(self.edgeset), self.edgeset_buckets, None, _ptr(self.fused), _ptr(self.colrev),
                        _ptr(self.colrev16))

    def _validate_flags(self, start, check_sorted, stream) -> int:
        with torch.cuda.device(self.device):
            flags = torch.zeros(1, dtype=torch.int32, device=self.device)
            torch.cuda.current_stream(self.device).synchronize()  # the zero fill lands before a launch on another stream
            csr = self.csr()
            _lib.check(_lib.lib().walk_b200_csr_validate(
                C.byref(csr), _ptr(start), 0 if start is None else start.numel(), int(check_sorted),
                flags.data_ptr(), _stream_handle(stream, self.device)))
            return _take_flags(flags, stream, self.device)

    def validate(self, start: Optional[torch.Tensor] = None, *, check_sorted: bool = True, stream=None):
        """Raise ValueError when the CSR (and, if given, the start nodes) is malformed."""
        f = self._validate_flags(start, check_sorted, stream)
        if f:
            raise ValueError(f"malformed graph input, status flags 0x{f:x}: {describe_flags(f)}")

    def check_rows_sorted(self, stream=None) -> bool:
        """Whether every row of ``col`` is strictly ascending -- what the binary-search membership test of
        node2vec needs, and what the reference's linear ``is_neighbor`` scan
        (``random_walks/BiasedRandomWalk.cpp:20-28``) does not. Checked once per graph (one pass over the
        CSR); any other defect found on the way (ids out of range, a broken ``rowptr``) raises."""
        if self.rows_sorted is None:
            f = self._validate_flags(None, True, stream)
            other = f & ~_lib.FLAG_UNSORTED_ROW
            if other:
                raise ValueError(f"malformed graph input, status flags 0x{other:x}: {describe_flags(other)}")
            self.rows_sorted = not (f & _lib.FLAG_UNSORTED_ROW)
        return self.rows_sorted

    def edgeset_fits(self) -> bool:
        """Whether this device has room left for the edge hash set and the reverse positions (together
        about 28 bytes per edge while they are built, 24 afterwards)."""
        free, _ = torch.cuda.mem_get_info(self.device)
        cached = torch.cuda.memory_reserved(self.device) - torch.cuda.memory_allocated(self.device)
        return 28 * self.num_edges * 1.2 + (256 << 20) < free + cached


def describe_flags(f: int) -> str:
    names = [(_lib.FLAG_BAD_NODE, "node id out of range"), (_lib.FLAG_BAD_EDGE, "edge index out of range (rand outside [0,1)?)"),
             (_lib.FLAG_ATTEMPT_CAP, "rejection attempt cap hit"), (_lib.FLAG_BAD_ROWPTR, "rowptr malformed"),
             (_lib.FLAG_DESC_OVERFLOW, "row descriptor overflow"), (_lib.FLAG_UNSORTED_ROW, "row not strictly ascending"),
             (_lib.FLAG_EDGESET_FULL, "edge hash set overflow")]
    return "; ".join(n for b, n in names if f & b) or "none"


# ---- graph caches: keyed on storage identity + version, holding the keyed tensors alive
_GRAPH_CACHE: "OrderedDict[tuple, WalkGraph]" = OrderedDict()
_HOST_CACHE: "OrderedDict[tuple, HostGraph]" = OrderedDict()
_CACHE_SIZE = 4


def clear_caches() -> None:
    _GRAPH_CACHE.clear()
    for g in _HOST_CACHE.values():
        g.close()
    _HOST_CACHE.clear()


def _key(rowptr, col, symmetric):
    return (rowptr.data_ptr(), rowptr.numel(), rowptr._version, col.data_ptr(), col.numel(), col._version,
            str(rowptr.device), bool(symmetric))


def prepare_graph(rowptr, col, *, symmetric: bool = False, edgeset: bool = False, fused: bool = False,
                  validate: bool = False, trifilter: bool = False) -> "WalkGraph":
    """Build (or fetch from a small cache) the device-side graph for these CSR tensors."""
    k = _key(rowptr, col, symmetric)
    g = _GRAPH_CACHE.get(k)
    if g is not None and edgeset:
        g.build_edgeset()
    if g is not None and fused:
        g.build_fused()
    if g is not None and trifilter:
        g.build_trifilter()
    if g is None:
        g = WalkGraph(rowptr, col, symmetric=symmetric, edgeset=edgeset, fused=fused, validate=validate,
                      trifilter=trifilter)
        _GRAPH_CACHE[k] = g
        while len(_GRAPH_CACHE) > _CACHE_SIZE:
            _GRAPH_CACHE.popitem(last=False)
    else:
        _GRAPH_CACHE.move_to_end(k)
    return g


class HostGraph:
    """A CSR graph given as host arrays, uploaded once and kept resident on one device."""

    def __init__(self, rowptr, col, *, symmetric: bool = False, edgeset: bool = False, fused: bool = False,
                 validate: bool = False, device=None, trifilter: bool = False):
        self.rowptr = _require(_as_cpu_tensor(rowptr), "rowptr", torch.int64)
        self.col = _require(_as_cpu_tensor(col), "col", torch.int64)
        self.num_nodes = self.rowptr.numel() - 1
        self.num_edges = self.col.numel()
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        if trifilter and not (symmetric and edgeset):
            raise ValueError("the triangle filter needs a graph declared undirected (symmetric=True) and the edge hash set "
                             "(edgeset=True)")
        h = C.c_void_p(None)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().walk_b200_graph_create(
                self.rowptr.data_ptr(), _ptr(self.col), self.num_nodes, self.num_edges,
                (_lib.CSR_SYMMETRIC if symmetric else 0) | (_lib.CSR_WANT_EDGESET if edgeset else 0)
                | (_lib.CSR_WANT_FUSED if fused else 0)
                | (_lib.CSR_WANT_TRIFILTER if trifilter else 0),
                int(validate), C.byref(h)))
        self._h = h

    def device_bytes(self) -> int:
        b = C.c_int64(0)
        _lib.check(_lib.lib().walk_b200_graph_device_bytes(self._h, C.byref(b)))
        return int(b.value)

    def close(self):
        if getattr(self, "_h", None):
            _lib.lib().walk_b200_graph_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _as_cpu_tensor(a):
    if isinstance(a, torch.Tensor):
        return a
    return torch.from_numpy(np.ascontiguousarray(a))


def _fingerprint(t: torch.Tensor) -> tuple:
    """Cheap content sample of a host array (ends, and a position-weighted sum of at most 2^17 evenly spaced
    entries): host arrays, numpy ones above all, carry no version counter, so an edit in place would
    otherwise go unseen and a stale resident graph would be walked. A cached graph is a snapshot of the
    arrays it was made from; an edit this sample misses needs ``clear_caches()`` or an explicit
    :class:`HostGraph`."""
    n = t.numel()
    if n == 0:
        return (0,)
    sample = t[::max(1, n >> 16)]
    weights = torch.arange(sample.numel(), dtype=torch.int64) % 1021 + 1
    return (int(t[0]), int(t[-1]), int((sample * weights).sum()))


def _host_graph(rowptr, col, symmetric, validate, edgeset=False, fused=False, trifilter=False):
    k = (_key(rowptr, col, symmetric) + (bool(edgeset), bool(fused), bool(trifilter)) + _fingerprint(rowptr)
         + _fingerprint(col))
    g = _HOST_CACHE.get(k)
    if g is None:
        g = HostGraph(rowptr, col, symmetric=symmetric, edgeset=edgeset, fused=fused, validate=validate,
                      trifilter=trifilter)
        _HOST_CACHE[k] = g
        while len(_HOST_CACHE) > _CACHE_SIZE:
            _, old = _HOST_CACHE.popitem(last=False)
            old.close()
    else:
        _HOST_CACHE.move_to_end(k)
    return g


def read_status(graph: WalkGraph, stream=None) -> int:
    """Wait for ``stream`` (the one the walks were launched on; ``None`` = torch's current stream), then
    return and clear the status flags kernels raised on this graph."""
    return _take_flags(graph.flags, stream, graph.device)


def _check_walk_length(walk_length):
    if not isinstance(walk_length, (int, np.integer)) or isinstance(walk_length, bool):
        raise TypeError("walk_length must be an int")
    if walk_length < 0 or walk_length > 2**31 - 2:
        raise ValueError("walk_length out of range")
    return int(walk_length)


def _finish(graph, out, e_out, check, return_edges, stream=None):
    if check:
        f = read_status(graph, stream)
        if f:
            raise RuntimeError(f"walk kernel raised status flags 0x{f:x}: {describe_flags(f)}")
    return (out, e_out) if return_edges else out


def _devices(devices):
    out = []
    for d in devices:
        d = torch.device("cuda", d) if isinstance(d, int) else torch.device(d)
        if d.type != "cuda":
            raise ValueError(f"devices must name CUDA devices, got {d}")
        out.append(torch.device("cuda", torch.cuda.current_device() if d.index is None else d.index))
    if not out:
        raise ValueError("devices is empty")
    return out


_REPLICAS: "OrderedDict[tuple, tuple]" = OrderedDict()


def _replica(rowptr, col, dev):
    """The CSR on ``dev``: the caller's tensors if they live there, else a copy made once (device to
    device, over NVLink where the GPUs are connected) and kept while the source tensors are unchanged."""
    if rowptr.device == dev:
        return rowptr, col
    k = _key(rowptr, col, False) + (str(dev),)
    hit = _REPLICAS.get(k)
    if hit is None:
        hit = (rowptr, col, rowptr.to(dev), col.to(dev))  # the source tensors are held so their addresses stay theirs
        _REPLICAS[k] = hit
        while len(_REPLICAS) > 2 * _CACHE_SIZE:
            _REPLICAS.popitem(last=False)
    else:
        _REPLICAS.move_to_end(k)
    return hit[2], hit[3]


def _across_devices(call, rowptr, col, start, rand, L, devices, gather, return_edges, base, stride):
    """One host thread drives several GPUs: device ``g`` of ``G`` walks the contiguous block
    ``shard_range(n, G, g)`` of the start rows on a replica of the CSR (launches are asynchronous, so the
    devices run at the same time); draws are indexed by the global row, so the blocks are exactly the rows
    of the single-device result. ``gather=False`` returns the list of per-device blocks, ``gather=True``
    one matrix on ``start``'s device (device-to-device copies, each ordered after its block's kernel)."""
    from .sharding import shard_range
    devs = _devices(devices)
    n = start.numel()
    home = start.device
    blocks, edges = [], []
    full = torch.empty((n, L + 1), dtype=torch.int64, device=home) if gather else None
    full_e = torch.empty((n, L), dtype=torch.int64, device=home) if gather and return_edges else None
    for r, dev in enumerate(devs):
        b, e = shard_range(n, len(devs), r)
        rp, cl = _replica(rowptr, col, dev)
        s_blk = start[b:e].to(dev, non_blocking=True)
        r_blk = None if rand is None else rand.reshape(n, -1)[b:e].to(dev, non_blocking=True)
        # rank 0 of a gather on its own device writes its block in place
        out = full[b:e] if gather and dev == home else None
        res = call(rp, cl, s_blk, r_blk, base + b * stride, stride, out)
        blocks.append(res[0] if return_edges else res)
        if return_edges:
            edges.append(res[1])
    if not gather:
        return list(zip(blocks, edges)) if return_edges else blocks
    for r, dev in enumerate(devs):
        b, e = shard_range(n, len(devs), r)
        if blocks[r].data_ptr() != full[b:e].data_ptr():
            full[b:e].copy_(blocks[r], non_blocking=True)
        if return_edges:
            full_e[b:e].copy_(edges[r], non_blocking=True)
    return (full, full_e) if return_edges else full


def random_walk(rowptr, col, start, rand, walk_length, *, stream=None, return_edges: bool = False,
                check: bool = False, out: Optional[torch.Tensor] = None, graph: Optional[WalkGraph] = None,
                fused: bool = False, seed: int = 0, walk_index_base: int = 0, walk_index_stride: int = 1,
                validate: bool = False, devices=None, gather: bool = False):
    """Uniform CSR random walk (``random_walk`` of the reference, ``bindings.cpp:12-21``).

    Step ``l`` of walk ``w`` moves from ``v`` to ``col[rowptr[v] + int(rand[w, l] * deg(v))]``
    with the reference's float32 arithmetic (``random_walks/RandomWalk.cpp:45-54``); a node
    without out-edges keeps the walk in place. Returns int64 ``[n, walk_length + 1]``.

    Extra keyword-only options (not in the reference): ``return_edges`` also returns the
    edge ids ``[n, walk_length]`` the reference computes but never exposes; ``check``
    synchronises and raises if the kernel met malformed input; ``out`` supplies the output
    tensor; ``graph`` passes a prepared :class:`WalkGraph` instead of ``rowptr``/``col``;
    ``fused=True`` builds (once per graph, 16 bytes per edge) fused edge records that make a step
    one gather instead of two -- worth it when many calls walk the same graph. ``rand=None``
    (CUDA tensors only) lets the kernel generate the draws itself from a Philox stream keyed by
    ``seed`` and indexed by the global walk (``walk_index_base + row * walk_index_stride``);
    ``mlx_cluster_b200._lib.uniform_draws`` replays that stream on the host.
    ``validate=True`` first checks the CSR and the start nodes on the device (the reference checks
    nothing, ``random_walks/RandomWalk.cpp:33-38``) and raises ``ValueError`` on a malformed input.
    ``devices=[...]`` (CUDA tensors only) splits the start rows in contiguous blocks over these GPUs of
    this process, each walking a replica of the CSR, and returns the list of per-device blocks, or with
    ``gather=True`` the one matrix on ``start``'s device; one process per GPU goes through
    :func:`mlx_cluster_b200.sharded_walk` instead.
    """
    L = _check_walk_length(walk_length)
    if not isinstance(start, torch.Tensor) or not start.is_cuda:
        if devices is not None:
            raise ValueError("devices= needs CUDA tensors; host arrays walk on the resident graph's device")
        return _random_walk_host(rowptr, col, start, rand, L, return_edges, out, fused, validate)
    dev = start.device
    if devices is not None:
        if graph is not None or out is not None:
            raise ValueError("devices= builds its own per-device graphs and outputs: pass rowptr/col, not graph=/out=")
        rp = _require(rowptr, "rowptr", torch.int64, dev)
        cl = _require(col, "col", torch.int64, dev)
        if rand is not None and rand.numel() != start.numel() * L:
            raise ValueError(f"rand must hold n * walk_length = {start.numel() * L} values, has {rand.numel()}")

        def call(rp_d, cl_d, s_blk, r_blk, b, st, o):
            return random_walk(rp_d, cl_d, s_blk, r_blk, L, return_edges=return_edges, check=check, out=o, fused=fused,
                               seed=seed, walk_index_base=b, walk_index_stride=st, validate=validate)
        return _across_devices(call, rp, cl, start, rand, L, devices, gather, return_edges, int(walk_index_base),
                               int(walk_index_stride))
    g = graph if graph is not None else prepare_graph(_require(rowptr, "rowptr", torch.int64, dev),
                                                      _require(col, "col", torch.int64, dev), fused=fused)
    _require(start, "start", torch.int64, g.device)
    n = start.numel()
    if rand is not None:
        _require(rand, "rand", torch.float32, g.device)
        if rand.numel() != n * L:
            raise ValueError(f"rand must hold n * walk_length = {n * L} values, has {rand.numel()}")
    if validate:
        g.validate(start, check_sorted=False, stream=stream)
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty((n, L + 1), dtype=torch.int64, device=dev)
        else:
            _require(out, "out", torch.int64, dev)
            if out.numel() != n * (L + 1):
                raise ValueError("out has the wrong size")
        e_out = torch.empty((n, L), dtype=torch.int64, device=dev) if return_edges else None
        csr = g.csr()
        if rand is None:
            _lib.check(_lib.lib().walk_b200_uniform_walk_philox(
                C.byref(csr), _ptr(start), n, L, int(seed) & (2**64 - 1), int(walk_index_base),
                int(walk_index_stride), _ptr(out), _ptr(e_out), g.flags.data_ptr(), _stream_handle(stream, dev)))
        else:
            _lib.check(_lib.lib().walk_b200_uniform_walk(
                C.byref(csr), _ptr(start), _ptr(rand), n, L, _ptr(out), _ptr(e_out),
                g.flags.data_ptr(), _stream_handle(stream, dev)))
    return _finish(g, out, e_out, check, return_edges, stream)


def _membership_ready(g: WalkGraph, edgeset, stream, allow_auto: bool = True, q: float = 1.0) -> None:
    """Bring a graph into a state the node2vec kernels answer exactly on.

    ``edgeset=True`` builds the edge hash set now, ``False`` never does, ``"auto"`` (the default of
    :func:`rejection_sampling`) builds it on the graph's second node2vec call when the device has room:
    the set and the reverse positions that come with it triple the graph's memory and take about as long to
    build as one fast walk launch, which pays from the second launch on (the first call of a graph that is
    walked only once runs the binary-search kernel and allocates nothing). Without a hash set the membership
    test is a binary search over ``col``, which needs every row sorted; the reference's linear scan does not
    (``random_walks/BiasedRandomWalk.cpp:20-28``). So the rows are checked once per graph, and an unsorted
    CSR gets the hash set (exact for any CSR) regardless -- or, with ``edgeset=False``, is refused.
    A graph that keeps being walked (``_FILTER_AFTER_CALLS`` node2vec calls) with membership tests in play
    (``q > 1``) and that turns out to be undirected -- every edge has its reverse, read off the reverse positions
    in one pass -- also gets the triangle filter, if the device has room for 16 more bytes per edge."""
    if g.num_edges == 0:
        return
    if g.edgeset is not None:
        _maybe_filter(g, edgeset, stream, allow_auto, q)
        return
    if edgeset is True:
        g.build_edgeset(stream=stream)
        return
    if not g.check_rows_sorted(stream=stream):
        if edgeset is False:
            raise ValueError("a row of col is not sorted ascending: the binary-search membership test needs sorted "
                             "rows; pass edgeset=True (or leave the default) to use the edge hash set instead")
        g.build_edgeset(stream=stream)
        return
    if allow_auto and edgeset == "auto" and g.n2v_calls >= 1 and g.num_nodes < 2**32 - 1 and g.edgeset_fits():
        g.build_edgeset(stream=stream)


_FILTER_AFTER_CALLS = 16  # the filter takes about 20 launches' time to build and saves a fifth of every launch after


def _maybe_filter(g: WalkGraph, edgeset, stream, allow_auto: bool, q: float) -> None:
    if not (allow_auto and edgeset == "auto") or g.colrev16 is not None or g.colrev is None:
        return
    if g.n2v_calls < _FILTER_AFTER_CALLS or not q > 1.0 or g.filter_declined:
        return
    free, _ = torch.cuda.mem_get_info(g.device)
    cached = torch.cuda.memory_reserved(g.device) - torch.cuda.memory_allocated(g.device)
    if not g.symmetric:
        # undirected <=> no edge lacks its reverse (reverse position 0xffffffff in the upper half of colrev)
        with torch.cuda.device(g.device):
            _sync_stream(stream, g.device)
            undirected = True
            for c0 in range(0, g.num_edges, 1 << 26):  # in slices: the temporaries of one pass would double the graph
                part = g.colrev[c0:c0 + (1 << 26)]
                if bool(((part >> 32) & 0xffffffff).eq(0xffffffff).any().item()):
                    undirected = False
                    break
        if not undirected:
            g.filter_declined = True
            return
        g.symmetric = True
    if 16 * g.num_edges * 1.2 + (256 << 20) > free + cached:
        g.filter_declined = True
        return
    g.build_trifilter(stream=stream)


def rejection_sampling(rowptr, col, start, walk_length, p, q, *, stream=None, seed: int = 0,
                       walk_index_base: int = 0, walk_index_stride: int = 1, symmetric: bool = False,
                       edgeset="auto",
                       return_edges: bool = False,
                       return_counters: bool = False, check: bool = False,
                       out: Optional[torch.Tensor] = None, graph: Optional[WalkGraph] = None,
                       validate: bool = False, devices=None, gather: bool = False, trifilter: bool = False):
    """node2vec biased walk by rejection sampling (``rejection_sampling`` of the reference,
    ``bindings.cpp:35-45``; loop at ``random_walks/BiasedRandomWalk.cpp:52-99``).

    The reference draws from the C library's global ``rand()``; here the draws are a
    Philox4x32-10 stream keyed by ``seed`` and indexed by (global walk index, step,
    attempt), so a call is reproducible, re-entrant and independent of how walks are
    sharded (row ``i`` of this call is global walk ``walk_index_base + i * walk_index_stride``).
    ``symmetric=True`` asserts an undirected graph and lets the membership test search the previous
    node's row. ``edgeset`` chooses how "is the previous node a neighbour of the candidate" is answered:
    ``True`` builds (once per graph, 16 bytes per edge, plus 8 for the reverse positions) an exact edge
    hash set that answers with about one 32-byte read, for any CSR; ``False`` keeps the binary search
    over ``col`` (rows must be sorted: checked once per graph, an unsorted CSR raises); ``"auto"``
    (default) walks a graph's first call with the binary search and builds the hash set on its second
    call if the device has room (and, from its 17th call on, the triangle filter if the graph proves to be
    undirected and ``q > 1``), and always builds it for a CSR whose rows are not sorted (a prepared
    ``graph=`` is only checked for sorted rows and otherwise walked with the structures it has). None of
    this changes a result. ``trifilter=True`` (with ``symmetric=True``: undirected graphs only) also builds the
    triangle filter -- seconds per graph, after which a walk at p=0.25, q=4 gathers about half as much; for
    graphs that are walked many times. ``validate``, ``devices`` and ``gather`` as in :func:`random_walk`.
    Returns int64 ``[n, walk_length + 1]``.
    """
    L = _check_walk_length(walk_length)
    p, q = float(p), float(q)
    if edgeset not in (True, False, "auto"):
        raise ValueError("edgeset must be True, False or 'auto'")
    if not isinstance(start, torch.Tensor) or not start.is_cuda:
        if devices is not None:
            raise ValueError("devices= needs CUDA tensors; host arrays walk on the resident graph's device")
        return _rejection_sampling_host(rowptr, col, start, L, p, q, seed, walk_index_base, symmetric,
                                        return_edges, out, edgeset, walk_index_stride, validate, trifilter)
    dev = start.device
    if devices is not None:
        if graph is not None or out is not None or return_counters:
            raise ValueError("devices= builds its own per-device graphs and outputs: pass rowptr/col, "
                             "not graph=/out=/return_counters=")
        rp = _require(rowptr, "rowptr", torch.int64, dev)
        cl = _require(col, "col", torch.int64, dev)

        def call(rp_d, cl_d, s_blk, r_blk, b, st, o):
            return rejection_sampling(rp_d, cl_d, s_blk, L, p, q, seed=seed, walk_index_base=b, walk_index_stride=st,
                                      symmetric=symmetric, edgeset=edgeset, return_edges=return_edges, check=check,
                                      out=o, validate=validate, trifilter=trifilter)
        return _across_devices(call, rp, cl, start, None, L, devices, gather, return_edges, int(walk_index_base),
                               int(walk_index_stride))
    if trifilter and not symmetric and graph is None:
        raise ValueError("trifilter=True needs symmetric=True: the triangle filter is only valid on an undirected graph")
    g = graph if graph is not None else prepare_graph(_require(rowptr, "rowptr", torch.int64, dev),
                                                      _require(col, "col", torch.int64, dev),
                                                      symmetric=symmetric, trifilter=trifilter)
    _require(start, "start", torch.int64, g.device)
    n = start.numel()
    if validate:
        g.validate(start, check_sorted=False, stream=stream)
    # a graph the caller prepared keeps the structures it was given, except that unsorted rows get the hash set
    _membership_ready(g, edgeset, stream, allow_auto=graph is None, q=q)
    g.n2v_calls += 1
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty((n, L + 1), dtype=torch.int64, device=dev)
        else:
            _require(out, "out", torch.int64, dev)
            if out.numel() != n * (L + 1):
                raise ValueError("out has the wrong size")
        e_out = torch.empty((n, L), dtype=torch.int64, device=dev) if return_edges else None
        counters = torch.zeros(len(_lib.COUNTER_NAMES), dtype=torch.int64, device=dev) if return_counters else None
        if counters is not None:
            torch.cuda.current_stream(dev).synchronize()  # zeroed before a launch on another stream adds to them
        csr = g.csr()
        _lib.check(_lib.lib().walk_b200_node2vec_walk(
            C.byref(csr), _ptr(start), n, L, p, q, int(seed) & (2**64 - 1), int(walk_index_base),
            int(walk_index_stride), _ptr(out), _ptr(e_out), g.flags.data_ptr(), _ptr(counters), _stream_handle(stream, dev)))
    res = _finish(g, out, e_out, check, return_edges, stream)
    if return_counters:
        _sync_stream(stream, dev)
        cnt = dict(zip(_lib.COUNTER_NAMES, (int(x) for x in counters.tolist())))
        return (*res, cnt) if isinstance(res, tuple) else (res, cnt)
    return res


# ---- host-array path ---------------------------------------------------------------

def _host_out(n, L, out):
    if out is None:
        return torch.empty((n, L + 1), dtype=torch.int64, pin_memory=True)
    _require(out, "out", torch.int64)
    if out.is_cuda or out.numel() != n * (L + 1):
        raise ValueError("out must be a CPU int64 tensor of n * (walk_length + 1) elements")
    return out


def _random_walk_host(rowptr, col, start, rand, L, return_edges, out, fused=False, validate=False):
    rowptr, col = _as_cpu_tensor(rowptr), _as_cpu_tensor(col)
    start = _require(_as_cpu_tensor(start), "start", torch.int64)
    rand = _require(_as_cpu_tensor(rand), "rand", torch.float32)
    n = start.numel()
    if rand.numel() != n * L:
        raise ValueError(f"rand must hold n * walk_length = {n * L} values, has {rand.numel()}")
    g = _host_graph(rowptr, col, False, 2 if validate else 0, fused=fused)
    out = _host_out(n, L, out)
    e_out = torch.empty((n, L), dtype=torch.int64, pin_memory=True) if return_edges else None
    with torch.cuda.device(g.device):
        _lib.check(_lib.lib().walk_b200_uniform_walk_host(g._h, _ptr(start), _ptr(rand), n, L, _ptr(out), _ptr(e_out)))
    return (out, e_out) if return_edges else out


def _rejection_sampling_host(rowptr, col, start, L, p, q, seed, base, symmetric, return_edges, out, edgeset=False,
                             stride=1, validate=False, trifilter=False):
    rowptr, col = _as_cpu_tensor(rowptr), _as_cpu_tensor(col)
    start = _require(_as_cpu_tensor(start), "start", torch.int64)
    n = start.numel()
    if edgeset == "auto":
        # a resident graph is made to be walked again and again: build the hash set with the upload when the
        # graph (with it, about 5x the bytes of col) fits half the device, else keep the binary search
        free, _ = torch.cuda.mem_get_info()
        edgeset = col.numel() * 40 + rowptr.numel() * 16 < free // 2
    # without the hash set the membership test is a binary search: the upload then checks that rows are sorted
    # (validate mode 1) and refuses the graph otherwise; with it, rows may come in any order (mode 2)
    if trifilter and not symmetric:
        raise ValueError("trifilter=True needs symmetric=True: the triangle filter is only valid on an undirected graph")
    g = _host_graph(rowptr, col, symmetric, 1 if not edgeset else (2 if validate else 0), bool(edgeset),
                    trifilter=bool(trifilter and edgeset))
    out = _host_out(n, L, out)
    e_out = torch.empty((n, L), dtype=torch.int64, pin_memory=True) if return_edges else None
    with torch.cuda.device(g.device):
        _lib.check(_lib.lib().walk_b200_node2vec_walk_host(g._h, _ptr(start), n, L, p, q, int(seed) & (2**64 - 1),
                                                           int(base), int(stride), _ptr(out), _ptr(e_out)))
    return (out, e_out) if return_edges else out


def context_windows(walks: torch.Tensor, context_size: int, *, stream=None, out: Optional[torch.Tensor] = None):
    """All runs of ``context_size`` consecutive nodes of every walk: int64
    ``[n * (walk_length + 2 - context_size), context_size]``, column 0 the centre node and the rest
    its skip-gram context -- the input of node2vec's positive-pair loss. Same values as
    ``walks.unfold(1, context_size, 1).reshape(-1, context_size)``, produced by one streaming kernel."""
    _require(walks, "walks", torch.int64)
    if not walks.is_cuda or walks.dim() != 2:
        raise ValueError("walks must be a 2-D CUDA tensor [n, walk_length + 1]")
    n, row = walks.shape
    cs = int(context_size)
    if cs < 1 or cs > row:
        raise ValueError(f"context_size must be in [1, {row}]")
    rows_out = n * (row + 1 - cs)
    dev = walks.device
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty((rows_out, cs), dtype=torch.int64, device=dev)
        else:
            _require(out, "out", torch.int64, dev)
            if out.numel() != rows_out * cs:
                raise ValueError("out has the wrong size")
        _lib.check(_lib.lib().walk_b200_context_windows(_ptr(walks), n, row - 1, cs, _ptr(out), _stream_handle(stream, dev)))
    return out


def csr_from_edges(src: torch.Tensor, dst: torch.Tensor, num_nodes: int, *, symmetrize: bool = True,
                   drop_self_loops: bool = True, dedupe: bool = True, stream=None, check: bool = True):
    """Edge list -> ``(rowptr, col)`` on the device, rows sorted ascending, ``rowptr`` over all
    ``num_nodes`` nodes (isolated nodes keep their empty rows -- the host recipe of the reference's
    demos, ``tests/test_random_walk.py:22-28`` there, loses them).

    ``src``/``dst``: int64 CUDA tensors of equal length. ``symmetrize`` also inserts every edge
    reversed, ``dedupe`` keeps one copy of a repeated edge. With ``check`` an endpoint outside
    ``[0, num_nodes)`` raises; without it such edges are silently left out. The call synchronises
    once, to learn the number of edges and trim ``col``.
    """
    _require(src, "src", torch.int64)
    _require(dst, "dst", torch.int64, src.device if src.is_cuda else None)
    if not src.is_cuda or src.dim() != 1 or dst.shape != src.shape:
        raise ValueError("src and dst must be 1-D CUDA tensors of equal length")
    dev = src.device
    m, n = src.numel(), int(num_nodes)
    options = ((_lib.BUILD_SYMMETRIZE if symmetrize else 0) | (_lib.BUILD_DROP_SELF_LOOPS if drop_self_loops else 0) |
               (_lib.BUILD_DEDUPE if dedupe else 0))
    with torch.cuda.device(dev):
        need = C.c_uint64(0)
        _lib.check(_lib.lib().walk_b200_csr_build_scratch_bytes(m, n, options, C.byref(need)))
        scratch = torch.empty(max(int(need.value), 256), dtype=torch.uint8, device=dev)
        rowptr = torch.empty(n + 1, dtype=torch.int64, device=dev)
        col = torch.empty(max(1, m * (2 if symmetrize else 1)), dtype=torch.int64, device=dev)
        flags = torch.zeros(1, dtype=torch.int32, device=dev)
        src, dst = src.contiguous(), dst.contiguous()
        _lib.check(_lib.lib().walk_b200_csr_build(_ptr(src), _ptr(dst), m, n, options, _ptr(scratch), int(need.value),
                                                  _ptr(rowptr), _ptr(col), _ptr(flags), _stream_handle(stream, dev)))
        if isinstance(stream, torch.cuda.Stream):
            stream.synchronize()
        elif stream is not None:
            torch.cuda.synchronize(dev)
        nnz = int(rowptr[-1].item())
        if check and int(flags.item()) & _lib.FLAG_BAD_NODE:
            raise _lib.WalkError(_lib.ERR_DEVICE_FLAGS, "edge list holds a node id outside [0, num_nodes)")
    return rowptr, col[:nnz]


def negative_walks(start: torch.Tensor, walk_length: int, num_nodes: int, *, seed: int = 0, row_index_base: int = 0,
                   row_index_stride: int = 1, stream=None, out: Optional[torch.Tensor] = None):
    """Negative samples shaped like walks: int64 ``[n, walk_length + 1]`` with column 0 = ``start`` and
    the other columns node ids drawn uniformly from ``[0, num_nodes)`` (Philox4x32-10, key = ``seed``,
    indexed by global row and column, so shards of the rows reproduce the unsharded result). Feed it to
    :func:`context_windows` like a walk matrix to get the negative pairs of the skip-gram loss."""
    _require(start, "start", torch.int64)
    if not start.is_cuda or start.dim() != 1:
        raise ValueError("start must be a 1-D CUDA tensor")
    n, L = start.numel(), int(walk_length)
    dev = start.device
    with torch.cuda.device(dev):
        if out is None:
            out = torch.empty((n, L + 1), dtype=torch.int64, device=dev)
        else:
            _require(out, "out", torch.int64, dev)
            if out.numel() != n * (L + 1) or not out.is_contiguous():
                raise ValueError("out has the wrong size or is not contiguous")
        _lib.check(_lib.lib().walk_b200_negative_walks(_ptr(start.contiguous()), n, L, int(num_nodes), int(seed),
                                                       int(row_index_base), int(row_index_stride), _ptr(out),
                                                       _stream_handle(stream, dev)))
    return out
