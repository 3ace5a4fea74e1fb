"""ctypes binding of ``libwalk_b200.so`` -- the only route from Python to the kernels.

There is deliberately no fallback: if the library is missing or a call fails, the
caller gets an exception.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libwalk_b200.so"

OK = 0
ERR_INVALID_ARG, ERR_BAD_PQ, ERR_CUDA, ERR_CSR_INVALID, ERR_UNSUPPORTED, ERR_DEVICE_FLAGS = 1, 2, 3, 4, 5, 6
FLAG_BAD_NODE, FLAG_BAD_EDGE, FLAG_ATTEMPT_CAP, FLAG_BAD_ROWPTR = 0x1, 0x2, 0x4, 0x8
FLAG_DESC_OVERFLOW, FLAG_UNSORTED_ROW, FLAG_EDGESET_FULL = 0x10, 0x20, 0x80
CSR_SYMMETRIC, CSR_WANT_EDGESET, CSR_WANT_FUSED, CSR_WANT_TRIFILTER = 0x1, 0x2, 0x4, 0x8
COUNTER_NAMES = ("loads", "attempts", "membership", "probes",
                 "steps_deg0", "steps_deg1", "steps_sampled", "steps_first", "formula_probes", "gathers16", "filtered")

# every symbol include/walk_b200.h declares
EXPORTS = (
    "walk_b200_abi_version", "walk_b200_last_error", "walk_b200_launch_count", "walk_b200_last_kernel",
    "walk_b200_uniform_walk", "walk_b200_uniform_walk_philox", "walk_b200_uniform_draw",
    "walk_b200_uniform_draws", "walk_b200_node2vec_walk", "walk_b200_rowdesc_pack",
    "walk_b200_csr_validate", "walk_b200_edgeset_buckets", "walk_b200_edgeset_build", "walk_b200_revpos_build", "walk_b200_colrev_build", "walk_b200_trifilter_build", "walk_b200_fused_build", "walk_b200_philox4x32_10", "walk_b200_node2vec_draw",
    "walk_b200_node2vec_thresholds", "walk_b200_shard_range", "walk_b200_shard_count_cyclic",
    "walk_b200_graph_create", "walk_b200_graph_destroy", "walk_b200_graph_csr",
    "walk_b200_graph_device_bytes", "walk_b200_uniform_walk_host", "walk_b200_node2vec_walk_host",
    "walk_b200_graph_host_transport", "walk_b200_host_widen_probe",
    "walk_b200_l2_window_set", "walk_b200_l2_window_clear",
    "walk_b200_set_tuning", "walk_b200_get_tuning",
    "walk_b200_uniform_walk_noalloc", "walk_b200_gather_probe", "walk_b200_gather_probe_ex", "walk_b200_context_windows",
    "walk_b200_csr_build_scratch_bytes", "walk_b200_csr_build",
    "walk_b200_negative_walks", "walk_b200_negative_draw",
)
BUILD_SYMMETRIZE, BUILD_DROP_SELF_LOOPS, BUILD_DEDUPE = 0x1, 0x2, 0x4
NOALLOC_MAX_NODES = 1 << 20


class Csr(C.Structure):
    _fields_ = [("rowptr", C.c_void_p), ("col", C.c_void_p), ("num_nodes", C.c_int64),
                ("num_edges", C.c_int64), ("rowdesc", C.c_void_p), ("flags", C.c_uint32),
                ("reserved", C.c_uint32), ("edgeset", C.c_void_p), ("edgeset_buckets", C.c_uint64),
                ("revpos", C.c_void_p), ("fused", C.c_void_p), ("colrev", C.c_void_p), ("colrev16", C.c_void_p)]


class WalkError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"walk_b200 error {code}: {message}")
        self.code = code


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m mlx_cluster_b200.build` "
            "(needs nvcc). This package has no CPU implementation.")
    L = C.CDLL(str(LIB_PATH))
    vp, i64, i32, u64, u32, dbl = C.c_void_p, C.c_int64, C.c_int32, C.c_uint64, C.c_uint32, C.c_double
    L.walk_b200_abi_version.restype = C.c_int
    L.walk_b200_last_error.restype = C.c_char_p
    L.walk_b200_launch_count.restype = u64
    L.walk_b200_last_kernel.restype = C.c_char_p
    L.walk_b200_uniform_walk.argtypes = [C.POINTER(Csr), vp, vp, i64, i32, vp, vp, vp, vp]
    L.walk_b200_uniform_walk_philox.argtypes = [C.POINTER(Csr), vp, i64, i32, u64, u64, u64, vp, vp, vp, vp]
    L.walk_b200_uniform_draw.argtypes = [u64, u64, u32, C.POINTER(C.c_float)]
    L.walk_b200_uniform_draw.restype = None
    L.walk_b200_uniform_draws.argtypes = [u64, u64, u64, i64, i32, vp]
    L.walk_b200_uniform_draws.restype = None
    L.walk_b200_node2vec_walk.argtypes = [C.POINTER(Csr), vp, i64, i32, dbl, dbl, u64, u64, u64, vp, vp, vp, vp, vp]
    L.walk_b200_rowdesc_pack.argtypes = [vp, i64, i64, vp, vp, vp]
    L.walk_b200_csr_validate.argtypes = [C.POINTER(Csr), vp, i64, i32, vp, vp]
    L.walk_b200_edgeset_buckets.argtypes = [i64, C.POINTER(u64)]
    L.walk_b200_edgeset_build.argtypes = [C.POINTER(Csr), vp, u64, vp, vp]
    L.walk_b200_revpos_build.argtypes = [C.POINTER(Csr), vp, vp, vp]
    L.walk_b200_colrev_build.argtypes = [C.POINTER(Csr), vp, vp, vp]
    L.walk_b200_trifilter_build.argtypes = [C.POINTER(Csr), vp, i64, vp, vp]
    L.walk_b200_fused_build.argtypes = [C.POINTER(Csr), vp, vp, vp]
    L.walk_b200_philox4x32_10.argtypes = [vp, vp, vp]
    L.walk_b200_philox4x32_10.restype = None
    L.walk_b200_node2vec_draw.argtypes = [u64, u64, u32, u32, C.POINTER(u32), C.POINTER(u32)]
    L.walk_b200_node2vec_draw.restype = None
    L.walk_b200_node2vec_thresholds.argtypes = [dbl, dbl, C.POINTER(dbl * 3), C.POINTER(u32 * 3)]
    L.walk_b200_shard_range.argtypes = [i64, i32, i32, C.POINTER(i64), C.POINTER(i64)]
    L.walk_b200_shard_count_cyclic.argtypes = [i64, i32, i32, C.POINTER(i64)]
    L.walk_b200_graph_create.argtypes = [vp, vp, i64, i64, u32, i32, C.POINTER(vp)]
    L.walk_b200_graph_destroy.argtypes = [vp]
    L.walk_b200_graph_csr.argtypes = [vp, C.POINTER(Csr)]
    L.walk_b200_graph_device_bytes.argtypes = [vp, C.POINTER(i64)]
    L.walk_b200_uniform_walk_host.argtypes = [vp, vp, vp, i64, i32, vp, vp]
    L.walk_b200_node2vec_walk_host.argtypes = [vp, vp, i64, i32, dbl, dbl, u64, u64, u64, vp, vp]
    L.walk_b200_graph_host_transport.argtypes = [vp, C.POINTER(i32), C.POINTER(dbl), C.POINTER(dbl)]
    L.walk_b200_host_widen_probe.argtypes = [C.c_size_t, C.POINTER(dbl)]
    L.walk_b200_l2_window_set.argtypes = [vp, C.c_size_t, C.c_float, vp, C.POINTER(C.c_size_t)]
    L.walk_b200_l2_window_clear.argtypes = [vp]
    L.walk_b200_uniform_walk_noalloc.argtypes = [vp, vp, i64, i64, vp, vp, i64, i32, vp, vp, vp, vp]
    L.walk_b200_context_windows.argtypes = [vp, i64, i32, i32, vp, vp]
    L.walk_b200_negative_walks.argtypes = [vp, i64, i32, i64, C.c_uint64, C.c_uint64, C.c_uint64, vp, vp]
    L.walk_b200_negative_draw.argtypes = [C.c_uint64, C.c_uint64, C.c_uint32, i64, C.POINTER(i64)]
    L.walk_b200_csr_build_scratch_bytes.argtypes = [i64, i64, C.c_uint32, C.POINTER(C.c_uint64)]
    L.walk_b200_csr_build.argtypes = [vp, vp, i64, i64, C.c_uint32, vp, C.c_uint64, vp, vp, vp, vp]
    L.walk_b200_gather_probe.argtypes = [C.c_size_t, i32, C.POINTER(dbl)]
    L.walk_b200_gather_probe_ex.argtypes = [C.c_size_t, i32, i32, i32, i32, i32, C.POINTER(dbl)]
    L.walk_b200_set_tuning.argtypes = [C.c_char_p, i32]
    L.walk_b200_get_tuning.argtypes = [C.c_char_p, C.POINTER(i32)]
    for name in EXPORTS:  # AttributeError here = the built library is older than the header
        getattr(L, name)
    _lib = L
    return L


def check(rc: int) -> None:
    if rc != OK:
        raise WalkError(rc, lib().walk_b200_last_error().decode("utf-8", "replace"))


def launch_count() -> int:
    return int(lib().walk_b200_launch_count())


def last_kernel() -> str:
    """Name of the kernel this thread launched last through the library."""
    return lib().walk_b200_last_kernel().decode()


def set_tuning(key: str, value: int) -> None:
    check(lib().walk_b200_set_tuning(key.encode(), int(value)))


def get_tuning(key: str) -> int:
    v = C.c_int32(0)
    check(lib().walk_b200_get_tuning(key.encode(), C.byref(v)))
    return int(v.value)


def philox4x32_10(counter, key):
    import numpy as np
    c = np.asarray(counter, dtype=np.uint32).copy()
    k = np.asarray(key, dtype=np.uint32).copy()
    o = np.zeros(4, dtype=np.uint32)
    lib().walk_b200_philox4x32_10(c.ctypes.data, k.ctypes.data, o.ctypes.data)
    return o


def node2vec_draw(seed: int, walk: int, step: int, attempt: int):
    c, a = C.c_uint32(0), C.c_uint32(0)
    lib().walk_b200_node2vec_draw(seed, walk, step, attempt, C.byref(c), C.byref(a))
    return int(c.value), int(a.value)


def uniform_draws(seed: int, num_walks: int, walk_length: int, walk_index_base: int = 0, walk_index_stride: int = 1):
    """The float32 [num_walks, walk_length] draws the kernel generates for these walks (host replay)."""
    import numpy as np
    out = np.empty((num_walks, walk_length), dtype=np.float32)
    lib().walk_b200_uniform_draws(seed, walk_index_base, walk_index_stride, num_walks, walk_length, out.ctypes.data)
    return out


def node2vec_thresholds(p: float, q: float):
    prob = (C.c_double * 3)()
    cuts = (C.c_uint32 * 3)()
    check(lib().walk_b200_node2vec_thresholds(p, q, C.byref(prob), C.byref(cuts)))
    return tuple(prob), tuple(cuts)


def gather_probe(array_bytes: int = 2 << 30, iters: int = 32, *, chains: int = 1, gather_bytes: int = 8,
                 fetch_bytes: int = 64, threads_per_sm: int = 0) -> float:
    """Dependent random gathers per second this device sustains out of DRAM (``chains`` of them in
    flight per thread, ``gather_bytes`` each, the L2 fetching ``fetch_bytes`` per miss)."""
    r = C.c_double(0.0)
    check(lib().walk_b200_gather_probe_ex(array_bytes, iters, chains, gather_bytes, fetch_bytes, threads_per_sm,
                                          C.byref(r)))
    return float(r.value)


def host_transport(graph_handle) -> int:
    """1 if the host entry points move this graph's walk matrices as int32 (widened on the host), 0 if as int64."""
    n = C.c_int32(0)
    check(lib().walk_b200_graph_host_transport(graph_handle, C.byref(n), None, None))
    return int(n.value)


def host_transport_rates(graph_handle):
    """(pinned device-to-host GB/s, widening threads' int64 output GB/s) measured when the graph was created."""
    d, w = C.c_double(0.0), C.c_double(0.0)
    check(lib().walk_b200_graph_host_transport(graph_handle, None, C.byref(d), C.byref(w)))
    return float(d.value), float(w.value)


def host_widen_probe(out_bytes: int = 256 << 20) -> float:
    r = C.c_double(0.0)
    check(lib().walk_b200_host_widen_probe(out_bytes, C.byref(r)))
    return float(r.value)


def shard_count_cyclic(num_walks: int, world_size: int, rank: int) -> int:
    c = C.c_int64(0)
    check(lib().walk_b200_shard_count_cyclic(num_walks, world_size, rank, C.byref(c)))
    return int(c.value)


def edgeset_buckets(num_edges: int) -> int:
    b = C.c_uint64(0)
    check(lib().walk_b200_edgeset_buckets(num_edges, C.byref(b)))
    return int(b.value)


def shard_range(num_walks: int, world_size: int, rank: int):
    b, e = C.c_int64(0), C.c_int64(0)
    check(lib().walk_b200_shard_range(num_walks, world_size, rank, C.byref(b), C.byref(e)))
    return int(b.value), int(e.value)


def negative_draw(seed: int, row: int, k: int, num_nodes: int) -> int:
    """Host replay of draw ``k`` of global row ``row`` of ``walk_b200_negative_walks``."""
    v = C.c_int64(0)
    check(lib().walk_b200_negative_draw(seed, row, k, num_nodes, C.byref(v)))
    return int(v.value)
