"""ctypes front end to the parity checkers. TEST INFRASTRUCTURE ONLY.

Only the test suite, the smoke check and the bench's CPU-baseline legs may import
this package. The product package never does: it has no CPU path.

``uniform_walk`` / ``node2vec_walk`` call the C restatement (``walk_oracle.c``);
``ref_random_walk`` / ``ref_rejection_sampling`` call the reference's own
``eval_cpu`` loops when the compiled reference library is available
(``have_ref()``).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import numpy as np

from . import build as _build

_HERE = Path(__file__).resolve().parent
_I64P = np.ctypeslib.ndpointer(dtype=np.int64, flags="C_CONTIGUOUS")
_F32P = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")

_oracle = None
_ref = None

COUNTER_NAMES = (
    "attempts", "membership_ref", "membership_needed", "scan_elems", "bsearch_probes",
    "steps_deg0", "steps_deg1", "steps_sampled", "steps_first", "steps_capped",
)


def _opt(arr):
    return None if arr is None else arr.ctypes.data_as(C.c_void_p)


def _load_oracle():
    global _oracle
    if _oracle is None:
        so = _build.ORACLE_SO
        if not so.exists() or _build._stale(so, [_HERE / "walk_oracle.c"]):
            _build.build_oracle()
        lib = C.CDLL(str(so))
        lib.oracle_philox4x32_10.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
        lib.oracle_uniform_walk.argtypes = [_I64P, _I64P, _I64P, _F32P, C.c_int64, C.c_int,
                                            _I64P, C.c_void_p]
        lib.oracle_node2vec_thresholds.argtypes = [C.c_double, C.c_double, C.c_void_p]
        lib.oracle_accept_cut.argtypes = [C.c_double]
        lib.oracle_accept_cut.restype = C.c_uint32
        lib.oracle_counter_count.restype = C.c_int
        lib.oracle_node2vec_walk.argtypes = [_I64P, _I64P, _I64P, C.c_int64, C.c_int, C.c_double,
                                             C.c_double, C.c_int, C.c_uint64, C.c_uint64, C.c_uint64,
                                             _I64P, C.c_void_p, C.c_void_p, C.c_uint32]
        assert lib.oracle_counter_count() == len(COUNTER_NAMES)
        _oracle = lib
    return _oracle


def _load_ref():
    global _ref
    if _ref is None:
        so = _build.build_ref()
        if so is None or not Path(so).exists():
            return None
        lib = C.CDLL(str(so))
        lib.ref_random_walk.restype = C.c_double
        lib.ref_random_walk.argtypes = [_I64P, C.c_int64, _I64P, C.c_int64, _I64P, C.c_int64, _F32P,
                                        C.c_int, C.c_void_p, C.c_void_p]
        lib.ref_rejection_sampling.restype = C.c_double
        lib.ref_rejection_sampling.argtypes = [_I64P, C.c_int64, _I64P, C.c_int64, _I64P, C.c_int64,
                                               C.c_int, C.c_double, C.c_double, C.c_uint,
                                               C.c_void_p, C.c_void_p]
        lib.ref_factory_shapes.argtypes = [C.c_int64, C.c_int, C.c_int, C.c_void_p]
        lib.ref_rand_max.restype = C.c_int
        _ref = lib
    return _ref


def have_ref() -> bool:
    return _load_ref() is not None


def _i64(a):
    return np.ascontiguousarray(a, dtype=np.int64)


# --------------------------------------------------------------------------- restatement

def philox4x32_10(counter, key):
    """One Philox4x32-10 block: 4 counter words, 2 key words -> 4 output words."""
    lib = _load_oracle()
    c = np.asarray(counter, dtype=np.uint32).copy()
    k = np.asarray(key, dtype=np.uint32).copy()
    o = np.zeros(4, dtype=np.uint32)
    lib.oracle_philox4x32_10(c.ctypes.data, k.ctypes.data, o.ctypes.data)
    return o


def thresholds(p: float, q: float):
    lib = _load_oracle()
    o = np.zeros(3, dtype=np.float64)
    lib.oracle_node2vec_thresholds(p, q, o.ctypes.data)
    return o


def accept_cut(prob: float) -> int:
    return int(_load_oracle().oracle_accept_cut(prob))


def uniform_walk(rowptr, col, start, rand, walk_length: int, return_edges: bool = False):
    lib = _load_oracle()
    rowptr, col, start = _i64(rowptr), _i64(col), _i64(start)
    n = start.shape[0]
    rand = np.ascontiguousarray(rand, dtype=np.float32).reshape(n, walk_length) if walk_length else \
        np.zeros((n, 0), dtype=np.float32)
    n_out = np.empty((n, walk_length + 1), dtype=np.int64)
    e_out = np.empty((n, walk_length), dtype=np.int64) if return_edges else None
    if col.size == 0:
        col = np.zeros(1, dtype=np.int64)
    if rand.size == 0:
        rand = np.zeros(1, dtype=np.float32)
    lib.oracle_uniform_walk(rowptr, col, start if n else np.zeros(1, np.int64), rand, n, walk_length,
                            n_out if n_out.size else np.zeros(1, np.int64), _opt(e_out))
    return (n_out, e_out) if return_edges else n_out


def node2vec_walk(rowptr, col, start, walk_length: int, p: float, q: float, *, seed: int = 0,
                  walk_index_base: int = 0, walk_index_stride: int = 1, draw_mode: int = 1,
                  return_edges: bool = False,
                  return_counters: bool = False, max_attempts: int = 0):
    """draw_mode 1: Philox stream (key=seed, counter=(walk, step, attempt));
    draw_mode 0: libc rand() in the reference's call order (seed it with ``srand``).
    ``max_attempts`` 0 is the reference's unbounded rejection loop; a positive value makes a step
    stand still (edge id -1) once that many candidates were rejected, as the CUDA path does."""
    lib = _load_oracle()
    rowptr, col, start = _i64(rowptr), _i64(col), _i64(start)
    n = start.shape[0]
    n_out = np.empty((n, walk_length + 1), dtype=np.int64)
    e_out = np.empty((n, walk_length), dtype=np.int64) if return_edges else None
    cnt = np.zeros(len(COUNTER_NAMES), dtype=np.int64)
    if col.size == 0:
        col = np.zeros(1, dtype=np.int64)
    lib.oracle_node2vec_walk(rowptr, col, start if n else np.zeros(1, np.int64), n, walk_length,
                             p, q, draw_mode, seed, walk_index_base, walk_index_stride,
                             n_out if n_out.size else np.zeros(1, np.int64), _opt(e_out), cnt.ctypes.data,
                             int(max_attempts))
    res = [n_out]
    if return_edges:
        res.append(e_out)
    if return_counters:
        res.append(dict(zip(COUNTER_NAMES, (int(x) for x in cnt))))
    return res[0] if len(res) == 1 else tuple(res)


def libc_srand(seed: int) -> None:
    C.CDLL(None).srand(C.c_uint(seed))


# --------------------------------------------------------------------------- compiled reference

def ref_random_walk(rowptr, col, start, rand, walk_length: int, return_edges=False, return_seconds=False):
    lib = _load_ref()
    if lib is None:
        raise RuntimeError("compiled reference library not available")
    rowptr, col, start = _i64(rowptr), _i64(col), _i64(start)
    n = start.shape[0]
    rand = np.ascontiguousarray(rand, dtype=np.float32)
    n_out = np.empty((n, walk_length + 1), dtype=np.int64)
    e_out = np.empty((n, walk_length), dtype=np.int64) if return_edges else None
    secs = lib.ref_random_walk(rowptr, rowptr.size, col if col.size else np.zeros(1, np.int64), col.size,
                               start if n else np.zeros(1, np.int64), n,
                               rand.reshape(-1) if rand.size else np.zeros(1, np.float32),
                               walk_length, _opt(n_out), _opt(e_out))
    res = [n_out]
    if return_edges:
        res.append(e_out)
    if return_seconds:
        res.append(secs)
    return res[0] if len(res) == 1 else tuple(res)


def ref_rejection_sampling(rowptr, col, start, walk_length: int, p: float, q: float, *,
                           srand_seed: int = 1, return_edges=False, return_seconds=False):
    lib = _load_ref()
    if lib is None:
        raise RuntimeError("compiled reference library not available")
    if walk_length < 1:
        raise ValueError("the reference's biased walk needs walk_length >= 1")
    rowptr, col, start = _i64(rowptr), _i64(col), _i64(start)
    n = start.shape[0]
    n_out = np.empty((n, walk_length + 1), dtype=np.int64)
    e_out = np.empty((n, walk_length), dtype=np.int64) if return_edges else None
    secs = lib.ref_rejection_sampling(rowptr, rowptr.size, col if col.size else np.zeros(1, np.int64),
                                      col.size, start if n else np.zeros(1, np.int64), n, walk_length,
                                      p, q, srand_seed, _opt(n_out), _opt(e_out))
    res = [n_out]
    if return_edges:
        res.append(e_out)
    if return_seconds:
        res.append(secs)
    return res[0] if len(res) == 1 else tuple(res)


def ref_factory_shapes(n: int, walk_length: int, which: int):
    lib = _load_ref()
    o = np.zeros(4, dtype=np.int32)
    lib.ref_factory_shapes(n, walk_length, which, o.ctypes.data)
    return tuple(int(x) for x in o)


def ref_rand_max() -> int:
    return int(_load_ref().ref_rand_max())
