"""ctypes binding of the C oracle (oracle/spdnn_oracle.c).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

_lib = None


def lib():
    global _lib
    if _lib is None:
        path = _build.build_oracle()
        _lib = C.CDLL(path)
        _lib.spdnn_oracle_infer.restype = C.c_int64
        _lib.spdnn_oracle_infer.argtypes = [
            C.c_int, C.c_int, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_float, C.c_float,
            C.c_float, C.c_int64, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int]
        _lib.spdnn_oracle_layer_raw.restype = None
        _lib.spdnn_oracle_layer_raw.argtypes = [
            C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_int64, C.c_void_p, C.c_void_p, C.c_int]
        _lib.spdnn_oracle_max_threads.restype = C.c_int
    return _lib


def max_threads() -> int:
    return int(lib().spdnn_oracle_max_threads())


def infer(y0: np.ndarray, layers, bias: float, clip: float = 32.0, first_image: int = 0, value: float = 0.0625,
          threads: int = 0, prune: bool = True, want_activations: bool = True):
    """``layers``: sequence of ``(rows int32[N,K] (-1 padding), vals float32[N,K] or None)``.
    Returns (categories int32[count], activations float32[count,N] or None, live int64[L])."""
    layers = list(layers)
    y0 = np.ascontiguousarray(y0, dtype=np.float32)
    batch, n = y0.shape
    k = layers[0][0].shape[1] if layers else 0
    rows = [np.ascontiguousarray(r, dtype=np.int32) for r, _ in layers]
    vals = [None if v is None else np.ascontiguousarray(v, dtype=np.float32) for _, v in layers]
    assert all(r.shape == (n, k) for r in rows)
    nl = len(layers)
    rp = (C.c_void_p * max(nl, 1))(*[r.ctypes.data for r in rows])
    vp = (C.c_void_p * max(nl, 1))(*[None if v is None else v.ctypes.data for v in vals])
    cats = np.empty(max(batch, 1), dtype=np.int32)
    act = np.empty((max(batch, 1), n), dtype=np.float32) if want_activations else None
    live = np.zeros(max(nl, 1), dtype=np.int64)
    cnt = lib().spdnn_oracle_infer(n, nl, k, rp, vp, value, bias, clip, batch, y0.ctypes.data, first_image,
                                   cats.ctypes.data, None if act is None else act.ctypes.data, live.ctypes.data,
                                   threads, 1 if prune else 0)
    if cnt < 0:
        raise MemoryError("oracle allocation failed")
    return cats[:cnt].copy(), (None if act is None else act[:cnt].copy()), live[:nl]


def layer_raw(y: np.ndarray, rows: np.ndarray, vals, value: float = 0.0625, threads: int = 0) -> np.ndarray:
    y = np.ascontiguousarray(y, dtype=np.float32)
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    n, k = rows.shape
    v = None if vals is None else np.ascontiguousarray(vals, dtype=np.float32)
    out = np.empty_like(y)
    lib().spdnn_oracle_layer_raw(n, k, rows.ctypes.data, None if v is None else v.ctypes.data, value, y.shape[0],
                                 y.ctypes.data, out.ctypes.data, threads)
    return out
