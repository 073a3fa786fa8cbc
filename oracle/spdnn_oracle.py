"""CPU oracle (numpy) for the sparse-DNN inference loop.  TEST INFRASTRUCTURE
ONLY: the product never imports this file; tests, the smoke check and the
benchmark's CPU-baseline leg use it as the checker.

It restates the reference's arithmetic for the loop
``Y <- min(32, ReLU(Y W + b))``:

* one layer's raw product follows ``CpuSpmm::run_and_cmp``
  (src/utils/cpu_spmm.h:11-43): for every image, ``res[out] += in * val`` over
  the COO sorted by (output, input) (sort at src/utils/matrix.h:245-253), i.e.
  each output accumulates its terms in ASCENDING INPUT-NEURON order, starting
  from 0.0f, in fp32, product rounded before the add;
* the epilogue is ``__ReLU(acc + bias)`` with
  ``x<0 ? 0 : x>32 ? 32 : x`` (src/microbenchmark/all_network.cu:8-10, 57, 108, 147);
* an image survives a layer when any of its activations is non-zero
  (all_network.cu:57-59, 455-463); dead images are dropped from the work list;
* the category list is the ascending list of original image numbers alive
  after the last layer (the reference only prints their count, all_network.cu:508).

Parity status: pinned against the reference's own ``CpuSpmm`` /
``CpuSpmmFuse`` code compiled from its sources (oracle/build.py, ``_ref/ref_harness``);
the reference holds no golden vectors and the challenge's truth-category files
are not available, so parity against the official data set is unpinned.
"""
from __future__ import annotations

import numpy as np


def layer_raw(y: np.ndarray, rows: np.ndarray, vals: np.ndarray | None, value: float = 0.0625) -> np.ndarray:
    """Raw ``Y W`` for one layer.  ``y`` float32 [B, N]; ``rows`` int32 [N, K]
    (ascending per column, entries < 0 are padding); ``vals`` float32 [N, K] or
    None for the constant ``value``."""
    y = np.ascontiguousarray(y, dtype=np.float32)
    b, n = y.shape
    k = rows.shape[1]
    acc = np.zeros((b, rows.shape[0]), dtype=np.float32)
    for j in range(k):
        r = rows[:, j]
        valid = r >= 0
        w = np.float32(value) if vals is None else vals[:, j].astype(np.float32)
        term = y[:, np.where(valid, r, 0)] * w          # fp32 product, rounded
        if not valid.all():
            term = np.where(valid[None, :], term, np.float32(0.0))
        acc = acc + term                                  # fp32 add, rounded
    return acc


def relu_clip(x: np.ndarray, clip: float = 32.0) -> np.ndarray:
    x = np.asarray(x, dtype=np.float32)
    return np.where(x < 0, np.float32(0), np.where(x > np.float32(clip), np.float32(clip), x)).astype(np.float32)


def infer(y0: np.ndarray, layers, bias: float, clip: float = 32.0, first_image: int = 0,
          keep_layers: bool = False):
    """Run all layers.  ``layers`` is an iterable of ``(rows, vals_or_None)``.

    Returns ``(categories int32[], activations float32[count, N], live int64[L])``
    (and the per-layer activations of the live images when ``keep_layers``).
    Categories are ascending global image numbers (``first_image`` + index)."""
    y = np.ascontiguousarray(y0, dtype=np.float32)
    ids = np.arange(first_image, first_image + y.shape[0], dtype=np.int64)
    live = []
    kept = []
    bias32 = np.float32(bias)
    for rows, vals in layers:
        if y.shape[0]:
            out = np.empty((y.shape[0], rows.shape[0]), dtype=np.float32)
            step = max(1, (1 << 22) // max(rows.shape[0], 1))
            for s in range(0, y.shape[0], step):
                out[s:s + step] = relu_clip(layer_raw(y[s:s + step], rows, vals) + bias32, clip)
            alive = (out != 0).any(axis=1)
            y = out[alive]
            ids = ids[alive]
        else:
            y = np.zeros((0, rows.shape[0]), dtype=np.float32)
        live.append(y.shape[0])
        if keep_layers:
            kept.append((ids.copy(), y.copy()))
    res = (ids.astype(np.int32), y, np.asarray(live, dtype=np.int64))
    return res + (kept,) if keep_layers else res


def csc_to_rows(col_ptr: np.ndarray, row_idx: np.ndarray, val: np.ndarray | None):
    """General CSC -> padded per-column lists sorted by ascending row
    (rows int32 [N, K] with -1 padding, vals float32 [N, K] or None)."""
    n = len(col_ptr) - 1
    cnt = np.diff(col_ptr)
    k = int(cnt.max()) if n else 0
    rows = np.full((n, k), -1, dtype=np.int32)
    vals = None if val is None else np.zeros((n, k), dtype=np.float32)
    for c in range(n):
        s, e = col_ptr[c], col_ptr[c + 1]
        order = np.argsort(row_idx[s:e], kind="stable")
        rows[c, : e - s] = row_idx[s:e][order]
        if vals is not None:
            vals[c, : e - s] = val[s:e][order]
    return rows, vals
