"""Writes a case file for oracle/ref_harness.cpp: a small network, its inputs and the
oracle's per-layer raw products and activations (unpruned, as the reference's CPU checkers
compute them).  TEST INFRASTRUCTURE ONLY."""
from __future__ import annotations

import struct

import numpy as np

from . import spdnn_oracle as npo


def write_case(path: str, y0: np.ndarray, layer_rows, bias: float, value: float = 0.0625, vals=None,
               tsv_dir: str | None = None) -> dict:
    """``layer_rows``: list of int32 [N, K] (ascending per column).  Returns the arrays that
    were written so a caller can reuse them."""
    y0 = np.ascontiguousarray(y0, dtype=np.float32)
    batch, n = y0.shape
    acts, raws = [], []
    y = y0
    with open(path, "wb") as f:
        f.write(b"SPDNNC01")
        f.write(struct.pack("<iiif", n, batch, len(layer_rows), float(bias)))
        f.write(y0.tobytes())
        for l, rows in enumerate(layer_rows):
            v = None if vals is None else vals[l]
            raw = npo.layer_raw(y, rows, v, value)
            act = npo.relu_clip(raw + np.float32(bias))
            k = rows.shape[1]
            b = np.repeat(np.arange(1, n + 1, dtype=np.int32), k)
            a = (rows.reshape(-1) + 1).astype(np.int32)
            vv = np.full(a.size, value, dtype=np.float32) if v is None else v.reshape(-1).astype(np.float32)
            keep = a > 0
            a, b, vv = a[keep], b[keep], vv[keep]
            # the reference reads triplets in any order; shuffle to prove order independence
            perm = np.random.default_rng(1234 + l).permutation(a.size)
            a, b, vv = a[perm], b[perm], vv[perm]
            f.write(struct.pack("<i", a.size))
            f.write(a.tobytes()); f.write(b.tobytes()); f.write(vv.tobytes())
            f.write(raw.astype(np.float32).tobytes()); f.write(act.astype(np.float32).tobytes())
            if tsv_dir is not None:
                with open(f"{tsv_dir}/n{n}-l{l + 1}.tsv", "w") as t:
                    for x, yy, z in zip(a.tolist(), b.tolist(), vv.tolist()):
                        t.write(f"{x}\t{yy}\t{z!r}\n")
            raws.append(raw); acts.append(act)
            y = act
    return {"raw": raws, "act": acts}
