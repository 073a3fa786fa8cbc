"""Runs the reference's own GPU inference loop (src/microbenchmark/snig.cu, built as
oracle/_ref/ref_snig by oracle/build.py) on a generated network and parses what it prints.
TEST INFRASTRUCTURE ONLY: the tests use the per-layer survivor counts as a second pin of the
oracle, the benchmark reports its kernel time beside this repository's."""
from __future__ import annotations

import os
import re
import struct
import subprocess
import tempfile

import numpy as np

from . import build as _build


def available() -> str | None:
    """Path of the built harness, or None (the reference tree and nvcc are needed to build it)."""
    return _build.build_ref_snig()


def write_case(path: str, net, layers: int, y0: np.ndarray) -> None:
    """``net``: generator network (layer_rows, pattern_id, bias); ``y0``: binary [batch, N]."""
    n = net.neurons
    pid_of, distinct = [], {}
    for l in range(layers):
        pid = net.pattern_id(l)
        if pid not in distinct:
            distinct[pid] = (len(distinct), np.ascontiguousarray(net.layer_rows(l), dtype=np.int32))
        pid_of.append(distinct[pid][0])
    k = next(iter(distinct.values()))[1].shape[1]
    with open(path, "wb") as f:
        f.write(b"SPDNNS01")
        f.write(struct.pack("<iiiiif", n, y0.shape[0], layers, k, len(distinct), float(net.bias)))
        f.write(np.asarray(pid_of, dtype=np.int32).tobytes())
        for _, rows in sorted(distinct.values(), key=lambda t: t[0]):
            f.write(rows.tobytes())
        f.write(np.packbits(np.asarray(y0) != 0, axis=1, bitorder="little").tobytes())


def run(net, layers: int, y0: np.ndarray, timeout: float = 600.0) -> dict:
    """Returns {"live": per-layer survivor counts, "kernel_ms": total, "layer_ms": [...], "sec_size": s}."""
    exe = available()
    if exe is None:
        raise RuntimeError("oracle/_ref/ref_snig is not built")
    with tempfile.TemporaryDirectory(prefix="spdnn_snig_") as d:
        case = os.path.join(d, "case.bin")
        write_case(case, net, layers, y0)
        r = subprocess.run([exe, case, d], capture_output=True, text=True, timeout=timeout)
    if r.returncode != 0:
        raise RuntimeError(f"ref_snig failed ({r.returncode}): {r.stderr[-400:]}")
    live, ms = [], []
    for m in re.finditer(r"layer = (\d+), batch = (\d+), time = ([0-9.eE+-]+)", r.stdout):
        live.append(int(m.group(2)))
        ms.append(float(m.group(3)))
    total = re.search(r"Kernel Exec Time \[SNIG\] = ([0-9.eE+-]+)ms", r.stdout)
    sec = re.search(r"sec_size = (\d+)", r.stdout)
    if len(live) != layers or total is None:
        raise RuntimeError("could not parse the output of ref_snig: " + r.stdout[-400:])
    return {"live": np.asarray(live, dtype=np.int64), "kernel_ms": float(total.group(1)), "layer_ms": ms,
            "sec_size": int(sec.group(1)) if sec else None}
