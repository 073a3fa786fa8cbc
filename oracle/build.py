"""Builds the test oracle.  Nothing built here is part of the shipped library.

    python oracle/build.py          # liboracle.so (C restatement) and, when the reference
                                    # tree is present, _ref/ref_harness and _ref/ref_snig

``_ref/ref_harness`` is the reference's own CPU checkers (src/utils/cpu_spmm.h,
src/utils/cpu_spmm_fuse.h), ``_ref/ref_snig`` its structure-agnostic GPU inference loop
(src/microbenchmark/snig.cu), both compiled from the reference's sources where they lie; only
the binaries land in ``oracle/_ref/`` (git-ignored).  No reference source is copied.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference's source tree: the directory named by SPDNN_REFERENCE, else a `reference` folder beside
# this repository (where the build container keeps it); absent on the GPU box, which uses the built binary
REF = os.environ.get("SPDNN_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def _compilers(names):
    seen = []
    for c in names:
        p = shutil.which(c) if c and not os.path.isabs(c) else c
        if p and os.path.exists(p) and p not in seen:
            seen.append(p)
    return seen


def _newer(target, *sources):
    return os.path.exists(target) and all(os.path.getmtime(target) >= os.path.getmtime(s) for s in sources)


def build_oracle(force: bool = False) -> str:
    """Compile spdnn_oracle.c into liboracle.so (OpenMP when a compiler supports it)."""
    src = os.path.join(HERE, "spdnn_oracle.c")
    out = os.path.join(HERE, "liboracle.so")
    if not force and _newer(out, src):
        return out
    errors = []
    for omp in (["-fopenmp"], []):
        for cc in _compilers(["/usr/bin/gcc", "gcc", os.environ.get("CC", ""), "cc"]):
            cmd = [cc, "-O2", "-ffp-contract=off", "-shared", "-fPIC", *omp, "-o", out, src]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode == 0:
                return out
            errors.append(" ".join(cmd) + "\n" + r.stderr[-400:])
    raise RuntimeError("could not build the oracle:\n" + "\n".join(errors))


def build_ref(force: bool = False) -> str | None:
    """Compile the harness against the reference headers; None when the reference is absent
    and no earlier build exists."""
    src = os.path.join(HERE, "ref_harness.cpp")
    out = os.path.join(HERE, "_ref", "ref_harness")
    if not os.path.isdir(os.path.join(REF, "src", "utils")):
        return out if os.path.exists(out) else None
    if not force and _newer(out, src):
        return out
    os.makedirs(os.path.dirname(out), exist_ok=True)
    errors = []
    for cxx in _compilers(["/usr/bin/g++", "g++", os.environ.get("CXX", ""), "c++"]):
        cmd = [cxx, "-std=c++11", "-O3", "-pthread", "-I" + os.path.join(REF, "src"), "-o", out, src]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode == 0:
            return out
        errors.append(" ".join(cmd) + "\n" + r.stderr[-400:])
    raise RuntimeError("could not build the reference harness:\n" + "\n".join(errors))


def build_ref_snig(force: bool = False) -> str | None:
    """Compile the harness around the reference's structure-agnostic GPU loop (src/microbenchmark/snig.cu) with
    nvcc, for sm_100a; None when neither the reference nor an earlier build is there."""
    src = os.path.join(HERE, "ref_snig_harness.cu")
    out = os.path.join(HERE, "_ref", "ref_snig")
    if not os.path.isfile(os.path.join(REF, "src", "microbenchmark", "snig.cu")):
        return out if os.path.exists(out) else None
    if not force and _newer(out, src):
        return out
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return out if os.path.exists(out) else None
    os.makedirs(os.path.dirname(out), exist_ok=True)
    ccbin = ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", *ccbin, "-std=c++14", "-O2", "-w", "-I" + os.path.join(REF, "src"),
           "-o", out, src]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("could not build the SNIG harness:\n" + " ".join(cmd) + "\n" + r.stderr[-800:])
    return out


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_oracle(force))
    print(build_ref(force))
    print(build_ref_snig(force))
