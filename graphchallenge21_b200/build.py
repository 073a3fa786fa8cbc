"""In-tree build of the CUDA library and the C++ drivers for sm_100a.

    python -m graphchallenge21_b200.build [--force]

Produces ``graphchallenge21_b200/libspdnn_b200.so`` (kernels + C ABI), the drivers
``graphchallenge21_b200/bin/{network,multi_gpu,main}`` that keep the reference's command
lines (src/network.cpp:58-64, src/multi_gpu.cpp:66-68) and the measurement programs of
``csrc/tools`` (``bin/add_chain_ceiling``).  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB = os.path.join(PKG, "libspdnn_b200.so")
BIN = os.path.join(PKG, "bin")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _host_cxx() -> list[str]:
    # a system g++ is preferred over a toolchain wrapper that may lack its runtime specs
    for cand in ("/usr/bin/g++",):
        if os.path.exists(cand):
            return ["-ccbin", cand]
    return []


def _stale(target: str, sources: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + r.stdout[-2000:] + r.stderr[-4000:])


def _sources(*names: str) -> list[str]:
    out = [os.path.join(CSRC, n) for n in names]
    out.append(os.path.join(PKG, "..", "include", "spdnn_b200.h"))
    return out


def build_library(force: bool = False) -> str:
    # every source and header of the library: a header that is not listed would leave a stale build behind
    deps = _sources(*sorted(n for n in os.listdir(CSRC) if n.endswith((".cu", ".cuh", ".h"))))
    if force or _stale(LIB, deps):
        _run([_nvcc(), *ARCH, *_host_cxx(), "-lineinfo", "-O3", "-std=c++17", "-shared", "-Xcompiler", "-fPIC",
              "-o", LIB, os.path.join(CSRC, "spdnn_api.cu"), os.path.join(CSRC, "spdnn_static.cu")])
    return LIB


def build_drivers(force: bool = False) -> list[str]:
    os.makedirs(BIN, exist_ok=True)
    built = []
    ddir = os.path.join(CSRC, "drivers")
    if not os.path.isdir(ddir):
        return built
    common = [os.path.join(ddir, f) for f in sorted(os.listdir(ddir)) if f.endswith(".h")]
    for name in ("network", "multi_gpu", "main"):
        src = os.path.join(ddir, name + ".cpp")
        if not os.path.exists(src):
            continue
        out = os.path.join(BIN, name)
        if force or _stale(out, [src, LIB, *common]):
            _run([_nvcc(), *_host_cxx(), "-O2", "-std=c++17", "-o", out, src, "-I" + os.path.join(PKG, "..", "include"),
                  "-L" + PKG, "-lspdnn_b200", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/..", "-Xcompiler", "-pthread"])
        built.append(out)
    return built


def build_tools(force: bool = False) -> list[str]:
    """Stand-alone measurement programs (csrc/tools): no library, no inputs; they print what the hardware sustains on
    one inner loop of the library, the ceiling its profile is compared with."""
    os.makedirs(BIN, exist_ok=True)
    built = []
    tdir = os.path.join(CSRC, "tools")
    if not os.path.isdir(tdir):
        return built
    for f in sorted(os.listdir(tdir)):
        if not f.endswith(".cu"):
            continue
        src, out = os.path.join(tdir, f), os.path.join(BIN, f[:-3])
        if force or _stale(out, [src]):
            _run([_nvcc(), *ARCH, *_host_cxx(), "-lineinfo", "-O3", "-std=c++17", "-o", out, src])
        built.append(out)
    return built


def build_all(force: bool = False) -> str:
    lib = build_library(force)
    build_drivers(force)
    build_tools(force)
    return lib


if __name__ == "__main__":
    print(build_all("--force" in sys.argv))
