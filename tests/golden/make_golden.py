"""Generates the committed golden vectors of tests/golden/.

    python tests/golden/make_golden.py

Each case is a seeded synthetic network and input (graphchallenge21_b200.generator), run
through the numpy oracle; before a file is written the same case is fed to the reference's
own CPU checkers (oracle/_ref/ref_harness: CpuSpmm::run_and_cmp per layer through the
reference's TSV loader, src/utils/cpu_spmm.h:11-55, src/utils/matrix.h:255-282), so the
stored outputs are reference-verified to the reference's tolerance (1e-3 absolute).  The
reference tree is needed only here, not when the tests run.
"""
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images  # noqa: E402
from oracle import build, make_case, spdnn_oracle as npo  # noqa: E402

CASES = [
    # name, neurons, layers, batch, pattern, bias override, input kind
    ("radix16_n1024_l24_b96", 1024, 24, 96, "radix16", None, "blobs"),
    ("random_n1024_l6_b80", 1024, 6, 80, "random", None, "mixed"),
    ("radix16_n4096_l10_b40", 4096, 10, 40, "radix16", None, "blobs"),
]


def mixed_density_images(neurons, batch, seed=0xABCD, lo=0.05, hi=0.6):
    from graphchallenge21_b200.generator import rand_unit
    idx = np.arange(batch * neurons, dtype=np.uint64).reshape(batch, neurons)
    dens = lo + (hi - lo) * rand_unit(seed, 3, np.arange(batch, dtype=np.uint64))
    return (rand_unit(seed, 4, idx) < dens[:, None]).astype(np.float32)


def main():
    harness = build.build_ref()
    if harness is None:
        raise SystemExit("reference tree not available: golden vectors must be generated where it is")
    for name, n, layers, batch, pattern, bias, kind in CASES:
        net = SyntheticNetwork(n, layers, pattern, bias=bias)
        y0 = synthetic_images(n, batch) if kind == "blobs" else mixed_density_images(n, batch)
        rows = [net.layer_rows(l) for l in range(layers)]
        with tempfile.TemporaryDirectory() as d:
            make_case.write_case(os.path.join(d, "c.bin"), y0, rows, float(net.bias), tsv_dir=d)
            r = subprocess.run([harness, "verify", os.path.join(d, "c.bin"), d], capture_output=True, text=True)
            if r.returncode != 0 or "REF_VERIFY_OK" not in r.stdout:
                raise SystemExit(f"{name}: reference checker disagrees\n{r.stdout[-500:]}{r.stderr[-500:]}")
        cats, act, live = npo.infer(y0, [(r, None) for r in rows], float(net.bias))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), neurons=n, layers=layers, batch=batch,
                            pattern=pattern, bias=np.float32(net.bias), seed=net.seed,
                            y0_bits=np.packbits(y0.astype(bool), axis=1), categories=cats, live=live,
                            activations=act.astype(np.float32))
        print(name, "survivors", len(cats), "live", live.tolist())


if __name__ == "__main__":
    main()
