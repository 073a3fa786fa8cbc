"""CPU tests: the oracle against the golden vectors and the reference's own CPU checkers."""
import glob
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT, mixed_density_images, rows_of
from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images
from oracle import build, make_case, spdnn_oracle as npo

GOLDEN = sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "*.npz")))


def load_golden(path):
    g = np.load(path)
    n, layers, batch = int(g["neurons"]), int(g["layers"]), int(g["batch"])
    net = SyntheticNetwork(n, layers, str(g["pattern"]), seed=int(g["seed"]), bias=float(g["bias"]))
    y0 = np.unpackbits(g["y0_bits"], axis=1)[:, :n].astype(np.float32)
    return g, net, y0


def test_golden_files_exist():
    assert len(GOLDEN) >= 3


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_c_oracle_matches_golden(path, oracle):
    g, net, y0 = load_golden(path)
    layers = [(r, None) for r in rows_of(net)]
    cats, act, live = oracle.infer(y0, layers, float(net.bias))
    assert np.array_equal(cats, g["categories"])
    assert np.array_equal(live, g["live"])
    assert np.array_equal(act, g["activations"])          # bit-exact
    # unpruned (as the reference's CPU loop runs) gives the same answer
    cats2, act2, live2 = oracle.infer(y0, layers, float(net.bias), prune=False)
    assert np.array_equal(cats2, cats) and np.array_equal(act2, act) and np.array_equal(live2, live)


def test_numpy_and_c_oracle_agree_general_values(oracle):
    n, b, layers = 256, 40, 5
    rng = np.random.default_rng(7)
    y0 = mixed_density_images(n, b)
    rows, vals = [], []
    for l in range(layers):
        k = 12
        r = np.sort(np.stack([rng.choice(n, k, replace=False) for _ in range(n)]), axis=1).astype(np.int32)
        r[rng.random((n, k)) < 0.15] = -1                    # ragged columns
        r = np.where(r < 0, np.iinfo(np.int32).max, r)
        r.sort(axis=1)
        r[r == np.iinfo(np.int32).max] = -1
        rows.append(r)
        vals.append(rng.uniform(0.02, 0.25, (n, k)).astype(np.float32))
    lay = list(zip(rows, vals))
    c1, a1, l1 = npo.infer(y0, lay, -0.2)
    c2, a2, l2 = oracle.infer(y0, lay, -0.2)
    assert np.array_equal(c1, c2) and np.array_equal(l1, l2) and np.array_equal(a1, a2)
    assert 0 < len(c1) < b


def test_empty_batch_and_all_dead(oracle):
    net = SyntheticNetwork(1024, 4, "random")
    layers = [(r, None) for r in rows_of(net)]
    c, a, l = oracle.infer(np.zeros((0, 1024), np.float32), layers, float(net.bias))
    assert len(c) == 0 and l.tolist() == [0, 0, 0, 0]
    c, a, l = oracle.infer(np.zeros((5, 1024), np.float32), layers, float(net.bias))
    assert len(c) == 0 and l.tolist() == [0, 0, 0, 0]


def test_first_image_offsets_categories(oracle):
    net = SyntheticNetwork(1024, 6, "radix16")
    y0 = synthetic_images(1024, 64, first_image=1000)
    layers = [(r, None) for r in rows_of(net)]
    c0, _, _ = oracle.infer(y0, layers, float(net.bias), first_image=0)
    c1, _, _ = oracle.infer(y0, layers, float(net.bias), first_image=1000)
    assert np.array_equal(c0 + 1000, c1)


@pytest.fixture(scope="module")
def harness():
    h = build.build_ref()
    if h is None:
        pytest.skip("reference tree not present and no prebuilt oracle/_ref/ref_harness")
    return h


def test_reference_cpu_checker_accepts_oracle(harness, tmp_path):
    """CpuSpmm::run_and_cmp (src/utils/cpu_spmm.h) recomputes every layer from the TSV files it
    loads itself and aborts on a mismatch > 1e-3."""
    net = SyntheticNetwork(1024, 5, "radix16")
    y0 = synthetic_images(1024, 24)
    make_case.write_case(str(tmp_path / "c.bin"), y0, rows_of(net), float(net.bias), tsv_dir=str(tmp_path))
    r = subprocess.run([harness, "verify", str(tmp_path / "c.bin"), str(tmp_path)], capture_output=True, text=True)
    assert r.returncode == 0 and "REF_VERIFY_OK" in r.stdout, r.stdout[-400:] + r.stderr[-400:]


def test_reference_cpu_checker_rejects_wrong_numbers(harness, tmp_path):
    net = SyntheticNetwork(1024, 2, "radix16")
    y0 = synthetic_images(1024, 8)
    p = str(tmp_path / "c.bin")
    make_case.write_case(p, y0, rows_of(net), float(net.bias))
    blob = bytearray(open(p, "rb").read())
    # corrupt one raw value of layer 0 (header 24 B, input, nnz word, three triplet arrays)
    off = 24 + 8 * 1024 * 4 + 4 + 3 * 32 * 1024 * 4
    blob[off:off + 4] = np.float32(5.0).tobytes()
    open(p, "wb").write(bytes(blob))
    r = subprocess.run([harness, "verify", p], capture_output=True, text=True)
    assert r.returncode != 0


def test_reference_fused_checker_accepts_oracle_clip_chain(harness, tmp_path):
    """CpuSpmmFuse::run_and_cmp (src/utils/cpu_spmm_fuse.h) chains layers with the clip; its
    bias argument is an int, so the case uses bias 0."""
    net = SyntheticNetwork(1024, 3, "radix16", bias=0.0)
    y0 = synthetic_images(1024, 16)
    make_case.write_case(str(tmp_path / "c.bin"), y0, rows_of(net), 0.0)
    r = subprocess.run([harness, "fuse", str(tmp_path / "c.bin")], capture_output=True, text=True)
    assert r.returncode == 0 and "REF_FUSE_OK" in r.stdout, r.stdout[-400:] + r.stderr[-400:]
