"""GPU tests of the drivers that keep the reference's command lines (src/network.cpp,
src/multi_gpu.cpp, src/main.cpp) and of their Python mirror, on TSV files in the
reference's format."""
import io
import os
import re
import subprocess

import numpy as np
import pytest

from conftest import ROOT, rows_of
from graphchallenge21_b200 import build, formats, generator, network
from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images

pytestmark = pytest.mark.gpu

N, B, L = 1024, 300, 10


@pytest.fixture(scope="module")
def data(tmp_path_factory, oracle):
    d = tmp_path_factory.mktemp("data")
    net = SyntheticNetwork(N, L, "radix16")
    for l in range(L):
        a, b, v = net.layer_coo_1based(l)
        p = np.random.default_rng(l).permutation(a.size)        # file order is arbitrary
        formats.write_layer_tsv(formats.weight_file_name(str(d), N, l), a[p], b[p], v[p])
    y0 = synthetic_images(N, B)
    formats.write_input_tsv(formats.input_file_name(str(d), N), *generator.dense_to_coo_1based(y0))
    cats, _, live = oracle.infer(y0, [(r, None) for r in rows_of(net)], float(net.bias))
    build.build_all()
    return str(d), cats, live


def run(exe, args, data_dir, cwd, extra_env=None):
    env = dict(os.environ, SPDNN_DATA_DIR=data_dir, **(extra_env or {}))
    r = subprocess.run([os.path.join(build.BIN, exe), *map(str, args)], capture_output=True, text=True, env=env,
                       cwd=cwd, timeout=300)
    assert r.returncode == 0, r.stdout[-1500:] + r.stderr[-1500:]
    return r.stdout


def test_network_driver(data, tmp_path):
    d, cats, live = data
    out = run("network", [N, B, L], d, str(tmp_path))
    got = [int(m.group(2)) for m in re.finditer(r"^layer (\d+), batch = (\d+)$", out, re.M)]
    assert got == live.tolist()
    assert "[BEGIN]..." in out and "[END]..." in out and "Kernel Exec Time [20-uiuc-row-succ] = " in out
    assert np.array_equal(formats.read_categories(str(tmp_path / f"neuron{N}-l{L}-categories.tsv")), cats)
    assert "Challenge" not in out                       # no truth file next to the data yet
    formats.write_categories(formats.truth_file_name(d, N, L), cats)
    assert f"Challenge PASSED: {len(cats)} categories" in run("network", [N, B, L], d, str(tmp_path))
    formats.write_categories(formats.truth_file_name(d, N, L), cats[1:])
    assert "Challenge FAILED" in run("network", [N, B, L], d, str(tmp_path))
    os.remove(formats.truth_file_name(d, N, L))
    assert "Usage: exe neuron batch layer" in run("network", [N, B], d, str(tmp_path))
    # the batch argument truncates the input file like the reference's reader
    out = run("network", [N, 100, L], d, str(tmp_path))
    assert np.array_equal(formats.read_categories(str(tmp_path / f"neuron{N}-l{L}-categories.tsv")), cats[cats < 100])


def test_multi_gpu_driver(data, tmp_path):
    import torch
    d, cats, live = data
    for gpus in sorted({1, min(2, torch.cuda.device_count())}):
        out = run("multi_gpu", [N, B, L], d, str(tmp_path), {"SPDNN_GPUS": str(gpus)})
        assert f"task_count = {gpus}" in out and "GPU[0] [BEGIN]..." in out
        assert np.array_equal(formats.read_categories(str(tmp_path / f"neuron{N}-l{L}-categories.tsv")), cats)


def test_single_layer_testbed(data, tmp_path):
    d, _, _ = data
    out = run("main", [3, N, 256], d, str(tmp_path))
    assert "Compare with cpu result [Success]" in out


def test_missing_file_is_reported(data, tmp_path):
    d, _, _ = data
    env = dict(os.environ, SPDNN_DATA_DIR=d)
    r = subprocess.run([os.path.join(build.BIN, "network"), str(N), str(B), str(L + 1)], capture_output=True, text=True,
                       env=env, cwd=str(tmp_path))
    assert r.returncode != 0 and "does not exists" in r.stdout


def test_python_mirror_run_network(data, tmp_path):
    d, cats, live = data
    buf = io.StringIO()
    got = network.run_network(N, B, L, d, out=buf, categories_path=str(tmp_path / "c.tsv"))
    assert np.array_equal(got, cats)
    lines = [int(m.group(1)) for m in re.finditer(r"^layer \d+, batch = (\d+)$", buf.getvalue(), re.M)]
    assert lines == live.tolist()
    assert np.array_equal(formats.read_categories(str(tmp_path / "c.tsv")), cats)
    # single process, no process group: run_multi_gpu degenerates to one shard
    got2 = network.run_multi_gpu(N, B, L, d, out=io.StringIO())
    assert np.array_equal(got2, cats)
