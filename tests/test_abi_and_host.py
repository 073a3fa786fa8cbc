"""CPU tests: the C-ABI library loads and exports what the header declares; host logic."""
import ctypes as C
import io
import os
import re
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from conftest import ROOT
from graphchallenge21_b200 import _lib, formats, generator, network
from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images


def header_symbols():
    txt = open(os.path.join(ROOT, "include", "spdnn_b200.h")).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(spdnn_[a-z_0-9]+)\s*\(", txt)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = header_symbols()
    assert len(names) >= 18
    for n in names:
        assert hasattr(lib, n), n
        assert n in _lib.SYMBOLS, f"{n} declared in the header but not bound"
    assert b"sm_100a" in lib.spdnn_version()


def test_stats_struct_matches_header_size():
    # int32, int32, int64, float, float, double, int64, int32, int32
    assert C.sizeof(_lib.Stats) == 48


def test_inspect_layer_without_gpu():
    lib = _lib.load()
    for pattern, want_classes in (("radix16", 64), ("random", 1024)):
        net = SyntheticNetwork(1024, 3, pattern)
        cp, ri, v = net.layer_csc(1)
        cls, k, uni = C.c_int(), C.c_int(), C.c_int()
        rc = lib.spdnn_inspect_layer_csc(1024, cp.ctypes.data, ri.ctypes.data, v.ctypes.data, C.byref(cls), C.byref(k),
                                         C.byref(uni))
        assert rc == 0 and cls.value == want_classes and k.value == 32 and uni.value == 1
    # non power-of-two weights are not "uniform"; malformed layers are rejected
    v2 = np.full_like(v, 0.1)
    assert lib.spdnn_inspect_layer_csc(1024, cp.ctypes.data, ri.ctypes.data, v2.ctypes.data, None, None, C.byref(uni)) == 0
    assert uni.value == 0
    bad = ri.copy(); bad[5] = 4096
    assert lib.spdnn_inspect_layer_csc(1024, cp.ctypes.data, bad.ctypes.data, None, None, None, None) == -1


def test_network_analysis_in_value_ids():
    """Host logic of the resident kernel's tables: value ids chain from layer to layer."""
    n, L = 1024, 9
    net = SyntheticNetwork(n, L, "radix16")
    r = network.inspect_network(n, [net.layer_csc(l) for l in range(L)])
    assert r["classes"][:5].tolist() == [64] * 5 and r["classes"].max() == 64
    assert r["classes"][5] == 32                                 # stride N/2: columns g and g + 32 read the same rows
    assert r["v_in"].tolist() == [n] + r["classes"][:-1].tolist()   # layer 0 reads neurons, the rest value ids
    assert r["form"].tolist() == [0] + [1] * (L - 1)             # 16-wide butterfly blocks alternate two ids
    net = SyntheticNetwork(n, 3, "random")
    r = network.inspect_network(n, [net.layer_csc(l) for l in range(3)])
    assert r["classes"].tolist() == [n] * 3 and r["v_in"].tolist() == [n] * 3 and r["form"].tolist() == [0] * 3
    # a layer after one with repeated columns merges columns that differ only in equivalent rows
    cp, ri, v = SyntheticNetwork(n, 2, "radix16").layer_csc(0)
    rnd = SyntheticNetwork(n, 2, "random").layer_csc(1)
    r = network.inspect_network(n, [(cp, ri, v), rnd])
    assert r["classes"][0] == 64 and r["v_in"][1] == 64 and r["form"][1] == 0 and r["classes"][1] <= n


def test_generator_is_deterministic_and_well_formed():
    for pattern in ("radix16", "random"):
        a = SyntheticNetwork(1024, 8, pattern).layer_rows(3)
        b = SyntheticNetwork(1024, 8, pattern).layer_rows(3)
        assert np.array_equal(a, b) and a.shape == (1024, 32)
        assert (np.diff(a, axis=1) > 0).all() and a.min() >= 0 and a.max() < 1024
        # every input neuron feeds 32 outputs on average; radix16 exactly
        cnt = np.bincount(a.reshape(-1), minlength=1024)
        assert cnt.sum() == 32 * 1024 and (pattern == "random" or (cnt == 32).all())
    y = synthetic_images(1024, 200)
    assert set(np.unique(y)) <= {0.0, 1.0} and 0.10 < y.mean() < 0.20
    assert np.array_equal(synthetic_images(1024, 50, first_image=100), synthetic_images(1024, 150)[100:])
    h = generator.hash_reorder(np.arange(1024), 1024)
    assert np.array_equal(generator.hash_reorder_inverse(h, 1024), np.arange(1024))


def test_radix16_is_block_butterfly_in_permuted_numbering():
    n = 1024
    net = SyntheticNetwork(n, 8, "radix16")
    for layer, stride in ((0, 16), (1, 32), (5, 512), (6, 32)):
        rows = net.layer_rows(layer)
        for c in (0, 17, 513, 1023):
            cp = int(generator.hash_reorder(c, n))
            rp = np.sort(generator.hash_reorder(rows[c], n))
            base = cp // 16 * 16
            want = np.sort(np.concatenate([base + np.arange(16), (base + stride + np.arange(16)) % n]))
            assert np.array_equal(rp, want)


def test_formats_round_trip(tmp_path):
    net = SyntheticNetwork(1024, 2, "radix16")
    a, b, v = net.layer_coo_1based(1)
    p = formats.weight_file_name(str(tmp_path), 1024, 1)
    formats.write_layer_tsv(p, a, b, v)
    a2, b2, v2 = formats.read_layer_tsv(p)
    assert np.array_equal(a, a2) and np.array_equal(b, b2) and np.array_equal(v, v2)
    y = synthetic_images(1024, 10)
    img, neu, val = generator.dense_to_coo_1based(y)
    formats.write_input_tsv(formats.input_file_name(str(tmp_path), 1024), img, neu, val)
    i2, n2, _ = formats.read_input_tsv(formats.input_file_name(str(tmp_path), 1024), 4)
    assert i2.max() == 4 and np.array_equal(n2, neu[img <= 4])
    formats.write_weights_bin(str(tmp_path / "w.bin"), [net.layer_coo_1based(l) for l in range(2)])
    got = list(formats.read_weights_bin(str(tmp_path / "w.bin"), 1024, 2))
    assert np.array_equal(got[1][0], a) and np.array_equal(got[1][2], v)
    formats.write_input_bin(str(tmp_path / "i.bin"), img, neu, val)
    i3, n3, v3 = formats.read_input_bin(str(tmp_path / "i.bin"))
    assert np.array_equal(i3, img) and np.array_equal(n3, neu)
    formats.write_categories(str(tmp_path / "c.tsv"), np.array([0, 5, 9]))
    assert formats.read_categories(str(tmp_path / "c.tsv")).tolist() == [0, 5, 9]
    assert formats.compare_categories([0, 5, 9], str(tmp_path / "c.tsv"))["passed"]
    v = formats.compare_categories([0, 9, 11], str(tmp_path / "c.tsv"))
    assert not v["passed"] and v["missing"] == [5] and v["extra"] == [11]
    assert formats.compare_categories([0, 5], str(tmp_path / "c.tsv"), batch=6)["passed"]


def test_shard_bounds_cover_batch():
    for batch, world in ((60000, 8), (6000, 2), (7, 4), (0, 2), (33, 32)):
        cuts = [network.shard_bounds(batch, world, r) for r in range(world)]
        assert cuts[0][0] == 0 and cuts[-1][1] == batch
        assert all(cuts[i][1] == cuts[i + 1][0] for i in range(world - 1))
    assert network.shard_bounds(6001, 2, 0) == (0, 3001)      # the reference's (batch + 1) / 2


def test_create_without_gpu_returns_status_not_crash():
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(network.SpDNNError) as e:
        network.SpDNN(1024, 2, -0.3)
    assert e.value.code == -2


WORKER = textwrap.dedent("""
    import os, sys, io
    sys.path.insert(0, {root!r})
    import numpy as np
    import torch.distributed as dist
    from graphchallenge21_b200 import network
    from oracle import c_oracle

    class OracleEngine:
        # stands in for the GPU context so that the sharding / gather logic runs on CPU
        def __init__(self, n, l, bias, device):
            self.n, self.l, self.bias, self.layers_ = n, l, bias, {{}}
            self.neurons, self.layers = n, l
        def set_layer_coo(self, layer, a, b, v, index_base=1):
            order = np.lexsort((a, b))
            self.layers_[layer] = (a[order].reshape(self.n, 32) - index_base).astype(np.int32)
        def set_input_coo(self, img, neu, val, batch, first, index_base=1):
            self.y0 = np.zeros((batch, self.n), np.float32)
            self.y0[img - index_base, neu - index_base] = val
            self.first = first
        def infer(self):
            self.c, _, self.live = c_oracle.infer(self.y0, [(self.layers_[i], None) for i in range(self.l)], self.bias,
                                                  first_image=self.first, threads=2)
        def layer_live(self): return self.live
        def categories(self): return self.c
        def close(self): pass

    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
    out = io.StringIO()
    cats = network.run_multi_gpu(1024, 50, 6, {data!r}, out=out, engine_factory=OracleEngine)
    np.save(os.path.join({data!r}, f"cats{{sys.argv[1]}}.npy"), cats)
    assert "GPU[" in out.getvalue()
    dist.destroy_process_group()
""")


def test_multi_rank_sharding_and_gather_gloo(tmp_path, oracle):
    """world_size 2 on CPU: contiguous shards, replicated weights, one final gather."""
    n, batch, layers = 1024, 50, 6
    net = SyntheticNetwork(n, layers, "radix16")
    for l in range(layers):
        formats.write_layer_tsv(formats.weight_file_name(str(tmp_path), n, l), *net.layer_coo_1based(l))
    y0 = synthetic_images(n, batch)
    formats.write_input_tsv(formats.input_file_name(str(tmp_path), n), *generator.dense_to_coo_1based(y0))
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT, port=29500 + os.getpid() % 2000, data=str(tmp_path)))
    procs = [subprocess.Popen([sys.executable, str(script), str(r)], stderr=subprocess.PIPE, text=True) for r in range(2)]
    for p in procs:
        try:
            _, err = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            raise
        assert p.returncode == 0, err[-2000:]
    want, _, _ = oracle.infer(y0, [(net.layer_rows(l), None) for l in range(layers)], float(net.bias))
    for r in range(2):
        assert np.array_equal(np.load(tmp_path / f"cats{r}.npy"), want)
    assert 0 < len(want) < batch


def test_bit_matrix_layout_of_binary_inputs():
    """pack_bits: bit (n & 7) of byte n >> 3 of row i = neuron n of image i, rows padded to whole 32-bit words
    (what spdnn_set_input_bits documents)."""
    rng = np.random.default_rng(3)
    for n in (1024, 72, 33):
        y = (rng.random((5, n)) < 0.3).astype(np.float32) * np.float32(2.5)       # any non-zero value counts as set
        bits = network.pack_bits(y)
        assert bits.dtype == np.uint8 and bits.shape == (5, (n + 31) // 32 * 4)
        back = np.unpackbits(bits, axis=1, bitorder="little")[:, :n]
        assert np.array_equal(back, (y != 0).astype(np.uint8))
        assert not np.unpackbits(bits, axis=1, bitorder="little")[:, n:].any()


def test_image_generator_does_not_depend_on_its_thread_count():
    a = synthetic_images(4096, 300, first_image=17)
    b = synthetic_images(4096, 300, first_image=17, threads=4)
    assert np.array_equal(a, b)
    assert np.array_equal(synthetic_images(4096, 10, first_image=27), a[10:20])


def test_reference_arm_prints_the_bench_line():
    """`bench.py --impl reference`: the reference's CPU loop on a bounded sample, one JSON line with the keys of
    the bench contract (runs without a GPU)."""
    import json
    import subprocess
    import sys
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--config", "0", "--steps", "1",
                        "--warmup", "0", "--cpu-seconds", "0.5"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "edges/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] in ("reference", "port") and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["value"] == line["value"] and line["e2e"]["h2d_bytes_per_step"] == 0
    assert line["config"]["workload"].startswith("N=1024")
