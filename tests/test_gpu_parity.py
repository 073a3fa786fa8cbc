"""GPU parity tests: the CUDA path through the C ABI against the oracle, bit for bit."""
import ctypes as C
import glob
import os

import numpy as np
import pytest

from conftest import ROOT, mixed_density_images, rows_of
from graphchallenge21_b200 import SpDNN, SpDNNError, _lib, generator, network
from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images

pytestmark = pytest.mark.gpu

GOLDEN = sorted(glob.glob(os.path.join(ROOT, "tests", "golden", "*.npz")))
REL_TOL = 1e-5        # stated tolerance for activations; the tests below get 0 (bit-exact)
_LARGE_WANT = {}      # oracle results shared by the parametrised cases of one input


def run_gpu(net, y0, first=0, how="dense", layers=None, vals=None, clip=32.0, alias=False, order=None):
    n, L = net.neurons, (net.layers if layers is None else layers)
    with SpDNN(n, L, float(net.bias), clip=clip) as g:
        if alias:
            g.set_network(net)           # equal layers declared once, then spdnn_set_layer_same_as
        for l in ([] if alias else (order or range(L))):
            if vals is None:
                g.set_layer_csc(l, *net.layer_csc(l))
            else:
                g.set_layer_rows(l, net.layer_rows(l), vals[l])
        if how == "dense":
            g.set_input_dense(y0, first)
        elif how == "coo":
            img, neu, val = generator.dense_to_coo_1based(y0)
            g.set_input_coo(img, neu, val, y0.shape[0], first, index_base=1)
        elif how == "device":
            import torch
            g.set_input_dense(torch.from_numpy(y0).cuda(), first)
        elif how == "bits":
            g.set_input_bits(network.pack_bits(y0), first)
        elif how == "bits_device":
            import torch
            g.set_input_bits(torch.from_numpy(network.pack_bits(y0)).cuda(), first)
        res = g.infer()
        return g.categories().copy(), g.activations(), g.layer_live().copy(), res


def check(got, want):
    cats, act, live, res = got
    wc, wa, wl = want
    assert np.array_equal(live, wl), (live.tolist(), wl.tolist())
    assert np.array_equal(cats, wc)
    assert res.survivors == len(wc)
    assert act.shape == wa.shape
    if wa.size:
        rel = np.abs(act - wa) / np.maximum(np.abs(wa), 1e-30)
        assert rel.max() <= REL_TOL
        assert np.array_equal(act, wa), "activations are expected to be bit-exact"


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
@pytest.mark.parametrize("how", ["dense", "coo", "device", "bits", "bits_device"])
def test_golden_vectors(path, how):
    g = np.load(path)
    n, L = int(g["neurons"]), int(g["layers"])
    net = SyntheticNetwork(n, L, str(g["pattern"]), seed=int(g["seed"]), bias=float(g["bias"]))
    y0 = np.unpackbits(g["y0_bits"], axis=1)[:, :n].astype(np.float32)
    check(run_gpu(net, y0, how=how), (g["categories"], g["activations"], g["live"]))


@pytest.mark.parametrize("pattern,n,L,b", [("radix16", 1024, 120, 6000), ("radix16", 4096, 30, 777),
                                           ("random", 1024, 12, 1500), ("radix16", 16384, 12, 100),
                                           ("radix16", 4096, 60, 2000), ("radix16", 16384, 24, 300),
                                           ("radix16", 65536, 14, 64), ("random", 4096, 8, 300)])
def test_against_oracle(pattern, n, L, b, oracle):
    net = SyntheticNetwork(n, L, pattern)
    y0 = synthetic_images(n, b) if pattern == "radix16" else mixed_density_images(n, b)
    want = oracle.infer(y0, [(r, None) for r in rows_of(net)], float(net.bias), first_image=500)
    got = run_gpu(net, y0, first=500)
    check(got, want)
    assert 0 < len(want[0]) < b          # the case exercises compaction


@pytest.mark.parametrize("env", [{"SPDNN_RESIDENT": "0"}, {"SPDNN_RESIDENT_TI": "8"}, {"SPDNN_RESIDENT_TI": "4"},
                                 {"SPDNN_CHUNK_FIRST": "1", "SPDNN_CHUNK_MAX": "3"}, {"SPDNN_CHUNK_FIRST": "64"},
                                 {"SPDNN_STAGE_TABLES": "0"}, {"SPDNN_EXACT_SHORTCUT": "1"}, {"SPDNN_RESIDENT_IPT": "4"},
                                 {"SPDNN_BIT_FORM": "0"}, {"SPDNN_DENSE_DIRECT": "1"}, {"SPDNN_LAZY_EXPAND": "0"},
                                 {"SPDNN_RESIDENT_TI": "16"}, {"SPDNN_REPS_ONLY": "0"}, {"SPDNN_BINARY_FRONT": "0"},
                                 {"SPDNN_RESIDENT": "2"}, {"SPDNN_COUNT_FRONT": "0"},
                                 {"SPDNN_RESIDENT": "0", "SPDNN_COUNT_FRONT": "0"}])
def test_kernel_paths_agree(env, monkeypatch, oracle):
    """The per-layer kernel, and the shared-memory-resident kernel at every group size and chunk
    schedule, give the same bits as the oracle."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    for pattern, n, L, b in (("radix16", 1024, 40, 1000), ("random", 1024, 9, 700)):
        net = SyntheticNetwork(n, L, pattern)
        y0 = synthetic_images(n, b) if pattern == "radix16" else mixed_density_images(n, b)
        want = oracle.infer(y0, [(r, None) for r in rows_of(net)], float(net.bias), first_image=7)
        check(run_gpu(net, y0, first=7), want)
        check(run_gpu(net, y0, first=7, how="bits"), want)
        check(run_gpu(net, y0, first=7, how="coo"), want)


@pytest.mark.parametrize("n,L,b", [(1024, 30, 777), (4096, 20, 300), (16384, 12, 100), (65536, 10, 40)])
@pytest.mark.parametrize("how", ["dense", "device", "coo", "bits", "bits_device"])
def test_binary_inputs_in_every_format(n, L, b, how, oracle):
    """A binary input is kept as one bit per activation whatever format it arrives in, and layer 0 is computed
    from the bits (by the first chunk while it loads, or by the per-layer kernel); same bits as the oracle."""
    net = SyntheticNetwork(n, L, "radix16")
    y0 = synthetic_images(n, b, first_image=31)
    key = ("binary", n, L, b)
    if key not in _LARGE_WANT:
        _LARGE_WANT[key] = oracle.infer(y0, [(r, None) for r in rows_of(net)], float(net.bias), first_image=9)
    check(run_gpu(net, y0, first=9, how=how, alias=True), _LARGE_WANT[key])


@pytest.mark.parametrize("odd_image", [0, 40, 299])
@pytest.mark.parametrize("how", ["dense", "device", "coo"])
def test_one_value_that_is_not_binary_switches_the_pass_to_floats(odd_image, how, oracle, monkeypatch):
    """The input is staged in pieces of 32 images; the one value that is neither 0 nor 1 sits in the first, a
    middle or the last piece, so pieces converted before it exist as bits only and are rebuilt as floats."""
    monkeypatch.setenv("SPDNN_STAGE_KB", "128")          # 32 images of 1024 floats per copy
    n, L, b = 1024, 12, 300
    net = SyntheticNetwork(n, L, "radix16")
    y0 = synthetic_images(n, b)
    on = np.nonzero(y0[odd_image])[0]
    y0[odd_image, on[: len(on) // 2]] = np.float32(1.75)
    want = oracle.infer(y0, [(r, None) for r in rows_of(net)], float(net.bias))
    check(run_gpu(net, y0, how=how), want)


def test_dense_input_read_in_place(oracle, monkeypatch):
    """With SPDNN_DENSE_DIRECT=1 a dense input is read in place by the first launch (16-byte
    loads when the matrix is aligned, 4-byte loads when it is not); a caller's device buffer is
    not modified, and the same context then takes triplets (the other captured pass) with the
    same result."""
    import torch
    monkeypatch.setenv("SPDNN_DENSE_DIRECT", "1")
    n, L, b = 1024, 30, 1000
    net = SyntheticNetwork(n, L, "radix16")
    y0 = synthetic_images(n, b)
    want = oracle.infer(y0, [(r, None) for r in rows_of(net)], float(net.bias), first_image=3)
    buf = torch.zeros(b * n + 8, dtype=torch.float32, device="cuda")
    with SpDNN(n, L, float(net.bias)) as g:
        for l in range(L):
            g.set_layer_csc(l, *net.layer_csc(l))
        for shift in (0, 1, 4):
            view = buf[shift:shift + b * n].view(b, n)
            view.copy_(torch.from_numpy(y0))
            g.set_input_dense(view, 3)
            res = g.infer()
            check((g.categories().copy(), g.activations(), g.layer_live().copy(), res), want)
            assert torch.equal(view.cpu(), torch.from_numpy(y0))
        img, neu, val = generator.dense_to_coo_1based(y0)
        g.set_input_coo(img, neu, val, b, 3, index_base=1)
        res = g.infer()
        check((g.categories().copy(), g.activations(), g.layer_live().copy(), res), want)
        g.set_input_dense(y0, 3)                       # host matrix: staged, then read in place
        res = g.infer()
        check((g.categories().copy(), g.activations(), g.layer_live().copy(), res), want)


_BIT_FORM_WANT = {}


@pytest.mark.parametrize("env", [{}, {"SPDNN_BIT_FORM": "0"}, {"SPDNN_CHUNK_FIRST": "1", "SPDNN_CHUNK_MAX": "3"},
                                 {"SPDNN_RESIDENT_TI": "8"}, {"SPDNN_STAGE_TABLES": "0"}, {"SPDNN_RESIDENT_IPT": "4"},
                                 {"SPDNN_TABLE_GROUP": "1"}, {"SPDNN_TABLE_GROUP": "2", "SPDNN_TABLE_RING": "2"},
                                 {"SPDNN_ALT2_SMALL_BLOCKS": "0"}, {"SPDNN_WORD_RING": "2"}, {"SPDNN_BITS_FIRST": "1"},
                                 {"SPDNN_BITS_FIRST": "1", "SPDNN_BITS_THREADS": "1024", "SPDNN_CHUNK_FIRST": "40"},
                                 {"SPDNN_BITS_SMALL": "1"}, {"SPDNN_BITS_SMALL": "1", "SPDNN_BITS_FIRST": "1"}])
@pytest.mark.parametrize("bias,clip,n,L", [(-0.3, 32.0, 1024, 70), (0.0, 32.0, 1024, 70), (-32.0, 32.0, 1024, 70), (0.01, 32.0, 1024, 70),
                                           (-0.3, 8.0, 1024, 70), (-1.0, 2.5, 1024, 70), (-0.35, 32.0, 4096, 50), (0.0, 16.0, 4096, 50)])
def test_bit_form_of_saturated_activations(bias, clip, n, L, env, monkeypatch, oracle):  # noqa: E302
    """Blocks whose activations are all exactly 0 or clip continue as one word per row and come
    back to floats in the layer where an output is not saturated; the bits are those of the
    float form for every bias and clip.  The batch holds runs of images that are saturated from
    the start (so whole blocks start a chunk in the bit form), images scaled off the 1/16 grid,
    all-clip images and ordinary ones; N = 4096 has 256 classes per layer (all warps of a block
    work in the bit form), N = 1024 at most 64 (one warp)."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    b = 640
    net = SyntheticNetwork(n, L, "radix16", bias=bias)
    y0 = synthetic_images(n, b)
    y0[128:320] *= np.float32(clip)
    y0[320:400:3] *= np.float32(0.37 * clip)
    y0[400:440] = np.float32(clip)
    key = (bias, clip, n)
    if key not in _BIT_FORM_WANT:
        _BIT_FORM_WANT[key] = oracle.infer(y0, [(r, None) for r in rows_of(net)], bias, clip=clip)
    check(run_gpu(net, y0, clip=clip), _BIT_FORM_WANT[key])


def _large_case(oracle, bias, clip, n, L, b):
    """Batch with every kind of image the bit form distinguishes: ordinary blobs, runs that are
    saturated from the start (whole 32-image blocks begin a chunk as words), values off the
    1/16 grid, all-clip images and all-zero images."""
    net = SyntheticNetwork(n, L, "radix16", bias=bias)
    y0 = synthetic_images(n, b)
    y0[32:64] *= np.float32(clip)
    y0[64:80:3] *= np.float32(0.37 * clip)
    y0[80:88] = np.float32(clip)
    y0[40:44] = 0.0           # all-zero images inside a saturated tile: they die in the tile's first layer of the bit form
    key = (bias, clip, n, L, b)
    if key not in _LARGE_WANT:
        _LARGE_WANT[key] = oracle.infer(y0, [(r, None) for r in rows_of(net)], bias, clip=clip, first_image=11)
    return net, y0, _LARGE_WANT[key]


@pytest.mark.parametrize("env", [{}, {"SPDNN_BIT_FORM": "0"}, {"SPDNN_STAGE_TABLES": "0"}, {"SPDNN_RESIDENT_TI": "8"},
                                 {"SPDNN_RESIDENT_TI": "4"}, {"SPDNN_WORD_RING": "2"}, {"SPDNN_CHUNK_FIRST": "3", "SPDNN_CHUNK_GROWTH": "2"},
                                 {"SPDNN_BITS_KERNEL": "0"}, {"SPDNN_BITS_FIRST": "1"}, {"SPDNN_BITS_FIRST": "1", "SPDNN_BITS_THREADS": "128"},
                                 {"SPDNN_BITS_FIRST": "1", "SPDNN_STAGE_TABLES": "0"}, {"SPDNN_BITS_FIRST": "1", "SPDNN_TABLE_GROUP": "1", "SPDNN_TABLE_RING": "2"},
                                 {"SPDNN_BITS_FIRST": "1", "SPDNN_CHUNK_FIRST": "1", "SPDNN_CHUNK_MAX": "3"},
                                 {"SPDNN_BITS_FIRST": "1", "SPDNN_TABLE_CACHE": "0"}, {"SPDNN_TWO_BLOCKS": "0"},
                                 {"SPDNN_COUNT_FRONT": "0"}, {"SPDNN_ALT2_THREADS": "256"},
                                 {"SPDNN_ALT2_THREADS": "256", "SPDNN_RESIDENT_TI": "8", "SPDNN_BITS_KERNEL": "0"}],
                         ids=lambda e: ",".join(f"{k[6:]}={v}" for k, v in e.items()) or "default")
@pytest.mark.parametrize("bias,clip,n,L,b", [(-0.4, 32.0, 16384, 80, 96), (-0.45, 32.0, 65536, 48, 96)])
def test_bit_form_at_the_large_network_sizes(bias, clip, n, L, b, env, monkeypatch, oracle):
    """N = 16384 (1024 classes per layer) and N = 65536 (4096 classes): every warp of a block works
    on a layer of the bit form, the tables are staged in small groups or read from global memory,
    and the float form runs 16, 8 or 4 images per block.  These are the launch shapes of the two
    largest challenge networks (the reference needed its 64-bit build for them,
    src/microbenchmark/out_memory.cu:24,35,58)."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    net, y0, want = _large_case(oracle, bias, clip, n, L, b)
    check(run_gpu(net, y0, first=11, clip=clip, alias=True), want)
    assert 0 < len(want[0]) < b


@pytest.mark.parametrize("n,L,b", [(4096, 240, 200), (16384, 130, 96)])
def test_long_networks_enter_and_leave_the_bit_form_in_mid_chunk(n, L, b, oracle):
    """Long enough for the chunks to grow to hundreds of layers with >= 256 classes per layer:
    blocks enter the bit form in the middle of a chunk, images die inside it."""
    net, y0, want = _large_case(oracle, float(SyntheticNetwork(n, 1).bias), 32.0, n, L, b)
    check(run_gpu(net, y0, first=11, alias=True), want)


@pytest.mark.parametrize("n,b", [(16384, 64), (65536, 32)])
def test_full_depth_of_the_largest_networks(n, b, oracle):
    """All 1920 layers of the two largest challenge networks on a small batch, against the oracle."""
    L = 1920
    net = SyntheticNetwork(n, L, "radix16")
    y0 = synthetic_images(n, b, first_image=77)
    want = oracle.infer(y0, [(r, None) for r in rows_of(net)], float(net.bias), first_image=77)
    check(run_gpu(net, y0, first=77, alias=True), want)
    assert 0 < len(want[0]) < b


def test_layers_without_a_host_copy_mix_with_resident_chunks(oracle, monkeypatch):
    """The canonical form of a layer is kept on the host only within a budget; a layer without it runs in
    the per-layer kernel and must then write ALL rows, because the resident chunk behind it has no class
    representatives to read through.  Layers are declared back to front so that layer 0 is the one that
    does not fit the budget."""
    monkeypatch.setenv("SPDNN_HOST_BUDGET_MB", "3")          # six of the eight distinct 512 KB layers
    n, L, b = 4096, 20, 300
    net = SyntheticNetwork(n, L, "radix16")
    y0 = synthetic_images(n, b)
    want = oracle.infer(y0, [(r, None) for r in rows_of(net)], float(net.bias))
    check(run_gpu(net, y0, order=list(range(L - 1, -1, -1))), want)
    monkeypatch.setenv("SPDNN_HOST_BUDGET_MB", "0")          # nothing kept: every layer in the per-layer kernel
    check(run_gpu(net, y0), want)


@pytest.mark.parametrize("pattern,n,L,b,budget_mb", [("random", 4096, 10, 300, 1), ("random", 1024, 12, 500, 1),
                                                     ("radix16", 4096, 30, 300, 0), ("radix16", 1024, 40, 700, 0)])
def test_weights_streamed_from_host_memory(pattern, n, L, b, budget_mb, oracle, monkeypatch):
    """Layers beyond the device budget for weights keep their tables in page-locked host memory and are
    copied into two device slots by a second stream while the layer before runs (the reference's
    out-of-core variant, src/microbenchmark/out_memory.cu:315-329, 368-388).  Budget 1 MB: the first
    layer(s) stay on the device (and may run in resident chunks), the rest are streamed; budget 0: all are."""
    monkeypatch.setenv("SPDNN_WEIGHT_BUDGET_MB", str(budget_mb))
    net = SyntheticNetwork(n, L, pattern)
    y0 = synthetic_images(n, b) if pattern == "radix16" else mixed_density_images(n, b)
    want = oracle.infer(y0, [(r, None) for r in rows_of(net)], float(net.bias), first_image=5)
    check(run_gpu(net, y0, first=5), want)
    check(run_gpu(net, y0, first=5, how="bits"), want)
    assert 0 < len(want[0]) < b


@pytest.mark.parametrize("env", [{}, {"SPDNN_BITS_FIRST": "1"}, {"SPDNN_BITS_FIRST": "1", "SPDNN_BITS_THREADS": "128"},
                                 {"SPDNN_BITS_FIRST": "1", "SPDNN_CHUNK_FIRST": "2", "SPDNN_CHUNK_GROWTH": "2"}, {"SPDNN_BITS_KERNEL": "0"}],
                         ids=lambda e: ",".join(f"{k[6:]}={v}" for k, v in e.items()) or "default")
@pytest.mark.parametrize("n,L,b,bias,clip", [(1024, 48, 600, -0.3, 32.0), (4096, 24, 200, -0.35, 32.0), (1024, 30, 300, 0.01, 8.0),
                                             (1024, 30, 300, -3.0, 2.5)])
def test_count_form_on_networks_without_structure(n, L, b, bias, clip, env, monkeypatch, oracle):
    """Pattern 'random' has no repeated columns, so every class gathers 32 rows; tiles whose activations are all 0
    or clip run a chunk as words with each output decided by the count of clip-valued inputs.  The batch mixes
    densities (some images saturate, some die, some stay in between for a while) with images that are
    saturated from the start and values off the grid."""
    for k, v in env.items():
        monkeypatch.setenv(k, v)
    net = SyntheticNetwork(n, L, "random", bias=bias)
    y0 = mixed_density_images(n, b)
    y0[32:96] = (mixed_density_images(n, 64, seed=77, lo=0.5, hi=0.95) * np.float32(clip))
    y0[96:104:3] *= np.float32(0.37 * clip)
    key = ("count", n, L, b, bias, clip)
    if key not in _LARGE_WANT:
        _LARGE_WANT[key] = oracle.infer(y0, [(r, None) for r in rows_of(net)], bias, clip=clip, first_image=2)
    check(run_gpu(net, y0, first=2, clip=clip), _LARGE_WANT[key])


def test_positive_bias_all_zero_inputs_stay_alive(oracle):
    """With a positive bias even an all-zero input has non-zero activations after layer 0, so
    nothing is ever dropped (every image is in the work list until a layer zeroes it,
    all_network.cu:455-463)."""
    n, L, b = 1024, 6, 200
    net = SyntheticNetwork(n, L, "radix16", bias=0.01)
    y0 = synthetic_images(n, b)
    y0[::4] = 0.0
    want = oracle.infer(y0, [(r, None) for r in rows_of(net)], 0.01)
    got = run_gpu(net, y0)
    check(got, want)
    assert len(want[0]) == b


def test_alternating_pairs_with_k16(oracle):
    """The alternating-pair table form with K != 32 (runtime-K code path) and weight 1/8."""
    from conftest import paired_group_network
    n, L, b = 256, 6, 300
    rows = paired_group_network(n, L)
    vals = [np.full((n, 16), 0.125, np.float32) for _ in range(L)]

    class Net:
        neurons, layers, bias = n, L, np.float32(-0.4)
        def layer_rows(self, l): return rows[l]
    from graphchallenge21_b200 import network
    csc = [((np.arange(n + 1) * 16).astype(np.int32), r.reshape(-1), v.reshape(-1)) for r, v in zip(rows, vals)]
    info = network.inspect_network(n, csc)
    assert info["form"].tolist() == [0] + [1] * (L - 1) and info["classes"].max() <= n // 8
    y0 = mixed_density_images(n, b)
    want = oracle.infer(y0, list(zip(rows, vals)), -0.4, value=0.125)
    got = run_gpu(Net(), y0, vals=vals)
    check(got, want)
    assert 0 < len(want[0]) < b


@pytest.mark.parametrize("budget_mb", [None, 0])
def test_general_weights_and_ragged_columns(oracle, budget_mb, monkeypatch):
    if budget_mb is not None:
        monkeypatch.setenv("SPDNN_WEIGHT_BUDGET_MB", str(budget_mb))       # every layer streamed from host memory
    n, b, L = 512, 200, 6
    rng = np.random.default_rng(11)
    y0 = mixed_density_images(n, b)
    rows, vals = [], []
    for l in range(L):
        k = 20 if l % 2 else 37           # 37 -> padded to 40: the generic-K kernel
        r = np.sort(np.stack([rng.choice(n, k, replace=False) for _ in range(n)]), axis=1).astype(np.int64)
        drop = rng.random((n, k)) < 0.1
        r[drop] = n + 1
        r.sort(axis=1)
        r[r == n + 1] = -1
        rows.append(r.astype(np.int32))
        vals.append(rng.uniform(0.02, 0.2, (n, k)).astype(np.float32))

    class Net:
        neurons, layers, bias = n, L, np.float32(-0.25)
        def layer_rows(self, l): return rows[l]
    # the oracle wants one K for all layers: pad the shorter layers on its side
    kmax = max(r.shape[1] for r in rows)
    prow = [np.pad(r, ((0, 0), (0, kmax - r.shape[1])), constant_values=-1) for r in rows]
    pval = [np.pad(v, ((0, 0), (0, kmax - v.shape[1]))) for v in vals]
    want = oracle.infer(y0, list(zip(prow, pval)), -0.25)
    got = run_gpu(Net(), y0, vals=vals)
    check(got, want)


def test_uniform_non_power_of_two_weight_uses_general_path(oracle):
    n, b, L = 1024, 300, 5
    net = SyntheticNetwork(n, L, "radix16")
    y0 = synthetic_images(n, b)
    vals = [np.full((n, 32), 0.07, np.float32) for _ in range(L)]
    want = oracle.infer(y0, [(net.layer_rows(l), vals[l]) for l in range(L)], float(net.bias))
    with SpDNN(n, L, float(net.bias)) as g:
        for l in range(L):
            g.set_layer_rows(l, net.layer_rows(l), vals[l])
        assert g.layer_info(0) == {"classes": 64, "k": 32, "uniform": False}
        g.set_input_dense(y0)
        res = g.infer()
        check((g.categories().copy(), g.activations(), g.layer_live().copy(), res), want)


def test_edge_batches(oracle):
    n, L = 1024, 8
    net = SyntheticNetwork(n, L, "radix16")
    layers = [(r, None) for r in rows_of(net)]
    with SpDNN(n, L, float(net.bias)) as g:
        for l in range(L):
            g.set_layer_csc(l, *net.layer_csc(l))
        # the same context serves batches of different sizes, empty and all-dead included
        for b in (1, 31, 32, 33, 0, 257, 64):
            y0 = synthetic_images(n, b, first_image=3 * b)
            g.set_input_dense(y0, 10)
            res = g.infer()
            want = oracle.infer(y0, layers, float(net.bias), first_image=10)
            check((g.categories().copy(), g.activations(), g.layer_live().copy(), res), want)
        y0 = np.zeros((40, n), np.float32)
        g.set_input_dense(y0)
        assert g.infer().survivors == 0 and len(g.categories()) == 0 and g.layer_live().tolist() == [0] * L


def test_infer_is_repeatable_and_input_is_consumed():
    n, L, b = 1024, 10, 500
    net = SyntheticNetwork(n, L, "radix16")
    y0 = synthetic_images(n, b)
    with SpDNN(n, L, float(net.bias)) as g:
        for l in range(L):
            g.set_layer_csc(l, *net.layer_csc(l))
        outs = []
        for _ in range(3):
            g.set_input_dense(y0)
            g.infer()
            outs.append((g.categories().copy(), g.activations()))
        assert all(np.array_equal(outs[0][0], o[0]) and np.array_equal(outs[0][1], o[1]) for o in outs)
        # passes queued back to back without waiting in between: the last one's results are what is fetched
        for k in range(3):
            g.set_input_dense(y0[: b - 100 * (2 - k)])
            g.infer_async()
        res = g.sync()
        assert res.batch == b and np.array_equal(g.categories(), outs[0][0]) and np.array_equal(g.activations(), outs[0][1])
        with pytest.raises(SpDNNError) as e:
            g.infer()
        assert e.value.code == -4


def test_error_paths():
    n, L = 1024, 2
    net = SyntheticNetwork(n, L, "radix16")
    with SpDNN(n, L, float(net.bias)) as g:
        cp, ri, v = net.layer_csc(0)
        bad = ri.copy(); bad[7] = n
        with pytest.raises(SpDNNError):
            g.set_layer_csc(0, cp, bad, v)
        with pytest.raises(SpDNNError):
            g.set_layer_csc(5, cp, ri, v)
        g.set_layer_csc(0, cp, ri, v)
        g.set_input_dense(synthetic_images(n, 8))
        with pytest.raises(SpDNNError) as e:      # layer 1 missing
            g.infer()
        assert e.value.code == -4
        g.set_layer_csc(1, *net.layer_csc(1))
        # out-of-range input triplet: reported by the device-side check, context stays usable
        g.set_input_coo(np.array([1, 99], np.int32), np.array([1, 1], np.int32), None, 8, 0, 1)
        with pytest.raises(SpDNNError) as e:
            g.infer()
        assert e.value.code == -5
        g.set_input_dense(synthetic_images(n, 8))
        g.infer()
    with pytest.raises(SpDNNError):
        SpDNN(n, L, -0.3, device=99)


def test_shards_compose(oracle):
    """Batch sharding: running two halves with their global offsets gives the two halves of
    the full category list (what the multi-GPU path relies on)."""
    n, L, b = 1024, 20, 900
    net = SyntheticNetwork(n, L, "radix16")
    y0 = synthetic_images(n, b)
    full = run_gpu(net, y0)[0]
    lo = run_gpu(net, y0[:450], first=0)[0]
    hi = run_gpu(net, y0[450:], first=450)[0]
    assert np.array_equal(np.concatenate([lo, hi]), full)


def test_full_size_properties_config1():
    """N=1024, L=1920, B=60000 (too slow for the CPU oracle in full): size-independent
    properties -- deterministic across runs, survivors saturate to {0, 32}, live counts never
    grow, and the first 6000 images give exactly the categories of a 6000-image run."""
    n, L, b = 1024, 1920, 60000
    net = SyntheticNetwork(n, L, "radix16")
    y0 = synthetic_images(n, b)
    with SpDNN(n, L, float(net.bias)) as g:
        for l in range(L):
            g.set_layer_csc(l, *net.layer_csc(l))
        g.set_input_dense(y0)
        r1 = g.infer()
        c1, live1 = g.categories().copy(), g.layer_live().copy()
        a1 = g.activations()
        g.set_input_dense(y0[:6000])
        g.infer()
        c2 = g.categories().copy()
    assert (np.diff(live1) <= 0).all() and live1[-1] == len(c1) == r1.survivors
    assert 0.05 * b < len(c1) < 0.8 * b
    assert (np.diff(c1) > 0).all()
    assert np.isin(a1, (0.0, 32.0)).all() and (a1 != 0).any(axis=1).all()
    assert np.array_equal(c2, c1[c1 < 6000])
    assert r1.kernel_launches >= 2
