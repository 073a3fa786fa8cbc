"""Seeded random sweep of the inference path against the oracle: network length, batch size,
bias, clip, input kind (ordinary, saturated from the start, off the 1/16 grid), input format
and the launch-shape switches are drawn together, so that combinations no hand-written case
lists get a turn (blocks that enter and leave the bit form in mid-chunk, partial last blocks,
chunks of one layer, ...).  Everything is compared bit for bit."""
import os
import random

import numpy as np
import pytest

from graphchallenge21_b200 import SpDNN, SyntheticNetwork, generator, synthetic_images
from graphchallenge21_b200.generator import mixed_density_images

pytestmark = pytest.mark.gpu

SWITCHES = [{}, {"SPDNN_RESIDENT_TI": "16"}, {"SPDNN_RESIDENT_TI": "8"}, {"SPDNN_TABLE_GROUP": "4"}, {"SPDNN_WORD_RING": "3"},
            {"SPDNN_CHUNK_FIRST": "3", "SPDNN_CHUNK_GROWTH": "2"}, {"SPDNN_STAGE_TABLES": "0"}, {"SPDNN_RESIDENT_IPT": "4"},
            {"SPDNN_ALT2_SMALL_BLOCKS": "0"}, {"SPDNN_CHUNK_MAX": "5"}, {"SPDNN_LAZY_EXPAND": "0"}, {"SPDNN_DENSE_DIRECT": "1"},
            {"SPDNN_RESIDENT_TI": "4"}, {"SPDNN_WORD_RING": "2"}, {"SPDNN_BITS_KERNEL": "0"},
            {"SPDNN_BITS_FIRST": "1"}, {"SPDNN_BITS_FIRST": "1", "SPDNN_CHUNK_FIRST": "2"}, {"SPDNN_BITS_FIRST": "1", "SPDNN_BITS_THREADS": "256"},
            {"SPDNN_BINARY_FRONT": "0"}, {"SPDNN_RESIDENT": "0"},
            {"SPDNN_BITS_FIRST": "1", "SPDNN_TABLE_CACHE": "0"}, {"SPDNN_COUNT_FRONT": "0"},
            {"SPDNN_BITS_SMALL": "1"}, {"SPDNN_BITS_SMALL": "1", "SPDNN_BITS_FIRST": "1"}, {"SPDNN_EXACT_SHORTCUT": "1"},
            {"SPDNN_EXACT_SHORTCUT": "1", "SPDNN_BIT_FORM": "0"}, {"SPDNN_ALT2_THREADS": "256"}, {"SPDNN_TWO_BLOCKS": "0"}]


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_configurations_match_the_oracle(seed, monkeypatch, oracle):
    rng = random.Random(seed)
    for it in range(14):
        n = rng.choice([1024, 1024, 1024, 4096, 4096, 16384, 65536])
        L = rng.randint(5, {1024: 200, 4096: 50, 16384: 40, 65536: 24}[n])
        b = rng.choice([1, 31, 32, 33, 100, 257, 640, 1500, 3000] if n <= 4096 else [1, 31, 33, 64, 100])
        bias = rng.choice([-0.3, -0.3, -0.35, 0.0, -1.0, -32.0, 0.01, -0.0625, -16.0])
        clip = rng.choice([32.0, 32.0, 32.0, 8.0, 2.5, 1.0, 100.0])
        for k in [k for k in os.environ if k.startswith("SPDNN_") and k not in ("SPDNN_B200_LIB", "SPDNN_DATA_DIR")]:
            monkeypatch.delenv(k)
        for k, v in rng.choice(SWITCHES).items():
            monkeypatch.setenv(k, v)
        net = SyntheticNetwork(n, L, "radix16", bias=bias)
        kind = rng.choice(["blobs", "mixed", "saturated", "three kinds"])
        if kind == "mixed":
            y0 = mixed_density_images(n, b, first_image=it * 1000)
        else:
            y0 = synthetic_images(n, b, first_image=it * 1000)
            if kind == "saturated":
                y0 *= np.float32(clip)
            elif kind == "three kinds":
                y0[::3] *= np.float32(clip)
                y0[1::3] *= np.float32(0.37 * clip)
        want_c, want_a, want_l = oracle.infer(y0, [(net.layer_rows(l), None) for l in range(L)], bias, clip=clip, first_image=7)
        with SpDNN(n, L, bias, clip=clip) as g:
            if rng.random() < 0.5:
                g.set_network(net)
            else:
                for l in range(L):
                    g.set_layer_csc(l, *net.layer_csc(l))
            fmt = rng.random()
            if fmt < 0.25 and kind in ("blobs", "mixed"):
                from graphchallenge21_b200.network import pack_bits
                g.set_input_bits(pack_bits(y0), 7)
            elif fmt < 0.6:
                g.set_input_dense(y0, 7)
            else:
                img, neu, val = generator.dense_to_coo_1based(y0)
                g.set_input_coo(img, neu, val, b, 7, index_base=1)
            g.infer()
            what = (seed, it, n, L, b, bias, clip, kind)
            assert np.array_equal(g.layer_live(), want_l), what
            assert np.array_equal(g.categories(), want_c), what
            assert np.array_equal(g.activations(), want_a), what
