import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def rows_of(net, layers=None):
    return [net.layer_rows(l) for l in range(net.layers if layers is None else layers)]


@pytest.fixture(scope="session")
def oracle():
    from oracle import c_oracle
    c_oracle.lib()
    return c_oracle


def mixed_density_images(neurons, batch, seed=0xABCD, lo=0.05, hi=0.6):
    """Binary inputs whose per-image density is spread over [lo, hi]: keeps a share of the
    images alive on networks without locality (pattern 'random')."""
    from graphchallenge21_b200.generator import mixed_density_images as gen
    return gen(neurons, batch, seed, lo, hi)


def paired_group_network(n=256, layers=6, group=16):
    """A network whose layers alternate, in value ids, between two ids with K = 16 terms:
    column c (group g = c // 16, parity p = c % 2) reads all 16 neurons of group
    (g + shift(layer, p)) mod G.  Sorted by neuron the terms alternate even, odd, even, ...; all
    even (odd) neurons of a group form one class of the layer before.  Returns rows per layer."""
    g_count = n // group
    out = []
    for l in range(layers):
        rows = np.empty((n, group), dtype=np.int32)
        for c in range(n):
            g, p = c // group, c % 2
            h = (g + (l + 1) * (1 + 2 * p)) % g_count
            rows[c] = np.arange(group * h, group * h + group)
        out.append(rows)
    return out
