"""The reference's own CUDA implementation beside the oracle and this library.

oracle/_ref/ref_snig is the reference's structure-agnostic GPU inference loop
(src/microbenchmark/snig.cu:19-120 kernel, :124-257 host loop) compiled from the reference's sources
and driven through its own matrix type, as src/SNIG.cpp does.  It prints the number of images that
still hold a non-zero activation after every layer; those counts must equal the oracle's and the
library's.  (Its sums are accumulated with shared-memory atomics in no fixed order, so activations
agree only to rounding and are not compared.)"""
import numpy as np
import pytest

from graphchallenge21_b200 import SpDNN
from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,L,b", [(1024, 48, 700), (4096, 24, 256)])
def test_reference_gpu_loop_survivor_counts(n, L, b, oracle):
    from oracle import ref_snig
    if ref_snig.available() is None:
        pytest.skip("oracle/_ref/ref_snig was not built (needs the reference tree and nvcc at build time)")
    net = SyntheticNetwork(n, L, "radix16")
    y0 = synthetic_images(n, b, first_image=123)
    ref = ref_snig.run(net, L, y0)
    _, _, want_live = oracle.infer(y0, [(net.layer_rows(l), None) for l in range(L)], float(net.bias), want_activations=False)
    assert np.array_equal(ref["live"], want_live), (ref["live"].tolist(), want_live.tolist())
    with SpDNN(n, L, float(net.bias)) as g:
        g.set_network(net)
        g.set_input_dense(y0)
        g.infer()
        assert np.array_equal(g.layer_live(), ref["live"])
    assert 0 < want_live[-1] < b
