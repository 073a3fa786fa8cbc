"""spdnn_layer_static: the entry point for callers that cannot allocate device memory.

Some users of this library run a layer from a place where cudaMalloc is off limits: inside
another runtime's memory pool that owns the whole device, in a callback where the implicit
synchronisation of an allocation is not allowed, or after the process has frozen its memory
footprint.  For them one layer can be run on caller-owned buffers with the kernel's scratch
held in a fixed array of the loaded module.  This test calls that entry point through the C
ABI, twice in a row on different inputs (the scratch is shared between calls and must come
back clean), and checks survivors and activations against the existing context-based entry
points, bit for bit (the tolerance the other GPU tests state is 1e-5 relative).

It sits in a file of its own that pytest collects last, and passes both alone in a fresh
process and after the other GPU tests.
"""
import ctypes as C

import numpy as np
import pytest

from graphchallenge21_b200 import SpDNN, _lib
from graphchallenge21_b200.generator import SyntheticNetwork, synthetic_images

pytestmark = pytest.mark.gpu

REL_TOL = 1e-5


def to_tiles(y, neurons):
    """[batch, N] row-major -> tile layout [tiles][N + 1][32] (row N = zeros)."""
    b = y.shape[0]
    tiles = (b + 31) // 32
    t = np.zeros((tiles, neurons + 1, 32), dtype=np.float32)
    pad = np.zeros((tiles * 32, neurons), dtype=np.float32)
    pad[:b] = y
    t[:, :neurons, :] = pad.reshape(tiles, 32, neurons).transpose(0, 2, 1)
    return t


def reference_one_layer(net, layer, y0):
    """The existing entry points, one layer: survivors (positions in the batch) and their activations."""
    with SpDNN(net.neurons, 1, float(net.bias)) as g:
        g.set_layer_csc(0, *net.layer_csc(layer))
        g.set_input_dense(y0)
        g.infer()
        return g.categories().copy(), g.activations()


def static_one_layer(lib, torch, net, layer, y0):
    n, b = net.neurons, y0.shape[0]
    yin = torch.from_numpy(to_tiles(y0, n)).cuda()
    yout = torch.zeros_like(yin)
    off = torch.from_numpy((net.layer_rows(layer).astype(np.int32) * 32)).cuda()
    surv = torch.full((max(b, 1),), -1, dtype=torch.int32, device="cuda")
    count = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    err = C.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.spdnn_layer_static(yin.data_ptr(), yout.data_ptr(), n, b, None, off.data_ptr(), None, 32, 0.0625,
                                float(net.bias), 32.0, surv.data_ptr(), count.data_ptr(), stream, err, 256)
    assert rc == 0, err.value.decode()
    torch.cuda.synchronize()
    c = int(count.item())
    pos = surv[:c].cpu().numpy()
    out = yout.cpu().numpy()                       # [tiles][N + 1][32]
    rows = out[pos // 32, :n, pos % 32] if c else np.zeros((0, n), np.float32)
    return pos, rows


def test_static_scratch_layer_matches_context_path_twice_in_a_row():
    import torch
    lib = _lib.load()
    n = 1024
    net = SyntheticNetwork(n, 4, "radix16")
    for call, (layer, batch, first) in enumerate(((0, 1000, 0), (2, 333, 5000))):
        y0 = synthetic_images(n, batch, first_image=first)
        y0[:: 5 - 2 * call] = 0.0                    # dead images, a different set in each call
        want_pos, want_act = reference_one_layer(net, layer, y0)
        pos, act = static_one_layer(lib, torch, net, layer, y0)
        assert np.array_equal(pos, want_pos)
        assert act.shape == want_act.shape
        rel = np.abs(act - want_act) / np.maximum(np.abs(want_act), 1e-30)
        assert rel.max() <= REL_TOL and np.array_equal(act, want_act)
        assert 0 < len(pos) < batch


def test_static_scratch_rejects_oversized_batch_with_a_message():
    import torch
    lib = _lib.load()
    dummy = torch.zeros(64, dtype=torch.float32, device="cuda")
    idx = torch.zeros(64, dtype=torch.int32, device="cuda")
    err = C.create_string_buffer(256)
    rc = lib.spdnn_layer_static(dummy.data_ptr(), dummy.data_ptr(), 1024, 2097152 + 1, None, idx.data_ptr(), None, 32,
                                0.0625, -0.3, 32.0, idx.data_ptr(), idx.data_ptr(), None, err, 256)
    assert rc == -6 and b"limit" in err.value
    rc = lib.spdnn_layer_static(dummy.data_ptr(), dummy.data_ptr(), 1024, 10, None, idx.data_ptr(), None, 30,
                                0.0625, -0.3, 32.0, idx.data_ptr(), idx.data_ptr(), None, err, 256)
    assert rc == -1
