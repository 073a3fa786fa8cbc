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


def static_call(lib, torch, yin, n, live_in, rows, vals, bias, positions=None, w=0.0625):
    """One call of the entry point on a tile buffer that is already on the device.  rows: int [n, k]
    input neurons per output neuron (-1 = padding); vals: float [n, k] or None (uniform weight w).
    Returns (yout tiles on the device, survivor positions on the device, their count)."""
    k = rows.shape[1]
    off = np.where(rows < 0, n, rows).astype(np.int32) * 32
    off_d = torch.from_numpy(off).cuda()
    vals_d = None if vals is None else torch.from_numpy(np.ascontiguousarray(vals, np.float32)).cuda()
    yout = torch.zeros_like(yin)
    surv = torch.full((max(live_in, 1),), -1, dtype=torch.int32, device="cuda")
    count = torch.full((1,), -1, dtype=torch.int32, device="cuda")
    err = C.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.spdnn_layer_static(yin.data_ptr(), yout.data_ptr(), n, live_in, None if positions is None else positions.data_ptr(),
                                off_d.data_ptr(), None if vals_d is None else vals_d.data_ptr(), k, w, float(bias), 32.0,
                                surv.data_ptr(), count.data_ptr(), stream, err, 256)
    assert rc == 0, err.value.decode()
    torch.cuda.synchronize()
    return yout, surv, int(count.item())


def rows_at(yout, pos, n):
    out = yout.cpu().numpy()                       # [tiles][N + 1][32]
    return out[pos // 32, :n, pos % 32] if len(pos) else np.zeros((0, n), np.float32)


def static_one_layer(lib, torch, net, layer, y0):
    n, b = net.neurons, y0.shape[0]
    yin = torch.from_numpy(to_tiles(y0, n)).cuda()
    yout, surv, c = static_call(lib, torch, yin, n, b, net.layer_rows(layer), None, net.bias)
    pos = surv[:c].cpu().numpy()
    return pos, rows_at(yout, pos, n)


def test_static_scratch_layer_matches_context_path_twice_in_a_row():
    import torch
    from oracle import c_oracle
    lib = _lib.load()
    n = 1024
    net = SyntheticNetwork(n, 4, "radix16")
    for call, (layer, batch, first) in enumerate(((0, 1000, 0), (2, 333, 5000))):
        y0 = synthetic_images(n, batch, first_image=first)
        y0[:: 5 - 2 * call] = 0.0                    # dead images, a different set in each call
        want_pos, want_act = reference_one_layer(net, layer, y0)
        pos, act = static_one_layer(lib, torch, net, layer, y0)
        # and against the CPU oracle, which shares no code with either entry point
        o_pos, o_act, _ = c_oracle.infer(y0, [(net.layer_rows(layer), None)], float(net.bias))
        assert np.array_equal(pos, o_pos) and np.array_equal(act, o_act)
        assert np.array_equal(pos, want_pos)
        assert act.shape == want_act.shape
        rel = np.abs(act - want_act) / np.maximum(np.abs(want_act), 1e-30)
        assert rel.max() <= REL_TOL and np.array_equal(act, want_act)
        assert 0 < len(pos) < batch


def test_static_scratch_chained_calls_general_weights_and_empty_batch():
    """Two layers chained through the survivor positions of the first call (in_positions), explicit
    weights with ragged columns padded to k = 8 (the general-K, per-entry-weight kernel), and a call
    with no images at all; each compared with the CPU oracle."""
    import torch
    from oracle import c_oracle
    lib = _lib.load()
    n, b, k = 512, 203, 8
    rng = np.random.default_rng(5)
    rows, vals = [], []
    for _ in range(2):
        r = np.sort(np.stack([rng.choice(n, k, replace=False) for _ in range(n)]), axis=1).astype(np.int64)
        r[rng.random((n, k)) < 0.15] = n + 1
        r.sort(axis=1)
        r[r == n + 1] = -1
        rows.append(r.astype(np.int32))
        vals.append(rng.uniform(0.1, 0.6, (n, k)).astype(np.float32))
    y0 = (rng.random((b, n)) < 0.1).astype(np.float32)
    y0[::7] = 0.0
    bias = -0.5
    yin = torch.from_numpy(to_tiles(y0, n)).cuda()
    y1, surv1, c1 = static_call(lib, torch, yin, n, b, rows[0], vals[0], bias)
    p1 = surv1[:c1].cpu().numpy()
    w1 = c_oracle.infer(y0, [(rows[0], vals[0])], bias)
    assert np.array_equal(p1, w1[0]) and np.array_equal(rows_at(y1, p1, n), w1[1]) and 0 < c1 < b
    # second layer reads the survivors of the first through their positions; y1's row `neurons` is zero
    # because the buffer was created zeroed and the entry point never writes that row
    y2, surv2, c2 = static_call(lib, torch, y1, n, c1, rows[1], vals[1], bias, positions=surv1)
    p2 = surv2[:c2].cpu().numpy()
    w2 = c_oracle.infer(y0, [(rows[0], vals[0]), (rows[1], vals[1])], bias)
    assert np.array_equal(p1[p2], w2[0]) and np.array_equal(rows_at(y2, p2, n), w2[1])
    # no images: the count comes back 0 and the scratch stays clean for the call after it
    _, _, c0 = static_call(lib, torch, yin, n, 0, rows[0], vals[0], bias)
    assert c0 == 0
    y1b, surv1b, c1b = static_call(lib, torch, yin, n, b, rows[0], vals[0], bias)
    assert c1b == c1 and torch.equal(surv1b[:c1b], surv1[:c1]) and torch.equal(y1b, y1)


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
    rc = lib.spdnn_layer_static(dummy.data_ptr(), dummy.data_ptr(), 1 << 26, 10, None, idx.data_ptr(), None, 32,
                                0.0625, -0.3, 32.0, idx.data_ptr(), idx.data_ptr(), None, err, 256)
    assert rc == -1
