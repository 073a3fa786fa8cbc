"""Host-side mirror of the reference's drivers over the C ABI (include/spdnn_b200.h).

``SpDNN`` wraps one context (one GPU).  ``run_network`` keeps the contract of the
reference's single-GPU executable (src/network.cpp:56-125: argv ``neuron batch layer``,
``../data`` files, the ``layer l, batch = k`` lines and the total kernel time) and
``run_multi_gpu`` that of its MPI driver (src/multi_gpu.cpp:57-155: every rank takes a
contiguous slice of the images, weights replicated, no exchange inside the layer loop),
with ``torch.distributed`` ranks in place of MPI ranks and a final gather of the surviving
image numbers that the reference does not perform.
"""
from __future__ import annotations

import ctypes as C
import os
import sys
from dataclasses import dataclass

import numpy as np

from . import _lib, formats
from .generator import BIAS_BY_NEURONS


class SpDNNError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"spdnn error {code}: {message}")
        self.code = code


@dataclass
class InferResult:
    layers: int
    batch: int
    survivors: int
    prepare_ms: float
    infer_ms: float
    algorithmic_bytes: float
    kernel_launches: int
    loop_launches: int = 0
    resident_group: int = 0

    @property
    def edges(self) -> float:
        return float(self.batch) * 32.0 * self.layers    # multiply by neurons for the metric


def _ptr(a):
    return None if a is None else C.c_void_p(a.ctypes.data)


class SpDNN:
    """One inference context on one GPU."""

    def __init__(self, neurons: int, layers: int, bias: float | None = None, clip: float = 32.0, device: int = 0):
        self._lib = _lib.load()
        self.neurons, self.layers = int(neurons), int(layers)
        if bias is None:
            bias = BIAS_BY_NEURONS[neurons]      # src/network.cpp:73-78
        self.bias, self.clip, self.device = float(bias), float(clip), int(device)
        self._ctx = C.c_void_p()
        rc = self._lib.spdnn_create(C.byref(self._ctx), device, neurons, layers, bias, clip)
        if rc != 0:
            msg = self._lib.spdnn_last_error(self._ctx).decode() if self._ctx else "allocation failed"
            if self._ctx:
                self._lib.spdnn_destroy(self._ctx)
                self._ctx = C.c_void_p()
            raise SpDNNError(rc, msg)
        self.batch = 0

    # -- plumbing --------------------------------------------------------------
    def _check(self, rc: int):
        if rc != 0:
            raise SpDNNError(rc, self._lib.spdnn_last_error(self._ctx).decode())

    def close(self):
        if getattr(self, "_ctx", None):
            self._lib.spdnn_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def set_stream(self, cuda_stream: int | None):
        """Enqueue on the caller's CUDA stream (its handle as an integer, e.g.
        ``torch.cuda.current_stream().cuda_stream``); ``None`` restores the context's own."""
        self._check(self._lib.spdnn_set_stream(self._ctx, C.c_void_p(cuda_stream or 0)))

    # -- layers ----------------------------------------------------------------
    def set_layer_csc(self, layer: int, col_ptr, row_idx, val=None):
        col_ptr = np.ascontiguousarray(col_ptr, dtype=np.int32)
        row_idx = np.ascontiguousarray(row_idx, dtype=np.int32)
        if col_ptr.shape != (self.neurons + 1,):
            raise SpDNNError(-1, f"col_ptr must have {self.neurons + 1} entries")
        if row_idx.size != int(col_ptr[-1]):
            raise SpDNNError(-1, "row_idx size must equal col_ptr[-1]")
        if val is not None:
            val = np.ascontiguousarray(val, dtype=np.float32)
            if val.size != row_idx.size:
                raise SpDNNError(-1, "val size must equal row_idx size")
        self._check(self._lib.spdnn_set_layer_csc(self._ctx, layer, _ptr(col_ptr), _ptr(row_idx), _ptr(val)))

    def set_layer_same_as(self, layer: int, other_layer: int):
        """Layer ``layer`` is the matrix of ``other_layer`` (set before): no data is passed again."""
        self._check(self._lib.spdnn_set_layer_same_as(self._ctx, layer, other_layer))

    def set_network(self, net):
        """All layers of a generated network (``layer_csc(l)``, ``pattern_id(l)``): layers with equal
        pattern ids are declared once and aliased afterwards."""
        first = {}
        for l in range(self.layers):
            pid = net.pattern_id(l) if hasattr(net, "pattern_id") else l
            if pid in first:
                self.set_layer_same_as(l, first[pid])
            else:
                self.set_layer_csc(l, *net.layer_csc(l))
                first[pid] = l

    def set_layer_rows(self, layer: int, rows, vals=None):
        """``rows`` int [N, K]: the K input neurons of every output neuron (entries < 0 are skipped)."""
        rows = np.asarray(rows)
        n, k = rows.shape
        if (rows >= 0).all():
            col_ptr = (np.arange(n + 1, dtype=np.int64) * k).astype(np.int32)
            self.set_layer_csc(layer, col_ptr, rows.reshape(-1), None if vals is None else np.asarray(vals).reshape(-1))
            return
        keep = rows >= 0
        col_ptr = np.concatenate([[0], np.cumsum(keep.sum(axis=1))]).astype(np.int32)
        self.set_layer_csc(layer, col_ptr, rows[keep], None if vals is None else np.asarray(vals)[keep])

    def set_layer_coo(self, layer: int, in_neuron, out_neuron, val=None, index_base: int = 1):
        a = np.ascontiguousarray(in_neuron, dtype=np.int32)
        b = np.ascontiguousarray(out_neuron, dtype=np.int32)
        v = None if val is None else np.ascontiguousarray(val, dtype=np.float32)
        if a.size != b.size or (v is not None and v.size != a.size):
            raise SpDNNError(-1, "triplet arrays differ in length")
        self._check(self._lib.spdnn_set_layer_coo(self._ctx, layer, a.size, _ptr(a), _ptr(b), _ptr(v), index_base))

    def layer_info(self, layer: int):
        cls, k, uni = C.c_int(), C.c_int(), C.c_int()
        self._check(self._lib.spdnn_get_layer_info(self._ctx, layer, C.byref(cls), C.byref(k), C.byref(uni)))
        return {"classes": cls.value, "k": k.value, "uniform": bool(uni.value)}

    # -- inputs ----------------------------------------------------------------
    def set_input_dense(self, y0, first_global_id: int = 0):
        """``y0``: [batch, N] float32, a numpy array / CPU torch tensor (host path) or a CUDA
        torch tensor on this context's device (device path, no host copy)."""
        if hasattr(y0, "is_cuda"):                     # torch tensor
            if y0.dim() != 2 or y0.shape[1] != self.neurons:
                raise SpDNNError(-1, f"input must be [batch, {self.neurons}]")
            import torch
            if y0.dtype != torch.float32 or not y0.is_contiguous():
                raise SpDNNError(-1, "input must be contiguous float32")
            self.batch = int(y0.shape[0])
            if y0.is_cuda:
                if y0.device.index != self.device:
                    raise SpDNNError(-1, "input tensor lives on another device")
                fn = self._lib.spdnn_set_input_dense_device
            else:
                fn = self._lib.spdnn_set_input_dense
            self._check(fn(self._ctx, C.c_void_p(y0.data_ptr()), self.batch, first_global_id))
            return
        y0 = np.ascontiguousarray(y0, dtype=np.float32)
        if y0.ndim != 2 or y0.shape[1] != self.neurons:
            raise SpDNNError(-1, f"input must be [batch, {self.neurons}]")
        self.batch = int(y0.shape[0])
        self._check(self._lib.spdnn_set_input_dense(self._ctx, _ptr(y0), self.batch, first_global_id))

    def set_input_coo(self, img, neuron, val, batch: int, first_global_id: int = 0, index_base: int = 1):
        i = np.ascontiguousarray(img, dtype=np.int32)
        n = np.ascontiguousarray(neuron, dtype=np.int32)
        v = None if val is None else np.ascontiguousarray(val, dtype=np.float32)
        if i.size != n.size or (v is not None and v.size != i.size):
            raise SpDNNError(-1, "triplet arrays differ in length")
        self.batch = int(batch)
        self._check(self._lib.spdnn_set_input_coo(self._ctx, i.size, _ptr(i), _ptr(n), _ptr(v), batch, first_global_id,
                                                  index_base))

    def set_input_bits(self, bits, first_global_id: int = 0):
        """``bits``: uint8 [batch, row_bytes] bit matrix, bit (n & 7) of byte n >> 3 of row i = neuron n of image
        i is 1.0 (``pack_bits`` makes it); a numpy array / CPU torch tensor (host path) or a CUDA torch tensor."""
        if hasattr(bits, "is_cuda"):
            import torch
            if bits.dim() != 2 or bits.dtype != torch.uint8 or not bits.is_contiguous():
                raise SpDNNError(-1, "bit matrix must be contiguous uint8 [batch, row_bytes]")
            self.batch = int(bits.shape[0])
            fn = self._lib.spdnn_set_input_bits_device if bits.is_cuda else self._lib.spdnn_set_input_bits
            self._check(fn(self._ctx, C.c_void_p(bits.data_ptr()), int(bits.shape[1]), self.batch, first_global_id))
            return
        bits = np.ascontiguousarray(bits, dtype=np.uint8)
        if bits.ndim != 2:
            raise SpDNNError(-1, "bit matrix must be [batch, row_bytes]")
        self.batch = int(bits.shape[0])
        self._check(self._lib.spdnn_set_input_bits(self._ctx, _ptr(bits), int(bits.shape[1]), self.batch, first_global_id))

    # -- the loop --------------------------------------------------------------
    @staticmethod
    def _result(s: _lib.Stats) -> InferResult:
        return InferResult(s.layers, s.batch, int(s.survivors), float(s.prepare_ms), float(s.infer_ms),
                           float(s.algorithmic_bytes), int(s.kernel_launches), int(s.loop_launches), int(s.resident_group))

    def infer(self) -> InferResult:
        s = _lib.Stats()
        self._check(self._lib.spdnn_infer(self._ctx, C.byref(s)))
        return self._result(s)

    def infer_async(self):
        self._check(self._lib.spdnn_infer_async(self._ctx))

    def sync(self) -> InferResult:
        s = _lib.Stats()
        self._check(self._lib.spdnn_sync(self._ctx, C.byref(s)))
        return self._result(s)

    # -- results ---------------------------------------------------------------
    def layer_live(self) -> np.ndarray:
        live = np.zeros(self.layers, dtype=np.int32)
        self._check(self._lib.spdnn_get_layer_live(self._ctx, _ptr(live), live.size))
        return live

    def categories(self, out=None) -> np.ndarray:
        """Ascending global image numbers alive after the last layer (0-based + first_global_id)."""
        cap = max(self.batch, 1)
        ids = out if out is not None else np.empty(cap, dtype=np.int32)
        cnt = C.c_int()
        self._check(self._lib.spdnn_get_categories(self._ctx, _ptr(ids), ids.size, C.byref(cnt)))
        return ids[: cnt.value]

    def activations(self) -> np.ndarray:
        count = len(self.categories())
        y = np.empty((count, self.neurons), dtype=np.float32)
        self._check(self._lib.spdnn_get_activations(self._ctx, _ptr(y) if count else None, count))
        return y


def pack_bits(y0: np.ndarray) -> np.ndarray:
    """[batch, N] array -> the bit matrix ``set_input_bits`` takes (non-zero = 1), rows padded to whole 32-bit words."""
    y0 = np.asarray(y0)
    b, n = y0.shape
    out = np.zeros((b, (n + 31) // 32 * 4), dtype=np.uint8)
    out[:, : (n + 7) // 8] = np.packbits(y0 != 0, axis=1, bitorder="little")
    return out


def inspect_network(neurons: int, layer_csc) -> dict:
    """Host-only analysis of a network (no GPU): per layer the classes in value ids, the value
    ids read and the resident kernel's table form (0 = K gathers, 1 = alternating pair).
    ``layer_csc``: sequence of (col_ptr, row_idx, val_or_None)."""
    lib = _lib.load()
    keep, cps, ris, vs = [], [], [], []
    for cp, ri, v in layer_csc:
        cp = np.ascontiguousarray(cp, dtype=np.int32); ri = np.ascontiguousarray(ri, dtype=np.int32)
        v = None if v is None else np.ascontiguousarray(v, dtype=np.float32)
        keep.append((cp, ri, v))
        cps.append(cp.ctypes.data); ris.append(ri.ctypes.data); vs.append(None if v is None else v.ctypes.data)
    n = len(keep)
    arr = lambda xs: (C.c_void_p * max(n, 1))(*xs)
    classes, v_in, form = (np.zeros(max(n, 1), dtype=np.int32) for _ in range(3))
    rc = lib.spdnn_inspect_network_csc(neurons, n, arr(cps), arr(ris), arr(vs), _ptr(classes), _ptr(v_in), _ptr(form))
    if rc != 0:
        raise SpDNNError(rc, "malformed layer")
    return {"classes": classes[:n], "v_in": v_in[:n], "form": form[:n]}


# ---- the reference's drivers ---------------------------------------------------------------

def load_network_from_files(net: SpDNN, data_dir: str, log=None):
    """Every rank/driver reads all layers (src/network.cpp:97-121, src/multi_gpu.cpp:116-145)."""
    for l in range(net.layers):
        path = formats.weight_file_name(data_dir, net.neurons, l)
        a, b, v = formats.read_layer_tsv(path)
        net.set_layer_coo(l, a, b, v, index_base=1)
        if log:
            log(f"[{path}] to COO success!")


def shard_bounds(batch: int, world: int, rank: int):
    """Contiguous slice [lo, hi) of the images for ``rank`` (src/microbenchmark/multi_gpu/multi_gpu.cu:251-258
    with the slice length ceil(batch/world) in place of the hard-wired (batch+1)/2 of src/multi_gpu.cpp:151)."""
    per = (batch + world - 1) // world
    lo = min(rank * per, batch)
    return lo, min(lo + per, batch)


def run_network(neuron: int, batch: int, layer: int, data_dir: str = "../data", device: int = 0, out=None,
                categories_path: str | None = None):
    """``./single.out neuron batch layer`` (src/network.cpp:56-125).  Returns the 0-based
    category list; prints the reference's progress lines to ``out`` (default stdout)."""
    out = out or sys.stdout
    say = lambda s: print(s, file=out)
    say("[BEGIN]...")
    img, neu, val = formats.read_input_tsv(formats.input_file_name(data_dir, neuron), batch)
    for i in np.nonzero(val != 1.0)[0][:16]:
        say(f"read input {img[i]}, {val[i]:f}")                      # src/network.cpp:49-51
    say(f"Read Input success! read_numeber = {img.size}")
    say("Read Input success!")
    with SpDNN(neuron, layer, BIAS_BY_NEURONS[neuron], 32.0, device) as net:
        load_network_from_files(net, data_dir, say)
        net.set_input_coo(img, neu, val, batch, 0, index_base=1)
        res = net.infer()
        for l, k in enumerate(net.layer_live().tolist()):
            say(f"layer {l}, batch = {k}")                            # all_network.cu:508
        say(f"Kernel Exec Time [20-uiuc-row-succ] = {res.infer_ms}ms")  # all_network.cu:522
        upper = res.algorithmic_bytes / 1e9 / 700.0 * 1000.0          # the reference's 700 GB/s model, :335-340
        say(f"Kernel Exec Upper Time = {upper}ms")
        cats = net.categories().copy()
    if categories_path:
        formats.write_categories(categories_path, cats)
    truth = formats.truth_file_name(data_dir, neuron, layer)
    if os.path.exists(truth):                     # the challenge's truth categories, when they were downloaded
        v = formats.compare_categories(cats, truth, batch)
        say(f"Challenge {'PASSED' if v['passed'] else 'FAILED'}: {v['got']} categories, truth {v['truth']}")
    say("[END]...")
    return cats


def gather_categories(local_ids: np.ndarray, group=None, capacity: int | None = None) -> np.ndarray:
    """The one exchange step: every rank's ascending list of surviving global image numbers
    is gathered on all ranks and concatenated in rank order (slices are contiguous, so the
    result is ascending).  Uses ``torch.distributed`` (NCCL or gloo) when initialised.
    ``capacity``: an upper bound of any rank's list length that every rank knows (the largest
    shard); with it the exchange is ONE all-gather of ``capacity + 1`` int32 per rank (count, then
    the numbers), without it the counts are exchanged first."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return np.asarray(local_ids, dtype=np.int32)
    world = dist.get_world_size(group)
    backend = dist.get_backend(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if backend == "nccl" else torch.device("cpu")
    local = np.ascontiguousarray(local_ids, dtype=np.int32)
    if capacity is not None:
        if len(local) > capacity:
            raise ValueError("more survivors than the stated capacity")
        mine = np.empty(capacity + 1, dtype=np.int32)
        mine[0] = len(local)
        mine[1:1 + len(local)] = local
        mine[1 + len(local):] = -1
        everyone = torch.empty(world * (capacity + 1), dtype=torch.int32, device=dev)
        dist.all_gather_into_tensor(everyone, torch.from_numpy(mine).to(dev), group=group)
        got = everyone.cpu().numpy().reshape(world, capacity + 1)
        return np.concatenate([got[r, 1:1 + got[r, 0]] for r in range(world)]).astype(np.int32)
    n_local = torch.tensor([len(local)], dtype=torch.int64, device=dev)
    counts = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
    dist.all_gather(counts, n_local, group=group)
    counts = [int(c.item()) for c in counts]
    cap = max(max(counts), 1)
    buf = torch.full((cap,), -1, dtype=torch.int32, device=dev)
    if len(local):
        buf[: len(local)] = torch.from_numpy(local).to(dev)
    parts = [torch.empty(cap, dtype=torch.int32, device=dev) for _ in range(world)]
    dist.all_gather(parts, buf, group=group)
    return np.concatenate([p[:c].cpu().numpy() for p, c in zip(parts, counts)]).astype(np.int32)


def run_multi_gpu(neuron: int, batch: int, layer: int, data_dir: str = "../data", out=None, engine_factory=None):
    """``mpirun -np G ./run_multi_gpu neuron batch layer`` (src/multi_gpu.cpp:57-155) with
    ``torch.distributed`` ranks: rank r runs images [r*ceil(B/G), ...) on GPU LOCAL_RANK and
    the survivors are gathered at the end.  ``engine_factory(neuron, layer, bias, device)``
    may replace the context class (used by host-logic tests)."""
    import os
    import torch.distributed as dist
    out = out or sys.stdout
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    device = int(os.environ.get("LOCAL_RANK", rank))
    say = lambda s: print(f"GPU[{rank}] {s}", file=out)
    say("[BEGIN]...")
    img, neu, val = formats.read_input_tsv(formats.input_file_name(data_dir, neuron), batch)
    say("Read Input success!")
    lo, hi = shard_bounds(batch, world, rank)
    keep = (img > lo) & (img <= hi)                     # img is 1-based
    factory = engine_factory or (lambda n, l, b, d: SpDNN(n, l, b, 32.0, d))
    net = factory(neuron, layer, BIAS_BY_NEURONS[neuron], device)
    try:
        load_network_from_files(net, data_dir, None)
        net.set_input_coo(img[keep] - lo, neu[keep], val[keep], hi - lo, lo, index_base=1)
        net.infer()
        live = net.layer_live()
        for l in range(0, layer, 100):
            say(f"[GPU {device}], Layer {l}, Batch = {int(live[l])}")    # multi_gpu.cu:517-518
        local = np.asarray(net.categories()).copy()
    finally:
        net.close()
    say("[END]...")
    return gather_categories(local, capacity=(batch + world - 1) // world)
