"""Seeded synthetic stand-ins for the Graph Challenge sparse-DNN data set.

The reference ships no data (its ``../data`` tree is git-ignored) and reads
``../data/neuron{N}/n{N}-l{k}.tsv`` weight layers and
``../data/sparse-images-{N}.tsv`` inputs (src/network.cpp:14-19, 33-54).  This
module produces networks and inputs with the same shapes and value
distributions: N x N layers with exactly 32 non-zeros per column, every value
0.0625, the per-size biases of src/network.cpp:73-78, and binary inputs on a
sqrt(N) x sqrt(N) pixel grid.

Two sparsity patterns are offered.

``radix16``
    RadiX-Net-like.  The pattern is defined in the reference's hash-permuted
    neuron numbering (src/reorder/hash.h:14-22) where it is a butterfly of
    16-wide blocks: the inputs of output ``c`` are ``16*floor(c/16) + [0,16)``
    and the same run shifted by ``stride`` (mod N), with ``stride = 16`` for
    layer 0 and ``16 * 2**k``, k cycling over 1..T-1, afterwards (the strides of
    src/microbenchmark/all_network.cu:316-327 and the type-1 layer counts T of
    src/network.cpp:80-85).  It is then written through the inverse permutation,
    so in file numbering the pattern looks scattered, as the challenge files do.

``random``
    Every column draws 32 distinct rows uniformly at random.

Everything is a pure function of (seed, coordinates) through a counter-based
64-bit mixer, so any slice can be regenerated anywhere without shipping files.
"""
from __future__ import annotations

import numpy as np

NNZ_PER_COL = 32
WEIGHT_VALUE = np.float32(0.0625)
CLIP = np.float32(32.0)

# src/network.cpp:73-78
BIAS_BY_NEURONS = {1024: -0.3, 4096: -0.35, 16384: -0.4, 65536: -0.45}
# src/network.cpp:80-85 (number of "type-1" butterfly layers)
TYPE1_BY_NEURONS = {1024: 6, 4096: 8, 16384: 10, 65536: 12}

_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_GOLD = np.uint64(0x9E3779B97F4A7C15)


def mix64(x):
    """splitmix64 finaliser on uint64 arrays (wrap-around arithmetic)."""
    x = np.asarray(x, dtype=np.uint64)
    with np.errstate(over="ignore"):
        x = (x ^ (x >> np.uint64(30))) * _M1
        x = (x ^ (x >> np.uint64(27))) * _M2
        x = x ^ (x >> np.uint64(31))
    return x


def rand_u64(seed, stream, index):
    """Counter-based random uint64: a function of (seed, stream, index) only."""
    with np.errstate(over="ignore"):
        s = mix64(np.uint64(seed) + _GOLD * np.uint64(stream + 1))
        return mix64(s ^ (np.asarray(index, dtype=np.uint64) * _GOLD + _GOLD))


def rand_unit(seed, stream, index):
    """Uniform float64 in [0, 1) from the top 53 bits of ``rand_u64``."""
    return (rand_u64(seed, stream, index) >> np.uint64(11)).astype(np.float64) * (1.0 / (1 << 53))


def default_bias(neurons: int) -> float:
    if neurons in BIAS_BY_NEURONS:
        return BIAS_BY_NEURONS[neurons]
    # between the tabulated sizes: same trend (-0.05 per factor 4)
    return -0.3 - 0.05 * (np.log2(max(neurons, 1)) - 10.0) / 2.0


def hash_buckets(neurons: int) -> int:
    """Bucket count the reference uses: N/16 (src/network.cpp:66-71)."""
    return max(neurons // 16, 1)


def hash_reorder(v, neurons: int):
    """``h(v) = v div buckets + (v mod buckets) * (N div buckets)`` (src/reorder/hash.h:14-22)."""
    b = hash_buckets(neurons)
    v = np.asarray(v)
    return v // b + (v % b) * (neurons // b)


def hash_reorder_inverse(h, neurons: int):
    b = hash_buckets(neurons)
    w = neurons // b
    h = np.asarray(h)
    return (h % w) * b + h // w


class SyntheticNetwork:
    """L layers of an N x N matrix with exactly 32 non-zeros per column."""

    def __init__(self, neurons: int, layers: int, pattern: str = "radix16", seed: int = 0x5EED0000,
                 bias: float | None = None):
        if pattern not in ("radix16", "random"):
            raise ValueError("pattern must be 'radix16' or 'random'")
        if neurons < 64 or neurons % 32:
            raise ValueError("neurons must be a multiple of 32 and at least 64")
        self.neurons = int(neurons)
        self.layers = int(layers)
        self.pattern = pattern
        self.seed = int(seed)
        self.bias = np.float32(default_bias(neurons) if bias is None else bias)
        self.clip = CLIP
        self.value = WEIGHT_VALUE
        self._cache: dict[int, np.ndarray] = {}

    # -- pattern bookkeeping -------------------------------------------------
    def _num_strides(self) -> int:
        # strides 16*2^k must stay below N: k = 0 .. log2(N/16)-1
        return max(int(np.log2(self.neurons // 16)), 1)

    def pattern_id(self, layer: int) -> int:
        """Layers with equal ``pattern_id`` have identical matrices."""
        if self.pattern == "random":
            return layer
        if layer == 0:
            return 0
        t = min(TYPE1_BY_NEURONS.get(self.neurons, self._num_strides()), self._num_strides())
        if t <= 1:
            return 0
        return 1 + (layer - 1) % (t - 1)

    def num_patterns(self) -> int:
        return len({self.pattern_id(l) for l in range(self.layers)})

    # -- layers --------------------------------------------------------------
    def layer_rows(self, layer: int) -> np.ndarray:
        """int32 [N, 32]: for every output neuron (column of W) its 32 input
        neurons (rows of W) in ascending order."""
        pid = self.pattern_id(layer)
        if pid not in self._cache:
            rows = self._radix16_rows(pid) if self.pattern == "radix16" else self._random_rows(pid)
            rows.setflags(write=False)
            if len(self._cache) > 64:
                self._cache.clear()
            self._cache[pid] = rows
        return self._cache[pid]

    def _radix16_rows(self, k: int) -> np.ndarray:
        n = self.neurons
        stride = 16 << k
        cp = np.arange(n, dtype=np.int64)            # column, permuted numbering
        base = (cp // 16) * 16
        run = np.arange(16, dtype=np.int64)
        rows_p = np.concatenate([base[:, None] + run[None, :],
                                 (base[:, None] + stride + run[None, :]) % n], axis=1)
        rows_f = hash_reorder_inverse(rows_p, n)      # file numbering
        col_f = hash_reorder_inverse(cp, n)
        out = np.empty((n, NNZ_PER_COL), dtype=np.int32)
        out[col_f] = np.sort(rows_f, axis=1).astype(np.int32)
        return out

    def _random_rows(self, layer: int) -> np.ndarray:
        n = self.neurons
        idx = np.arange(n * NNZ_PER_COL, dtype=np.uint64).reshape(n, NNZ_PER_COL)
        rows = (rand_u64(self.seed, 1000 + layer, idx) % np.uint64(n)).astype(np.int64)
        rows.sort(axis=1)
        attempt = 0
        while True:
            bad = np.nonzero((np.diff(rows, axis=1) == 0).any(axis=1))[0]
            if bad.size == 0:
                break
            attempt += 1
            sub = idx[bad] + np.uint64(attempt) * np.uint64(n * NNZ_PER_COL)
            rows[bad] = np.sort((rand_u64(self.seed, 1000 + layer, sub) % np.uint64(n)).astype(np.int64), axis=1)
        return rows.astype(np.int32)

    def layer_csc(self, layer: int):
        """(col_ptr int32[N+1], row_idx int32[32N], val float32[32N]) of layer ``layer``."""
        rows = self.layer_rows(layer)
        col_ptr = (np.arange(self.neurons + 1, dtype=np.int64) * NNZ_PER_COL).astype(np.int32)
        val = np.full(rows.size, self.value, dtype=np.float32)
        return col_ptr, np.ascontiguousarray(rows).reshape(-1), val

    def layer_coo_1based(self, layer: int):
        """The triplets of the reference's layer file, ``a b v`` with a = input
        neuron, b = output neuron, both 1-based (src/utils/matrix.h:273-277)."""
        rows = self.layer_rows(layer)
        b = np.repeat(np.arange(1, self.neurons + 1, dtype=np.int32), NNZ_PER_COL)
        a = rows.reshape(-1) + 1
        v = np.full(a.size, self.value, dtype=np.float32)
        return a, b, v


def synthetic_images(neurons: int, batch: int, seed: int = 0x1A6E5, first_image: int = 0,
                     density: float = 0.15, discs: int = 3, threads: int = 1) -> np.ndarray:
    """Binary float32 [batch, N] inputs: per image ``discs`` filled discs of
    random centre and radius on the sqrt(N) x sqrt(N) grid (stroke-like blobs),
    scaled so that about ``density`` of the pixels are 1.0.  Image ``i`` of the
    result is global image ``first_image + i`` and depends on nothing else
    (``threads`` only spreads the work over host threads)."""
    g = int(round(np.sqrt(neurons)))
    if g * g != neurons:
        raise ValueError("neurons must be a perfect square")
    out = np.empty((batch, neurons), dtype=np.float32)
    # mean radius so that `discs` discs cover ~density of the grid after the
    # typical overlap and border clipping (calibrated factor 1.17)
    r_mean = g * np.sqrt(density * 1.17 / (np.pi * discs))
    yy, xx = np.meshgrid(np.arange(g, dtype=np.float32), np.arange(g, dtype=np.float32), indexing="ij")
    chunk = max(1, min(batch, (1 << 22) // max(neurons, 1)))

    def fill(s):
        e = min(batch, s + chunk)
        ids = np.arange(first_image + s, first_image + e, dtype=np.uint64)
        on = np.zeros((e - s, g, g), dtype=bool)
        for d in range(discs):
            key = ids * np.uint64(16) + np.uint64(d * 3)
            cx = (rand_unit(seed, 7, key) * g).astype(np.float32)
            cy = (rand_unit(seed, 7, key + np.uint64(1)) * g).astype(np.float32)
            rr = ((0.55 + 0.9 * rand_unit(seed, 7, key + np.uint64(2))) * r_mean).astype(np.float32)
            d2 = (xx[None] - cx[:, None, None]) ** 2 + (yy[None] - cy[:, None, None]) ** 2
            on |= d2 <= (rr * rr)[:, None, None]
        out[s:e] = on.reshape(e - s, neurons)

    starts = range(0, batch, chunk)
    if threads > 1 and len(starts) > 1:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(threads) as pool:
            list(pool.map(fill, starts))
    else:
        for s in starts:
            fill(s)
    return out


def mixed_density_images(neurons: int, batch: int, seed: int = 0xABCD, lo: float = 0.05, hi: float = 0.6,
                         first_image: int = 0) -> np.ndarray:
    """Binary float32 [batch, N] inputs without spatial structure whose per-image density is
    spread uniformly over [lo, hi].  On networks without locality (pattern 'random') a
    15 %-dense image dies within three layers; the dense end of this mix survives, which makes
    it the input of the generality tests and of the 'random' benchmark runs."""
    ids = np.arange(first_image, first_image + batch, dtype=np.uint64)
    idx = ids[:, None] * np.uint64(neurons) + np.arange(neurons, dtype=np.uint64)[None, :]
    dens = lo + (hi - lo) * rand_unit(seed, 3, ids)
    return (rand_unit(seed, 4, idx) < dens[:, None]).astype(np.float32)


def dense_to_coo_1based(dense: np.ndarray, first_image: int = 0):
    """The triplets of the reference's input file, ``img neuron val`` 1-based
    (src/network.cpp:33-54)."""
    img, neuron = np.nonzero(dense)
    return (img + 1 + first_image).astype(np.int32), (neuron + 1).astype(np.int32), dense[img, neuron].astype(np.float32)
