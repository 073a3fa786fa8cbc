"""Readers and writers for the reference's on-disk formats.

* weight layer ``neuron{N}/n{N}-l{k}.tsv``: lines ``a b v`` (1-based), ``W[a][b] = v`` with
  a the input neuron and b the output neuron (src/utils/matrix.h:255-282, T == false);
* inputs ``sparse-images-{N}.tsv``: lines ``img neuron val`` (1-based); only ``img <= batch``
  is kept (src/network.cpp:33-54);
* binary variants of the side benchmarks (benchmark/cusparse/cusparse.cu:335-357, 362-383):
  ``neuron{N}.bin`` = per layer ``int32 row[nnz], int32 col[nnz], float val[nnz]`` (1-based),
  ``sparse-images-{N}.bin`` = ``int32 neuron[nnz], int32 image[nnz], float val[nnz]``;
* category list ``neuron{N}-l{L}-categories.tsv``: one 1-based surviving image number per
  line (tools/get_dataset.sh:15; the reference never writes one).
"""
from __future__ import annotations

import os

import numpy as np


def weight_file_name(data_dir: str, neurons: int, layer: int) -> str:
    """Path of 0-based layer ``layer`` (src/network.cpp:14-19)."""
    return os.path.join(data_dir, f"neuron{neurons}", f"n{neurons}-l{layer + 1}.tsv")


def input_file_name(data_dir: str, neurons: int) -> str:
    return os.path.join(data_dir, f"sparse-images-{neurons}.tsv")


def _read_triplets(path: str):
    if not os.path.exists(path):
        raise FileNotFoundError(f"FILE:{path} does not exists.")
    try:
        import pandas as pd
        df = pd.read_csv(path, sep=r"\s+", header=None, names=["a", "b", "v"],
                         dtype={"a": np.int32, "b": np.int32, "v": np.float32}, engine="c")
        return df["a"].to_numpy(), df["b"].to_numpy(), df["v"].to_numpy()
    except ImportError:
        arr = np.loadtxt(path, dtype=np.float64, ndmin=2)
        return arr[:, 0].astype(np.int32), arr[:, 1].astype(np.int32), arr[:, 2].astype(np.float32)


def read_layer_tsv(path: str):
    """(in_neuron, out_neuron, val), 1-based, in file order."""
    return _read_triplets(path)


def write_layer_tsv(path: str, in_neuron, out_neuron, val) -> None:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
        for a, b, v in zip(np.asarray(in_neuron).tolist(), np.asarray(out_neuron).tolist(), np.asarray(val).tolist()):
            f.write(f"{a}\t{b}\t{v!r}\n")


def read_input_tsv(path: str, batch: int):
    """(img, neuron, val), 1-based, restricted to img <= batch."""
    img, neuron, val = _read_triplets(path)
    keep = img <= batch
    return img[keep], neuron[keep], val[keep]


def write_input_tsv(path: str, img, neuron, val) -> None:
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
        for a, b, v in zip(np.asarray(img).tolist(), np.asarray(neuron).tolist(), np.asarray(val).tolist()):
            f.write(f"{a}\t{b}\t{v!r}\n")


def write_categories(path: str, ids_zero_based) -> None:
    """One 1-based image number per line."""
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    with open(path, "w") as f:
        for i in np.asarray(ids_zero_based).tolist():
            f.write(f"{i + 1}\n")


def read_categories(path: str) -> np.ndarray:
    """0-based image numbers from a category file."""
    txt = open(path).read().split()
    return np.asarray([int(float(t)) - 1 for t in txt], dtype=np.int32)


def write_weights_bin(path: str, layers) -> None:
    """``layers``: iterable of (in_neuron, out_neuron, val) 1-based triplets, one per layer."""
    with open(path, "wb") as f:
        for a, b, v in layers:
            f.write(np.asarray(a, dtype=np.int32).tobytes())
            f.write(np.asarray(b, dtype=np.int32).tobytes())
            f.write(np.asarray(v, dtype=np.float32).tobytes())


def read_weights_bin(path: str, neurons: int, layers: int, nnz_per_layer: int | None = None):
    """Yields (in_neuron, out_neuron, val) per layer from ``neuron{N}.bin``."""
    nnz = 32 * neurons if nnz_per_layer is None else nnz_per_layer
    with open(path, "rb") as f:
        for _ in range(layers):
            a = np.fromfile(f, dtype=np.int32, count=nnz)
            b = np.fromfile(f, dtype=np.int32, count=nnz)
            v = np.fromfile(f, dtype=np.float32, count=nnz)
            if v.size != nnz:
                raise ValueError(f"{path}: truncated layer")
            yield a, b, v


def write_input_bin(path: str, img, neuron, val) -> None:
    with open(path, "wb") as f:
        f.write(np.asarray(neuron, dtype=np.int32).tobytes())
        f.write(np.asarray(img, dtype=np.int32).tobytes())
        f.write(np.asarray(val, dtype=np.float32).tobytes())


def read_input_bin(path: str, batch: int | None = None):
    """(img, neuron, val) 1-based from ``sparse-images-{N}.bin``."""
    nnz = os.path.getsize(path) // 12
    with open(path, "rb") as f:
        neuron = np.fromfile(f, dtype=np.int32, count=nnz)
        img = np.fromfile(f, dtype=np.int32, count=nnz)
        val = np.fromfile(f, dtype=np.float32, count=nnz)
    if batch is not None:
        keep = img <= batch
        img, neuron, val = img[keep], neuron[keep], val[keep]
    return img, neuron, val


def truth_file_name(data_dir: str, neurons: int, layers: int) -> str:
    """The challenge's truth file for a network, next to the data (tools/get_dataset.sh:15)."""
    return os.path.join(data_dir, f"neuron{neurons}-l{layers}-categories.tsv")


def compare_categories(ids_zero_based, truth_path: str, batch: int | None = None) -> dict:
    """Compares a category list with a truth file (1-based image numbers, one per line; only
    images <= batch count when the run used a truncated batch).  Returns the verdict and the
    differences."""
    truth = read_categories(truth_path)
    if batch is not None:
        truth = truth[truth < batch]
    got = np.asarray(ids_zero_based, dtype=np.int64)
    missing = np.setdiff1d(truth, got)
    extra = np.setdiff1d(got, truth)
    return {"passed": missing.size == 0 and extra.size == 0, "truth": int(truth.size), "got": int(got.size),
            "missing": missing[:16].tolist(), "extra": extra[:16].tolist()}
