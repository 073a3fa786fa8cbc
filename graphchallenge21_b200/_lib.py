"""ctypes binding of libspdnn_b200.so (include/spdnn_b200.h).

There is no fallback: if the library is missing it is built with nvcc, and if that is not
possible the import fails loudly.  Nothing here computes on the CPU.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# SPDNN_B200_LIB may point at another build of the same library (e.g. one compiled with
# different tuning macros); by default the in-tree build is used.
LIB_PATH = os.environ.get("SPDNN_B200_LIB") or os.path.join(PKG, "libspdnn_b200.so")

OK = 0


class Stats(C.Structure):
    _fields_ = [("layers", C.c_int32), ("batch", C.c_int32), ("survivors", C.c_int64), ("prepare_ms", C.c_float),
                ("infer_ms", C.c_float), ("algorithmic_bytes", C.c_double), ("kernel_launches", C.c_int64),
                ("loop_launches", C.c_int32), ("resident_group", C.c_int32)]


# every entry point include/spdnn_b200.h declares
SYMBOLS = {
    "spdnn_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_float, C.c_float]),
    "spdnn_set_layer_csc": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "spdnn_set_layer_same_as": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "spdnn_set_layer_coo": (C.c_int, [C.c_void_p, C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int]),
    "spdnn_set_input_dense": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "spdnn_set_input_dense_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int]),
    "spdnn_set_input_coo": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]),
    "spdnn_set_input_bits": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int]),
    "spdnn_set_input_bits_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int]),
    "spdnn_infer": (C.c_int, [C.c_void_p, C.POINTER(Stats)]),
    "spdnn_infer_async": (C.c_int, [C.c_void_p]),
    "spdnn_sync": (C.c_int, [C.c_void_p, C.POINTER(Stats)]),
    "spdnn_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "spdnn_get_layer_live": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int]),
    "spdnn_get_categories": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_int)]),
    "spdnn_get_activations": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64]),
    "spdnn_get_layer_info": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "spdnn_inspect_layer_csc": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int),
                                          C.POINTER(C.c_int)]),
    "spdnn_inspect_network_csc": (C.c_int, [C.c_int, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                            C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p, C.c_void_p]),
    "spdnn_layer_static": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                     C.c_float, C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_char_p,
                                     C.c_int]),
    "spdnn_last_error": (C.c_char_p, [C.c_void_p]),
    "spdnn_destroy": (None, [C.c_void_p]),
    "spdnn_version": (C.c_char_p, []),
}

_lib = None


def load():
    """Load (building first if needed) the CUDA library; raises if that is impossible."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        if os.environ.get("SPDNN_B200_LIB"):
            raise FileNotFoundError(LIB_PATH)
        from . import build
        build.build_library()
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)      # AttributeError here = the library does not match the header
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib
