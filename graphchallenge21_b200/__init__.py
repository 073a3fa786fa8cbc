"""B200 (sm_100a) implementation of the Graph Challenge sparse-DNN inference loop
``Y <- min(32, ReLU(Y W + b))``: a drop-in for the GPU execution functions of
CGCL-codes/Graphchallenge21 (src/microbenchmark/all_network.cu, multi_gpu/multi_gpu.cu).

``SpDNN`` mirrors the C ABI (include/spdnn_b200.h); ``run_network`` /
``run_multi_gpu`` mirror the reference's drivers (src/network.cpp, src/multi_gpu.cpp).
"""
from .network import SpDNN, SpDNNError, InferResult, run_network, run_multi_gpu  # noqa: F401
from .generator import SyntheticNetwork, synthetic_images  # noqa: F401

__all__ = ["SpDNN", "SpDNNError", "InferResult", "run_network", "run_multi_gpu", "SyntheticNetwork",
           "synthetic_images"]
