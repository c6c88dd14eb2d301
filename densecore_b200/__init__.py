"""densecore_b200: DenseCore's quantized decode hot path on NVIDIA B200.

The compute lives in libdc_b200.so (hand-written sm_100a CUDA behind the C ABI
of include/dc_b200.h).  This package is the Python host-side mirror of the
reference's op interface, used by the tests and the benchmark.
"""
from .blocks import (GGML_TYPE_F16, GGML_TYPE_F32, GGML_TYPE_Q4_K, GGML_TYPE_Q6_K, QK_K, row_bytes)
from ._lib import DcError
from .ops import Context, KVCache, Weight
from .model import Config, Model, dense_0p8b, moe_35b_a3b, tensor_seed
from .spec import speculative_decode
from .sched import Scheduler

__all__ = ["Context", "Weight", "KVCache", "Model", "Config", "dense_0p8b", "moe_35b_a3b", "tensor_seed", "speculative_decode", "Scheduler", "DcError", "GGML_TYPE_F32", "GGML_TYPE_F16", "GGML_TYPE_Q4_K", "GGML_TYPE_Q6_K",
           "QK_K", "row_bytes"]
