"""B200-native runtime behind the ncnn-compiler C ABI: Python binding for tests and benchmarks.

The product is libncnn_b200.so (C++/CUDA, sources under csrc/, C ABI in
include/ncnn_b200.h).  This package only loads it through ctypes and mirrors the
way the reference's tests drive a compiled model: load, call the entry point with
contiguous fp32 [C][H][W] buffers, read a status code.
"""
from .runtime import (DynamicModel, Model, MultiModel, multi_partition, NcnnB200Error, describe, lib_path, load_library, op_dequantize,
                      op_quantize, op_requantize, inner_product_int8_noalloc, FP32_SPLIT, TF32, FP32_CUDA)
from . import zoo  # noqa: F401
from .sharding import gather_outputs, shard_range

__all__ = ["DynamicModel", "Model", "MultiModel", "multi_partition", "NcnnB200Error", "describe", "lib_path", "load_library", "op_quantize",
           "op_dequantize", "op_requantize", "inner_product_int8_noalloc", "zoo", "shard_range", "gather_outputs", "FP32_SPLIT", "TF32", "FP32_CUDA"]
