"""vkml_b200: a B200 (sm_100a) execution backend behind vkML's backend interface.

The product is the CUDA library ``lib/libvkml_b200.so`` with the C ABI declared in
``include/vkml_b200.h``; ``adapter/`` holds the C++ class that plugs it into vkML as
a ``vkml::Backend``.  This Python package is a thin ctypes mirror of that backend
interface for tests, benchmarks and scripting.
"""
from .backend import (Backend, DeviceTensor, Storage, Error, ShapeError, DTypeError, DeviceError,
                      OutOfMemoryError, InternalError, COMPUTE_SYNC, COMPUTE_GRAD_SYNC, GEMM_3XTF32,
                      GEMM_TF32, GEMM_FP32)
from .graph import DType, Op, NodeDesc, TensorDesc, op_name
from . import graph

__all__ = ["Backend", "DeviceTensor", "Storage", "DType", "Op", "NodeDesc", "TensorDesc", "graph",
           "op_name", "Error", "ShapeError", "DTypeError", "DeviceError", "OutOfMemoryError",
           "InternalError", "COMPUTE_SYNC", "COMPUTE_GRAD_SYNC", "GEMM_3XTF32", "GEMM_TF32", "GEMM_FP32"]
