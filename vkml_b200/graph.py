"""Host-side mirror of the part of vkML's graph layer the backend reads:
``OpKind`` (include/vkml/graph/op.h:30-139), ``DType`` (include/vkml/core/dtype.h:17-23),
the op parameter PODs (op.h:226-318) and a strided tensor description equal to
``vkml::Shape`` + the node address (include/vkml/core/shape.h:60-153).
"""
from __future__ import annotations

import ctypes
import enum
import struct
from dataclasses import dataclass, field
from typing import Sequence

import numpy as np

from . import _abi


class DType(enum.IntEnum):
    F32 = 0
    F16 = 1
    I32 = 2
    I64 = 3
    BOOL = 4

    @property
    def itemsize(self) -> int:
        return {0: 4, 1: 2, 2: 4, 3: 8, 4: 1}[int(self)]

    @property
    def numpy(self):
        return {0: np.float32, 1: np.float16, 2: np.int32, 3: np.int64, 4: np.uint8}[int(self)]

    @staticmethod
    def of(np_dtype) -> "DType":
        dt = np.dtype(np_dtype)
        table = {np.dtype(np.float32): DType.F32, np.dtype(np.float16): DType.F16,
                 np.dtype(np.int32): DType.I32, np.dtype(np.int64): DType.I64,
                 np.dtype(np.uint8): DType.BOOL, np.dtype(np.bool_): DType.BOOL}
        if dt not in table:
            raise TypeError(f"vkml_b200: no vkML dtype for numpy dtype {dt}")
        return table[dt]


_OP_NAMES = """input const full arange rand reshape permute slice broadcast squeeze unsqueeze
contiguous cast cat add sub mul scaled_add div pow maximum minimum equal less greater less_equal
greater_equal not_equal neg abs sign square sqrt rsqrt reciprocal exp log erf erfc sin cos tanh
sigmoid relu gelu silu clamp sum mean max min prod argmax argmin matmul softmax log_softmax im2col
col2im max_pool2d max_pool2d_backward index_select scatter_add slice_backward where triu tril""".split()

Op = enum.IntEnum("Op", {name.upper(): i for i, name in enumerate(_OP_NAMES)})
OP_COUNT = len(_OP_NAMES)


def op_name(op: int) -> str:
    return _OP_NAMES[int(op)]


# -- op parameter PODs, packed exactly as the C++ structs lay them out (x86-64) --

def reduce_params(axes: Sequence[int], ndim: int, keepdim: bool = False) -> bytes:
    mask = 0
    for a in axes:
        mask |= 1 << (a % ndim if ndim else 0)
    return struct.pack("<I?", mask, keepdim)


def axis_params(axis: int) -> bytes:
    return struct.pack("<i", axis)


def scaled_add_params(alpha: float, beta: float) -> bytes:
    return struct.pack("<ff", alpha, beta)


def clamp_params(lo, hi) -> bytes:
    return struct.pack("<ff??", 0.0 if lo is None else lo, 0.0 if hi is None else hi,
                       lo is not None, hi is not None)


def full_params(value: float) -> bytes:
    return struct.pack("<d", value)


def arange_params(start: float, step: float) -> bytes:
    return struct.pack("<dd", start, step)


def rand_params(seed: int, offset: int) -> bytes:
    return struct.pack("<QQ", seed, offset)


def tri_params(diagonal: int) -> bytes:
    return struct.pack("<i", diagonal)


def slice_params(axis: int, start: int, stop: int, step: int) -> bytes:
    return struct.pack("<i4xqqq", axis, start, stop, step)


def unfold_params(kernel, stride, padding, dilation, image) -> bytes:
    return struct.pack("<10i", kernel[0], kernel[1], stride[0], stride[1], padding[0], padding[1],
                       dilation[0], dilation[1], image[0], image[1])


@dataclass
class TensorDesc:
    """A strided view of memory: address, extents, BYTE strides, dtype."""
    data: int
    dims: tuple
    strides: tuple
    dtype: DType

    @property
    def ndim(self) -> int:
        return len(self.dims)

    @property
    def numel(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    @property
    def nbytes(self) -> int:
        return self.numel * self.dtype.itemsize

    @staticmethod
    def contiguous(data: int, dims: Sequence[int], dtype: DType) -> "TensorDesc":
        dims = tuple(int(d) for d in dims)
        strides, acc = [], dtype.itemsize
        for d in reversed(dims):
            strides.append(acc)
            acc *= d
        return TensorDesc(int(data or 0), dims, tuple(reversed(strides)), dtype)

    def to_c(self) -> _abi.Tensor:
        if self.ndim > _abi.MAX_DIMS:
            raise ValueError(f"rank {self.ndim} exceeds {_abi.MAX_DIMS}")
        t = _abi.Tensor()
        t.data = self.data or None
        t.ndim = self.ndim
        t.dtype = int(self.dtype)
        for i in range(_abi.MAX_DIMS):
            t.dims[i] = self.dims[i] if i < self.ndim else 1
            t.strides[i] = self.strides[i] if i < self.ndim else 0
        return t


@dataclass
class NodeDesc:
    """One computed node: op, output view, source views, raw OpParams bytes."""
    op: int
    out: TensorDesc
    src: list = field(default_factory=list)
    params: bytes = b""

    def to_c(self) -> _abi.Node:
        n = _abi.Node()
        n.op = int(self.op)
        n.n_src = len(self.src)
        n.out = self.out.to_c()
        for i, s in enumerate(self.src):
            n.src[i] = s.to_c()
        if self.params:
            ctypes.memmove(n.params, bytes(self.params), min(len(self.params), _abi.PARAM_BYTES))
        return n


def pack_nodes(nodes: Sequence[NodeDesc]):
    arr = (_abi.Node * max(len(nodes), 1))()
    for i, n in enumerate(nodes):
        arr[i] = n.to_c()
    return arr
