"""Shared test machinery: three evaluators of one node-descriptor interface and
the seeded case generator.

``OracleImpl``  -- oracle/libvkml_oracle.so, the C restatement (host memory)
``RefImpl``     -- oracle/_ref/libvkml_ref.so, the reference CPU backend compiled
                  from its own sources (host memory)
``CudaImpl``    -- the product: vkml_b200 through the C ABI (device memory)

A source operand is a numpy array VIEW: transposes, slices and ``np.broadcast_to``
give exactly the byte strides / stride-0 broadcasts vkML's view ops produce, and the
array's ``.base`` chain tells the CUDA evaluator which buffer to upload.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

import vkml_b200
from vkml_b200 import _abi, graph
from vkml_b200.graph import DType, NodeDesc, Op, TensorDesc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_SO = os.path.join(ROOT, "oracle", "libvkml_oracle.so")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libvkml_ref.so")
REF_B200_SO = os.path.join(ROOT, "oracle", "_ref", "libvkml_ref_b200.so")

STATUS_OK = 0


def host_desc(a: np.ndarray) -> TensorDesc:
    return TensorDesc(a.ctypes.data if a.size else (a.ctypes.data or 0), a.shape, a.strides, DType.of(a.dtype))


def root_of(a: np.ndarray) -> np.ndarray:
    while isinstance(a.base, np.ndarray):
        a = a.base
    return a


class HostImpl:
    """Evaluates descriptors on host memory through a `compute(nodes, n)` C function."""

    def __init__(self, path: str, symbol: str):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        self.fn = getattr(self.lib, symbol)
        self.fn.restype = C.c_int
        self.fn.argtypes = [C.POINTER(_abi.Node), C.c_size_t]

    def run_status(self, op, srcs, out_shape, out_dtype, params=b""):
        out = np.zeros(out_shape, dtype=DType(out_dtype).numpy)
        node = NodeDesc(int(op), host_desc(out), [host_desc(s) for s in srcs], params)
        c = node.to_c()
        rc = self.fn(C.byref(c), 1)
        return rc, out

    def run(self, op, srcs, out_shape, out_dtype, params=b""):
        rc, out = self.run_status(op, srcs, out_shape, out_dtype, params)
        assert rc == STATUS_OK, f"{type(self).__name__}: status {rc} for op {graph.op_name(op)}"
        return out


class OracleImpl(HostImpl):
    def __init__(self):
        super().__init__(ORACLE_SO, "vkml_oracle_compute")


class RefImpl(HostImpl):
    def __init__(self):
        super().__init__(REF_SO, "vkml_ref_compute")


class CudaImpl:
    def __init__(self, backend: vkml_b200.Backend):
        self.b = backend

    def _upload(self, view: np.ndarray, cache: dict):
        root = root_of(view)
        key = id(root)
        if key not in cache:
            flat = np.ascontiguousarray(root).reshape(-1) if root.flags["C_CONTIGUOUS"] else None
            assert flat is not None, "roots of test operands are contiguous"
            st = self.b.allocate(max(root.nbytes, 1))
            if root.nbytes:
                self.b.copy_from_host(st, 0, flat)
            cache[key] = (st, root)
        st, root = cache[key]
        offset = view.ctypes.data - root.ctypes.data if view.size else 0
        return TensorDesc(st.data + offset, view.shape, view.strides, DType.of(view.dtype))

    def run(self, op, srcs, out_shape, out_dtype, params=b"", sync_check=True):
        cache = {}
        descs = [self._upload(s, cache) for s in srcs]
        dt = DType(out_dtype)
        out_desc = TensorDesc.contiguous(0, out_shape, dt)
        st = self.b.allocate(out_desc.nbytes)
        out_desc.data = st.data
        node = NodeDesc(int(op), out_desc, descs, params)
        assert self.b.supports(node), f"backend declines op {graph.op_name(op)}"
        self.b.compute([node])
        out = np.empty(out_shape, dtype=dt.numpy)
        if out.nbytes:
            self.b.copy_to_host(out, st, 0)
        if sync_check:
            self.b.synchronize()
        return out


# ---------------------------------------------------------------------------
# layouts
# ---------------------------------------------------------------------------

def layouts(rng: np.random.Generator, shape, dtype=np.float32, scale=1.0):
    """Yield (tag, view) pairs of the same logical values under different strides:
    dense, transposed storage, a strided slice of a larger buffer, and an offset
    view -- the layout generator of vkML's device-vs-CPU suite
    (tests/python/vkvalidate.py:211-259)."""
    shape = tuple(shape)
    vals = (rng.standard_normal(shape) * scale).astype(dtype)
    yield "dense", vals.copy()
    if len(shape) >= 2:
        perm = list(range(len(shape)))
        perm[-1], perm[-2] = perm[-2], perm[-1]
        stored = np.ascontiguousarray(vals.transpose(perm))
        yield "transposed", stored.transpose(perm)
    if len(shape) >= 1 and shape[-1] > 0:
        big_shape = shape[:-1] + (shape[-1] * 2 + 3,)
        big = rng.standard_normal(big_shape).astype(dtype)
        view = big[..., 1:1 + 2 * shape[-1]:2]
        view[...] = vals
        yield "strided", view
    if len(shape) >= 1:
        big = rng.standard_normal((shape[0] + 2,) + shape[1:]).astype(dtype)
        view = big[1:1 + shape[0]]
        view[...] = vals
        yield "offset", view


ELEMENT_SIZES = [0, 1, 7, 255, 256, 257, 1000, 100_000]
