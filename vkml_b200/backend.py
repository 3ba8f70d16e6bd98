"""Host-side mirror of ``vkml::Backend`` (include/vkml/backend/api/backend.h:49-125)
over the C ABI: same method names, argument meaning and error behaviour, so code
and tests written against vkML's backend interface read the same here.

Errors cross the C boundary as status codes and are raised as the exception
types vkML maps to Python (bindings/module.cpp:243-250).
"""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _abi
from .graph import DType, NodeDesc, TensorDesc, pack_nodes


class Error(RuntimeError):
    """vkml::Error"""


class ShapeError(Error):
    pass


class DTypeError(Error):
    pass


class DeviceError(Error):
    pass


class OutOfMemoryError(Error):
    pass


class InternalError(Error):
    pass


_STATUS_EXC = {
    1: ShapeError, 2: DTypeError, 3: DeviceError, 4: IndexError, 5: NotImplementedError,
    6: InternalError, 7: OutOfMemoryError, 8: ValueError, 9: DeviceError,
}

COMPUTE_SYNC = 1
COMPUTE_GRAD_SYNC = 2
GEMM_3XTF32, GEMM_TF32, GEMM_FP32 = 0, 1, 2


class Storage:
    """vkml::Storage (include/vkml/core/storage.h:29-55): an owned device byte
    range. Dropping the last reference returns the block to the backend's cache;
    that is safe while kernels using it are queued (stream-ordered reuse)."""

    def __init__(self, backend: "Backend", data: int, nbytes: int):
        self._backend = backend
        self.data = data
        self.nbytes = nbytes

    def __del__(self):
        b, self._backend = getattr(self, "_backend", None), None
        if b is not None and self.data and b._ctx:
            b._lib.b200_free(b._ctx, self.data)


class Backend:
    """One CUDA device behind vkML's backend interface."""

    def __init__(self, cuda_ordinal: int = 0):
        self._lib = _abi.load()
        if self._lib.b200_abi_version() != 1:
            raise DeviceError("vkml_b200: ABI version mismatch")
        ctx = C.c_void_p()
        rc = self._lib.b200_create(cuda_ordinal, C.byref(ctx))
        if rc != 0:
            raise DeviceError(
                f"vkml_b200: cannot open CUDA device {cuda_ordinal}: "
                f"{self._lib.b200_status_name(rc).decode()} (no CPU fallback exists)")
        self._ctx = ctx
        self.ordinal = cuda_ordinal
        caps = _abi.Caps()
        self._check(self._lib.b200_get_caps(self._ctx, C.byref(caps)), "capabilities")
        self._caps = caps

    # -- describe -----------------------------------------------------------
    @property
    def name(self) -> str:
        return "b200:" + self._caps.name.decode()

    @property
    def device(self) -> str:
        # registered under vkML's "vulkan:N" device slot (include/vkml/core/device.h:9-12)
        return f"vulkan:{self.ordinal}"

    def capabilities(self) -> dict:
        c = self._caps
        return {
            "name": c.name.decode(), "compute_capability": (c.cc_major, c.cc_minor),
            "shader_core_count": c.sm_count, "subgroup_size": c.warp_size,
            "max_workgroup_invocations": c.max_threads_per_block,
            "max_shared_memory_bytes": c.max_shared_memory_bytes,
            "total_memory_bytes": c.total_memory_bytes,
            "min_buffer_alignment": c.min_buffer_alignment,
            "asynchronous": True, "host_accessible_buffers": False, "unified_memory": False,
        }

    # -- memory ---------------------------------------------------------------
    def allocate(self, nbytes: int) -> Storage:
        """Allocator::allocate: zero bytes yields a Storage with null data."""
        ptr = C.c_void_p()
        self._check(self._lib.b200_alloc(self._ctx, nbytes, C.byref(ptr)), "allocate")
        return Storage(self, ptr.value or 0, nbytes)

    # -- compute --------------------------------------------------------------
    def supports(self, node: NodeDesc) -> bool:
        c = node.to_c()
        return bool(self._lib.b200_supports(C.byref(c)))

    def matmul_kernel(self, node: NodeDesc) -> tuple:
        """(kernel, reason) a matmul node would get, taken by itself: fp32_simt, tcgen05_3xtf32 (operand
        planes), tcgen05_3xtf32_stream (streamed operand) or tcgen05_3xtf32_direct (operands read directly)."""
        c = node.to_c()
        name, why = C.create_string_buffer(64), C.create_string_buffer(160)
        self._check(self._lib.b200_matmul_kernel(self._ctx, C.byref(c), name, 64, why, 160), "matmul_kernel")
        return name.value.decode(), why.value.decode()

    def compute(self, nodes: Sequence[NodeDesc], flags: int = 0) -> None:
        """Backend::compute: ordered when this returns, not necessarily finished."""
        self.compute_packed(pack_nodes(nodes), len(nodes), flags)

    def compute_packed(self, packed, n: int, flags: int = 0) -> None:
        self._check(self._lib.b200_compute(self._ctx, packed, n, flags), "compute")

    # -- copies ---------------------------------------------------------------
    def copy_from_host(self, dst: Storage, dst_offset: int, src, nbytes: int | None = None) -> None:
        buf = np.ascontiguousarray(src) if not isinstance(src, int) else None
        n = nbytes if nbytes is not None else buf.nbytes
        if n == 0:
            return
        if dst_offset < 0 or dst_offset + n > dst.nbytes:
            raise IndexError(f"copy_from_host writes {n} bytes at offset {dst_offset} into a "
                             f"{dst.nbytes}-byte storage")
        ptr = src if isinstance(src, int) else buf.ctypes.data
        self._check(self._lib.b200_copy_from_host(self._ctx, dst.data + dst_offset, ptr, n),
                    "copy_from_host")

    def copy_to_host(self, dst: np.ndarray, src: Storage, src_offset: int, nbytes: int | None = None) -> None:
        n = nbytes if nbytes is not None else dst.nbytes
        if n == 0:
            return
        if src_offset < 0 or src_offset + n > src.nbytes:
            raise IndexError(f"copy_to_host reads {n} bytes at offset {src_offset} from a "
                             f"{src.nbytes}-byte storage")
        assert dst.flags["C_CONTIGUOUS"]
        self._check(self._lib.b200_copy_to_host(self._ctx, dst.ctypes.data, src.data + src_offset, n),
                    "copy_to_host")

    def copy_device_to_device(self, copies: Sequence[tuple]) -> None:
        """copies: (dst Storage, dst_offset, src Storage, src_offset, nbytes); disjoint ranges."""
        arr = (_abi.Copy * max(len(copies), 1))()
        for i, (d, doff, s, soff, n) in enumerate(copies):
            if doff < 0 or doff + n > d.nbytes or soff < 0 or soff + n > s.nbytes:
                raise IndexError("copy_device_to_device range exceeds a storage")
            arr[i].dst = (d.data + doff) or None
            arr[i].src = (s.data + soff) or None
            arr[i].nbytes = n
        self._check(self._lib.b200_copy_device_to_device(self._ctx, arr, len(copies)),
                    "copy_device_to_device")

    def synchronize(self) -> None:
        self._check(self._lib.b200_synchronize(self._ctx), "synchronize")

    # -- policy / introspection -------------------------------------------------
    def set_gemm_precision(self, precision: int) -> None:
        self._check(self._lib.b200_set_gemm_precision(self._ctx, precision), "set_gemm_precision")

    def stats(self) -> dict:
        s = _abi.Stats()
        self._check(self._lib.b200_get_stats(self._ctx, C.byref(s)), "stats")
        return {name: getattr(s, name) for name, _ in s._fields_}

    def set_profiling(self, enabled: bool) -> None:
        """Bracket every kernel launch with device timestamps (VulkanBackend::set_profiling)."""
        self._check(self._lib.b200_profile_enable(self._ctx, 1 if enabled else 0), "profile_enable")

    def last_profile(self, capacity: int = 65536) -> list:
        """[(label, gpu_ms)] in launch order since the last read; synchronises."""
        buf = (_abi.ProfileRecord * capacity)()
        n = C.c_size_t(0)
        self._check(self._lib.b200_profile_read(self._ctx, buf, capacity, C.byref(n)), "profile_read")
        return [(buf[i].label.decode(), float(buf[i].ms)) for i in range(n.value)]

    def span_graph_stats(self) -> tuple:
        """(spans served by launching a kept CUDA graph, graphs captured) since the context was created."""
        hits, captures = C.c_uint64(0), C.c_uint64(0)
        self._check(self._lib.b200_span_graph_stats(self._ctx, C.byref(hits), C.byref(captures)), "span_graph_stats")
        return int(hits.value), int(captures.value)

    def timer_begin(self) -> None:
        self._check(self._lib.b200_timer_begin(self._ctx), "timer_begin")

    def timer_end(self) -> float:
        """Device milliseconds since timer_begin, on the context's stream; synchronises."""
        ms = C.c_float(0)
        self._check(self._lib.b200_timer_end(self._ctx, C.byref(ms)), "timer_end")
        return float(ms.value)

    def alloc_host(self, nbytes: int) -> np.ndarray:
        """Page-locked host bytes as a uint8 array (freed with free_host)."""
        ptr = C.c_void_p()
        self._check(self._lib.b200_alloc_host(self._ctx, nbytes, C.byref(ptr)), "alloc_host")
        arr = np.ctypeslib.as_array((C.c_uint8 * nbytes).from_address(ptr.value))
        self._pinned = getattr(self, "_pinned", {})
        self._pinned[arr.ctypes.data] = ptr.value
        return arr

    def free_host(self, arr: np.ndarray) -> None:
        ptr = getattr(self, "_pinned", {}).pop(arr.ctypes.data, None)
        if ptr is not None:
            self._check(self._lib.b200_free_host(self._ctx, ptr), "free_host")

    def trim(self) -> None:
        self._check(self._lib.b200_trim(self._ctx), "trim")

    @property
    def stream(self) -> int:
        return self._lib.b200_stream(self._ctx) or 0

    # -- data parallel ----------------------------------------------------------
    def dist_unique_id(self) -> bytes:
        buf = C.create_string_buffer(_abi.UNIQUE_ID_BYTES)
        self._check(self._lib.b200_dist_unique_id(buf), "dist_unique_id")
        return buf.raw

    def dist_init(self, rank: int, world: int, unique_id: bytes, timeout_ms: int | None = None) -> None:
        """Join a data-parallel job.  With `timeout_ms`, ranks that do not all arrive in time end
        the call with DeviceError (timeout) and an aborted communicator instead of blocking."""
        buf = C.create_string_buffer(unique_id, _abi.UNIQUE_ID_BYTES)
        if timeout_ms is None:
            self._check(self._lib.b200_dist_init(self._ctx, rank, world, buf), "dist_init")
        else:
            self._check(self._lib.b200_dist_init_deadline(self._ctx, rank, world, buf, timeout_ms), "dist_init")

    def dist_all_reduce_mean(self, data: int, count: int) -> None:
        self._check(self._lib.b200_dist_all_reduce_mean(self._ctx, data, count), "all_reduce")

    def dist_wait(self) -> None:
        self._check(self._lib.b200_dist_wait(self._ctx), "dist_wait")

    def dist_mark_grad(self, data: int, count: int) -> None:
        self._check(self._lib.b200_dist_mark_grad(self._ctx, data, count), "dist_mark_grad")

    def dist_clear_grads(self) -> None:
        self._check(self._lib.b200_dist_clear_grads(self._ctx), "dist_clear_grads")

    def close(self) -> None:
        if self._ctx:
            self._lib.b200_destroy(self._ctx)
            self._ctx = None

    # -- helpers ----------------------------------------------------------------
    def _check(self, rc: int, where: str) -> None:
        if rc == 0:
            return
        detail = self._lib.b200_last_error(self._ctx) if self._ctx else b""
        msg = f"b200 backend: {where}: {self._lib.b200_status_name(rc).decode()}"
        if detail:
            msg += ": " + detail.decode(errors="replace")
        raise _STATUS_EXC.get(rc, InternalError)(msg)


class DeviceTensor:
    """A strided view over a Storage: the fields of a vkML node the backend reads
    (shape with byte strides, dtype, storage, storage_offset; node.h:69-157)."""

    def __init__(self, backend: Backend, storage: Storage, dims, strides, dtype: DType, offset: int = 0):
        self.backend = backend
        self.storage = storage
        self.dims = tuple(int(d) for d in dims)
        self.strides = tuple(int(s) for s in strides)
        self.dtype = DType(dtype)
        self.offset = offset

    # creation
    @staticmethod
    def empty(backend: Backend, dims, dtype: DType = DType.F32) -> "DeviceTensor":
        desc = TensorDesc.contiguous(0, dims, DType(dtype))
        return DeviceTensor(backend, backend.allocate(desc.nbytes), desc.dims, desc.strides, dtype)

    @staticmethod
    def from_host(backend: Backend, array: np.ndarray) -> "DeviceTensor":
        a = np.ascontiguousarray(array)
        t = DeviceTensor.empty(backend, a.shape, DType.of(a.dtype))
        backend.copy_from_host(t.storage, 0, a)
        return t

    @property
    def numel(self) -> int:
        n = 1
        for d in self.dims:
            n *= d
        return n

    @property
    def desc(self) -> TensorDesc:
        return TensorDesc((self.storage.data + self.offset) if self.storage.data else 0,
                          self.dims, self.strides, self.dtype)

    # views (no kernels: the executor resolves them by aliasing, backend.h:34-45)
    def transpose(self, a: int, b: int) -> "DeviceTensor":
        d, s = list(self.dims), list(self.strides)
        d[a], d[b] = d[b], d[a]
        s[a], s[b] = s[b], s[a]
        return DeviceTensor(self.backend, self.storage, d, s, self.dtype, self.offset)

    def reshape(self, dims) -> "DeviceTensor":
        desc = TensorDesc.contiguous(0, dims, self.dtype)
        assert self.is_contiguous() and desc.numel == self.numel
        return DeviceTensor(self.backend, self.storage, desc.dims, desc.strides, self.dtype, self.offset)

    def broadcast_to(self, dims) -> "DeviceTensor":
        dims = tuple(dims)
        pad = len(dims) - len(self.dims)
        d = (1,) * pad + self.dims
        s = (0,) * pad + self.strides
        out_s = []
        for have, want, st in zip(d, dims, s):
            if have == want:
                out_s.append(st)
            else:
                assert have == 1
                out_s.append(0)
        return DeviceTensor(self.backend, self.storage, dims, out_s, self.dtype, self.offset)

    def is_contiguous(self) -> bool:
        if self.numel == 0:
            return True
        expected = self.dtype.itemsize
        for d, s in zip(reversed(self.dims), reversed(self.strides)):
            if d == 1:
                continue
            if s != expected:
                return False
            expected *= d
        return True

    def numpy(self) -> np.ndarray:
        """Synchronising read of a CONTIGUOUS tensor (Tensor::to_host makes a
        Contiguous node first when strided; callers here do the same)."""
        assert self.is_contiguous()
        out = np.empty(self.dims, dtype=self.dtype.numpy)
        self.backend.copy_to_host(out, self.storage, self.offset, out.nbytes)
        return out
