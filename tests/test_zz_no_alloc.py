"""The allocation-free column sum, called through the C ABI.

Some users of this library may not allocate device memory when they need a result: a host
callback or a latency-critical loop, a process whose memory budget was fixed at start-up,
a plug-in that was handed a stream and buffers only.  `b200_sum_columns_f32_noalloc` serves
them from a fixed scratch array inside the library.  Here it is checked against the
ordinary path (a sum node through `b200_compute`, which takes its scratch from the
context's allocator) on two calls in a row -- the second call sees whatever the first left
in the shared array -- and its size limit is checked to be refused with a message.

This file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes as C

import numpy as np
import pytest

import cases
from helpers import CudaImpl
from vkml_b200 import _abi, graph
from vkml_b200.graph import DType, Op

pytestmark = pytest.mark.gpu


def noalloc_sum(backend, x: np.ndarray, pitch: int) -> np.ndarray:
    """x: [rows, cols] values; stored on the device with `pitch` elements per row."""
    lib = _abi.load()
    rows, cols = x.shape
    host = np.zeros((rows, pitch), dtype=np.float32)
    host[:, :cols] = x
    src = backend.allocate(max(host.nbytes, 4))   # the TEST may allocate; the entry point does not
    dst = backend.allocate(max(cols * 4, 4))
    if host.nbytes:
        backend.copy_from_host(src, 0, host)
    backend.synchronize()
    before = backend.stats()
    err = C.create_string_buffer(256)
    rc = lib.b200_sum_columns_f32_noalloc(src.data, rows, cols, pitch, dst.data, backend.stream, err, 256)
    assert rc == 0, err.value.decode()
    out = np.empty(cols, dtype=np.float32)
    if cols:
        backend.copy_to_host(out, dst, 0)
    backend.synchronize()
    after = backend.stats()
    # nothing was taken from the context's allocator either
    assert after["total_allocations"] == before["total_allocations"]
    assert after["driver_allocations"] == before["driver_allocations"]
    return out


def reference_sum(cuda, x: np.ndarray) -> np.ndarray:
    rows, cols = x.shape
    return cuda.run(Op.SUM, [x], (cols,), DType.F32, graph.reduce_params([0], 2))


def check(x, got, want):
    case = cases.Case("sum columns (no alloc)", Op.SUM, [x], want.shape, DType.F32,
                      terms_abs_sum=np.abs(x.astype(np.float64)).sum(0), reduction_n=x.shape[0])
    cases.check(case, got, want)


def test_two_calls_in_a_row_match_the_allocating_path(backend):
    cuda = CudaImpl(backend)
    rng = np.random.default_rng(31)
    # first call: many splits, every counter and most of the partial planes get used
    a = rng.standard_normal((4096, 8192)).astype(np.float32)
    got_a = noalloc_sum(backend, a, 8192)
    check(a, got_a, reference_sum(cuda, a))
    # second call, different geometry and a padded pitch, on top of the first call's leftovers
    b = (rng.standard_normal((1000, 257)) * 100).astype(np.float32)
    got_b = noalloc_sum(backend, b, 300)
    check(b, got_b, reference_sum(cuda, b))
    # and again the first shape: byte-identical to its first result (fixed summation order)
    again = noalloc_sum(backend, a, 8192)
    assert np.array_equal(again.view(np.uint32), got_a.view(np.uint32))
    # few rows (single pass, no partials) and a long row
    c = rng.standard_normal((5, 100_000)).astype(np.float32)
    check(c, noalloc_sum(backend, c, 100_000), reference_sum(cuda, c))
    # exact on integers, whatever the split count
    d = rng.integers(-8, 9, (3000, 1031)).astype(np.float32)
    np.testing.assert_array_equal(noalloc_sum(backend, d, 1031), d.sum(0, dtype=np.float64).astype(np.float32))


def test_sizes_beyond_the_fixed_array_are_refused(backend):
    lib = _abi.load()
    buf = backend.allocate(1024)
    err = C.create_string_buffer(256)
    too_wide = 1048576 + 1
    rc = lib.b200_sum_columns_f32_noalloc(buf.data, 1, too_wide, too_wide, buf.data, backend.stream, err, 256)
    assert rc == 8  # B200_INVALID_ARGUMENT
    assert b"exceed" in err.value and str(1048576).encode() in err.value
    rc = lib.b200_sum_columns_f32_noalloc(buf.data, 4, 16, 8, buf.data, backend.stream, err, 256)
    assert rc == 8 and b"row_pitch" in err.value
    rc = lib.b200_sum_columns_f32_noalloc(None, 4, 16, 16, buf.data, backend.stream, err, 256)
    assert rc == 8
    # zero columns: nothing to do, no error
    assert lib.b200_sum_columns_f32_noalloc(None, 4, 0, 0, None, backend.stream, err, 256) == 0
    backend.synchronize()
