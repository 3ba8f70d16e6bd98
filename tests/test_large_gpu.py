"""Index spaces beyond 2^31 elements: the 64-bit paths of the elementwise, transposing and
reduction kernels.  Inputs are built on the device from small broadcast vectors (nothing of
this size crosses PCIe); results are checked on sampled rows and through reductions."""
import numpy as np
import pytest

import vkml_b200
from vkml_b200 import DeviceTensor, NodeDesc, Op, graph
from vkml_b200.graph import DType

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend():
    b = vkml_b200.Backend(0)
    yield b
    b.trim()


def _rows(backend, t, rows, cols, picks):
    out = {}
    for r in picks:
        buf = np.empty(cols, dtype=np.float32)
        backend.copy_to_host(buf, t.storage, int(r) * cols * 4, buf.nbytes)
        out[int(r)] = buf
    return out


def test_two_billion_element_tensors(backend):
    rows, cols = 65536 + 24, 32768            # 2 148 270 080 elements, 8.6 GB per tensor
    assert rows * cols > 2 ** 31
    c = (np.arange(rows) % 1021).astype(np.float32)      # small integers: every sum below is exact
    r = (np.arange(cols) % 1019).astype(np.float32)
    tc = DeviceTensor.from_host(backend, c.reshape(rows, 1))
    tr = DeviceTensor.from_host(backend, r.reshape(1, cols))
    x = DeviceTensor.empty(backend, (rows, cols))
    # x[i, j] = c[i] + r[j]: both operands are stride-0 broadcasts, the output index is 64-bit
    backend.compute([NodeDesc(Op.ADD, x.desc, [tc.broadcast_to((rows, cols)).desc, tr.broadcast_to((rows, cols)).desc])])
    picks = [0, 1, 4095, 65535, 65536, rows - 1]
    for i, got in _rows(backend, x, rows, cols, picks).items():
        np.testing.assert_array_equal(got, c[i] + r)

    # transposing copy of the whole thing: y[j, i] = x[i, j] through the shared-memory tile kernel
    y = DeviceTensor.empty(backend, (cols, rows))
    backend.compute([NodeDesc(Op.CONTIGUOUS, y.desc, [x.transpose(0, 1).desc])])
    for j, got in _rows(backend, y, cols, rows, [0, 1, 777, cols - 1]).items():
        np.testing.assert_array_equal(got, c + r[j])

    # flat 128-bit path past 2^31 elements, in place of nothing: z = -x, checked at the far end
    z = DeviceTensor.empty(backend, (rows * cols,))
    backend.compute([NodeDesc(Op.NEG, z.desc, [x.reshape((rows * cols,)).desc])])
    tail = np.empty(cols, dtype=np.float32)
    backend.copy_to_host(tail, z.storage, (rows * cols - cols) * 4, tail.nbytes)
    np.testing.assert_array_equal(tail, -(c[rows - 1] + r))
    del z

    # reductions over the 2^31+ space: column sums (kept axis 32768 wide, 65560 terms each) and the
    # total; every partial sum is an integer below 2^24 per column, so the column sums are exact
    col_sum = DeviceTensor.empty(backend, (1, cols))
    backend.compute([NodeDesc(Op.SUM, col_sum.desc, [x.desc], graph.reduce_params([0], 2, True))])
    want_cols = c.astype(np.float64).sum() + rows * r.astype(np.float64)
    got_cols = col_sum.numpy().reshape(-1).astype(np.float64)
    np.testing.assert_allclose(got_cols, want_cols, rtol=1e-6)
    row_max = DeviceTensor.empty(backend, (rows,))
    backend.compute([NodeDesc(Op.MAX, row_max.desc, [x.desc], graph.reduce_params([1], 2, False))])
    np.testing.assert_array_equal(row_max.numpy(), c + r.max())
    arg = DeviceTensor.empty(backend, (rows,), DType.I64)
    backend.compute([NodeDesc(Op.ARGMAX, arg.desc, [x.desc], graph.reduce_params([1], 2, False))])
    np.testing.assert_array_equal(arg.numpy(), np.full(rows, int(np.argmax(r)), dtype=np.int64))
    total = DeviceTensor.empty(backend, ())
    backend.compute([NodeDesc(Op.MEAN, total.desc, [x.desc], graph.reduce_params([], 2, False))])
    want_mean = c.astype(np.float64).mean() + r.astype(np.float64).mean()
    assert abs(float(total.numpy()) - want_mean) <= 1e-5 * want_mean
    backend.synchronize()
