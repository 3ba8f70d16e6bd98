"""CUDA path vs the CPU oracle on identical seeded inputs, through the C ABI.

Integer, index and ordering ops are compared bit-exactly; floating ops under the
tolerance vkML itself applies between its GPU and CPU backends (tests/cases.py).
"""
import json
import os

import numpy as np
import pytest

import cases
from helpers import CudaImpl, OracleImpl
from vkml_b200 import graph
from vkml_b200.graph import DType, Op

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def oracle():
    return OracleImpl()


@pytest.fixture(scope="module")
def cuda(backend):
    return CudaImpl(backend)


def _run_family(gen, cuda, oracle, backend):
    n = 0
    failures = []
    for case in gen:
        want = oracle.run(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
        got = cuda.run(case.op, case.srcs, case.out_shape, case.out_dtype, case.params, sync_check=False)
        try:
            cases.check(case, got, want)
        except AssertionError as e:
            failures.append(str(e))
        n += 1
    backend.synchronize()
    assert not failures, f"{len(failures)}/{n} cases failed:\n" + "\n".join(failures[:20])
    return n


def test_elementwise(cuda, oracle, backend):
    assert _run_family(cases.elementwise_cases(), cuda, oracle, backend) >= 390


def test_f16_storage(cuda, oracle, backend):
    """F16 operands and results through every kernel family (widened, computed in f32, narrowed
    once): exact ops bit-identical to the CPU backend's Half kernels, the rest within one f16 ulp."""
    assert _run_family(cases.f16_cases(), cuda, oracle, backend) >= 38


def test_creation(cuda, oracle, backend):
    assert _run_family(cases.creation_cases(), cuda, oracle, backend) >= 25


def test_cast(cuda, oracle, backend):
    assert _run_family(cases.cast_cases(), cuda, oracle, backend) >= 14


def test_reduce(cuda, oracle, backend):
    assert _run_family(cases.reduce_cases(), cuda, oracle, backend) >= 500


def test_softmax(cuda, oracle, backend):
    assert _run_family(cases.softmax_cases(), cuda, oracle, backend) >= 100


def test_matmul_fp32(cuda, oracle, backend):
    backend.set_gemm_precision(2)
    try:
        assert _run_family(cases.matmul_cases(), cuda, oracle, backend) >= 70
    finally:
        backend.set_gemm_precision(0)


def test_matmul_default_precision(cuda, oracle, backend):
    """3xTF32 on the tensor cores where the shape is eligible, fp32 FMA elsewhere:
    both inside the backward-error bound of the fp32 dot product."""
    assert _run_family(cases.matmul_cases(), cuda, oracle, backend) >= 70


def test_matmul_tensor_core_3xtf32(cuda, oracle, backend):
    """tcgen05 path with the 3xTF32 split: inside the fp32 backward-error bound AND
    inside the relative Frobenius bound 1e-5*sqrt(K) the path is specified to."""
    n = 0
    backend.set_profiling(True)
    for case in cases.matmul_tc_cases():
        want = oracle.run(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
        got = cuda.run(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
        cases.check(case, got, want)
        rel = np.linalg.norm((got.astype(np.float64) - want).ravel()) / np.linalg.norm(want.astype(np.float64).ravel())
        assert rel < 1e-5 * np.sqrt(case.reduction_n), f"{case.name}: relative Frobenius error {rel:.3g}"
        assert rel < 1e-5, f"{case.name}: 3xTF32 should be near fp32-grade, got {rel:.3g}"
        n += 1
    labels = [l for l, _ in backend.last_profile()]
    backend.set_profiling(False)
    # every case really ran on the tensor cores (operand planes or the streamed operand)
    assert sum(l.startswith("matmul.tcgen05_3xtf32") for l in labels) == n, labels
    assert not any(l == "matmul.fp32_simt" for l in labels)
    # ... and the products bound by memory on the streamed-operand kernel: every case named for it,
    # both operand layouts, a tall W against a short K
    streamed = sum(l == "matmul.tcgen05_3xtf32_stream" for l in labels)
    named = sum("/stream-" in c.name for c in cases.matmul_tc_cases())
    assert named >= 14 and streamed >= named + 4, (streamed, named)


def test_matmul_tensor_core_both_operand_schemes(oracle, monkeypatch):
    """The two ways operands reach the tensor cores -- TF32 planes written to HBM first, or fp32
    tiles split inside the kernel -- each forced for every eligible shape: both inside the bounds
    against the oracle, and bit-identical to each other (same split, same accumulation order)."""
    import vkml_b200
    from helpers import CudaImpl
    results = {}
    for operands in ("planes", "direct"):
        monkeypatch.setenv("VKML_B200_GEMM_OPERANDS", operands)
        b = vkml_b200.Backend(0)
        impl = CudaImpl(b)
        b.set_profiling(True)
        outs = []
        for case in cases.matmul_tc_cases():
            want = oracle.run(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
            got = impl.run(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
            cases.check(case, got, want)
            rel = np.linalg.norm((got.astype(np.float64) - want).ravel()) / np.linalg.norm(want.astype(np.float64).ravel())
            assert rel < 1e-5, f"{case.name}: {rel:.3g}"
            outs.append((case.name, got))
        labels = [l for l, _ in b.last_profile() if l.startswith("matmul.tcgen05")]
        b.set_profiling(False)
        assert len(labels) == len(outs)
        results[operands] = (outs, labels)
    assert all(l == "matmul.tcgen05_3xtf32" for l in results["planes"][1])
    # operands with a pitch that is not a multiple of 16 bytes cannot be read by TMA directly
    direct_labels = results["direct"][1]
    assert sum(l == "matmul.tcgen05_3xtf32_direct" for l in direct_labels) >= 10, direct_labels
    for (name, a), (_, d) in zip(results["planes"][0], results["direct"][0]):
        assert np.array_equal(a.view(np.uint32), d.view(np.uint32)), name


def test_matmul_tensor_core_tf32_opt_in(cuda, oracle, backend):
    """Plain TF32 is an explicit opt-in and is only held to TF32-grade error."""
    backend.set_gemm_precision(1)
    try:
        for case in list(cases.matmul_tc_cases())[:4]:
            want = oracle.run(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
            got = cuda.run(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
            rel = np.linalg.norm((got.astype(np.float64) - want).ravel()) / np.linalg.norm(want.astype(np.float64).ravel())
            assert 1e-6 < rel < 2e-3, f"{case.name}: TF32 relative Frobenius error {rel:.3g}"
    finally:
        backend.set_gemm_precision(0)


def test_movement(cuda, oracle, backend):
    assert _run_family(cases.movement_cases(), cuda, oracle, backend) >= 85


def test_golden_fixtures(cuda, backend):
    """Committed outputs of the reference CPU build: the GPU agrees with the
    reference itself, not only with the restatement."""
    data = np.load(os.path.join(GOLDEN, "reference_outputs.npz"))
    names = json.loads(str(data["__index__"]))
    by_name = {c.name: c for c in cases.all_cases(quick=True)}
    by_name.update({c.name: c for c in cases.f16_cases()})
    for i, name in enumerate(names):
        case = by_name[name]
        got = cuda.run(case.op, case.srcs, case.out_shape, case.out_dtype, case.params, sync_check=False)
        cases.check(case, got, data[f"out_{i}"])
    backend.synchronize()


def test_known_answers(cuda, backend):
    from test_oracle import _params
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        table = json.load(f)
    for spec in table:
        srcs = []
        for s in spec["srcs"]:
            if s.get("values") is None:
                a = np.full(s["shape"], s["fill"], dtype=np.float32)
                a.reshape(-1)[0] = s.get("first", s["fill"])
            else:
                a = np.array(s["values"], dtype=DType[s.get("dtype", "F32")].numpy).reshape(s["shape"])
            if s.get("transpose"):
                a = np.ascontiguousarray(a).T
            if "broadcast" in s:
                a = np.broadcast_to(a, s["broadcast"])
            srcs.append(a)
        out_dt = DType[spec.get("out_dtype", "F32")]
        got = cuda.run(Op[spec["op"].upper()], srcs, tuple(spec["out_shape"]), out_dt, _params(spec))
        want = np.array(spec["want"], dtype=out_dt.numpy).reshape(spec["out_shape"])
        np.testing.assert_allclose(got, want, rtol=spec.get("rtol", 1e-6), atol=spec.get("atol", 0),
                                   err_msg=spec["name"])


def test_out_of_range_index_is_reported(cuda, backend):
    """The CPU backend throws IndexError before any value is visible
    (kernels_movement.cpp:362,419); the device clamps, records it, and the error reaches the
    caller with the first read of a result -- copy_to_host alone, the framework's normal way
    of observing a tensor -- or at the next synchronize, whichever comes first."""
    table = np.arange(12, dtype=np.float32).reshape(4, 3)
    idx = np.array([0, 4], dtype=np.int64)
    with pytest.raises(IndexError):  # run() ends in copy_to_host, nothing else synchronises
        cuda.run(Op.INDEX_SELECT, [table, idx], (2, 3), DType.F32, graph.axis_params(0), sync_check=False)
    backend.synchronize()  # the word is cleared: the context stays usable
    from vkml_b200 import DeviceTensor, NodeDesc
    src = DeviceTensor.from_host(backend, table[:2].copy())
    bad = DeviceTensor.from_host(backend, np.array([0, -1], dtype=np.int64))
    out = DeviceTensor.empty(backend, (4, 3))
    backend.compute([NodeDesc(Op.SCATTER_ADD, out.desc, [src.desc, bad.desc], graph.axis_params(0))])
    with pytest.raises(IndexError):  # no read in between: reported by synchronize
        backend.synchronize()
    got = cuda.run(Op.INDEX_SELECT, [table, np.array([3, 0], dtype=np.int64)], (2, 3), DType.F32,
                   graph.axis_params(0))
    np.testing.assert_array_equal(got, table[[3, 0]])


def test_repeated_execution_is_byte_identical(cuda, backend):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((300, 5000)).astype(np.float32)
    p = graph.reduce_params([1], 2)
    a = cuda.run(Op.SUM, [x], (300,), DType.F32, p)
    for _ in range(3):
        assert np.array_equal(a.view(np.uint32), cuda.run(Op.SUM, [x], (300,), DType.F32, p).view(np.uint32))
    a2 = np.ascontiguousarray(rng.standard_normal((64, 512)).astype(np.float32))
    b2 = np.ascontiguousarray(rng.standard_normal((512, 96)).astype(np.float32))
    m = cuda.run(Op.MATMUL, [a2.reshape(1, 1, 64, 512), b2.reshape(1, 1, 512, 96)], (1, 1, 64, 96), DType.F32)
    for _ in range(3):
        again = cuda.run(Op.MATMUL, [a2.reshape(1, 1, 64, 512), b2.reshape(1, 1, 512, 96)], (1, 1, 64, 96), DType.F32)
        assert np.array_equal(m.view(np.uint32), again.view(np.uint32))


def test_scaled_add_is_bit_identical_to_the_composed_form(cuda, backend):
    rng = np.random.default_rng(1)
    a = rng.standard_normal(100_001).astype(np.float32)
    b = rng.standard_normal(100_001).astype(np.float32)
    alpha, beta = np.float32(0.9), np.float32(-0.1)
    fused = cuda.run(Op.SCALED_ADD, [a, b], a.shape, DType.F32, graph.scaled_add_params(alpha, beta))
    al = np.broadcast_to(alpha.reshape(()), a.shape)
    be = np.broadcast_to(beta.reshape(()), a.shape)
    pa = cuda.run(Op.MUL, [a, al], a.shape, DType.F32)
    pb = cuda.run(Op.MUL, [b, be], a.shape, DType.F32)
    composed = cuda.run(Op.ADD, [pa, pb], a.shape, DType.F32)
    assert np.array_equal(fused.view(np.uint32), composed.view(np.uint32))
    assert np.array_equal(fused.view(np.uint32), (a * alpha + b * beta).view(np.uint32))


def test_a_span_is_ordered(backend):
    """RAW and WAR hazards inside one compute() span: later nodes read what earlier
    nodes wrote, and a buffer freed mid-span and handed out again is not clobbered
    (the checks of vkML's tests/cpp/test_aliasing.cpp, on the stream model)."""
    import vkml_b200 as V
    from vkml_b200 import DeviceTensor, NodeDesc
    n = 1 << 20
    x = np.arange(n, dtype=np.float32)
    tx = DeviceTensor.from_host(backend, x)
    t1 = DeviceTensor.empty(backend, (n,))
    t2 = DeviceTensor.empty(backend, (n,))
    t3 = DeviceTensor.empty(backend, (n,))
    span = [NodeDesc(Op.ADD, t1.desc, [tx.desc, tx.desc]),      # t1 = 2x
            NodeDesc(Op.MUL, t2.desc, [t1.desc, t1.desc]),      # t2 = 4x^2   (RAW on t1)
            NodeDesc(Op.NEG, t1.desc, [tx.desc]),               # t1 = -x     (WAR on t1)
            NodeDesc(Op.ADD, t3.desc, [t1.desc, t2.desc])]      # t3 = 4x^2 - x
    backend.compute(span)
    want = (x + x) * (x + x) + (-x)
    np.testing.assert_array_equal(t3.numpy(), want)
    # free a buffer while its consumer is queued, reallocate, overwrite
    t4 = DeviceTensor.empty(backend, (n,))
    backend.compute([NodeDesc(Op.RELU, t4.desc, [t3.desc])])
    addr = t3.storage.data
    del t3
    t5 = DeviceTensor.empty(backend, (n,))
    backend.compute([NodeDesc(Op.FULL, t5.desc, [], graph.full_params(-7.0))])
    np.testing.assert_array_equal(t4.numpy(), np.maximum(want, 0))
    assert t5.storage.data == addr  # the cache really did hand the block out again
    st = backend.stats()
    assert st["kernel_launches"] > 0 and st["compute_calls"] > 0


def test_operand_planes_are_shared_inside_a_span_only(monkeypatch):
    """With the plane scheme: a matrix that feeds several tensor-core matmuls of one span (a
    layer's forward, its input gradient and its weight gradient) is split into TF32 planes once:
    the results are bit-identical to running each product in a span of its own, the split
    launches drop, and nothing survives the span (the operand is overwritten between two spans)."""
    import vkml_b200
    from vkml_b200 import DeviceTensor, NodeDesc
    monkeypatch.setenv("VKML_B200_GEMM_OPERANDS", "planes")
    backend = vkml_b200.Backend(0)
    rng = np.random.default_rng(31)
    b, k, n = 256, 1000, 384          # 1000: not a multiple of the 32-wide padding
    x = DeviceTensor.from_host(backend, rng.standard_normal((1, 1, b, k)).astype(np.float32))
    w = DeviceTensor.from_host(backend, rng.standard_normal((1, 1, n, k)).astype(np.float32))
    g = DeviceTensor.from_host(backend, rng.standard_normal((1, 1, b, n)).astype(np.float32))

    def products():
        y = DeviceTensor.empty(backend, (1, 1, b, n))
        dx = DeviceTensor.empty(backend, (1, 1, b, k))
        dw2 = DeviceTensor.empty(backend, (1, 1, k, n))
        nodes = [NodeDesc(Op.MATMUL, y.desc, [x.desc, w.transpose(2, 3).desc]),    # forward: x W^T
                 NodeDesc(Op.MATMUL, dx.desc, [g.desc, w.desc]),                    # input gradient: g W
                 NodeDesc(Op.MATMUL, dw2.desc, [x.transpose(2, 3).desc, g.desc])]   # weight gradient: x^T g
        return nodes, (y, dx, dw2)

    nodes, outs = products()
    before = backend.stats()["kernel_launches"]
    backend.compute(nodes)
    shared = [t.numpy() for t in outs]
    launches_shared = backend.stats()["kernel_launches"] - before

    nodes, outs = products()
    before = backend.stats()["kernel_launches"]
    for node in nodes:
        backend.compute([node])
    alone = [t.numpy() for t in outs]
    launches_alone = backend.stats()["kernel_launches"] - before
    for a, c in zip(shared, alone):
        assert np.array_equal(a.view(np.uint32), c.view(np.uint32))
    assert launches_alone - launches_shared == 3      # x, W and g are each split once instead of twice

    # the same span again after W changed: a stale plane would reproduce the old product
    w2 = rng.standard_normal((1, 1, n, k)).astype(np.float32)
    backend.copy_from_host(w.storage, 0, w2)
    nodes, outs = products()
    backend.compute(nodes)
    xh, gh = x.numpy()[0, 0].astype(np.float64), g.numpy()[0, 0].astype(np.float64)
    np.testing.assert_allclose(outs[0].numpy()[0, 0], xh @ w2[0, 0].astype(np.float64).T, rtol=0, atol=2e-3)
    np.testing.assert_allclose(outs[1].numpy()[0, 0], gh @ w2[0, 0].astype(np.float64), rtol=0, atol=2e-3)
    np.testing.assert_allclose(outs[2].numpy()[0, 0], xh.T @ gh, rtol=0, atol=2e-3)


def test_errors_leave_the_backend_usable(backend):
    """A node the backend does not know, a geometry that contradicts its tensors, a span that fails
    half way and an allocation nobody can satisfy all come back as status codes (the exception
    types vkML maps them to), and the context keeps working afterwards -- the contract behind
    vkML's RecordingGuard (vulkan_backend.cpp:1216-1222) and OutOfMemoryError (allocator.h:41-44)."""
    import vkml_b200 as V
    from vkml_b200 import DeviceTensor, NodeDesc
    from vkml_b200.backend import OutOfMemoryError, ShapeError
    x = DeviceTensor.from_host(backend, np.arange(12, dtype=np.float32).reshape(3, 4))
    y = DeviceTensor.empty(backend, (3, 4))
    z = DeviceTensor.empty(backend, (3, 4))
    # an op the backend does not know: NotImplementedError, nothing launched
    with pytest.raises(NotImplementedError):
        backend.compute([NodeDesc(999, DeviceTensor.empty(backend, (3,)).desc, [x.desc], graph.reduce_params([1], 2))])
    # operand extents that contradict the output's
    a = DeviceTensor.empty(backend, (1, 1, 4, 5))
    b = DeviceTensor.empty(backend, (1, 1, 6, 7))
    with pytest.raises(ShapeError):
        backend.compute([NodeDesc(Op.MATMUL, DeviceTensor.empty(backend, (1, 1, 4, 7)).desc, [a.desc, b.desc])])
    # a span whose second node is invalid: the first node's work is ordered and valid, the error is
    # reported, and the next span runs normally
    bad = NodeDesc(Op.IM2COL, DeviceTensor.empty(backend, (1, 9, 4)).desc, [x.desc],
                   graph.unfold_params((3, 3), (1, 1), (1, 1), (1, 1), (2, 2)))
    with pytest.raises((ShapeError, ValueError)):
        backend.compute([NodeDesc(Op.NEG, y.desc, [x.desc]), bad, NodeDesc(Op.RELU, z.desc, [x.desc])])
    np.testing.assert_array_equal(y.numpy(), -x.numpy())
    backend.compute([NodeDesc(Op.RELU, z.desc, [y.desc])])
    np.testing.assert_array_equal(z.numpy(), np.zeros((3, 4), np.float32))
    # an allocation larger than the device: OutOfMemoryError, and the allocator still serves
    with pytest.raises(OutOfMemoryError):
        backend.allocate(1 << 42)
    w = DeviceTensor.from_host(backend, np.ones(1000, dtype=np.float32))
    np.testing.assert_array_equal(w.numpy(), np.ones(1000, np.float32))
    backend.synchronize()


def test_an_expired_device_wait_becomes_a_timeout_and_the_context_survives(backend):
    """Every device-side wait is bounded.  A block that waits one millisecond on a barrier nobody
    arrives on gives up by itself; the host reports B200_TIMEOUT (vkML's DeviceError) at the next
    synchronisation, and the context keeps working afterwards."""
    from vkml_b200 import DeviceTensor
    from vkml_b200.backend import DeviceError
    backend.synchronize()
    rc = backend._lib.b200_debug_expire_wait(backend._ctx, 1_000_000)
    assert rc == 0
    with pytest.raises(DeviceError, match="timeout"):
        backend.synchronize()
    backend.synchronize()  # reported once, then cleared
    w = DeviceTensor.from_host(backend, np.arange(1000, dtype=np.float32))
    np.testing.assert_array_equal(w.numpy(), np.arange(1000, dtype=np.float32))


def test_device_copies(backend):
    from vkml_b200 import DeviceTensor
    rng = np.random.default_rng(4)
    a = rng.standard_normal(1000).astype(np.float32)
    ta = DeviceTensor.from_host(backend, a)
    tb = DeviceTensor.empty(backend, (1000,))
    tc = DeviceTensor.empty(backend, (500,))
    backend.copy_device_to_device([(tb.storage, 0, ta.storage, 0, 4000), (tc.storage, 0, ta.storage, 2000, 2000)])
    np.testing.assert_array_equal(tb.numpy(), a)
    np.testing.assert_array_equal(tc.numpy(), a[500:])
    with pytest.raises(IndexError):
        backend.copy_device_to_device([(tc.storage, 0, ta.storage, 0, 4000)])
    with pytest.raises(IndexError):
        backend.copy_from_host(tc.storage, 1999, a)
    z = backend.allocate(0)
    assert z.data == 0 and z.nbytes == 0


def test_which_kernel_a_product_gets(backend):
    """b200_matmul_kernel names the kernel a product would get, taken by itself, and the profile of
    the product run by itself agrees: CUDA cores for a tiny product, operand planes for a large
    square one, the streamed operand for a skinny one and for a convolution's weight gradient, the
    operands read directly where a byte model says the plane passes would cost more than the product."""
    from vkml_b200 import DeviceTensor, NodeDesc
    rng = np.random.default_rng(31)

    def dev(*shape):
        return DeviceTensor.from_host(backend, rng.standard_normal(shape).astype(np.float32))

    def product(a, b, shape):
        return NodeDesc(Op.MATMUL, DeviceTensor.empty(backend, shape).desc, [a.desc, b.desc])

    cases = [
        ("fp32_simt", product(dev(1, 1, 24, 40), dev(1, 1, 40, 24), (1, 1, 24, 24))),
        ("tcgen05_3xtf32", product(dev(1, 1, 1024, 1024), dev(1, 1, 1024, 1024), (1, 1, 1024, 1024))),
        ("tcgen05_3xtf32_stream", product(dev(1, 1, 64, 2048), dev(1, 1, 2048, 512), (1, 1, 64, 512))),
        ("tcgen05_3xtf32_stream", product(dev(1, 4, 128, 256), dev(1, 4, 576, 256).transpose(2, 3), (1, 4, 128, 576))),
        # the first convolution's weight gradient: N = 27 keeps it off the streamed-operand kernel
        ("tcgen05_3xtf32_direct", product(dev(1, 16, 64, 1024), dev(1, 16, 27, 1024).transpose(2, 3), (1, 16, 64, 27))),
    ]
    for want, node in cases:
        name, why = backend.matmul_kernel(node)
        assert name == want and why, (want, name, why)
        backend.set_profiling(True)
        backend.compute([node])
        labels = [l for l, _ in backend.last_profile()]
        backend.set_profiling(False)
        assert "matmul." + want in labels, (want, labels)


def test_a_span_that_comes_back_is_replayed_as_a_graph_with_fresh_data(oracle, monkeypatch):
    """The same span on the same buffers, seven times with new input data each time: from the third
    submission on it is one CUDA graph launch, and every result is the one the eager path gives
    (bit for bit) and the oracle confirms.  A different span on the same buffers is not mistaken for it."""
    import vkml_b200
    from vkml_b200 import DeviceTensor, NodeDesc
    rng = np.random.default_rng(23)
    results = {}
    for mode in ("1", "0"):
        monkeypatch.setenv("VKML_B200_SPAN_GRAPHS", mode)
        b = vkml_b200.Backend(0)
        x = DeviceTensor.empty(b, (1, 1, 96, 160))
        w = DeviceTensor.from_host(b, (np.random.default_rng(3).standard_normal((1, 1, 160, 64)) * 0.05).astype(np.float32))
        bias = DeviceTensor.from_host(b, np.random.default_rng(4).standard_normal((1, 1, 1, 64)).astype(np.float32))
        h, hb, r, e, sm, s = (DeviceTensor.empty(b, (1, 1, 96, 64)) for _ in range(6))
        tot = DeviceTensor.empty(b, (1, 1, 96, 1))
        bias_b = bias.broadcast_to((1, 1, 96, 64))
        span = [NodeDesc(Op.MATMUL, h.desc, [x.desc, w.desc]), NodeDesc(Op.ADD, hb.desc, [h.desc, bias_b.desc]),
                NodeDesc(Op.RELU, r.desc, [hb.desc]), NodeDesc(Op.EXP, e.desc, [r.desc]),
                NodeDesc(Op.LOG_SOFTMAX, sm.desc, [e.desc], graph.axis_params(3)),
                NodeDesc(Op.NEG, s.desc, [sm.desc]),
                NodeDesc(Op.SUM, tot.desc, [s.desc], graph.reduce_params([3], 4, keepdim=True))]
        outs = []
        data = np.random.default_rng(5)
        for _ in range(7):
            xs = data.standard_normal((1, 1, 96, 160)).astype(np.float32)
            b.copy_from_host(x.storage, 0, xs)
            b.compute(span)
            outs.append((xs, tot.numpy().copy(), sm.numpy().copy()))
        other = span[:3] + [NodeDesc(Op.NEG, e.desc, [r.desc])] + span[4:]   # same buffers, another function
        b.compute(other)
        outs.append((None, tot.numpy().copy(), sm.numpy().copy()))
        hits, captures = b.span_graph_stats()
        if mode == "1":
            assert captures == 1 and hits == 5, (hits, captures)
        else:
            assert captures == 0 and hits == 0
        results[mode] = outs
    for (xs, t1, s1), (_, t0, s0) in zip(results["1"], results["0"]):
        assert np.array_equal(t1.view(np.uint32), t0.view(np.uint32)) and np.array_equal(s1.view(np.uint32), s0.view(np.uint32))
    xs, t1, s1 = results["1"][6]
    wh = (np.random.default_rng(3).standard_normal((160, 64)) * 0.05).astype(np.float32)
    bh = np.random.default_rng(4).standard_normal((64,)).astype(np.float32)
    z = np.maximum(xs.reshape(96, 160).astype(np.float64) @ wh + bh, 0)
    ez = np.exp(z)
    want = ez - np.log(np.exp(ez - ez.max(1, keepdims=True)).sum(1, keepdims=True)) - ez.max(1, keepdims=True)
    assert np.allclose(s1.reshape(96, 64), want, rtol=2e-4, atol=2e-4)
    assert not np.array_equal(results["1"][7][2], results["1"][6][2])


def test_large_uploads_from_pageable_memory_arrive_intact(backend):
    """copy_from_host of pageable memory above a few MB is staged through pinned slots by several
    threads: sizes that are not a multiple of the chunk, sources that change between calls (every
    slot is reused), the source overwritten as soon as the call returns, and a kernel queued
    right behind the copy -- the bytes on the device are the bytes that were passed."""
    from vkml_b200 import DeviceTensor, NodeDesc
    rng = np.random.default_rng(17)
    for n in (3_000_001, 8_400_000 // 4, 40_000_003):
        dev = DeviceTensor.empty(backend, (1, 1, 1, n))
        out = DeviceTensor.empty(backend, (1, 1, 1, n))
        for _ in range(3):
            src = rng.standard_normal(n).astype(np.float32)
            want = src.copy()
            backend.copy_from_host(dev.storage, 0, src)
            src[:] = -1.0                                   # the call has returned: the source is the caller's again
            backend.compute([NodeDesc(Op.NEG, out.desc, [dev.desc])])
            assert np.array_equal(out.numpy().ravel(), -want)
            back = np.empty(n, np.float32)
            backend.copy_to_host(back, dev.storage, 0)
            assert np.array_equal(back, want)


def test_profiling_stats_timer_and_pinned_memory(backend):
    """The auxiliary ABI: per-launch device times, counters, the stream stopwatch, page-locked buffers."""
    from vkml_b200 import DeviceTensor, NodeDesc
    rng = np.random.default_rng(9)
    a = DeviceTensor.from_host(backend, rng.standard_normal((1, 1, 512, 512)).astype(np.float32))
    b = DeviceTensor.from_host(backend, rng.standard_normal((1, 1, 512, 512)).astype(np.float32))
    c = DeviceTensor.empty(backend, (1, 1, 512, 512))
    r = DeviceTensor.empty(backend, (1, 1, 512, 512))
    before = backend.stats()
    backend.set_profiling(True)
    backend.timer_begin()
    backend.compute([NodeDesc(Op.MATMUL, c.desc, [a.desc, b.desc]), NodeDesc(Op.RELU, r.desc, [c.desc])])
    ms = backend.timer_end()
    prof = backend.last_profile()
    backend.set_profiling(False)
    labels = [l for l, _ in prof]
    assert labels[:3] == ["matmul.split_a", "matmul.split_b", "matmul.tcgen05_3xtf32"] and labels[-1] == "relu", labels
    assert labels[3:-1] in ([], ["matmul.fold"])  # a split-K fold when the tiles alone cannot fill the machine
    assert all(t > 0 for _, t in prof) and 0 < sum(t for _, t in prof) <= ms * 1.5
    after = backend.stats()
    assert after["kernel_launches"] - before["kernel_launches"] == len(labels)
    assert after["nodes_computed"] - before["nodes_computed"] == 2
    assert after["compute_calls"] - before["compute_calls"] == 1
    assert backend.last_profile() == []  # reading clears, and nothing is recorded once disabled
    pin = backend.alloc_host(512 * 512 * 4)
    backend.copy_to_host(pin, r.storage, 0, pin.nbytes)
    got = np.frombuffer(pin, dtype=np.float32).reshape(512, 512).copy()
    backend.free_host(pin)
    np.testing.assert_array_equal(got, r.numpy().reshape(512, 512))
    assert (got >= 0).all() and got.max() > 0
    caps = backend.capabilities()
    assert caps["compute_capability"][0] == 10 and caps["shader_core_count"] >= 100 and caps["asynchronous"]
