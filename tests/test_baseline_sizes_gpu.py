"""Parity at the sizes the benchmark publishes, not at reduced ones.

* the fp32 GEMM sweep (1024^3 in full; 4096^3, 8192^3, the skinny 64x4096x4096 and the
  long-K 512x65536x512 on whole rows of C chosen across every M-tile) against the
  reference CPU matmul kernel (oracle/_ref, compiled from the reference's sources) run on
  the same rows of A on all host threads -- asserted against the relative Frobenius bound
  1e-5*sqrt(K) and against vkML's backward-error bound, with the measured error recorded;
* the inputs vkML uses to attack GEMM numerics (tests/python/test_invariants.py:496-531),
  tiled up to a shape the tensor-core kernel takes, with the reference's structural
  assertions (NaN / infinity / sign pattern equal to the CPU's);
* softmax, log_softmax, the row sum and cross-entropy forward AND backward at
  (65536,10), (8192,1000), (1024,32000);
* full-size training steps of the CNN (batch 256) and of the wide MLP (batch 2048) through
  the reference's own executor and the adapter, against fixtures the reference CPU backend
  produced once (tests/golden/make_full_size_steps.py).
"""
import ctypes as C
import json
import os
import sys

import numpy as np
import pytest

import cases
import training
from helpers import REF_B200_SO, REF_SO, CudaImpl, OracleImpl, host_desc
from vkml_b200 import DeviceTensor, NodeDesc, _abi, graph
from vkml_b200.graph import DType, Op

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
GOLDEN = os.path.join(HERE, "golden")
if GOLDEN not in sys.path:
    sys.path.insert(0, GOLDEN)  # the fixture generator holds the configurations
SEED = training.SEED_DATA
THREADS = os.cpu_count() or 1


def record(**fields):
    """Measured errors go to stdout and, when VKML_B200_TEST_RECORDS names a directory, into a
    JSON-lines file there."""
    line = json.dumps(fields)
    print(line)
    out = os.environ.get("VKML_B200_TEST_RECORDS", "")
    if out and os.path.isdir(out):
        with open(os.path.join(out, "parity_measured.jsonl"), "a") as f:
            f.write(line + "\n")


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libvkml_ref.so not built")
    lib = C.CDLL(REF_SO)
    lib.vkml_ref_matmul_mt.restype = C.c_int
    lib.vkml_ref_matmul_mt.argtypes = [C.POINTER(_abi.Node), C.c_int]
    return lib


def reference_matmul(ref, a, b):
    """A[m,k] . B[k,n] with the reference CPU kernel, row slabs on all host threads."""
    a4, b4 = a.reshape((1, 1) + a.shape), b.reshape((1, 1) + b.shape)
    out = np.zeros((1, 1, a.shape[0], b.shape[1]), dtype=np.float32)
    node = NodeDesc(int(Op.MATMUL), host_desc(out), [host_desc(a4), host_desc(b4)]).to_c()
    assert ref.vkml_ref_matmul_mt(C.byref(node), THREADS) == 0
    return out[0, 0]


def rel_frobenius(got, want):
    want64 = want.astype(np.float64)
    return float(np.linalg.norm(got.astype(np.float64) - want64) / np.linalg.norm(want64))


# (m, k, n, rows compared; 0 = all)
GEMM_SWEEP = [(1024, 1024, 1024, 0), (4096, 4096, 4096, 32), (8192, 8192, 8192, 64),
              (64, 4096, 4096, 0), (512, 65536, 512, 32)]


@pytest.mark.parametrize("m,k,n,n_rows", GEMM_SWEEP, ids=lambda v: str(v))
def test_gemm_sweep_against_the_reference_kernel(backend, ref, m, k, n, n_rows):
    """C = A.B, A and B ~ N(0,1), as one matmul node through Backend.compute (what bench.py
    times).  Compared rows are spread so that every M-tile of the kernel contributes one."""
    rng = np.random.default_rng(SEED)
    a = rng.standard_normal((m, k), dtype=np.float32)
    b = rng.standard_normal((k, n), dtype=np.float32)
    ta = DeviceTensor.from_host(backend, a.reshape(1, 1, m, k))
    tb = DeviceTensor.from_host(backend, b.reshape(1, 1, k, n))
    tc = DeviceTensor.empty(backend, (1, 1, m, n))
    backend.set_profiling(True)
    backend.compute([NodeDesc(Op.MATMUL, tc.desc, [ta.desc, tb.desc])])
    labels = [l for l, _ in backend.last_profile()]
    backend.set_profiling(False)
    got = tc.numpy()[0, 0]
    if n_rows:
        step = m // n_rows
        rows = np.arange(n_rows) * step + rng.integers(0, step, n_rows)
    else:
        rows = np.arange(m)
    a_rows = np.ascontiguousarray(a[rows])
    want = reference_matmul(ref, a_rows, b)
    got = got[rows]
    rel = rel_frobenius(got, want)
    tas = np.abs(a_rows.astype(np.float64)) @ np.abs(b.astype(np.float64))
    bound = cases.pairwise_gamma(k) * tas * 4.0
    worst = float(np.max(np.abs(got.astype(np.float64) - want) / bound))
    record(test="gemm_sweep", m=m, k=k, n=n, rows=int(len(rows)), outputs=int(got.size), kernels=labels,
           rel_frobenius=rel, bound=1e-5 * float(np.sqrt(k)), worst_fraction_of_backward_bound=worst)
    assert any(l.startswith("matmul.") for l in labels)
    assert rel < 1e-5 * np.sqrt(k), rel
    assert worst <= 1.0, worst
    assert np.all(np.isfinite(got))


def adversarial(name, rng, shape):
    """The input classes of vkML's adversarial GEMM test (tests/python/test_invariants.py:496-509)."""
    if name == "cancelling":  # alternating +-1e7: every dot product is exactly zero on the CPU
        return np.where((np.arange(shape[0] * shape[1]).reshape(shape) % 2) == 0, 1e7, -1e7).astype(np.float32)
    if name == "tiny":
        return (rng.standard_normal(shape) * 1e-30).astype(np.float32)
    if name == "huge":
        return (rng.standard_normal(shape) * 1e20).astype(np.float32)
    if name == "mixed-magnitude":
        return (rng.standard_normal(shape) * 10.0 ** rng.integers(-20, 20, shape)).astype(np.float32)
    if name == "subnormal":
        return (rng.standard_normal(shape) * 1e-42).astype(np.float32)
    if name == "exact-halves":
        return (rng.integers(-8, 8, shape) * 0.5).astype(np.float32)
    raise KeyError(name)


ADVERSARIAL = ["cancelling", "tiny", "huge", "mixed-magnitude", "subnormal", "exact-halves"]
OVERFLOWING = {"huge", "mixed-magnitude"}  # classes with products beyond the fp32 range


@pytest.mark.parametrize("name", ADVERSARIAL)
@pytest.mark.parametrize("shape", [(64, 96, 64), (256, 512, 256)], ids=["cuda-core-64x96x64", "tensor-core-256x512x256"])
def test_adversarial_gemm_inputs(backend, name, shape):
    """vkML's own shape (64x96 . 96x64, served by the fp32 CUDA-core kernel here) and the same
    classes at a shape the tensor-core 3xTF32 kernel takes.  The reference asserts structure,
    not value: the NaN pattern, the infinity pattern and the sign pattern equal the CPU's.  That
    holds for every class on the CUDA-core kernel and for every class without overflowing
    products on the tensor cores; for the two overflowing classes see the comment below."""
    m, k, n = shape
    rng = np.random.default_rng(ADVERSARIAL.index(name) + 1000 * m)
    a = adversarial(name, rng, (m, k)).reshape(1, 1, m, k)
    b = adversarial(name, rng, (k, n)).reshape(1, 1, k, n)
    with np.errstate(all="ignore"):
        want = OracleImpl().run(Op.MATMUL, [a, b], (1, 1, m, n), DType.F32)
    impl = CudaImpl(backend)
    backend.set_profiling(True)
    got = impl.run(Op.MATMUL, [a, b], (1, 1, m, n), DType.F32)
    labels = [l for l, _ in backend.last_profile()]
    backend.set_profiling(False)
    on_tensor_cores = any(l.startswith("matmul.tcgen05") for l in labels)
    assert on_tensor_cores == (m >= 256), labels
    nan_same = bool(np.array_equal(np.isnan(got), np.isnan(want)))
    inf_same = bool(np.array_equal(np.isinf(got), np.isinf(want)))
    sign_same = bool(np.array_equal(np.signbit(got), np.signbit(want)) or not np.all(np.isfinite(got)))
    nf_gpu, nf_cpu = ~np.isfinite(got), ~np.isfinite(want)
    record(test="adversarial", name=name, shape=list(shape), kernels=labels, nan_pattern_equal=nan_same,
           inf_pattern_equal=inf_same, sign_pattern_equal=sign_same, cpu_nonfinite=int(nf_cpu.sum()),
           gpu_nonfinite=int(nf_gpu.sum()), nonfinite_only_on_gpu=int((nf_gpu & ~nf_cpu).sum()),
           nonfinite_only_on_cpu=int((nf_cpu & ~nf_gpu).sum()))
    if on_tensor_cores and name in OVERFLOWING:
        # The one decided divergence.  Products beyond the fp32 range: the CPU rounds every product
        # to +-inf before it sums, so opposite infinities meet as NaN; the tensor core forms the
        # products of one instruction exactly and rounds their SUM, so a +huge and a -huge product
        # may cancel before anything overflows, and what does overflow arrives as an infinity.
        # Held instead: the non-finite outputs are a subset of the CPU's (the tensor cores never
        # invent one), an output the CPU lost to overflow and the tensor cores kept is finite in
        # exact arithmetic too, and everything finite on both sides is inside the usual bound.
        assert not np.any(nf_gpu & ~nf_cpu), f"{name}: non-finite on the GPU only"
        with np.errstate(all="ignore"):
            exact = a[0, 0].astype(np.float64) @ b[0, 0].astype(np.float64)
        kept = (nf_cpu & ~nf_gpu)[0, 0]
        assert np.all(np.abs(exact[kept]) < np.finfo(np.float32).max)
        both = ~nf_cpu & ~nf_gpu
        tas = np.abs(a[0, 0].astype(np.float64)) @ np.abs(b[0, 0].astype(np.float64))
        with np.errstate(all="ignore"):
            err = np.abs(got.astype(np.float64) - want)[0, 0]
        ok = err <= 4.0 * cases.pairwise_gamma(k) * tas
        assert np.all(ok | ~both[0, 0])
        return
    assert nan_same, f"{name}: NaN pattern differs"
    assert inf_same, f"{name}: infinity pattern differs"
    assert sign_same, f"{name}: sign pattern differs"
    if name == "cancelling":
        assert np.all(got == 0.0)  # no residue of the hi/lo split where the exact answer is zero
    if name == "exact-halves":
        assert np.array_equal(got, want)  # every product and sum is exact in either arithmetic


CONFIG3 = [(65536, 10), (8192, 1000), (1024, 32000)]


def config3_inputs(b, c):
    rng = np.random.default_rng(SEED)
    logits = (2.0 * rng.standard_normal((b, c))).astype(np.float32)  # N(0, 4)
    labels = rng.integers(0, c, b).astype(np.int64)
    return logits, labels


@pytest.mark.parametrize("b,c", CONFIG3)
def test_softmax_log_softmax_and_row_sum_at_full_shapes(backend, b, c):
    logits, _ = config3_inputs(b, c)
    impl, oracle = CudaImpl(backend), OracleImpl()
    for op in (Op.SOFTMAX, Op.LOG_SOFTMAX):
        want = oracle.run(op, [logits], (b, c), DType.F32, graph.axis_params(1))
        got = impl.run(op, [logits], (b, c), DType.F32, graph.axis_params(1))
        cases.check(cases.Case(f"{graph.op_name(op)}/{b}x{c}", op, [logits], (b, c), DType.F32), got, want)
        record(test="config3", op=graph.op_name(op), b=b, c=c,
               max_rel=float(np.max(np.abs(got - want) / np.maximum(np.abs(want), 1e-30))))
    params = graph.reduce_params([1], 2)
    want = oracle.run(Op.SUM, [logits], (b,), DType.F32, params)
    got = impl.run(Op.SUM, [logits], (b,), DType.F32, params)
    case = cases.Case(f"sum/{b}x{c}", Op.SUM, [logits], (b,), DType.F32, params,
                      terms_abs_sum=np.abs(logits.astype(np.float64)).sum(1), reduction_n=c)
    cases.check(case, got, want)
    record(test="config3", op="sum", b=b, c=c, max_abs=float(np.max(np.abs(got - want))))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(REF_B200_SO):
        pytest.skip("oracle/_ref/libvkml_ref_b200.so not built")
    lib = training.load(with_b200=True)
    f32p, i64p = C.POINTER(C.c_float), C.POINTER(C.c_int64)
    lib.vkml_ref_cross_entropy.restype = C.c_int
    lib.vkml_ref_cross_entropy.argtypes = [C.c_int, f32p, i64p, C.c_int64, C.c_int64, f32p, f32p]
    return lib


def cross_entropy(lib, device, logits, labels):
    b, c = logits.shape
    loss, grad = C.c_float(0), np.zeros((b, c), dtype=np.float32)
    f32p, i64p = C.POINTER(C.c_float), C.POINTER(C.c_int64)
    rc = lib.vkml_ref_cross_entropy(device, logits.ctypes.data_as(f32p), labels.ctypes.data_as(i64p), b, c,
                                    C.byref(loss), grad.ctypes.data_as(f32p))
    assert rc == 0, lib.vkml_ref_last_error().decode()
    return float(loss.value), grad


@pytest.mark.parametrize("b,c", CONFIG3)
def test_cross_entropy_forward_and_backward_at_full_shapes(lib, b, c):
    """cross_entropy(logits, labels) and backward() through the reference's own graph and autograd
    on both devices: the scalar loss (rtol = atol = 1e-5, vkML's policy for this composite,
    tests/python/tolerance.py:238-239) and d loss / d logits, which is (softmax - onehot) / b."""
    logits, labels = config3_inputs(b, c)
    cpu_loss, cpu_grad = cross_entropy(lib, training.CPU, logits, labels)
    gpu_loss, gpu_grad = cross_entropy(lib, training.B200, logits, labels)
    record(test="cross_entropy", b=b, c=c, cpu_loss=cpu_loss, gpu_loss=gpu_loss,
           grad_max_abs=float(np.max(np.abs(gpu_grad - cpu_grad))), grad_rel_frobenius=rel_frobenius(gpu_grad, cpu_grad))
    assert abs(gpu_loss - cpu_loss) <= 1e-5 + 1e-5 * abs(cpu_loss)
    np.testing.assert_allclose(gpu_grad, cpu_grad, rtol=1e-5, atol=1e-5 / b)
    # the closed form vkML's own test checks (tests/python/test_ops_vs_torch.py:909-923)
    x = logits.astype(np.float64)
    p = np.exp(x - x.max(1, keepdims=True))
    p /= p.sum(1, keepdims=True)
    p[np.arange(b), labels] -= 1.0
    np.testing.assert_allclose(gpu_grad, p / b, rtol=1e-4, atol=1e-6 / b)


def full_size_fixture():
    path = os.path.join(GOLDEN, "full_size_steps.npz")
    if not os.path.exists(path):
        pytest.skip("tests/golden/full_size_steps.npz missing")
    return np.load(path)


def rel(a, b):
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-12)))


def test_full_size_cnn_steps(lib):
    """Benchmark configuration 4 at its own size -- batch 256, conv 64/128/256, Linear 4096->100 --
    three steps of SGD with momentum through the reference's executor and the adapter: every loss
    within 1e-4 relative of the CPU backend's, sampled parameters within 1e-4 after the last step."""
    import make_full_size_steps as gen
    fx = full_size_fixture()
    params, x, y = training.cnn_problem(batch=gen.CNN_BATCH, steps=gen.CNN_STEPS, **gen.CNN)
    losses, p = training.train_cnn(lib, training.B200, params=params, x=x, y=y, batch=gen.CNN_BATCH,
                                   steps=gen.CNN_STEPS, lr=gen.CNN_LR, **gen.CNN)
    record(test="full_size_cnn", gpu_losses=[float(v) for v in losses], cpu_losses=[float(v) for v in fx["cnn_losses"]],
           params_max_abs=float(np.max(np.abs(p[fx["cnn_positions"]] - fx["cnn_params"]))))
    assert rel(losses, fx["cnn_losses"]) < 1e-4
    np.testing.assert_allclose(p[fx["cnn_positions"]], fx["cnn_params"], rtol=0, atol=1e-4)


def test_full_size_wide_mlp_steps(lib):
    """Benchmark configuration 5 at its own size -- 4096-8192-8192-8192-1000, batch 2048 -- two
    steps: the second loss depends on every gradient and on the optimiser's update."""
    import make_full_size_steps as gen
    fx = full_size_fixture()
    if "mlp_losses" not in fx:
        pytest.skip("the wide-MLP fixture has not been generated")
    ws, bs, x, y = training.mlp_problem(gen.MLP_WIDTHS, gen.MLP_BATCH, gen.MLP_STEPS, data="normal")
    losses, w, b = training.train_mlp(lib, training.B200, gen.MLP_WIDTHS, ws, bs, x, y, gen.MLP_BATCH,
                                      gen.MLP_STEPS, lr=gen.MLP_LR)
    record(test="full_size_wide_mlp", gpu_losses=[float(v) for v in losses],
           cpu_losses=[float(v) for v in fx["mlp_losses"]],
           weights_max_abs=float(np.max(np.abs(w[fx["mlp_positions"]] - fx["mlp_weights"]))),
           biases_max_abs=float(np.max(np.abs(b - fx["mlp_biases"]))))
    assert rel(losses, fx["mlp_losses"]) < 1e-4
    np.testing.assert_allclose(w[fx["mlp_positions"]], fx["mlp_weights"], rtol=0, atol=1e-4)
    np.testing.assert_allclose(b, fx["mlp_biases"], rtol=0, atol=1e-4)


def test_full_size_wide_mlp_one_step(lib):
    """The same configuration, one step on a problem of its own: the loss checks the forward pass, the
    sampled weights and every bias after the update check every gradient and the optimiser."""
    import make_full_size_steps as gen
    if not os.path.exists(gen.OUT_MLP1):
        pytest.skip("the one-step wide-MLP fixture has not been generated")
    fx = np.load(gen.OUT_MLP1)
    ws, bs, x, y = training.mlp_problem(gen.MLP_WIDTHS, gen.MLP_BATCH, 1, data="normal")
    losses, w, b = training.train_mlp(lib, training.B200, gen.MLP_WIDTHS, ws, bs, x, y, gen.MLP_BATCH, 1, lr=gen.MLP_LR)
    record(test="full_size_wide_mlp_one_step", gpu_losses=[float(v) for v in losses],
           cpu_losses=[float(v) for v in fx["mlp1_losses"]],
           weights_max_abs=float(np.max(np.abs(w[fx["mlp1_positions"]] - fx["mlp1_weights"]))),
           biases_max_abs=float(np.max(np.abs(b - fx["mlp1_biases"]))))
    assert rel(losses, fx["mlp1_losses"]) < 1e-4
    np.testing.assert_allclose(w[fx["mlp1_positions"]], fx["mlp1_weights"], rtol=0, atol=1e-4)
    np.testing.assert_allclose(b, fx["mlp1_biases"], rtol=0, atol=1e-4)
