"""Pins the CPU oracle (oracle/vkml_oracle.c) before anything trusts it:

1. against the known-answer vectors of vkML's own C++ tests
   (tests/cpp/test_ops.cpp:105-311, tests/cpp/test_core.cpp:30-62), transcribed in
   tests/golden/known_answers.json;
2. bit for bit against the reference CPU backend compiled from its own sources
   (oracle/_ref/libvkml_ref.so), over every seeded case the GPU parity tests use;
3. against the committed fixtures in tests/golden/*.npz, which hold outputs of
   that same reference build (so the pin survives where the reference tree and
   its build are absent).
"""
import ctypes as C
import json
import os

import numpy as np
import pytest

import cases
from cases import Case
from helpers import ORACLE_SO, REF_SO, OracleImpl, RefImpl
from vkml_b200 import graph
from vkml_b200.graph import DType, Op

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def oracle():
    return OracleImpl()


@pytest.fixture(scope="module")
def ref():
    if not os.path.exists(REF_SO):
        pytest.skip("oracle/_ref/libvkml_ref.so not built (needs the reference tree)")
    return RefImpl()


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a).view(np.uint8)


def _params(spec) -> bytes:
    kind = spec.get("params")
    if kind is None:
        return b""
    name, args = kind[0], kind[1:]
    return getattr(graph, name + "_params")(*args)


def test_known_answers_from_the_reference_tests(oracle):
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        table = json.load(f)
    assert len(table) >= 25
    for spec in table:
        srcs = []
        for s in spec["srcs"]:
            if s.get("values") is None:  # a constant run, optionally with a different first element
                a = np.full(s["shape"], s["fill"], dtype=np.float32)
                a.reshape(-1)[0] = s.get("first", s["fill"])
            else:
                a = np.array(s["values"], dtype=DType[s.get("dtype", "F32")].numpy).reshape(s["shape"])
            if s.get("transpose"):
                a = a.T
            if "broadcast" in s:
                a = np.broadcast_to(a, s["broadcast"])
            srcs.append(a)
        out_dt = DType[spec.get("out_dtype", "F32")]
        got = oracle.run(Op[spec["op"].upper()], srcs, tuple(spec["out_shape"]), out_dt, _params(spec))
        want = np.array(spec["want"], dtype=out_dt.numpy).reshape(spec["out_shape"])
        if "rtol" in spec:
            np.testing.assert_allclose(got, want, rtol=spec["rtol"], atol=spec.get("atol", 0), err_msg=spec["name"])
        else:
            np.testing.assert_array_equal(got, want, err_msg=spec["name"])


def test_fp16_tables(oracle):
    lib = oracle.lib
    lib.vkml_oracle_f32_to_f16.restype = C.c_uint16
    lib.vkml_oracle_f32_to_f16.argtypes = [C.c_float]
    lib.vkml_oracle_f16_to_f32.restype = C.c_float
    lib.vkml_oracle_f16_to_f32.argtypes = [C.c_uint16]
    rt = lambda v: lib.vkml_oracle_f16_to_f32(lib.vkml_oracle_f32_to_f16(v))
    for v in [0.0, 1.0, -1.0, 0.5, -0.5, 2.0, 1024.0, -65504.0, 65504.0]:
        assert rt(v) == v
    assert lib.vkml_oracle_f32_to_f16(5.9604645e-8) != 0 and rt(5.9604645e-8) > 0  # subnormals kept
    assert rt(3.0e-8) > 0
    assert np.isinf(rt(float("inf"))) and rt(float("-inf")) < 0 and np.isnan(rt(float("nan")))
    assert np.isinf(rt(1.0e30))
    # every half value survives half -> float -> half, and numpy agrees on the widening
    allh = np.arange(65536, dtype=np.uint16)
    wide = allh.view(np.float16).astype(np.float32)
    for h in range(0, 65536, 7):
        f = lib.vkml_oracle_f16_to_f32(h)
        if np.isnan(wide[h]):
            assert np.isnan(f)
        else:
            assert f == wide[h]
            assert lib.vkml_oracle_f32_to_f16(f) == h
    # round-to-nearest-even against numpy's conversion
    rng = np.random.default_rng(3)
    xs = np.concatenate([rng.standard_normal(2000).astype(np.float32) * s for s in (1e-7, 1e-4, 1.0, 1e3, 7e4)])
    want = xs.astype(np.float16).view(np.uint16)
    got = np.array([lib.vkml_oracle_f32_to_f16(float(x)) for x in xs], dtype=np.uint16)
    np.testing.assert_array_equal(got, want)


def _all_case_ids():
    return [c.name for c in cases.all_cases()]


def test_oracle_matches_reference_bit_for_bit(oracle, ref):
    """The restatement and the compiled reference CPU backend agree on every byte."""
    n = 0
    for case in cases.all_cases():
        if case.op == Op.CAST and case.name in ("cast/f32->i32", "cast/f32->i64"):
            pass  # in-range values only in these cases; out-of-range float->int is undefined in C++
        rc_r, want = ref.run_status(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
        rc_o, got = oracle.run_status(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
        assert rc_r == rc_o, f"{case.name}: status oracle {rc_o} vs reference {rc_r}"
        if rc_r != 0:
            continue
        assert got.dtype == want.dtype and got.shape == want.shape
        if not np.array_equal(bits(got), bits(want)):
            bad = np.argwhere(got != want)
            raise AssertionError(f"{case.name}: oracle differs from the reference at {bad[:3].tolist()}: "
                                 f"{got[tuple(bad[0])]!r} vs {want[tuple(bad[0])]!r}" if len(bad) else
                                 f"{case.name}: bit patterns differ (signed zero or NaN payload)")
        n += 1
    assert n > 800


def test_f16_storage_matches_reference_bit_for_bit(oracle, ref):
    """F16 operands and results: the restatement's widen / compute in f32 / narrow once composition
    against the compiled reference's Half kernels, every family, bit for bit."""
    n = 0
    for case in cases.f16_cases():
        rc_r, want = ref.run_status(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
        rc_o, got = oracle.run_status(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
        assert rc_r == 0 and rc_o == 0, f"{case.name}: status oracle {rc_o}, reference {rc_r}"
        assert got.dtype == want.dtype and got.shape == want.shape, case.name
        if not np.array_equal(bits(got), bits(want)):
            bad = np.argwhere(bits(got) != bits(want))
            raise AssertionError(f"{case.name}: oracle differs from the reference at {bad[:3].tolist()}: "
                                 f"{got[tuple(bad[0])]!r} vs {want[tuple(bad[0])]!r}")
        n += 1
    assert n >= 38


def test_index_errors_match_the_reference(oracle, ref):
    table = np.arange(12, dtype=np.float32).reshape(4, 3)
    for bad_index in (-1, 4):
        idx = np.array([0, bad_index], dtype=np.int64)
        for impl in (oracle, ref):
            rc, _ = impl.run_status(Op.INDEX_SELECT, [table, idx], (2, 3), DType.F32, graph.axis_params(0))
            assert rc == 4  # IndexError
            rc, _ = impl.run_status(Op.SCATTER_ADD, [table[:2], idx], (4, 3), DType.F32, graph.axis_params(0))
            assert rc == 4


def test_golden_fixtures(oracle):
    """Outputs of the reference build, generated by tests/golden/make_golden.py."""
    path = os.path.join(GOLDEN, "reference_outputs.npz")
    data = np.load(path)
    names = json.loads(str(data["__index__"]))
    assert len(names) >= 60
    by_name = {c.name: c for c in cases.all_cases(quick=True)}
    by_name.update({c.name: c for c in cases.f16_cases()})
    for i, name in enumerate(names):
        case = by_name[name]
        want = data[f"out_{i}"]
        got = oracle.run(case.op, case.srcs, case.out_shape, case.out_dtype, case.params)
        assert np.array_equal(bits(got), bits(want)), name
