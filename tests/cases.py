"""Seeded op cases shared by the oracle-pinning tests (CPU) and the CUDA parity
tests (GPU), with the tolerance each op is held to.

The tolerance table restates vkML's own device-vs-CPU policy
(tests/python/tolerance.py:89-278): EXACT for everything that moves bits,
selects an element, or is one correctly-rounded IEEE operation; a ULP budget for
the transcendental functions (libm on the CPU, CUDA's math library on the GPU);
relative 1e-5 for softmax; a backward-error bound gamma*sum|terms| for sums,
means and dot products whose summation ORDER differs between implementations.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from vkml_b200 import graph
from vkml_b200.graph import DType, Op

from helpers import ELEMENT_SIZES, layouts

FP32_EPS = float(np.finfo(np.float32).eps)
PAIRWISE_BLOCK = 32

# kind, ulp, rtol, atol
POLICY = {
    "exact": ("exact", 0, 0, 0),
    "div": ("ulp", 3, 0, 0), "sqrt": ("ulp", 3, 0, 0), "rsqrt": ("ulp", 3, 0, 0),
    "reciprocal": ("ulp", 3, 0, 0), "exp": ("ulp", 8, 0, 0), "log": ("ulp", 4, 0, 2.0 ** -21),
    "sin": ("ulp", 0, 0, 2.0 ** -11), "cos": ("ulp", 0, 0, 2.0 ** -11),
    "erf": ("rel", 0, 1e-6, 1e-7), "erfc": ("rel", 0, 1e-5, 1e-7), "tanh": ("rel", 0, 1e-5, 1e-7),
    "sigmoid": ("rel", 0, 1e-5, 1e-7), "gelu": ("rel", 0, 1e-5, 1e-7), "silu": ("rel", 0, 1e-5, 1e-7),
    "pow": ("ulp", 16, 0, 0), "arange": ("ulp", 4, 0, 0),
    "softmax": ("rel", 0, 1e-5, 1e-7), "log_softmax": ("rel", 0, 1e-5, 1e-5),
    "sum": ("backward", 0, 0, 0), "mean": ("backward", 0, 0, 0), "matmul": ("backward", 0, 0, 0),
}

EXACT_OPS = {"full", "rand", "contiguous", "cast", "cat", "index_select", "im2col", "max_pool2d",
             "max_pool2d_backward", "col2im", "scatter_add", "relu", "neg", "abs", "sign", "clamp",
             "maximum", "minimum", "where", "triu", "tril", "equal", "less", "greater", "less_equal",
             "greater_equal", "not_equal", "argmax", "argmin", "max", "min", "add", "sub", "mul",
             "square", "scaled_add", "slice_backward", "prod"}


def policy_for(op_name: str):
    if op_name in EXACT_OPS:
        return POLICY["exact"]
    return POLICY[op_name]


def ulp_distance(a, b):
    ai = a.astype(np.float32).view(np.int32).astype(np.int64)
    bi = b.astype(np.float32).view(np.int32).astype(np.int64)
    ai = np.where(ai < 0, np.int64(0x80000000) - ai, ai)
    bi = np.where(bi < 0, np.int64(0x80000000) - bi, bi)
    return np.abs(ai - bi)


def pairwise_gamma(n: int) -> float:
    if n <= 1:
        return 0.0
    return (PAIRWISE_BLOCK + np.log2(max(n / PAIRWISE_BLOCK, 1.0))) * FP32_EPS


@dataclass
class Case:
    name: str
    op: int
    srcs: list
    out_shape: tuple
    out_dtype: DType
    params: bytes = b""
    # for the backward-error bound: per-output sum|terms| and the term count
    terms_abs_sum: object = None
    reduction_n: int = 0

    @property
    def op_name(self) -> str:
        return graph.op_name(self.op)


def check(case: Case, got: np.ndarray, want: np.ndarray, exact_override: bool = False):
    """Assert `got` matches `want` under the case's policy (or bit-exactly)."""
    assert got.shape == want.shape, f"{case.name}: shape {got.shape} vs {want.shape}"
    assert got.dtype == want.dtype, f"{case.name}: dtype {got.dtype} vs {want.dtype}"
    if got.size == 0:
        return
    kind, ulp, rtol, atol = POLICY["exact"] if exact_override else policy_for(case.op_name)
    floating = np.issubdtype(got.dtype, np.floating)
    if got.dtype == np.float16 and kind != "exact":
        # F16 is storage: both sides compute in f32 and narrow once, so an f32 difference inside the
        # op's own policy can move the narrowed value by at most one f16 ulp (tests/python/test_f16.py
        # in vkML holds f16 results to 1e-3)
        nan_g, nan_w = np.isnan(got), np.isnan(want)
        assert np.array_equal(nan_g, nan_w), f"{case.name}: NaN pattern differs"
        gi = got.view(np.int16).astype(np.int64)
        wi = want.view(np.int16).astype(np.int64)
        gi = np.where(gi < 0, np.int64(0x8000) - gi, gi)
        wi = np.where(wi < 0, np.int64(0x8000) - wi, wi)
        bad = (np.abs(gi - wi) > 1) & ~nan_g
        if kind == "backward":
            # sums and dot products: the f32 results may differ by the backward-error bound (which
            # is many f16 ulps for an output that cancels to nearly zero) before the one narrowing
            bound = pairwise_gamma(case.reduction_n) * np.asarray(case.terms_abs_sum, dtype=np.float64) * 4.0
            bound = np.broadcast_to(bound.reshape(got.shape) if np.ndim(bound) else bound, got.shape)
            with np.errstate(invalid="ignore"):
                diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
                spacing = np.spacing(np.abs(want)).astype(np.float64)
            bad &= diff > bound + spacing
        if np.any(bad):
            idx = np.argwhere(bad)[0]
            raise AssertionError(f"{case.name} [f16 ulp]: {int(bad.sum())}/{bad.size} differ; first at {tuple(idx)}: "
                                 f"got {got[tuple(idx)]!r} want {want[tuple(idx)]!r}")
        return
    nan_g = np.zeros(got.shape, dtype=bool)
    if floating:
        nan_g, nan_w = np.isnan(got), np.isnan(want)
        assert np.array_equal(nan_g, nan_w), f"{case.name}: NaN pattern differs"
    if kind == "exact":
        # value comparison, NaN placement checked above (vkML's EXACT policy)
        bad = ((got != want) & ~nan_g) if floating else (got != want)
    elif kind == "ulp":
        diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
        bad = np.zeros(got.shape, dtype=bool)
        with np.errstate(invalid="ignore"):
            if ulp:
                bad |= (ulp_distance(got, want) > ulp) & ~nan_g & (got != want)
            else:
                bad |= (got != want) & ~nan_g
            if atol:
                bad &= diff > atol
    elif kind == "rel":
        bad = ~np.isclose(got, want, rtol=rtol, atol=atol, equal_nan=True)
    elif kind == "backward":
        bound = pairwise_gamma(case.reduction_n) * np.asarray(case.terms_abs_sum, dtype=np.float64) * 4.0
        with np.errstate(invalid="ignore"):
            diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
        bad = (diff > np.broadcast_to(bound.reshape(got.shape) if np.ndim(bound) else bound, got.shape)) & ~nan_g
        bad &= ~((got == want))
    else:
        raise AssertionError(kind)
    if np.any(bad):
        idx = np.argwhere(bad)[0]
        raise AssertionError(
            f"{case.name} [{kind}]: {int(bad.sum())}/{bad.size} elements differ; first at {tuple(idx)}: "
            f"got {got[tuple(idx)]!r} want {want[tuple(idx)]!r}")


# ---------------------------------------------------------------------------

UNARY = ["neg", "abs", "sign", "square", "sqrt", "rsqrt", "reciprocal", "exp", "log", "erf", "erfc",
         "sin", "cos", "tanh", "sigmoid", "relu", "gelu", "silu"]
BINARY = ["add", "sub", "mul", "div", "pow", "maximum", "minimum"]
COMPARE = ["equal", "less", "greater", "less_equal", "greater_equal", "not_equal"]


def _unary_input(rng, name, shape):
    x = rng.standard_normal(shape).astype(np.float32)
    if name in ("sqrt", "rsqrt", "log"):
        x = np.abs(x) + np.float32(0.05)
    if name in ("exp", "sin", "cos"):
        x = np.clip(x, -3, 3)
    if name == "reciprocal":
        x = np.where(np.abs(x) < 0.05, np.float32(0.5), x)
    return x.astype(np.float32)


def elementwise_cases(seed=1234, sizes=ELEMENT_SIZES, quick=False):
    rng = np.random.default_rng(seed)
    # dense 1-D at the block-edge sizes
    for name in UNARY:
        for n in (sizes if not quick else [257]):
            yield Case(f"{name}/n={n}", Op[name.upper()], [_unary_input(rng, name, (n,))], (n,), DType.F32)
    for name in BINARY:
        for n in (sizes if not quick else [257]):
            a = rng.standard_normal((n,)).astype(np.float32)
            b = rng.standard_normal((n,)).astype(np.float32)
            if name == "pow":
                a = np.abs(a) + np.float32(0.1)
            if name == "div":
                b = np.where(np.abs(b) < 0.05, np.float32(0.5), b).astype(np.float32)
            yield Case(f"{name}/n={n}", Op[name.upper()], [a, b], (n,), DType.F32)
    for name in COMPARE:
        n = 1000
        a = rng.integers(-3, 4, n).astype(np.float32)
        b = rng.integers(-3, 4, n).astype(np.float32)
        a[::17] = np.nan
        yield Case(f"{name}/n={n}", Op[name.upper()], [a, b], (n,), DType.BOOL)
    # NaN rules
    x = np.array([np.nan, -0.0, 0.0, 1.0, -1.0, np.inf, -np.inf, 1e-42, -1e-42], dtype=np.float32)
    for name in ("relu", "sign", "neg", "abs", "square"):
        yield Case(f"{name}/special", Op[name.upper()], [x], x.shape, DType.F32)
    y = x[::-1].copy()
    for name in ("maximum", "minimum", "add", "mul", "sub"):
        yield Case(f"{name}/special", Op[name.upper()], [x, y], x.shape, DType.F32)
    # layouts: every stride pattern, rank 2 and rank 4
    # (200, 132) and (3, 64, 68) mix whole 64x64 tiles (128-bit path) with ragged edge tiles
    for shape in [(33, 65), (3, 5, 17, 9), (64, 128), (255, 257), (200, 132), (3, 64, 68)]:
        for tag_a, a in layouts(rng, shape):
            yield Case(f"relu/{shape}/{tag_a}", Op.RELU, [a], shape, DType.F32)
            yield Case(f"contiguous/{shape}/{tag_a}", Op.CONTIGUOUS, [a], shape, DType.F32)
            for tag_b, b in layouts(rng, shape):
                yield Case(f"add/{shape}/{tag_a}+{tag_b}", Op.ADD, [a, b], shape, DType.F32)
                yield Case(f"scaled_add/{shape}/{tag_a}+{tag_b}", Op.SCALED_ADD, [a, b], shape, DType.F32,
                           graph.scaled_add_params(0.9, -0.1))
    # broadcasts as stride-0 views: bias rows, columns, channels, scalars
    a = rng.standard_normal((64, 128)).astype(np.float32)
    row = np.broadcast_to(rng.standard_normal((128,)).astype(np.float32), (64, 128))
    col = np.broadcast_to(rng.standard_normal((64, 1)).astype(np.float32), (64, 128))
    scalar = np.broadcast_to(np.float32(0.25).reshape(()), (64, 128))
    yield Case("add/row-broadcast", Op.ADD, [a, row], a.shape, DType.F32)
    a_t = np.ascontiguousarray(a.T).T
    yield Case("add/transposed+row-broadcast", Op.ADD, [a_t, row], a.shape, DType.F32)
    yield Case("mul/col-broadcast*transposed", Op.MUL, [col, a_t], a.shape, DType.F32)
    yield Case("mul/col-broadcast", Op.MUL, [a, col], a.shape, DType.F32)
    yield Case("div/scalar-broadcast", Op.DIV, [a, scalar], a.shape, DType.F32)
    yield Case("equal/both-broadcast", Op.EQUAL,
               [np.broadcast_to(np.arange(64, dtype=np.float32).reshape(64, 1) % 10, (64, 10)),
                np.broadcast_to(np.arange(10, dtype=np.float32).reshape(1, 10), (64, 10))], (64, 10), DType.BOOL)
    img = rng.standard_normal((4, 8, 6, 6)).astype(np.float32)
    chan = np.broadcast_to(rng.standard_normal((8, 1, 1)).astype(np.float32), (4, 8, 6, 6))
    yield Case("add/channel-broadcast", Op.ADD, [img, chan], img.shape, DType.F32)
    yield Case("contiguous/broadcast-materialise", Op.CONTIGUOUS,
               [np.broadcast_to(np.float32(3.5).reshape(()), (64,))], (64,), DType.F32)
    # where / clamp / scaled_add bit identity / tri
    cond = (rng.random((64, 128)) < 0.5).astype(np.uint8)
    b = rng.standard_normal((64, 128)).astype(np.float32)
    yield Case("where/dense", Op.WHERE, [cond, a, b], a.shape, DType.F32)
    yield Case("where/broadcast-zero", Op.WHERE, [cond, a, np.broadcast_to(np.float32(0).reshape(()), a.shape)],
               a.shape, DType.F32)
    yield Case("clamp/both", Op.CLAMP, [a], a.shape, DType.F32, graph.clamp_params(-0.5, 0.5))
    yield Case("clamp/lo", Op.CLAMP, [a], a.shape, DType.F32, graph.clamp_params(0.0, None))
    yield Case("clamp/hi", Op.CLAMP, [a], a.shape, DType.F32, graph.clamp_params(None, 0.0))
    for d in (-2, 0, 1):
        yield Case(f"triu/{d}", Op.TRIU, [a], a.shape, DType.F32, graph.tri_params(d))
        yield Case(f"tril/{d}", Op.TRIL, [a], a.shape, DType.F32, graph.tri_params(d))
    wt = np.ascontiguousarray(rng.standard_normal((784, 128)).astype(np.float32)).T  # [128,784] strides {1,128}
    vt = np.ascontiguousarray(rng.standard_normal((784, 128)).astype(np.float32)).T
    yield Case("scaled_add/transposed-grad", Op.SCALED_ADD, [vt, wt], (128, 784), DType.F32,
               graph.scaled_add_params(0.9, 1.0))
    p = rng.standard_normal((128, 784)).astype(np.float32)
    yield Case("scaled_add/param-update", Op.SCALED_ADD, [p, wt], (128, 784), DType.F32,
               graph.scaled_add_params(1.0, -0.1))


def creation_cases():
    for dt, v in [(DType.F32, 2.5), (DType.F32, 0.1), (DType.I64, 7.0), (DType.I32, -3.0),
                  (DType.BOOL, 1.0), (DType.BOOL, 0.0), (DType.F16, 0.1)]:
        for n in (0, 1, 257):
            yield Case(f"full/{dt.name}/{v}/n={n}", Op.FULL, [], (n,), dt, graph.full_params(v))
    yield Case("full/scalar", Op.FULL, [], (), DType.F32, graph.full_params(1.0))
    yield Case("arange/f32", Op.ARANGE, [], (1000,), DType.F32, graph.arange_params(0.0, 1.0))
    yield Case("arange/f32-frac", Op.ARANGE, [], (777,), DType.F32, graph.arange_params(-3.3, 0.37))
    yield Case("arange/i64", Op.ARANGE, [], (100,), DType.I64, graph.arange_params(5.0, 3.0))
    for seed, off, n in [(0, 0, 16), (20260728, 5, 1000), (2 ** 40 + 3, 2 ** 33, 257)]:
        yield Case(f"rand/{seed}/{off}", Op.RAND, [], (n,), DType.F32, graph.rand_params(seed, off))


def cast_cases(seed=7):
    rng = np.random.default_rng(seed)
    f = (rng.standard_normal(1000) * 100).astype(np.float32)
    f[:4] = [0.0, -0.0, 0.5, -0.5]
    i64 = rng.integers(-2 ** 40, 2 ** 40, 1000).astype(np.int64)
    small_i64 = rng.integers(0, 1000, 1000).astype(np.int64)
    i32 = rng.integers(-2 ** 31, 2 ** 31 - 1, 1000).astype(np.int32)
    bl = (rng.random(1000) < 0.5).astype(np.uint8)
    h = rng.standard_normal(1000).astype(np.float16)
    f16src = np.concatenate([f / 100, np.array([65504, 65520, 1e30, 6e-8, 3e-8, 5.96e-8, 1e-10, np.inf, -np.inf,
                                                np.nan, 6.1e-5, 6.0e-5, 1.0009765625, 1.00048828125],
                                               dtype=np.float32)]).astype(np.float32)
    yield Case("cast/f32->i32", Op.CAST, [f], f.shape, DType.I32)
    yield Case("cast/f32->i64", Op.CAST, [f], f.shape, DType.I64)
    yield Case("cast/f32->bool", Op.CAST, [f], f.shape, DType.BOOL)
    yield Case("cast/f32->f16", Op.CAST, [f16src], f16src.shape, DType.F16)
    yield Case("cast/f16->f32", Op.CAST, [h], h.shape, DType.F32)
    yield Case("cast/i32->f32", Op.CAST, [i32], i32.shape, DType.F32)
    yield Case("cast/i32->i64", Op.CAST, [i32], i32.shape, DType.I64)
    yield Case("cast/i64->f32", Op.CAST, [i64], i64.shape, DType.F32)
    yield Case("cast/labels->f32", Op.CAST, [small_i64], small_i64.shape, DType.F32)
    yield Case("cast/i64->i32", Op.CAST, [small_i64], small_i64.shape, DType.I32)
    yield Case("cast/bool->f32", Op.CAST, [bl], bl.shape, DType.F32)
    yield Case("cast/bool->i64", Op.CAST, [bl], bl.shape, DType.I64)
    yield Case("cast/f32->f32", Op.CAST, [f], f.shape, DType.F32)
    m = rng.standard_normal((16, 24)).astype(np.float32)
    yield Case("cast/f32->i64/transposed", Op.CAST, [np.ascontiguousarray(m.T).T], m.shape, DType.I64)


def reduce_cases(seed=99, quick=False):
    rng = np.random.default_rng(seed)

    def mk(name, x, axes, keepdim=False, tag=""):
        nd = x.ndim
        axes_n = [a % nd for a in axes] if axes else list(range(nd))
        out_shape = tuple((1 if i in axes_n else d) for i, d in enumerate(x.shape) if keepdim or i not in axes_n)
        is_arg = name in ("argmax", "argmin")
        n_red = int(np.prod([x.shape[a] for a in axes_n])) if axes_n else 1
        tas = np.sum(np.abs(x.astype(np.float64)), axis=tuple(axes_n), keepdims=keepdim)
        if name == "mean" and n_red:
            tas = tas / n_red
        return Case(f"{name}/{x.shape}/axes={axes}/{tag}", Op[name.upper()], [x], out_shape,
                    DType.I64 if is_arg else DType.F32, graph.reduce_params(axes, nd, keepdim),
                    terms_abs_sum=tas, reduction_n=n_red)

    shapes = [((6,), [[]]), ((2, 3), [[], [0], [1], [-1]]), ((64, 10), [[1], [0]]), ((64, 128), [[0], [1], []]),
              ((4, 8, 6, 6), [[0, 2, 3], [1], [3], [0]]), ((3, 5, 300), [[2], [0, 1]]),
              ((1, 7, 40, 27), [[1]]), ((100000,), [[]]), ((2, 70000), [[1]]), ((9, 1031), [[1], [0]]),
              ((3000, 33), [[0]])]
    if quick:
        shapes = shapes[:5]
    for shape, axes_list in shapes:
        for axes in axes_list:
            for tag, x in layouts(rng, shape):
                if tag in ("strided", "offset") and len(shape) == 1 and shape[0] > 1000:
                    continue
                for name in ("sum", "mean", "max", "min", "argmax", "argmin"):
                    if name in ("argmax", "argmin") and len(axes) != 1:
                        continue
                    yield mk(name, x, axes, keepdim=False, tag=tag)
            yield mk("sum", rng.standard_normal(shape).astype(np.float32), axes, keepdim=True, tag="keepdim")
    # ties, NaN and infinities: first extremum, NaN rules
    t = np.array([[1, 5, 5, 4], [2, 2, 1, 1], [np.nan, 3, 3, np.nan], [-np.inf, -np.inf, -np.inf, -np.inf],
                  [np.nan, np.nan, np.nan, np.nan], [np.inf, 1, np.inf, 0]], dtype=np.float32)
    for name in ("max", "min", "argmax", "argmin", "sum"):
        yield mk(name, t, [1], tag="ties-nan")
    # prod: multiplied in index order on both sides, so exact -- including the case a tree would get
    # wrong (1e20 and 1e-20 alternating: 1 in order, inf or 0 once regrouped)
    rngp = np.random.default_rng(seed + 7)
    xp = rngp.uniform(0.5, 1.5, (33, 17)).astype(np.float32)
    for axes in ([1], [0], []):
        yield mk("prod", xp, axes, tag="dense")
    yield mk("prod", np.ascontiguousarray(xp.T).T, [1], tag="transposed")
    yield mk("prod", xp, [0], keepdim=True, tag="keepdim")
    alt = np.tile(np.array([1e20, 1e-20], dtype=np.float32), 3000).reshape(3, 2000)
    yield mk("prod", alt, [1], tag="order-sensitive")
    yield mk("prod", rngp.uniform(0.9, 1.1, (4, 8, 6, 6)).astype(np.float32), [0, 2, 3], tag="multi-axis")
    wide = rng.integers(0, 4, (5, 5000)).astype(np.float32)  # many ties across lanes
    for name in ("argmax", "argmin", "max", "min"):
        yield mk(name, wide, [1], tag="many-ties")
        yield mk(name, np.ascontiguousarray(wide.T), [0], tag="many-ties-col")
    ones = np.ones((100000,), dtype=np.float32)
    yield mk("sum", ones, [], tag="ones")
    mixed = ones.copy()
    mixed[0] = 1e7
    yield mk("sum", mixed, [], tag="mixed-magnitude")
    yield mk("sum", np.zeros((0, 5), dtype=np.float32), [0], tag="empty-reduced")
    yield mk("mean", np.zeros((0, 5), dtype=np.float32), [0], tag="empty-reduced")
    yield mk("max", np.zeros((0, 5), dtype=np.float32), [0], tag="empty-reduced")


def softmax_cases(seed=5, quick=False):
    rng = np.random.default_rng(seed)
    shapes = [((64, 10), 1), ((256, 100), 1), ((7, 1000), 1), ((3, 4099), 1), ((2, 32000), 1), ((2, 50000), 1),
              ((33, 65), 0), ((4, 8, 6, 6), 1), ((5, 300, 7), 1), ((3,), 0), ((512, 33), 1)]
    if quick:
        shapes = shapes[:4]
    for shape, axis in shapes:
        for tag, x in layouts(rng, shape, scale=2.0):
            if tag != "dense" and np.prod(shape) > 200000:
                continue
            for name in ("softmax", "log_softmax"):
                yield Case(f"{name}/{shape}/axis={axis}/{tag}", Op[name.upper()], [x], shape, DType.F32,
                           graph.axis_params(axis))
    for vals in ([1000.0, 1001.0, 1002.0], [0.0, -200.0, -400.0], [-1e30, 0.0, 1e30],
                 [np.nan, 1.0, 2.0], [-np.inf, -np.inf, -np.inf], [np.inf, 1.0, 2.0], [88.0, 89.0, -104.0]):
        x = np.array([vals], dtype=np.float32)
        for name in ("softmax", "log_softmax"):
            yield Case(f"{name}/extreme/{vals}", Op[name.upper()], [x], x.shape, DType.F32, graph.axis_params(1))
    big = np.full((2, 2000), 1000.0, dtype=np.float32)
    big[:, ::7] = 1002.0
    yield Case("softmax/large-logits-wide", Op.SOFTMAX, [big], big.shape, DType.F32, graph.axis_params(1))
    if not quick:
        # many long dense rows: the persistent kernel that prefetches the next row while one is processed
        # (row lengths at both ends of its range, more rows than two per SM, a row of NaN and of -inf)
        rng2 = np.random.default_rng(seed + 100)
        for shape in ((300, 8200), (297, 32768)):
            x = (rng2.standard_normal(shape) * 2.0).astype(np.float32)
            x[5, 17] = np.nan
            x[7, :] = -np.inf
            x[9, 100] = np.inf
            for name in ("softmax", "log_softmax"):
                yield Case(f"{name}/{shape}/long-rows", Op[name.upper()], [x], shape, DType.F32, graph.axis_params(1))


def matmul_cases(seed=11, quick=False):
    rng = np.random.default_rng(seed)

    def mk(tag, a, b):
        a4 = a.reshape((1,) * (4 - a.ndim) + a.shape) if a.ndim < 4 else a
        b4 = b.reshape((1,) * (4 - b.ndim) + b.shape) if b.ndim < 4 else b
        bshape = np.broadcast_shapes(a4.shape[:2], b4.shape[:2])
        a4 = np.broadcast_to(a4, bshape + a4.shape[2:])
        b4 = np.broadcast_to(b4, bshape + b4.shape[2:])
        m, k, n = a4.shape[2], a4.shape[3], b4.shape[3]
        tas = np.abs(a4.astype(np.float64)) @ np.abs(b4.astype(np.float64))
        return Case(f"matmul/{tag}/{m}x{k}x{n}/batch={bshape}", Op.MATMUL, [a4, b4], bshape + (m, n), DType.F32,
                    terms_abs_sum=tas, reduction_n=k)

    def rnd(*shape):
        return rng.standard_normal(shape).astype(np.float32)

    yield mk("known", np.array([[1, 2, 3], [4, 5, 6]], np.float32), np.array([[7, 8], [9, 10], [11, 12]], np.float32))
    edge = [1, 2, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 128, 129, 255, 257]
    if quick:
        edge = [1, 17, 33, 64, 129]
    for s in edge:
        yield mk("square", rnd(s, s), rnd(s, s))
    for m, k, n in [(1, 1, 1), (31, 33, 31), (33, 31, 33), (64, 784, 128), (64, 128, 10), (64, 10, 128),
                    (784, 64, 128), (128, 64, 10), (5, 1000, 3), (130, 70, 260), (64, 4096, 64), (3, 2500, 200)]:
        yield mk("nn", rnd(m, k), rnd(k, n))
        yield mk("nt", rnd(m, k), np.ascontiguousarray(rnd(n, k)).T)
        yield mk("tn", np.ascontiguousarray(rnd(k, m)).T, rnd(k, n))
        if not quick:
            yield mk("tt", np.ascontiguousarray(rnd(k, m)).T, np.ascontiguousarray(rnd(n, k)).T)
    # batched: weights broadcast over the batch (conv forward), per-sample dW, sliced operand
    yield mk("conv-fwd", rnd(1, 1, 16, 27), rnd(1, 6, 27, 64))
    yield mk("conv-dw", rnd(1, 6, 16, 64), np.ascontiguousarray(rnd(1, 6, 27, 64)).transpose(0, 1, 3, 2))
    yield mk("conv-dcols", np.broadcast_to(np.ascontiguousarray(rnd(16, 27)).T.reshape(1, 1, 27, 16), (1, 6, 27, 16)),
             rnd(1, 6, 16, 64))
    yield mk("batch2", rnd(2, 3, 20, 30), rnd(2, 3, 30, 10))
    yield mk("batch-bcast-b", rnd(2, 2, 2, 2), np.eye(2, dtype=np.float32).reshape(1, 1, 2, 2))
    big = rnd(40, 100)
    yield mk("sliced", big[3:35, 10:74:2], rnd(32, 50))
    yield mk("empty-k", np.zeros((4, 0), np.float32), np.zeros((0, 5), np.float32))
    yield mk("empty-m", np.zeros((0, 4), np.float32), rnd(4, 5))


def matmul_tc_cases(seed=12):
    """Shapes large enough for the tensor-core path, with every operand-major
    combination, ragged edges in M, N and K, batches and broadcast batches."""
    rng = np.random.default_rng(seed)

    def rnd(*shape):
        return rng.standard_normal(shape).astype(np.float32)

    def mk(tag, a4, b4):
        bshape = np.broadcast_shapes(a4.shape[:2], b4.shape[:2])
        a4 = np.broadcast_to(a4, bshape + a4.shape[2:])
        b4 = np.broadcast_to(b4, bshape + b4.shape[2:])
        m, k, n = a4.shape[2], a4.shape[3], b4.shape[3]
        tas = np.abs(a4.astype(np.float64)) @ np.abs(b4.astype(np.float64))
        return Case(f"matmul-tc/{tag}/{m}x{k}x{n}/batch={bshape}", Op.MATMUL, [a4, b4], bshape + (m, n), DType.F32,
                    terms_abs_sum=tas, reduction_n=k)

    def t(x):  # same values, transposed storage
        return np.ascontiguousarray(np.swapaxes(x, -1, -2)).swapaxes(-1, -2)

    m, k, n = 300, 1000, 520
    yield mk("nn", rnd(1, 1, m, k), rnd(1, 1, k, n))
    yield mk("nt", rnd(1, 1, m, k), t(rnd(1, 1, k, n)))
    yield mk("tn", t(rnd(1, 1, m, k)), rnd(1, 1, k, n))
    yield mk("tt", t(rnd(1, 1, m, k)), t(rnd(1, 1, k, n)))
    yield mk("bn64", rnd(1, 1, 1025, 777), rnd(1, 1, 777, 50))
    yield mk("bn128", rnd(1, 1, 513, 513), rnd(1, 1, 513, 100))
    yield mk("bn256", rnd(1, 1, 2100, 96), rnd(1, 1, 96, 2500))
    yield mk("k33", rnd(1, 1, 1024, 33), rnd(1, 1, 33, 1024))
    yield mk("split-k", rnd(1, 1, 128, 8192), rnd(1, 1, 8192, 128))
    yield mk("skinny", rnd(1, 1, 64, 2048), t(rnd(1, 1, 2048, 512)))
    yield mk("batched", rnd(2, 3, 150, 200), rnd(2, 3, 200, 130))
    yield mk("conv-fwd-bcast-a", rnd(1, 1, 128, 576), rnd(1, 8, 576, 256))
    yield mk("conv-dw", rnd(1, 8, 128, 256), t(rnd(1, 8, 256, 576)))
    yield mk("conv-dcols-bcast-a", t(rnd(1, 1, 576, 128)), rnd(1, 8, 128, 256))
    yield mk("bcast-b", rnd(4, 1, 100, 300), rnd(1, 1, 300, 200))
    yield mk("conv1-k27-bcast-a", rnd(1, 1, 64, 27), rnd(1, 16, 27, 1024))     # K below one K-block
    big = rnd(1, 1, 700, 1200)
    yield mk("sliced", big[:, :, 5:605, 16:1016], rnd(1, 1, 1000, 300))
    # a small left operand and a right operand with n contiguous: the streamed-operand kernel
    yield mk("stream-skinny-splitk", rnd(1, 1, 64, 2048), rnd(1, 1, 2048, 512))
    yield mk("stream-ragged-m-n-k", rnd(1, 1, 100, 1333), rnd(1, 1, 1333, 260))
    yield mk("stream-two-m-tiles", rnd(1, 1, 256, 320), rnd(1, 3, 320, 384))
    yield mk("stream-batches-in-a-tile", rnd(1, 1, 256, 1152), rnd(1, 8, 1152, 64))       # conv3 forward: N = 64
    yield mk("stream-batches-in-a-tile-n32", rnd(1, 1, 48, 1024), rnd(2, 8, 1024, 32))
    yield mk("stream-w-transposed", t(rnd(1, 1, 200, 96)), rnd(1, 4, 96, 256))            # conv dcols: W^T view
    yield mk("stream-w-batched", rnd(1, 4, 128, 256), rnd(1, 4, 256, 192))
    wide = rnd(1, 1, 512, 640)
    yield mk("stream-pitched-s", rnd(1, 1, 96, 512), wide[:, :, :, 64:576])                # S is a column slice
    # ... and a right operand with K contiguous (a transposed view: a Linear weight, the column tensor
    # in a convolution's weight gradient), ragged in every extent, pitched, batched, several chunks of W
    yield mk("stream-kmajor-ragged", rnd(1, 1, 100, 652), t(rnd(1, 1, 652, 520)))
    yield mk("stream-kmajor-conv3-dw", rnd(1, 4, 256, 64), t(rnd(1, 4, 64, 1152)))
    tall = rnd(1, 4, 400, 300)                                                              # storage [n][k], k sliced
    yield mk("stream-kmajor-pitched", rnd(1, 4, 60, 256), tall[:, :, 8:392, 20:276].swapaxes(-1, -2))
    yield mk("stream-kmajor-splitk", rnd(1, 1, 48, 4096), t(rnd(1, 1, 4096, 256)))
    # a tall W against a short K: the column gradient of a convolution (W^T broadcast, N = 64: two batches per tile)
    yield mk("stream-tall-w-conv3-dcols", t(rnd(1, 1, 1152, 256)), rnd(1, 8, 256, 64))
    yield mk("stream-tall-w-ragged", rnd(1, 1, 700, 130), rnd(1, 3, 130, 200))


def movement_cases(seed=21, quick=False):
    rng = np.random.default_rng(seed)

    def unfold(n, c, h, w, k, s, p, d):
        oh = (h + 2 * p[0] - (d[0] * (k[0] - 1) + 1)) // s[0] + 1
        ow = (w + 2 * p[1] - (d[1] * (k[1] - 1) + 1)) // s[1] + 1
        return oh, ow, graph.unfold_params(k, s, p, d, (h, w))

    geos = [(2, 3, 8, 8, (3, 3), (1, 1), (1, 1), (1, 1)), (2, 4, 9, 7, (3, 2), (2, 1), (1, 0), (1, 1)),
            (1, 2, 10, 10, (3, 3), (1, 1), (2, 2), (2, 2)), (3, 1, 5, 5, (1, 1), (1, 1), (0, 0), (1, 1)),
            (2, 3, 6, 6, (2, 2), (2, 2), (0, 0), (1, 1)), (4, 3, 32, 32, (3, 3), (1, 1), (1, 1), (1, 1)),
            # dense, unit-stride geometries (planes grouped per block, 128-bit rows): odd plane counts,
            # a 5x5 window with padding 2, no padding, a non-square window, an 8x8 plane
            (5, 7, 16, 16, (3, 3), (1, 1), (1, 1), (1, 1)), (3, 5, 12, 20, (5, 5), (1, 1), (2, 2), (1, 1)),
            (2, 3, 10, 12, (3, 5), (1, 1), (0, 0), (1, 1)), (9, 13, 8, 8, (3, 3), (1, 1), (1, 1), (1, 1)),
            (1, 2, 64, 64, (3, 3), (1, 1), (1, 1), (1, 1))]
    if quick:
        geos = geos[:3]
    for n, c, h, w, k, s, p, d in geos:
        oh, ow, params = unfold(n, c, h, w, k, s, p, d)
        for tag, x in layouts(rng, (n, c, h, w)):
            yield Case(f"im2col/{(n, c, h, w)}/k={k}s={s}p={p}d={d}/{tag}", Op.IM2COL, [x],
                       (n, c * k[0] * k[1], oh * ow), DType.F32, params)
        for tag, cols in layouts(rng, (n, c * k[0] * k[1], oh * ow)):
            yield Case(f"col2im/{(n, c, h, w)}/k={k}s={s}p={p}d={d}/{tag}", Op.COL2IM, [cols], (n, c, h, w),
                       DType.F32, params)
    pools = [(2, 3, 8, 8, (2, 2), (2, 2), (0, 0), (1, 1)), (2, 2, 9, 9, (3, 3), (2, 2), (1, 1), (1, 1)),
             (1, 4, 7, 6, (3, 2), (1, 1), (1, 1), (1, 1)), (4, 8, 32, 32, (2, 2), (2, 2), (0, 0), (1, 1)),
             # 128-bit 2x2 paths: width a multiple of 8; an odd height (a leftover row) keeps the forward
             # vector path but sends the adjoint to the per-window kernel
             (3, 5, 16, 24, (2, 2), (2, 2), (0, 0), (1, 1)), (2, 3, 9, 8, (2, 2), (2, 2), (0, 0), (1, 1)),
             (1, 1, 2, 8, (2, 2), (2, 2), (0, 0), (1, 1))]
    for n, c, h, w, k, s, p, d in pools:
        oh, ow, params = unfold(n, c, h, w, k, s, p, d)
        x = rng.integers(0, 5, (n, c, h, w)).astype(np.float32)  # many ties: first-max rule matters
        g = rng.standard_normal((n, c, oh, ow)).astype(np.float32)
        for tag, xv in layouts(rng, (n, c, h, w)):
            xv[...] = x
            yield Case(f"max_pool2d/{(n, c, h, w)}/k={k}s={s}p={p}/{tag}", Op.MAX_POOL2D, [xv], (n, c, oh, ow),
                       DType.F32, params)
        yield Case(f"max_pool2d_backward/{(n, c, h, w)}/k={k}s={s}p={p}", Op.MAX_POOL2D_BACKWARD, [g, x],
                   (n, c, h, w), DType.F32, params)
        xr = rng.standard_normal((n, c, h, w)).astype(np.float32)
        yield Case(f"max_pool2d_backward/random/{(n, c, h, w)}/k={k}", Op.MAX_POOL2D_BACKWARD, [g, xr],
                   (n, c, h, w), DType.F32, params)
    # index_select / scatter_add: every axis, duplicates, strided index
    table = rng.standard_normal((50, 16)).astype(np.float32)
    idx = rng.integers(0, 50, 200).astype(np.int64)
    yield Case("index_select/rows", Op.INDEX_SELECT, [table, idx], (200, 16), DType.F32, graph.axis_params(0))
    idx_c = rng.integers(0, 16, 9).astype(np.int64)
    yield Case("index_select/cols", Op.INDEX_SELECT, [table, idx_c], (50, 9), DType.F32, graph.axis_params(1))
    yield Case("index_select/strided-index", Op.INDEX_SELECT, [table, np.repeat(idx, 2)[::2]], (200, 16), DType.F32,
               graph.axis_params(0))
    t3 = rng.standard_normal((4, 10, 6)).astype(np.float32)
    idx3 = rng.integers(0, 10, 7).astype(np.int64)
    yield Case("index_select/middle", Op.INDEX_SELECT, [t3, idx3], (4, 7, 6), DType.F32, graph.axis_params(1))
    yield Case("index_select/transposed", Op.INDEX_SELECT, [np.ascontiguousarray(table.T).T, idx], (200, 16),
               DType.F32, graph.axis_params(0))
    yield Case("index_select/i64-values", Op.INDEX_SELECT, [np.arange(50, dtype=np.int64) * 3, idx], (200,),
               DType.I64, graph.axis_params(0))
    src = rng.standard_normal((200, 16)).astype(np.float32)
    yield Case("scatter_add/rows", Op.SCATTER_ADD, [src, idx], (50, 16), DType.F32, graph.axis_params(0))
    dup = np.zeros(200, dtype=np.int64)  # every source into one destination: order-sensitive sum
    yield Case("scatter_add/all-duplicates", Op.SCATTER_ADD, [src * 1e3, dup], (3, 16), DType.F32,
               graph.axis_params(0))
    src3 = rng.standard_normal((4, 7, 6)).astype(np.float32)
    yield Case("scatter_add/middle", Op.SCATTER_ADD, [src3, idx3], (4, 10, 6), DType.F32, graph.axis_params(1))
    # long index lists (an Embedding backward): bucketed by destination on the device, several
    # chunks of 1024 indices, one destination that takes a third of them, a strided index tensor
    # (a generator of their own: the cases after these keep the inputs their golden outputs were made from)
    rng2 = np.random.default_rng(seed + 1000)
    big_idx = rng2.integers(0, 2000, 3000).astype(np.int64)
    big_idx[rng2.random(3000) < 0.3] = 777
    big_src = (rng2.standard_normal((3000, 32)) * 10.0 ** rng2.integers(-3, 4, (3000, 1))).astype(np.float32)
    yield Case("scatter_add/embedding-backward", Op.SCATTER_ADD, [big_src, big_idx], (2000, 32), DType.F32,
               graph.axis_params(0))
    yield Case("scatter_add/embedding-backward-strided-index", Op.SCATTER_ADD,
               [big_src, np.repeat(big_idx, 3)[::3]], (2000, 32), DType.F32, graph.axis_params(0))
    mid_idx = rng2.integers(0, 1000, 2500).astype(np.int64)
    mid_src = rng2.standard_normal((4, 2500, 16)).astype(np.float32)
    yield Case("scatter_add/long-middle", Op.SCATTER_ADD, [mid_src, mid_idx], (4, 1000, 16), DType.F32,
               graph.axis_params(1))
    yield Case("scatter_add/empty", Op.SCATTER_ADD, [np.zeros((0, 16), np.float32), np.zeros((0,), np.int64)],
               (5, 16), DType.F32, graph.axis_params(0))
    # cat / slice_backward
    a = rng.standard_normal((3, 4, 5)).astype(np.float32)
    for axis, other in [(0, (2, 4, 5)), (1, (3, 6, 5)), (2, (3, 4, 1))]:
        b = rng.standard_normal(other).astype(np.float32)
        out = list(a.shape)
        out[axis] += other[axis]
        yield Case(f"cat/axis={axis}", Op.CAT, [a, b], tuple(out), DType.F32, graph.axis_params(axis))
    yield Case("cat/transposed", Op.CAT, [np.ascontiguousarray(a.transpose(0, 2, 1)).transpose(0, 2, 1), a], (6, 4, 5),
               DType.F32, graph.axis_params(0))
    g = rng.standard_normal((3, 4, 5)).astype(np.float32)
    yield Case("slice_backward/axis1", Op.SLICE_BACKWARD, [g], (3, 11, 5), DType.F32, graph.slice_params(1, 2, 10, 2))
    yield Case("slice_backward/axis0", Op.SLICE_BACKWARD, [g], (5, 4, 5), DType.F32, graph.slice_params(0, 1, 4, 1))
    yield Case("slice_backward/axis2-strided-g", Op.SLICE_BACKWARD, [np.ascontiguousarray(g.transpose(0, 2, 1)).transpose(0, 2, 1)],
               (3, 4, 15), DType.F32, graph.slice_params(2, 0, 15, 3))


def f16_cases(seed=77):
    """F16 storage through every kernel family: operands and results are half, arithmetic is f32."""
    rng = np.random.default_rng(seed)

    def h(*shape, scale=1.0):
        return (rng.standard_normal(shape) * scale).astype(np.float16)

    H = DType.F16
    a, b = h(33, 65), h(33, 65)
    for name in ("add", "sub", "mul", "maximum", "minimum", "div"):
        bb = np.where(np.abs(b) < 0.05, np.float16(0.5), b).astype(np.float16) if name == "div" else b
        yield Case(f"f16/{name}", Op[name.upper()], [a, bb], a.shape, H)
    yield Case("f16/add/transposed+row-broadcast", Op.ADD,
               [np.ascontiguousarray(a.T).T, np.broadcast_to(h(65), (33, 65))], a.shape, H)
    yield Case("f16/scaled_add", Op.SCALED_ADD, [a, b], a.shape, H, graph.scaled_add_params(0.9, -0.1))
    for name in ("relu", "neg", "abs", "square", "exp", "tanh", "sigmoid", "sqrt"):
        x = np.abs(a) + np.float16(0.1) if name == "sqrt" else a
        yield Case(f"f16/{name}", Op[name.upper()], [x], x.shape, H)
    special = np.array([np.nan, -0.0, 0.0, 1.0, -1.0, np.inf, -np.inf, 6e-8, -6e-8, 65504.0], dtype=np.float16)
    yield Case("f16/relu/special", Op.RELU, [special], special.shape, H)
    yield Case("f16/add/overflow", Op.ADD, [special, special[::-1].copy()], special.shape, H)
    yield Case("f16/less", Op.LESS, [a, b], a.shape, DType.BOOL)
    yield Case("f16/where", Op.WHERE, [(rng.random((33, 65)) < 0.5).astype(np.uint8), a, b], a.shape, H)
    yield Case("f16/contiguous/transposed", Op.CONTIGUOUS, [np.ascontiguousarray(a.T).T], a.shape, H)
    yield Case("f16/cat", Op.CAT, [a, h(7, 65)], (40, 65), H, graph.axis_params(0))
    yield Case("f16/tril", Op.TRIL, [a], a.shape, H, graph.tri_params(0))
    # reductions: f32 accumulation, one narrowing
    x = h(40, 300)
    tas = np.abs(x.astype(np.float64))
    yield Case("f16/sum/rows", Op.SUM, [x], (40,), H, graph.reduce_params([1], 2), terms_abs_sum=tas.sum(1), reduction_n=300)
    yield Case("f16/mean/cols", Op.MEAN, [x], (1, 300), H, graph.reduce_params([0], 2, True),
               terms_abs_sum=tas.sum(0, keepdims=True) / 40, reduction_n=40)
    yield Case("f16/max/rows", Op.MAX, [x], (40,), H, graph.reduce_params([1], 2))
    yield Case("f16/argmax/rows", Op.ARGMAX, [x], (40,), DType.I64, graph.reduce_params([1], 2))
    yield Case("f16/softmax", Op.SOFTMAX, [h(17, 100, scale=2.0)], (17, 100), H, graph.axis_params(1))
    yield Case("f16/log_softmax", Op.LOG_SOFTMAX, [h(17, 100, scale=2.0)], (17, 100), H, graph.axis_params(1))
    # matmul: CUDA-core size and tensor-core size
    for m, k, n in ((48, 96, 40), (256, 512, 384)):
        a4, b4 = h(1, 1, m, k), h(1, 1, k, n)
        tas4 = np.abs(a4.astype(np.float64)) @ np.abs(b4.astype(np.float64))
        yield Case(f"f16/matmul/{m}x{k}x{n}", Op.MATMUL, [a4, b4], (1, 1, m, n), H, terms_abs_sum=tas4, reduction_n=k)
    # window and index movement
    img = h(2, 3, 8, 8)
    up = graph.unfold_params((3, 3), (1, 1), (1, 1), (1, 1), (8, 8))
    yield Case("f16/im2col", Op.IM2COL, [img], (2, 27, 64), H, up)
    yield Case("f16/col2im", Op.COL2IM, [h(2, 27, 64)], (2, 3, 8, 8), H, up)
    pool = graph.unfold_params((2, 2), (2, 2), (0, 0), (1, 1), (8, 8))
    ties = rng.integers(0, 5, (2, 3, 8, 8)).astype(np.float16)
    yield Case("f16/max_pool2d", Op.MAX_POOL2D, [ties], (2, 3, 4, 4), H, pool)
    yield Case("f16/max_pool2d_backward", Op.MAX_POOL2D_BACKWARD, [h(2, 3, 4, 4), ties], (2, 3, 8, 8), H, pool)
    table = h(50, 16)
    idx = rng.integers(0, 50, 200).astype(np.int64)
    yield Case("f16/index_select", Op.INDEX_SELECT, [table, idx], (200, 16), H, graph.axis_params(0))
    yield Case("f16/scatter_add", Op.SCATTER_ADD, [h(200, 16), idx], (50, 16), H, graph.axis_params(0))
    yield Case("f16/slice_backward", Op.SLICE_BACKWARD, [h(3, 4, 5)], (3, 11, 5), H, graph.slice_params(1, 2, 10, 2))


def all_cases(quick=False):
    yield from elementwise_cases(quick=quick)
    yield from creation_cases()
    yield from cast_cases()
    yield from reduce_cases(quick=quick)
    yield from softmax_cases(quick=quick)
    yield from matmul_cases(quick=quick)
    yield from movement_cases(quick=quick)
