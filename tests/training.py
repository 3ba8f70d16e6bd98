"""Drivers for whole training runs through the reference's own graph, autograd and
optimiser code (oracle/_ref, built from the reference sources), on its CPU
backend or on the B200 adapter.  Test infrastructure."""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from helpers import REF_B200_SO, REF_SO

SEED_DATA = 20260728     # data and weights seeds of the reference's examples
SEED_WEIGHTS = 20260729  # (examples/mnist/train.py:304, examples/cifar100/train.py:418)

CPU, B200 = 0, 1


def load(with_b200: bool):
    path = REF_B200_SO if with_b200 else REF_SO
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
    f32p, i64p = C.POINTER(C.c_float), C.POINTER(C.c_int64)
    lib.vkml_ref_train_mlp.restype = C.c_int
    lib.vkml_ref_train_mlp.argtypes = [C.c_int, i64p, C.c_int, f32p, f32p, f32p, i64p, C.c_int64, C.c_int,
                                       C.c_double, C.c_double, f32p]
    lib.vkml_ref_train_cnn.restype = C.c_int
    lib.vkml_ref_train_cnn.argtypes = [C.c_int] + [C.c_int64] * 6 + [f32p, f32p, i64p, C.c_int64, C.c_int,
                                                                    C.c_double, C.c_double, f32p]
    lib.vkml_ref_last_error.restype = C.c_char_p
    return lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def linear_init(rng, fan_in, shape):
    """torch-style uniform +-1/sqrt(fan_in), as python/vkml/nn.py:272-279,680-691."""
    bound = 1.0 / np.sqrt(fan_in)
    return rng.uniform(-bound, bound, size=shape).astype(np.float32)


def mlp_problem(widths, batch, steps, data="uniform", same_batch=False):
    rng_d = np.random.default_rng(SEED_DATA)
    rng_w = np.random.default_rng(SEED_WEIGHTS)
    ws, bs = [], []
    for fin, fout in zip(widths[:-1], widths[1:]):
        ws.append(linear_init(rng_w, fin, (fout, fin)))
        bs.append(linear_init(rng_w, fin, (fout,)))
    n = batch if same_batch else batch * steps
    x = rng_d.random((n, widths[0]), dtype=np.float32) if data == "uniform" else \
        rng_d.standard_normal((n, widths[0]), dtype=np.float32)
    y = rng_d.integers(0, widths[-1], n).astype(np.int64)
    if same_batch:
        x, y = np.tile(x, (steps, 1)), np.tile(y, steps)
    return ws, bs, x, y


def train_mlp(lib, device, widths, ws, bs, x, y, batch, steps, lr=0.1, momentum=0.9):
    w = np.concatenate([a.ravel() for a in ws]).astype(np.float32)
    b = np.concatenate([a.ravel() for a in bs]).astype(np.float32)
    wd = np.array(widths, dtype=np.int64)
    losses = np.zeros(steps, dtype=np.float32)
    rc = lib.vkml_ref_train_mlp(device, _p(wd, C.c_int64), len(widths) - 1, _p(w, C.c_float), _p(b, C.c_float),
                                _p(x, C.c_float), _p(y, C.c_int64), batch, steps, lr, momentum,
                                _p(losses, C.c_float))
    if rc != 0:
        raise RuntimeError(f"train_mlp failed ({rc}): {lib.vkml_ref_last_error().decode()}")
    return losses, w, b


def cnn_problem(cin, hw, c1, c2, c3, classes, batch, steps):
    rng_d = np.random.default_rng(SEED_DATA)
    rng_w = np.random.default_rng(SEED_WEIGHTS)
    feat = c3 * (hw // 8) ** 2
    parts = []
    for cout, ci in ((c1, cin), (c2, c1), (c3, c2)):
        parts.append(linear_init(rng_w, ci * 9, (cout, ci, 3, 3)))
        parts.append(linear_init(rng_w, ci * 9, (cout,)))
    parts.append(linear_init(rng_w, feat, (classes, feat)))
    parts.append(linear_init(rng_w, feat, (classes,)))
    params = np.concatenate([p.ravel() for p in parts]).astype(np.float32)
    x = rng_d.random((batch * steps, cin, hw, hw), dtype=np.float32)
    y = rng_d.integers(0, classes, batch * steps).astype(np.int64)
    return params, x, y


def train_cnn(lib, device, cin, hw, c1, c2, c3, classes, params, x, y, batch, steps, lr=0.05, momentum=0.9):
    p = params.copy()
    losses = np.zeros(steps, dtype=np.float32)
    rc = lib.vkml_ref_train_cnn(device, cin, hw, c1, c2, c3, classes, _p(p, C.c_float), _p(x, C.c_float),
                                _p(y, C.c_int64), batch, steps, lr, momentum, _p(losses, C.c_float))
    if rc != 0:
        raise RuntimeError(f"train_cnn failed ({rc}): {lib.vkml_ref_last_error().decode()}")
    return losses, p
