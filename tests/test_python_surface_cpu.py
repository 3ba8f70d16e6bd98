"""The pybind11 module behind vkML's Python package (vkml_b200/bindings/vkml_core.cpp) on a host
with no GPU: it imports, exports the names the package binds (src/python/bindings.cpp), falls back
to the CPU device with a reason, and the framework above it computes there.  Runs in a fresh
interpreter so the module's copy of the framework is the only one in the process."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
PYTHON = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "python")

SCRIPT = r"""
import json, sys
import numpy as np
sys.path.insert(0, sys.argv[1])
import vkml as V
from vkml import _vkml_core as core
device, why = V.best_device()
a = np.arange(12, dtype=np.float32).reshape(3, 4)
b = np.arange(8, dtype=np.float32).reshape(4, 2)
x = V.tensor(a, device=V.cpu, requires_grad=True)
y = V.sum(V.matmul(x, V.tensor(b, device=V.cpu)))
y.backward()
try:
    V.matmul(V.tensor(a, device=V.cpu), V.tensor(a, device=V.cpu)).numpy()
    shape_error = None
except Exception as e:
    shape_error = type(e).__name__
print(json.dumps({"names": sorted(n for n in dir(core) if not n.startswith("__")), "device": str(device),
                  "why": why, "value": float(y.item()), "grad": np.asarray(x.grad).tolist(),
                  "reports": len(V.vulkan_device_reports()), "shape_error": shape_error}))
"""


def test_the_module_imports_and_computes_without_a_gpu():
    if not os.path.isdir(os.path.join(PYTHON, "vkml")):
        pytest.skip("oracle/_ref/python/vkml not built")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES=os.environ.get("CUDA_VISIBLE_DEVICES", ""))
    run = subprocess.run([sys.executable, "-c", SCRIPT, PYTHON], capture_output=True, text=True, timeout=300, env=env)
    assert run.returncode == 0, run.stderr[-3000:]
    out = json.loads(run.stdout.strip().splitlines()[-1])
    for name in ("Tensor", "ShapeError", "Reduction", "cpu_device", "device_backend", "matmul", "cross_entropy",
                 "log_softmax", "im2col", "max_pool2d", "scatter_add", "index_select", "backward", "realize",
                 "vulkan_device_reports", "vulkan_stats", "vulkan_last_profile", "vulkan_profile_records",
                 "vulkan_set_profile_history", "decisions"):
        assert name in out["names"], name
    # (3x4)@(4x2) summed: sum_i sum_j sum_k a[i,k] b[k,j]; d/da = row sums of b
    assert out["value"] == pytest.approx(float((__import__("numpy").arange(12).reshape(3, 4)
                                                @ __import__("numpy").arange(8).reshape(4, 2)).sum()))
    assert out["grad"] == [[1.0, 5.0, 9.0, 13.0]] * 3
    assert out["shape_error"] == "ShapeError"
    if out["reports"] == 0:          # no GPU in this process: the package says why it stays on the CPU
        assert out["device"] == "cpu" and out["why"]
