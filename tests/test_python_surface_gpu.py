"""vkML's Python API on the B200: `V.best_device()`, `V.nn`, `V.optim`, `Tensor.backward()` and
`.numpy()` drive the CUDA backend through the pybind11 module `_vkml_core`
(vkml_b200/bindings/vkml_core.cpp) with the package itself unchanged.  The run happens in a fresh
interpreter so the module's copy of the framework is the only one in the process."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
PACKAGE = os.path.join(os.path.dirname(HERE), "oracle", "_ref", "python", "vkml")


def test_the_python_package_trains_on_the_device_it_picks():
    """MLP 784-128-10, batch 64, SGD lr 0.1 momentum 0.9, 100 steps through V.nn / V.optim on the
    CPU device and on the device best_device() returns: loss within 1e-4 relative at every step
    (the bar of vkML's own device-vs-CPU trajectory test, tests/python/test_vulkan_kernels.py:1575-1603,
    and of tests/python/test_nn_vs_torch.py:344-398), parameters within 1e-4."""
    if not os.path.isdir(PACKAGE):
        pytest.skip("oracle/_ref/python/vkml not built")
    run = subprocess.run([sys.executable, os.path.join(HERE, "python_surface_worker.py")], capture_output=True,
                         text=True, timeout=900)
    assert run.returncode == 0, run.stderr[-3000:]
    out = json.loads(run.stdout.strip().splitlines()[-1])
    assert not out["is_cpu"], out["why"]
    assert out["device"] == "vulkan:0" and "B200" in out["why"], out["why"]
    assert out["reports"][0]["supported"] and out["reports"][0]["missing_requirement"] == ""
    cpu, dev = np.array(out["cpu_losses"]), np.array(out["device_losses"])
    assert np.all(np.isfinite(cpu)) and np.all(np.isfinite(dev))  # (random labels: the loss need not fall)
    assert np.max(np.abs(dev - cpu) / np.abs(cpu)) < 1e-4, (dev[:5], cpu[:5])
    assert out["params_max_abs"] < 1e-4
    # the device really did the work: four submissions and some twenty launches per step (fused groups)
    assert out["submissions"] >= 300 and out["dispatches"] >= 1500
    assert out["shape_error"] == "ShapeError"
    assert any(label.startswith("matmul.") for label in out["profile"]) and "relu" in out["profile"]
    assert out["profile"][-1] == "submit"
