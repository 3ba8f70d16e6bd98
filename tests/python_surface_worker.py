"""Runs in a fresh interpreter (tests/test_python_surface_gpu.py starts it): vkML's own Python
package -- `V.best_device()`, `V.nn`, `V.optim`, `Tensor.backward()`, `.numpy()` -- trains the
MNIST-shaped MLP of the benchmark's first configuration on the CPU device and on the device
`best_device()` picks, from the same initial parameters and the same batches, and prints what
the test compares as one JSON line.  The package is the reference's (compiled to bytecode), its
native module is vkml_b200/bindings/vkml_core.cpp with the B200 adapter behind the device slot."""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "oracle", "_ref", "python"))

import vkml as V  # noqa: E402

STEPS, BATCH = 100, 64
SEED_DATA, SEED_WEIGHTS = 20260728, 20260729


def build():
    return V.nn.Sequential(V.nn.Flatten(), V.nn.Linear(784, 128), V.nn.ReLU(), V.nn.Linear(128, 10))


def train(device, state, x, y):
    model = build()
    model.load_state_dict(state)
    model.to(device)
    opt = V.optim.SGD(model.parameters(), lr=0.1, momentum=0.9)
    losses = []
    for s in range(STEPS):
        xb = V.tensor(x[s * BATCH:(s + 1) * BATCH], device=device)
        yb = V.tensor(y[s * BATCH:(s + 1) * BATCH], device=device)
        loss = V.cross_entropy(model(xb), yb)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses, {k: np.asarray(v) for k, v in model.state_dict().items()}


def main():
    device, why = V.best_device()
    rng_w = np.random.default_rng(SEED_WEIGHTS)
    state = {}
    for name, p in build().state_dict().items():
        fan_in = np.asarray(p).shape[-1] if np.asarray(p).ndim == 2 else {128: 784, 10: 128}[np.asarray(p).shape[0]]
        bound = 1.0 / np.sqrt(fan_in)
        state[name] = rng_w.uniform(-bound, bound, np.asarray(p).shape).astype(np.float32)
    rng_d = np.random.default_rng(SEED_DATA)
    x = rng_d.random((STEPS * BATCH, 1, 28, 28), dtype=np.float32)
    y = rng_d.integers(0, 10, STEPS * BATCH).astype(np.int64)
    cpu_losses, cpu_state = train(V.cpu, state, x, y)
    out = {"device": str(device), "why": why, "is_cpu": bool(device.is_cpu), "cpu_losses": cpu_losses,
           "reports": V.vulkan_device_reports(), "names": V.vulkan_device_names()}
    if not device.is_cpu:
        before = V.vulkan_stats(device.index)
        dev_losses, dev_state = train(device, state, x, y)
        V.vulkan_synchronize(device.index)
        after = V.vulkan_stats(device.index)
        out["device_losses"] = dev_losses
        out["params_max_abs"] = max(float(np.max(np.abs(cpu_state[k] - dev_state[k]))) for k in cpu_state)
        out["submissions"] = after["submissions"] - before["submissions"]
        out["dispatches"] = after["dispatches"] - before["dispatches"]
        # an error raised by the device reaches Python as the exception type the package documents
        a = V.tensor(np.ones((2, 3), np.float32), device=device)
        try:
            V.matmul(a, a).numpy()
            out["shape_error"] = None
        except ValueError as exc:
            out["shape_error"] = type(exc).__name__
        # per-dispatch device times through the package's profiling hooks
        V.vulkan_set_profiling(True, device.index)
        b = V.tensor(np.ones((512, 512), np.float32), device=device)
        V.relu(V.matmul(b, b)).numpy()
        out["profile"] = [label for label, _ in V.vulkan_last_profile(device.index)]
        V.vulkan_set_profiling(False, device.index)
    print(json.dumps(out))


if __name__ == "__main__":
    main()
