"""Runs the benchmark's two large training configurations at FULL size on the reference CPU
backend (oracle/_ref, built from the reference sources) and stores what the GPU tests compare
against under tests/golden/full_size_steps.npz:

  cnn_*   CNN, batch 256, 3x32x32 inputs, conv 64/128/256, Linear 4096->100, 3 steps
          (about a minute of CPU time);
  mlp_*   MLP 4096-8192-8192-8192-1000, batch 2048, N(0,1) inputs, 2 steps (hours of
          single-threaded CPU time: the reference's matmul walks a row-major B by columns).

For each: the loss of every step, and the values of SAMPLE parameters (positions drawn from
a fixed seed) after the last step -- they depend on every gradient and on the optimiser.
The problems are the seeded ones of tests/training.py, so the GPU side regenerates the
same inputs instead of storing them.

  mlp1_*  the same MLP, ONE step on a problem of its own (half the time), stored in a file of its
          own, full_size_steps_mlp1.npz, so that it can be generated beside the two-step run.

Run from the repository root:  python tests/golden/make_full_size_steps.py [cnn] [mlp] [mlp1]
"""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import training  # noqa: E402

OUT = os.path.join(HERE, "full_size_steps.npz")
OUT_MLP1 = os.path.join(HERE, "full_size_steps_mlp1.npz")
SAMPLE = 4096
SAMPLE_SEED = 20260730

CNN = dict(cin=3, hw=32, c1=64, c2=128, c3=256, classes=100)
CNN_BATCH, CNN_STEPS, CNN_LR = 256, 3, 0.05
MLP_WIDTHS, MLP_BATCH, MLP_STEPS, MLP_LR = [4096, 8192, 8192, 8192, 1000], 2048, 2, 0.1


def sample_positions(n):
    return np.sort(np.random.default_rng(SAMPLE_SEED).choice(n, size=min(SAMPLE, n), replace=False))


def main():
    which = set(sys.argv[1:]) or {"cnn", "mlp"}
    lib = training.load(with_b200=False)
    out = dict(np.load(OUT)) if os.path.exists(OUT) else {}
    if "cnn" in which:
        t0 = time.time()
        params, x, y = training.cnn_problem(batch=CNN_BATCH, steps=CNN_STEPS, **CNN)
        losses, p = training.train_cnn(lib, training.CPU, params=params, x=x, y=y, batch=CNN_BATCH,
                                       steps=CNN_STEPS, lr=CNN_LR, **CNN)
        pos = sample_positions(p.size)
        out.update(cnn_losses=losses, cnn_positions=pos, cnn_params=p[pos])
        print(f"cnn: losses {losses} in {time.time() - t0:.0f} s", flush=True)
        np.savez(OUT, **out)
    if "mlp" in which:
        t0 = time.time()
        ws, bs, x, y = training.mlp_problem(MLP_WIDTHS, MLP_BATCH, MLP_STEPS, data="normal")
        losses, w, b = training.train_mlp(lib, training.CPU, MLP_WIDTHS, ws, bs, x, y, MLP_BATCH, MLP_STEPS,
                                          lr=MLP_LR)
        pos = sample_positions(w.size)
        out.update(mlp_losses=losses, mlp_positions=pos, mlp_weights=w[pos], mlp_biases=b)
        print(f"mlp: losses {losses} in {time.time() - t0:.0f} s", flush=True)
        np.savez(OUT, **out)
    if "mlp1" in which:
        t0 = time.time()
        ws, bs, x, y = training.mlp_problem(MLP_WIDTHS, MLP_BATCH, 1, data="normal")
        losses, w, b = training.train_mlp(lib, training.CPU, MLP_WIDTHS, ws, bs, x, y, MLP_BATCH, 1, lr=MLP_LR)
        pos = sample_positions(w.size)
        print(f"mlp1: losses {losses} in {time.time() - t0:.0f} s", flush=True)
        np.savez(OUT_MLP1, mlp1_losses=losses, mlp1_positions=pos, mlp1_weights=w[pos], mlp1_biases=b)


if __name__ == "__main__":
    main()
