"""Records the backend traffic of whole training steps from the reference framework
and stores it as replayable programs under tests/golden/programs/.

The reference's own graph, autograd and optimiser code (oracle/_ref, built from the
reference sources) runs each model on a recording `vkml::Backend` that logs every
allocation, upload, compute span, device copy and download instead of executing it,
so a full-size step is recorded in milliseconds.  Buffer ids are then made relative
to the step that allocated them, the steady state is checked to be periodic (step 2
and step 3 encode identically), and prologue + steps 0..2 are written out.

Run from the repository root:  python tests/golden/make_programs.py
"""
import ctypes as C
import gzip
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import training  # noqa: E402

OUT = os.path.join(HERE, "programs")
STEPS = 4


def relativise(events):
    """Split a raw log at its step markers and rewrite buffer ids as (steps back, index)."""
    chunks, current = [[]], None
    for ev in events:
        if ev["ev"] == "step":
            chunks.append([])
            continue
        chunks[-1].append(ev)
    owner = {}  # raw id -> (chunk index, allocation index)
    out, lookback = [], 0
    for ci, chunk in enumerate(chunks):
        n_alloc = 0
        res = []

        def ref(raw):
            nonlocal lookback
            if raw is None or raw < 0:
                return None
            oc, j = owner[raw]
            if oc == 0:
                return ["pro", j]
            lookback = max(lookback, ci - oc)
            return [ci - oc, j]

        def tensor(t):
            return {"buf": ref(t["id"]), "off": t["off"], "dtype": t["dtype"], "dims": t["dims"],
                    "strides": t["strides"]}

        for ev in chunk:
            k = ev["ev"]
            if k == "alloc":
                owner[ev["id"]] = (ci, n_alloc)
                n_alloc += 1
                res.append({"ev": "alloc", "bytes": ev["bytes"]})
            elif k == "free":
                res.append({"ev": "free", "buf": ref(ev["id"])})
            elif k in ("h2d", "d2h"):
                res.append({"ev": k, "buf": ref(ev["id"]), "off": ev["off"], "bytes": ev["bytes"]})
            elif k == "d2d":
                res.append({"ev": "d2d", "copies": [[ref(d), do, ref(s), so, n] for d, do, s, so, n in ev["copies"]]})
            elif k == "compute":
                res.append({"ev": "compute", "grad_sync": ev["grad_sync"],
                            "nodes": [{"op": n["op"], "params": n["params"], "out": tensor(n["out"]),
                                       "src": [tensor(s) for s in n["src"]]} for n in ev["nodes"]]})
            elif k == "sync":
                res.append({"ev": "sync"})
        out.append(res)
    return out, lookback


def record(lib, name, meta, run):
    raw_path = os.path.join(OUT, name + ".raw.jsonl")
    lib.vkml_ref_record_begin(raw_path.encode())
    run()
    lib.vkml_ref_record_end()
    events = [json.loads(line) for line in open(raw_path)]
    os.remove(raw_path)
    chunks, lookback = relativise(events)
    prologue, steps = chunks[0], chunks[1:]
    # frees that happen after the last step (teardown) are not part of any step
    assert len(steps) == STEPS
    # trailing events of the last chunk (final parameter downloads, teardown frees) are dropped
    # by comparing only up to the length of the previous step
    s2, s3 = steps[2], steps[3][: len(steps[2])]
    assert json.dumps(s2) == json.dumps(s3), f"{name}: the steady state is not periodic"
    program = {"name": name, "meta": meta, "lookback": lookback, "prologue": prologue, "steps": steps[:3]}
    path = os.path.join(OUT, name + ".json.gz")
    with gzip.open(path, "wt", compresslevel=9) as f:
        json.dump(program, f, separators=(",", ":"))
    n_nodes = [sum(len(e["nodes"]) for e in s if e["ev"] == "compute") for s in steps[:3]]
    print(f"{name}: nodes per step {n_nodes}, lookback {lookback}, {os.path.getsize(path)} bytes")


def main():
    os.makedirs(OUT, exist_ok=True)
    lib = training.load(with_b200=False)
    lib.vkml_ref_record_begin.argtypes = [C.c_char_p]

    def mlp(name, widths, batch, lr=0.1):
        n_w = sum(a * b for a, b in zip(widths[:-1], widths[1:]))
        ws = [np.zeros(n_w, dtype=np.float32)]
        bs = [np.zeros(sum(widths[1:]), dtype=np.float32)]
        x = np.zeros(batch * widths[0], dtype=np.float32)
        y = np.zeros(batch, dtype=np.int64)
        record(lib, name, {"model": "mlp", "widths": widths, "batch": batch, "lr": lr, "momentum": 0.9},
               lambda: training.train_mlp(lib, 2, widths, ws, bs, x, y, batch, STEPS, lr=lr))

    def cnn(name, batch, c1, c2, c3, classes=100, cin=3, hw=32, lr=0.05):
        feat = c3 * (hw // 8) ** 2
        n_p = c1 * cin * 9 + c1 + c2 * c1 * 9 + c2 + c3 * c2 * 9 + c3 + classes * feat + classes
        params = np.zeros(n_p, dtype=np.float32)
        x = np.zeros(batch * cin * hw * hw, dtype=np.float32)
        y = np.zeros(batch, dtype=np.int64)
        record(lib, name, {"model": "cnn", "batch": batch, "cin": cin, "hw": hw, "c1": c1, "c2": c2, "c3": c3,
                           "classes": classes, "lr": lr, "momentum": 0.9},
               lambda: training.train_cnn(lib, 2, cin, hw, c1, c2, c3, classes, params, x, y, batch, STEPS, lr=lr))

    mlp("mlp_784_128_10_b64", [784, 128, 10], 64)                       # benchmark configuration 1 (MNIST MLP)
    mlp("mlp_wide_b2048", [4096, 8192, 8192, 8192, 1000], 2048)          # benchmark configuration 5 (wide MLP, per-GPU batch)
    mlp("mlp_wide_reduced_b128", [256, 512, 512, 512, 100], 128, lr=0.02)
    cnn("cnn_cifar_b256", 256, 64, 128, 256)                            # benchmark configuration 4 (CNN, per-GPU batch)
    cnn("cnn_reduced_b16", 16, 16, 32, 64)


if __name__ == "__main__":
    main()
