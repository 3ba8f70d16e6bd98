"""One rank of a data-parallel test run (started by test_dp_cpu.py / test_dp_gpu.py).

mode cpu-oracle : the reference CPU backend trains on this rank's shard; gradients are
                  averaged across ranks on the host with a gloo all-reduce.  This is the
                  N-rank oracle multi-GPU runs are compared with.
mode gpu-replay : the recorded program of the same model is replayed through the C ABI on
                  this rank's GPU with B200_COMPUTE_GRAD_SYNC (NCCL all-reduce of the span's
                  gradient sinks on the communication stream).
mode cpu-dropout: rank 1 leaves before the first exchange; rank 0 must get an error from
                  its collective within the process-group timeout, not hang.
Writes its per-step losses (and final parameters) to <out>.rank<r>.npz.
"""
import argparse
import ctypes as C
import datetime
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

import training  # noqa: E402


def shard(x, y, steps, global_batch, rank, world):
    b = global_batch // world
    xs = x.reshape(steps, global_batch, -1)[:, rank * b:(rank + 1) * b].reshape(steps * b, -1)
    ys = y.reshape(steps, global_batch)[:, rank * b:(rank + 1) * b].reshape(-1)
    return np.ascontiguousarray(xs), np.ascontiguousarray(ys), b


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--program", default="mlp_wide_reduced_b128")
    ap.add_argument("--widths", default="256,512,512,512,100")
    ap.add_argument("--batch", type=int, default=128, help="per-rank batch")
    ap.add_argument("--lr", type=float, default=0.02)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=20 if args.mode != "cpu-dropout" else 4))

    widths = [int(w) for w in args.widths.split(",")]
    global_batch = args.batch * world
    ws, bs, x, y = training.mlp_problem(widths, global_batch, args.steps, data="normal")
    xs, ys, b = shard(x, y, args.steps, global_batch, rank, world)

    if args.mode in ("cpu-oracle", "cpu-dropout"):
        lib = training.load(with_b200=False)
        hook_t = C.CFUNCTYPE(None, C.POINTER(C.c_float), C.c_int64, C.c_void_p)
        state = {"calls": 0, "error": ""}

        def hook(ptr, count, _user):
            try:
                if args.mode == "cpu-dropout" and rank == 1:
                    os._exit(0)  # leaves between steps, with nothing of its own in flight
                arr = np.ctypeslib.as_array(ptr, shape=(count,))
                t = torch.from_numpy(arr)
                dist.all_reduce(t)
                t /= world
                state["calls"] += 1
            except Exception as e:  # the collective failed: record it, keep the process alive
                state["error"] = f"{type(e).__name__}: {e}"

        cb = hook_t(hook)
        lib.vkml_ref_set_grad_hook.argtypes = [hook_t, C.c_void_p]
        lib.vkml_ref_set_grad_hook(cb, None)
        steps = 1 if args.mode == "cpu-dropout" else args.steps
        losses, w, bias = training.train_mlp(lib, training.CPU, widths, ws, bs, xs, ys, b, steps, lr=args.lr)
        np.savez(f"{args.out}.rank{rank}.npz", losses=losses, w=w, b=bias, calls=state["calls"],
                 error=np.array(state["error"]))
        if args.mode == "cpu-dropout":
            os._exit(0)  # do not wait in destroy_process_group for a rank that is gone
    elif args.mode == "gpu-replay":
        import vkml_b200
        from vkml_b200.replay import Replayer, load_program
        backend = vkml_b200.Backend(0)  # CUDA_VISIBLE_DEVICES selects this rank's GPU
        uid = [backend.dist_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        backend.dist_init(rank, world, uid[0])
        program = load_program(os.path.join(HERE, "golden", "programs", args.program + ".json.gz"))
        assert program["meta"]["batch"] == b and program["meta"]["widths"] == widths
        params = [p for pair in zip(ws, bs) for p in pair]
        cur = {"s": 0}

        def feed(tag, nbytes):
            if tag[0] == "pro":
                return params[tag[1]]
            s = cur["s"]
            return xs[s * b:(s + 1) * b] if tag[1] == 0 else ys[s * b:(s + 1) * b]

        r = Replayer(backend, program, feed, grad_sync=True)
        for s in range(args.steps):
            cur["s"] = s
            r.step()
        backend.synchronize()
        losses = np.array([d.view(np.float32)[0] for _, d in r.downloads if d.nbytes == 4], dtype=np.float32)
        np.savez(f"{args.out}.rank{rank}.npz", losses=losses, comm_bytes=backend.stats()["comm_bytes"])
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
