#!/usr/bin/env python
"""Benchmark of the backend hot path: fp32 GEMM C = A.B at 8192^3 through
vkML's matmul node (3xTF32 on the tcgen05 tensor cores), as whole-job TFLOP/s.

    python bench.py --gpus N --steps K --warmup W            (N > 1: under torchrun)
    python bench.py --impl reference ...                     the reference CPU path

One step = one matmul node through Backend.compute(): operand split pre-pass
(A and B), the tensor-core kernel, nothing skipped.  A, B ~ N(0,1) from a fixed
seed, generated on the host and uploaded once; operands (268 MB each) exceed L2.
`value` times K steps with the inputs resident in HBM, on the device, max over
ranks.  `e2e` times the same call with HOST buffers: pinned A and B are copied
up and C is copied back inside every timed step.  `roofline` is the tensor-core
kernel alone, from CUDA events around each launch on the launching stream.
`cpu_baseline` is the reference CPU backend's matmul kernel (compiled from the
reference's own sources into oracle/_ref/) on a bounded row slab of the same
product, on all host cores.  At N > 1 every rank runs the same GEMM on its own
operands (independent replicas: a GEMM node has no exchange step).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SEED_DATA = 20260728
# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch of the tensor-core kernel at 8192^3,
# quoted from an ncu capture of that kernel (4.565 GB read + 0.256 GB written); it is not
# re-measured in the run that prints it, and the line says so.
TRAFFIC_BYTES_PER_LAUNCH = 4820527104


def gemm_config(size, precision, world):
    """The `config` object of the contract line; both arms print the same one."""
    return {"workload": f"fp32 GEMM C=A.B, M=N=K={size}, A,B ~ N(0,1) seed {SEED_DATA}, one matmul node "
                        "through Backend.compute",
            "m": size, "n": size, "k": size, "precision": precision,  # the arithmetic of the B200 arm
            "cache": "operands (268 MB each at 8192) exceed L2; no flush needed",
            "parallelism": "independent replicas" if world > 1 else "single GPU"}


def reference_rows(size, cores):
    """Rows of A in one bounded sample of the reference CPU product: the same slab for the
    `cpu_baseline` object and for every step of `--impl reference`."""
    return int(min(size, 4 * cores))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--size", type=int, default=8192, help="M = N = K")
    ap.add_argument("--precision", default="3xtf32", choices=["3xtf32", "tf32", "fp32"])
    ap.add_argument("--workload", default="gemm", choices=["gemm", "ops", "gemm-sweep", "adapter-step"],
                    help="gemm: the contract line; ops: per-kernel HBM table of the memory-bound family; "
                         "gemm-sweep: every GEMM shape of the benchmark's sweep; adapter-step: full-size training "
                         "steps driven by the reference framework's own executor through the vkml::Backend adapter")
    ap.add_argument("--no-graphs", action="store_true", help="train object: replay every step eagerly")
    ap.add_argument("--filter", default="", help="ops workload: substring of the case names to run")
    ap.add_argument("--train", default="mlp_wide_b2048",
                    help="recorded training step replayed for the secondary `train` object "
                         "(a file under tests/golden/programs/, or 'none')")
    ap.add_argument("--train-steps", type=int, default=10)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, v in names.items():
                    if bits & v:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(0.004)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def make_operands(size: int, rank: int):
    rng = np.random.default_rng(SEED_DATA + rank)
    a = rng.standard_normal((size, size), dtype=np.float32)
    b = rng.standard_normal((size, size), dtype=np.float32)
    return a, b


# ---------------------------------------------------------------------------
# reference CPU path (oracle/_ref): used by --impl reference and by cpu_baseline
# ---------------------------------------------------------------------------

def reference_lib():
    from vkml_b200 import _abi
    path = os.path.join(ROOT, "oracle", "_ref", "libvkml_ref.so")
    if not os.path.exists(path):
        return None
    lib = C.CDLL(path)
    lib.vkml_ref_matmul_mt.restype = C.c_int
    lib.vkml_ref_matmul_mt.argtypes = [C.POINTER(_abi.Node), C.c_int]
    return lib


def reference_slab(lib, a, b, rows: int, threads: int):
    """(seconds, C[:rows]) of the reference matmul kernel for A[:rows] . B on `threads` host threads."""
    from vkml_b200.graph import DType, NodeDesc, Op, TensorDesc
    k, n = b.shape
    out = np.empty((rows, n), dtype=np.float32)
    node = NodeDesc(int(Op.MATMUL), TensorDesc.contiguous(out.ctypes.data, (1, 1, rows, n), DType.F32),
                    [TensorDesc.contiguous(a.ctypes.data, (1, 1, rows, k), DType.F32),
                     TensorDesc.contiguous(b.ctypes.data, (1, 1, k, n), DType.F32)])
    c = node.to_c()
    t0 = time.perf_counter()
    rc = lib.vkml_ref_matmul_mt(C.byref(c), threads)
    dt = time.perf_counter() - t0
    if rc != 0:
        raise RuntimeError(f"reference matmul failed with status {rc}")
    return dt, out


def cpu_baseline(a, b, passes: int = 2):
    """The reference CPU kernel on a bounded sample of the workload (the first rows of the product),
    timed on all host threads; also returns those rows of C, which the caller compares with the GPU's."""
    lib = reference_lib()
    cores = os.cpu_count() or 1
    size = a.shape[0]
    if lib is None:
        return None, None
    rows = reference_rows(size, cores)
    t, out = 0.0, None
    for _ in range(passes):
        dt, out = reference_slab(lib, a, b, rows, cores)
        t += dt
    flops = 2.0 * rows * size * size * passes
    return {"value": flops / t / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "reference",
            "sample": f"rows 0..{rows} of A: a {rows}x{size}x{size} slab of the {size}^3 product through the "
                      f"reference matmul kernel, {cores} host threads over row slabs, {passes} passes, {t:.1f} s",
            "seconds": t, "full_size_seconds_extrapolated": t / passes * size / rows}, out


def run_reference(args, rank, world):
    if rank != 0:
        return
    a, b = make_operands(args.size, 0)
    lib = reference_lib()
    base = {"impl": "reference", "metric": "fp32_gemm_tflops", "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": gemm_config(args.size, args.precision, world)}
    if lib is None:
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libvkml_ref.so is not built"}))
        return
    cores = os.cpu_count() or 1
    rows = reference_rows(args.size, cores)
    for _ in range(args.warmup):
        reference_slab(lib, a, b, rows, cores)
    t = 0.0
    for _ in range(args.steps):
        t += reference_slab(lib, a, b, rows, cores)[0]
    flops = 2.0 * rows * args.size * args.size * args.steps
    v = flops / t / 1e12
    sample = (f"each step: rows 0..{rows} of A ({rows}x{args.size}x{args.size} slab of the product) through the "
              f"reference CPU matmul kernel on {cores} host threads")
    base.update({"value": v, "ms_per_step": t / args.steps * 1e3, "sample": sample,
                 "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "reference", "sample": sample},
                 "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}})
    print(json.dumps(base))


# ---------------------------------------------------------------------------
# B200 arm
# ---------------------------------------------------------------------------

def run_b200(args, rank, local_rank, world):
    import vkml_b200
    from vkml_b200 import DeviceTensor, NodeDesc, Op, graph
    dist = None
    if world > 1:
        import torch
        import torch.distributed as td
        torch.cuda.set_device(local_rank)
        td.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank))
        dist = td

    backend = vkml_b200.Backend(local_rank)  # raises without the CUDA library or a device
    backend.set_gemm_precision({"3xtf32": 0, "tf32": 1, "fp32": 2}[args.precision])
    size = args.size
    a_host, b_host = make_operands(size, rank)
    a = DeviceTensor.from_host(backend, a_host).reshape((1, 1, size, size))
    b = DeviceTensor.from_host(backend, b_host).reshape((1, 1, size, size))
    c = DeviceTensor.empty(backend, (1, 1, size, size))
    node = NodeDesc(int(Op.MATMUL), c.desc, [a.desc, b.desc])
    packed = graph.pack_nodes([node])
    flops_per_step = 2.0 * size ** 3

    def barrier():
        backend.synchronize()
        if dist is not None:
            import torch
            torch.cuda.synchronize()
            dist.barrier()

    def max_over_ranks(ms: float) -> float:
        if dist is None:
            return ms
        import torch
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing ----
    for _ in range(max(args.warmup, 3)):
        backend.compute_packed(packed, 1)
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = backend.stats()["kernel_launches"]
    backend.timer_begin()
    for _ in range(args.steps):
        backend.compute_packed(packed, 1)
    ms = backend.timer_end()
    barrier()
    launches = backend.stats()["kernel_launches"] - launches0
    # a second pass of the same steps with an event pair around every launch: the per-kernel
    # durations behind `roofline` (kept out of the timed region, whose figure they would inflate)
    backend.set_profiling(True)
    for _ in range(args.steps):
        backend.compute_packed(packed, 1)
    records = backend.last_profile()
    backend.set_profiling(False)
    clocks = sampler.stop()
    ms = max_over_ranks(ms)
    value = flops_per_step * args.steps * world / (ms * 1e-3) / 1e12
    # the first rows of C as the timed launches left them, for the parity object below
    cores = os.cpu_count() or 1
    check_rows = reference_rows(size, cores)
    c_rows = np.empty((check_rows, size), dtype=np.float32)
    backend.copy_to_host(c_rows, c.storage, 0, c_rows.nbytes)

    # ---- roofline of the dominant kernel ----
    pk = peaks()
    by_label = {}
    for label, t in records:
        by_label.setdefault(label, []).append(t)
    main_label = max(by_label, key=lambda k: sum(by_label[k])) if by_label else None
    roofline = None
    kernel_share = {k: {"launches": len(v), "total_ms": sum(v)} for k, v in by_label.items()}
    if main_label is not None:
        avg_ms = sum(by_label[main_label]) / len(by_label[main_label])
        achieved = flops_per_step / (avg_ms * 1e-3) / 1e12
        passes = 3 if args.precision == "3xtf32" else 1
        # TF32 issues at half the bf16 rate; MEASURED_PEAKS.json has no TF32 entry, so the
        # denominator is half the measured bf16 burst figure.
        peak = pk["bf16_tflops"] / 2.0
        roofline = {"bound": "tensor", "kernel": main_label, "achieved": achieved, "peak": peak,
                    "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": TRAFFIC_BYTES_PER_LAUNCH if (size == 8192 and args.precision == "3xtf32") else None,
                    "traffic_source": "quoted from one ncu capture of this kernel at this size; not measured in this run",
                    "avg_launch_ms": avg_ms, "launches_timed": len(by_label[main_label]),
                    "tensor_pipe_tflops": achieved * passes, "tensor_pipe_frac": achieved * passes / peak,
                    "peak_source": f"{pk['source']}: bf16_tflops/2 (TF32 runs at half the bf16 rate)",
                    "note": "achieved counts the algorithmic 2*M*N*K once; 3xTF32 issues it three times on "
                            "the tensor pipe (tensor_pipe_*), so frac cannot exceed 1/3"}
        if args.precision == "fp32":
            roofline["bound"] = "fp32-simt"

    # ---- end to end with host buffers ----
    e2e = None
    if not args.no_e2e:
        nbytes = size * size * 4
        pin_a, pin_b, pin_c = backend.alloc_host(nbytes), backend.alloc_host(nbytes), backend.alloc_host(nbytes)
        pin_a[:] = a_host.view(np.uint8).reshape(-1)
        pin_b[:] = b_host.view(np.uint8).reshape(-1)
        e_steps = max(3, min(args.steps, 10))

        def e2e_step():
            backend.copy_from_host(a.storage, 0, pin_a.ctypes.data, nbytes)
            backend.copy_from_host(b.storage, 0, pin_b.ctypes.data, nbytes)
            backend.compute_packed(packed, 1)
            backend.copy_to_host(pin_c, c.storage, 0, nbytes)

        for _ in range(2):
            e2e_step()
        barrier()
        backend.timer_begin()
        t0 = time.perf_counter()
        for _ in range(e_steps):
            e2e_step()
        e_ms = backend.timer_end()
        wall_ms = (time.perf_counter() - t0) * 1e3
        barrier()
        e_ms = max_over_ranks(max(e_ms, wall_ms))
        e2e = {"value": flops_per_step * e_steps * world / (e_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": 2 * nbytes, "d2h_bytes_per_step": nbytes, "steps": e_steps,
               "ms_per_step": e_ms / e_steps}
        checksum = float(np.frombuffer(pin_c, dtype=np.float32)[:1024].sum())
        e2e["result_checksum_first_1024"] = checksum
        for p in (pin_a, pin_b, pin_c):
            backend.free_host(p)

    cpu, parity = None, None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu, ref_rows = cpu_baseline(a_host, b_host)
        if ref_rows is not None:
            # the rows the CPU baseline computed anyway, against the same rows of the timed result
            want = ref_rows.astype(np.float64)
            diff = c_rows.astype(np.float64) - want
            parity = {"rows": int(check_rows), "outputs": int(c_rows.size),
                      "rel_frobenius": float(np.linalg.norm(diff) / np.linalg.norm(want)),
                      "bound": 1e-5 * float(np.sqrt(size)), "max_abs": float(np.max(np.abs(diff))),
                      "against": "the reference CPU matmul kernel on the same operands (rows 0..%d of C)" % check_rows}

    del a, b, c, packed
    backend.trim()
    train = train_section(args, backend, rank, world, dist, barrier, max_over_ranks)

    if rank == 0:
        line = {
            "metric": "fp32_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None,
            "dtype": {"3xtf32": "f32 (3xTF32 split on tcgen05, fp32 accumulate)", "tf32": "tf32",
                      "fp32": "f32"}[args.precision],
            "data": "synthetic",
            "config": gemm_config(size, args.precision, world),
            "roofline": roofline, "cpu_baseline": cpu, "parity": parity, "e2e": e2e, "gpu_launches": launches,
            "kernels": kernel_share, "clocks": clocks, "train": train,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# secondary object: a whole training step, replayed from the framework's recorded traffic
# ---------------------------------------------------------------------------

def train_section(args, backend, rank, world, dist, barrier, max_over_ranks):
    """Samples/s of a recorded training step (forward, backward, SGD-momentum update, loss
    read-back) replayed through the C ABI; at N > 1 every rank runs the step on its own
    batch and the backward span's gradient sinks are all-reduced over NCCL while the span runs."""
    from vkml_b200.replay import Replayer, load_program
    path = os.path.join(ROOT, "tests", "golden", "programs", args.train + ".json.gz")
    if args.train == "none" or not os.path.exists(path):
        return None
    program = load_program(path)
    meta = program["meta"]
    rng = np.random.default_rng(SEED_DATA + 1 + rank)
    wrng = np.random.default_rng(SEED_DATA + 1)  # identical parameters on every rank
    batch = meta["batch"]
    if meta["model"] == "mlp":
        widths = meta["widths"]
        params = []
        for fin, fout in zip(widths[:-1], widths[1:]):
            bound = 1.0 / np.sqrt(fin)
            params.append(wrng.uniform(-bound, bound, (fout, fin)).astype(np.float32))
            params.append(wrng.uniform(-bound, bound, (fout,)).astype(np.float32))
        x_shape, classes = (batch, widths[0]), widths[-1]
        x = rng.standard_normal(x_shape, dtype=np.float32)
        desc = "MLP " + "-".join(map(str, widths))
    else:
        cin, hw, classes = meta["cin"], meta["hw"], meta["classes"]
        feat = meta["c3"] * (hw // 8) ** 2
        params = []
        for cout, ci in ((meta["c1"], cin), (meta["c2"], meta["c1"]), (meta["c3"], meta["c2"])):
            bound = 1.0 / np.sqrt(ci * 9)
            params.append(wrng.uniform(-bound, bound, (cout, ci, 3, 3)).astype(np.float32))
            params.append(wrng.uniform(-bound, bound, (cout,)).astype(np.float32))
        bound = 1.0 / np.sqrt(feat)
        params.append(wrng.uniform(-bound, bound, (classes, feat)).astype(np.float32))
        params.append(wrng.uniform(-bound, bound, (classes,)).astype(np.float32))
        x_shape = (batch, cin, hw, hw)
        x = rng.random(x_shape, dtype=np.float32)
        desc = f"CNN conv3x3 {meta['c1']}-{meta['c2']}-{meta['c3']} + Linear {feat}->{classes}"
    y = rng.integers(0, classes, batch).astype(np.int64)
    pin_x, pin_y = backend.alloc_host(x.nbytes), backend.alloc_host(y.nbytes)
    pin_x[:] = x.view(np.uint8).reshape(-1)
    pin_y[:] = y.view(np.uint8).reshape(-1)
    from vkml_b200.tape import Tape
    if world > 1:
        uid = [backend.dist_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        backend.dist_init(rank, world, uid[0])
    # The library's native step tape issues the recorded calls (one foreign call per step), so
    # the host side costs what the framework's C++ executor would, not a Python loop per node.
    tape = Tape(backend, program, grad_sync=world > 1)
    # steady-state steps as captured CUDA graphs (single GPU; gradient-synchronising steps replay eagerly)
    use_graphs = world == 1 and not args.no_graphs
    tape.enable_graphs(use_graphs)
    tape.run_prologue(params)
    first = [pin_x.ctypes.data, pin_y.ctypes.data]
    for _ in range(len(program["steps"]) - 1):   # the recorded first steps differ from the steady state
        tape.step(first)
    steady = tape.template_for_step(tape.steps_run)
    with_uploads = tape.upload_ptrs(steady, first)
    resident = tape.upload_ptrs(steady, [None, None])
    # a graph is captured the second time a step's addresses come up, and the allocator cycles
    # through at most six address sets for these programs: fourteen steps see every set twice
    warm = 14 if use_graphs else 3
    for _ in range(warm):
        tape.step_fast(with_uploads)
    for _ in range(warm):
        tape.step_fast(resident)
    backend.synchronize()
    barrier()
    k = max(3, args.train_steps)
    # end to end: x and labels uploaded from pinned host memory every step, loss read back
    l0 = backend.stats()["kernel_launches"]
    t0 = time.perf_counter()
    for _ in range(k):
        tape.step_fast(with_uploads)
    backend.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3)
    launches = (backend.stats()["kernel_launches"] - l0) / k
    barrier()
    # inputs resident: the recorded uploads are skipped (the buffers keep the last batch)
    backend.timer_begin()
    for _ in range(k):
        tape.step_fast(resident)
    dev_ms = max_over_ranks(backend.timer_end())
    barrier()
    # a separate, profiled pass for the per-kernel breakdown (events around every launch)
    backend.set_profiling(True)
    for _ in range(k):
        tape.step_fast(resident)
    records = backend.last_profile()
    backend.set_profiling(False)
    barrier()
    loss_last = float(tape.downloads[0].view(np.float32)[0]) if tape.downloads else None
    steps_total = tape.steps_run
    comm_bytes = int(backend.stats()["comm_bytes"] / max(1, steps_total))
    alone_ms = None
    if world > 1 and comm_bytes:
        # the same bytes all-reduced with nothing else on the GPU: the part of it that the
        # step does not hide is ms_per_step(N) - ms_per_step(1)
        buf = backend.allocate(comm_bytes)
        for _ in range(2):
            backend.dist_all_reduce_mean(buf.data, comm_bytes // 4)
            backend.dist_wait()
        barrier()
        backend.timer_begin()
        for _ in range(k):
            backend.dist_all_reduce_mean(buf.data, comm_bytes // 4)
            backend.dist_wait()
        alone_ms = max_over_ranks(backend.timer_end()) / k
        del buf
        barrier()
    by_label = {}
    for label, t in records:
        by_label[label] = by_label.get(label, 0.0) + t / k
    top = dict(sorted(by_label.items(), key=lambda kv: -kv[1]))
    counts = {}
    for label, _ in records:
        counts[label] = counts.get(label, 0) + 1.0 / k
    if use_graphs:
        # replayed graphs launch the step's kernels as graph nodes, which the library's launch
        # counter does not see: count the same step's kernels from the profiled (eager) pass
        launches = round(sum(counts.values()), 2)
    out = {"workload": f"{desc}, per-GPU batch {batch}, fp32, cross-entropy, SGD momentum 0.9: the framework's "
                       f"recorded step ({args.train}) replayed by the library's step tape",
           "samples_per_s": batch * world * k / (dev_ms * 1e-3), "ms_per_step": dev_ms / k,
           "e2e_samples_per_s": batch * world * k / (e2e_ms * 1e-3), "e2e_ms_per_step": e2e_ms / k,
           "h2d_bytes_per_step": int(x.nbytes + y.nbytes), "d2h_bytes_per_step": 4,
           "gpu_launches_per_step": launches, "steps": k, "n_gpus": world,
           "parallelism": f"dp{world}: batch sharded, NCCL all-reduce of gradient sinks overlapped with backward"
                          if world > 1 else "single GPU",
           "comm_bytes_per_step": comm_bytes, "all_reduce_alone_ms": alone_ms,
           "loss_last": loss_last, "host_side": "library step tape" + (", CUDA graphs" if use_graphs else ""),
           "tape": tape.stats(),
           "device_ms_per_step_by_kernel": {a: round(b, 4) for a, b in top.items()},
           "launches_per_step_by_kernel": {a: round(counts[a], 2) for a in top}}
    tape.close()
    backend.free_host(pin_x)
    backend.free_host(pin_y)
    return out


# ---------------------------------------------------------------------------
# memory-bound family: achieved HBM GB/s per kernel at the benchmark's shapes
# ---------------------------------------------------------------------------

def run_ops(args, local_rank):
    """One JSON line per case: algorithmic bytes / device time, against the measured HBM
    peak.  Every case rotates over enough independent buffer sets that consecutive
    launches cannot be served from the 126 MB L2."""
    import vkml_b200
    from vkml_b200 import DeviceTensor, NodeDesc, Op, graph
    from vkml_b200.graph import DType
    backend = vkml_b200.Backend(local_rank)
    pk = peaks()
    rng = np.random.default_rng(SEED_DATA)
    F32, I64, BOOL, F16 = DType.F32, DType.I64, DType.BOOL, DType.F16

    def dev(shape, dtype=F32, kind="normal"):
        n = int(np.prod(shape)) if len(shape) else 1
        if dtype == F32:
            host = rng.standard_normal(n, dtype=np.float32) if kind == "normal" else rng.random(n, dtype=np.float32)
        elif dtype == I64:
            host = rng.integers(0, 10, n).astype(np.int64)
        elif dtype == F16:
            host = rng.standard_normal(n, dtype=np.float32).astype(np.float16)
        else:
            host = (rng.random(n) < 0.5).astype(np.uint8)
        return DeviceTensor.from_host(backend, host.reshape(shape))

    cases = []

    def case(name, op, out_shape, out_dtype, make_srcs, params=b"", bytes_alg=None):
        cases.append((name, op, out_shape, out_dtype, make_srcs, params, bytes_alg))

    def T(t):  # transposed view of a 2-D tensor
        return t.transpose(0, 1)

    B, H = 2048, 8192
    case("add dense [2048,8192]", Op.ADD, (B, H), F32, lambda: [dev((B, H)), dev((B, H))], bytes_alg=12 * B * H)
    case("add bias row-broadcast [2048,8192]+[8192]", Op.ADD, (B, H), F32,
         lambda: [dev((B, H)), dev((H,)).broadcast_to((B, H))], bytes_alg=8 * B * H + 4 * H)
    case("add bias channel-broadcast [256,64,32,32]+[64,1,1]", Op.ADD, (256, 64, 32, 32), F32,
         lambda: [dev((256, 64, 32, 32)), dev((64, 1, 1)).broadcast_to((256, 64, 32, 32))],
         bytes_alg=8 * 256 * 64 * 1024)
    case("relu [2048,8192]", Op.RELU, (B, H), F32, lambda: [dev((B, H))], bytes_alg=8 * B * H)
    # half storage: the elementwise families read and write it directly (2 bytes per element each way)
    case("add f16 dense [4096,8192]", Op.ADD, (4096, H), F16, lambda: [dev((4096, H), F16), dev((4096, H), F16)],
         bytes_alg=6 * 4096 * H)
    case("relu f16 [4096,8192]", Op.RELU, (4096, H), F16, lambda: [dev((4096, H), F16)], bytes_alg=4 * 4096 * H)
    case("less_equal vs scalar [2048,8192] -> bool", Op.LESS_EQUAL, (B, H), BOOL,
         lambda: [dev((B, H)), dev(()).broadcast_to((B, H))], bytes_alg=5 * B * H)
    case("where(mask, g, 0) [2048,8192]", Op.WHERE, (B, H), F32,
         lambda: [dev((B, H), BOOL), dev((B, H)), dev(()).broadcast_to((B, H))], bytes_alg=9 * B * H)
    case("mul col-broadcast [2048,1000]*[2048,1]", Op.MUL, (B, 1000), F32,
         lambda: [dev((B, 1000)), dev((B, 1)).broadcast_to((B, 1000))], bytes_alg=8 * B * 1000)
    case("exp [8192,1000]", Op.EXP, (8192, 1000), F32, lambda: [dev((8192, 1000))], bytes_alg=8 * 8192 * 1000)
    case("full zeros [2048,8192]", Op.FULL, (B, H), F32, lambda: [], graph.full_params(0.0), bytes_alg=4 * B * H)
    case("cast bool->f32 [8192,1000]", Op.CAST, (8192, 1000), F32, lambda: [dev((8192, 1000), BOOL)],
         bytes_alg=5 * 8192 * 1000)
    case("cast i64->f32 [1<<24]", Op.CAST, (1 << 24,), F32, lambda: [dev((1 << 24,), I64)], bytes_alg=12 * (1 << 24))
    case("scaled_add dense [8192,8192]", Op.SCALED_ADD, (H, H), F32, lambda: [dev((H, H)), dev((H, H))],
         graph.scaled_add_params(0.9, 1.0), bytes_alg=12 * H * H)
    case("scaled_add one transposed operand [8192,8192]", Op.SCALED_ADD, (H, H), F32,
         lambda: [dev((H, H)), T(dev((H, H)))], graph.scaled_add_params(1.0, -0.1), bytes_alg=12 * H * H)
    case("scaled_add both transposed [8192,4096]", Op.SCALED_ADD, (H, 4096), F32,
         lambda: [T(dev((4096, H))), T(dev((4096, H)))], graph.scaled_add_params(0.9, 1.0), bytes_alg=12 * H * 4096)
    case("contiguous of transposed [8192,8192]", Op.CONTIGUOUS, (H, H), F32, lambda: [T(dev((H, H)))],
         bytes_alg=8 * H * H)
    case("contiguous of transposed [8200,8200] (pitch not a power of two)", Op.CONTIGUOUS, (8200, 8200), F32,
         lambda: [T(dev((8200, 8200)))], bytes_alg=8 * 8200 * 8200)
    case("sum columns [2048,8200]->[8200] (pitch not a power of two)", Op.SUM, (1, 8200), F32,
         lambda: [dev((B, 8200))], graph.reduce_params([0], 2, True), bytes_alg=4 * B * 8200)
    case("sum columns [16384,8192]->[8192] (537 MB)", Op.SUM, (1, H), F32, lambda: [dev((16384, H))],
         graph.reduce_params([0], 2, True), bytes_alg=4 * 16384 * H)
    case("relu [8192,8192] (537 MB)", Op.RELU, (H, H), F32, lambda: [dev((H, H))], bytes_alg=8 * H * H)
    case("softmax [8192,8000] (524 MB)", Op.SOFTMAX, (8192, 8000), F32, lambda: [dev((8192, 8000))],
         graph.axis_params(1), bytes_alg=8 * 8192 * 8000)
    case("sum rows [16384,8000]->[16384] (524 MB)", Op.SUM, (16384,), F32, lambda: [dev((16384, 8000))],
         graph.reduce_params([1], 2), bytes_alg=4 * 16384 * 8000)
    for (b, c) in [(65536, 10), (8192, 1000), (1024, 32000)]:
        case(f"sum rows [{b},{c}]->[{b}]", Op.SUM, (b,), F32, lambda b=b, c=c: [dev((b, c))],
             graph.reduce_params([1], 2), bytes_alg=4 * b * c + 4 * b)
        case(f"softmax [{b},{c}]", Op.SOFTMAX, (b, c), F32, lambda b=b, c=c: [dev((b, c), kind="normal")],
             graph.axis_params(1), bytes_alg=8 * b * c)
        case(f"log_softmax [{b},{c}]", Op.LOG_SOFTMAX, (b, c), F32, lambda b=b, c=c: [dev((b, c))],
             graph.axis_params(1), bytes_alg=8 * b * c)
        case(f"argmax rows [{b},{c}]", Op.ARGMAX, (b,), I64, lambda b=b, c=c: [dev((b, c))],
             graph.reduce_params([1], 2), bytes_alg=4 * b * c + 8 * b)
    case("sum columns [2048,8192]->[8192] (bias grad)", Op.SUM, (1, H), F32, lambda: [dev((B, H))],
         graph.reduce_params([0], 2, True), bytes_alg=4 * B * H + 4 * H)
    case("sum batch axis [1,256,128,576]->[1,1,128,576] (conv dW)", Op.SUM, (1, 1, 128, 576), F32,
         lambda: [dev((1, 256, 128, 576))], graph.reduce_params([1], 4, True), bytes_alg=4 * 256 * 128 * 576)
    case("sum N,H,W [256,64,32,32]->[1,64,1,1] (conv bias grad)", Op.SUM, (1, 64, 1, 1), F32,
         lambda: [dev((256, 64, 32, 32))], graph.reduce_params([0, 2, 3], 4, True), bytes_alg=4 * 256 * 64 * 1024)
    case("mean all [1<<26]", Op.MEAN, (), F32, lambda: [dev((1 << 26,))], graph.reduce_params([], 1),
         bytes_alg=4 * (1 << 26))
    up = graph.unfold_params
    case("im2col [256,64,16,16] k3 p1 -> [256,576,256]", Op.IM2COL, (256, 576, 256), F32,
         lambda: [dev((256, 64, 16, 16))], up((3, 3), (1, 1), (1, 1), (1, 1), (16, 16)),
         bytes_alg=4 * (256 * 64 * 256 + 256 * 576 * 256))
    case("col2im [256,576,256] -> [256,64,16,16]", Op.COL2IM, (256, 64, 16, 16), F32,
         lambda: [dev((256, 576, 256))], up((3, 3), (1, 1), (1, 1), (1, 1), (16, 16)),
         bytes_alg=4 * (256 * 64 * 256 + 256 * 576 * 256))
    case("max_pool2d 2x2 [256,64,32,32]", Op.MAX_POOL2D, (256, 64, 16, 16), F32,
         lambda: [dev((256, 64, 32, 32))], up((2, 2), (2, 2), (0, 0), (1, 1), (32, 32)),
         bytes_alg=4 * 256 * 64 * (1024 + 256))
    case("max_pool2d_backward 2x2 [256,64,32,32]", Op.MAX_POOL2D_BACKWARD, (256, 64, 32, 32), F32,
         lambda: [dev((256, 64, 16, 16)), dev((256, 64, 32, 32))], up((2, 2), (2, 2), (0, 0), (1, 1), (32, 32)),
         bytes_alg=4 * 256 * 64 * (1024 + 256 + 1024))
    case("index_select rows [50000,1024][8192]", Op.INDEX_SELECT, (8192, 1024), F32,
         lambda: [dev((50000, 1024)), DeviceTensor.from_host(backend, rng.integers(0, 50000, 8192).astype(np.int64))],
         graph.axis_params(0), bytes_alg=8 * 8192 * 1024)
    # an Embedding's backward: 8192 gradient rows added into a 50000-row table (every row of the
    # result is written, each source row is read once)
    case("scatter_add rows [8192,1024] -> [50000,1024]", Op.SCATTER_ADD, (50000, 1024), F32,
         lambda: [dev((8192, 1024)), DeviceTensor.from_host(backend, rng.integers(0, 50000, 8192).astype(np.int64))],
         graph.axis_params(0), bytes_alg=4 * 1024 * (8192 + 50000))

    results = []
    for name, op, out_shape, out_dtype, make_srcs, params, bytes_alg in cases:
        if args.filter and args.filter not in name:
            continue
        probe = make_srcs()
        set_bytes = sum(t.storage.nbytes for t in probe) + int(np.prod(out_shape) if len(out_shape) else 1) * out_dtype.itemsize
        n_sets = int(min(24, max(2, np.ceil(300e6 / max(set_bytes, 1)))))
        sets = [probe] + [make_srcs() for _ in range(n_sets - 1)]
        outs = [DeviceTensor.empty(backend, out_shape, out_dtype) for _ in range(n_sets)]
        packed = [graph.pack_nodes([NodeDesc(int(op), o.desc, [t.desc for t in srcs], params)])
                  for srcs, o in zip(sets, outs)]
        reps = max(args.steps, 20)
        for i in range(max(args.warmup, 3)):
            backend.compute_packed(packed[i % n_sets], 1)
        backend.synchronize()
        l0 = backend.stats()["kernel_launches"]
        backend.timer_begin()
        for i in range(reps):
            backend.compute_packed(packed[i % n_sets], 1)
        ms = backend.timer_end()
        launches = (backend.stats()["kernel_launches"] - l0) / reps
        us = ms * 1e3 / reps
        gbs = bytes_alg / (us * 1e-6) / 1e9
        row = {"op": name, "us": round(us, 2), "algorithmic_MB": round(bytes_alg / 1e6, 2), "GBps": round(gbs, 1),
               "frac_of_hbm": round(gbs / pk["hbm_gbs"], 3), "launches_per_call": launches, "buffer_sets": n_sets}
        results.append(row)
        print(json.dumps(row), flush=True)
        del sets, outs, packed, probe
        backend.trim()
    return results


def run_gemm_sweep(args, local_rank):
    """One JSON line per GEMM shape of the benchmark's GEMM sweep (squares, skinny M=64, long-K split-K) and
    of the wide-MLP / CNN training steps, per precision: device time of the whole matmul node."""
    import vkml_b200
    from vkml_b200 import DeviceTensor, NodeDesc, Op, graph
    backend = vkml_b200.Backend(local_rank)
    rng = np.random.default_rng(SEED_DATA)
    shapes = [("square 256", 1, 256, 256, 256, "nn"), ("square 1024", 1, 1024, 1024, 1024, "nn"),
              ("square 4096", 1, 4096, 4096, 4096, "nn"), ("square 8192", 1, 8192, 8192, 8192, "nn"),
              ("skinny M=64, K=N=4096", 1, 64, 4096, 4096, "nn"), ("long K=65536, M=N=512", 1, 512, 65536, 512, "nn"),
              ("wide MLP fwd 2048x4096 . W^T(8192)", 1, 2048, 4096, 8192, "nt"),
              ("wide MLP fwd 2048x8192 . W^T(8192)", 1, 2048, 8192, 8192, "nt"),
              ("wide MLP dX 2048x8192 . W(8192x8192)", 1, 2048, 8192, 8192, "nn"),
              ("wide MLP dW x^T(8192x2048) . g(2048x8192)", 1, 8192, 2048, 8192, "tn"),
              ("wide MLP head 2048x8192 . W^T(1000)", 1, 2048, 8192, 1000, "nt"),
              ("conv2 fwd W[128x576] bcast . cols[256][576x256]", 256, 128, 576, 256, "bn"),
              ("conv3 fwd W[256x1152] bcast . cols[256][1152x64]", 256, 256, 1152, 64, "bn"),
              ("conv1 fwd W[64x27] bcast . cols[256][27x1024]", 256, 64, 27, 1024, "bn"),
              ("conv1 dW g[256][64x1024] . cols^T[256][1024x27]", 256, 64, 1024, 27, "nT"),
              ("conv2 dcols W^T[576x128] bcast . g[256][128x256]", 256, 576, 128, 256, "Bn"),
              ("conv2 dW g[256][128x256] . cols^T[256][256x576]", 256, 128, 256, 576, "nT"),
              ("conv3 dcols W^T[1152x256] bcast . g[256][256x64]", 256, 1152, 256, 64, "Bn"),
              ("conv3 dW g[256][256x64] . cols^T[256][64x1152]", 256, 256, 64, 1152, "nT"),
              ("CNN head 256x4096 . W^T(100)", 1, 256, 4096, 100, "nt"),
              ("MNIST MLP 64x784 . W^T(128)", 1, 64, 784, 128, "nt")]
    for name, batch, m, k, n, kind in shapes:
        if args.filter and args.filter not in name:
            continue
        flops = 2.0 * batch * m * n * k
        # small products: ten nodes per submitted span, so that the stream never waits for the host
        # between them (one Python call per node would be the thing measured).  Every node of the span
        # has operands and a result of its OWN: nothing is shared between the nodes (no operand plane is
        # reused) and the ten operand sets together are larger than L2, so no node finds its input there.
        per_span = 10 if flops < 1e10 else 1
        if kind in ("bn", "Bn"):
            host_a = rng.standard_normal((k, m) if kind == "Bn" else (m, k), dtype=np.float32)
            host_b = rng.standard_normal((1, batch, k, n), dtype=np.float32)
        elif kind == "nT":
            host_a = rng.standard_normal((1, batch, m, k), dtype=np.float32)
            host_b = rng.standard_normal((1, batch, n, k), dtype=np.float32)
        else:
            host_a = rng.standard_normal((k, m) if kind[0] == "t" else (m, k), dtype=np.float32)
            host_b = rng.standard_normal((n, k) if kind[1] == "t" else (k, n), dtype=np.float32)

        def operands():
            a = DeviceTensor.from_host(backend, host_a)
            b = DeviceTensor.from_host(backend, host_b)
            if kind == "bn":   # A broadcast over the batch
                a = a.reshape((1, 1, m, k)).broadcast_to((1, batch, m, k))
            elif kind == "Bn":   # A = a transposed view of a broadcast [k, m] matrix (dcols = W^T . g)
                a = a.transpose(0, 1)
                a = DeviceTensor(backend, a.storage, (1, 1) + a.dims, (0, 0) + a.strides, a.dtype).broadcast_to(
                    (1, batch, m, k))
            elif kind == "nT":   # batched A, B = a transposed view of batched [n, k] storage (dW = g . cols^T)
                b = b.transpose(2, 3)
            else:
                a = (a.transpose(0, 1) if kind[0] == "t" else a)
                b = (b.transpose(0, 1) if kind[1] == "t" else b)
                a = DeviceTensor(backend, a.storage, (1, 1) + a.dims, (0, 0) + a.strides, a.dtype)
                b = DeviceTensor(backend, b.storage, (1, 1) + b.dims, (0, 0) + b.strides, b.dtype)
            return a, b, DeviceTensor.empty(backend, (1, batch, m, n))

        sets = [operands() for _ in range(per_span)]
        nodes = [NodeDesc(int(Op.MATMUL), c.desc, [a.desc, b.desc]) for a, b, c in sets]
        packed = graph.pack_nodes(nodes[:1])
        span = graph.pack_nodes(nodes)
        row = {"gemm": name, "batch": batch, "m": m, "k": k, "n": n, "layout": kind, "nodes_per_span": per_span}
        for prec, code in (("3xtf32", 0), ("tf32", 1), ("fp32", 2)):
            if prec == "fp32" and flops > 3e11:
                continue
            backend.set_gemm_precision(code)
            reps = (20 if flops < 1e11 else 5) // (2 if per_span > 1 else 1)
            for _ in range(3):
                backend.compute_packed(span, per_span)
            backend.synchronize()
            backend.timer_begin()
            for _ in range(reps):
                backend.compute_packed(span, per_span)
            ms = backend.timer_end() / (reps * per_span)
            backend.set_profiling(True)
            backend.compute_packed(packed, 1)
            rec = backend.last_profile()
            backend.set_profiling(False)
            row[prec] = {"ms": round(ms, 4), "tflops": round(flops / (ms * 1e-3) / 1e12, 2),
                         "kernel_ms": {l: round(t, 4) for l, t in rec}}
        print(json.dumps(row), flush=True)
        del sets, nodes, packed, span
        backend.trim()


def run_adapter_steps(args):
    """The drop-in route itself, timed: vkML's own graph, autograd, executor and optimiser code
    (compiled from the reference's sources, with the B200 adapter registered as its device) run
    full-size training steps -- the framework calls Backend::compute / copy_* / allocate exactly
    as it would on its own GPU backend.  Wall clock per step, uploads and loss read-back included;
    the `train` object of the contract line replays the same traffic without the framework above."""
    path = os.path.join(ROOT, "oracle", "_ref", "libvkml_ref_b200.so")
    if not os.path.exists(path):
        print(json.dumps({"workload": "adapter-step", "unavailable": "oracle/_ref/libvkml_ref_b200.so is not built"}))
        return
    lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
    f32p, i64p = C.POINTER(C.c_float), C.POINTER(C.c_int64)
    lib.vkml_ref_train_mlp.restype = C.c_int
    lib.vkml_ref_train_mlp.argtypes = [C.c_int, i64p, C.c_int, f32p, f32p, f32p, i64p, C.c_int64, C.c_int,
                                       C.c_double, C.c_double, f32p]
    lib.vkml_ref_train_cnn.restype = C.c_int
    lib.vkml_ref_train_cnn.argtypes = [C.c_int] + [C.c_int64] * 6 + [f32p, f32p, i64p, C.c_int64, C.c_int,
                                                                    C.c_double, C.c_double, f32p]
    lib.vkml_ref_step_seconds.restype = C.c_int
    lib.vkml_ref_step_seconds.argtypes = [C.POINTER(C.c_double), C.c_int]
    lib.vkml_ref_last_error.restype = C.c_char_p
    steps = max(6, args.train_steps)
    rng = np.random.default_rng(SEED_DATA + 1)

    def ptr(a, t):
        return a.ctypes.data_as(C.POINTER(t))

    def report(name, rc, batch):
        if rc != 0:
            print(json.dumps({"workload": "adapter-step", "model": name, "error": lib.vkml_ref_last_error().decode()}))
            return
        buf = (C.c_double * steps)()
        n = lib.vkml_ref_step_seconds(buf, steps)
        ms = [buf[i] * 1e3 for i in range(n)]
        steady = sorted(ms[3:])
        med = steady[len(steady) // 2]
        print(json.dumps({"workload": "adapter-step", "model": name, "per_gpu_batch": batch, "steps": n,
                          "ms_per_step": med, "samples_per_s": batch / (med * 1e-3), "first_steps_ms": ms[:3],
                          "path": "reference executor -> vkml::Backend adapter -> C ABI -> CUDA; wall clock per step "
                                  "with the batch uploaded and the loss read back"}), flush=True)

    widths = np.array([4096, 8192, 8192, 8192, 1000], dtype=np.int64)
    batch = 2048
    w = np.concatenate([rng.uniform(-1, 1, a * b).astype(np.float32) / np.float32(np.sqrt(a))
                        for a, b in zip(widths[:-1], widths[1:])])
    b = np.zeros(int(widths[1:].sum()), dtype=np.float32)
    x = rng.standard_normal((batch * steps, int(widths[0])), dtype=np.float32)
    y = rng.integers(0, int(widths[-1]), batch * steps).astype(np.int64)
    losses = np.zeros(steps, dtype=np.float32)
    rc = lib.vkml_ref_train_mlp(1, ptr(widths, C.c_int64), len(widths) - 1, ptr(w, C.c_float), ptr(b, C.c_float),
                                ptr(x, C.c_float), ptr(y, C.c_int64), batch, steps, 0.1, 0.9, ptr(losses, C.c_float))
    report("MLP 4096-8192-8192-8192-1000", rc, batch)
    del w, x
    batch, c1, c2, c3, classes = 256, 64, 128, 256, 100
    n_p = c1 * 27 + c1 + c2 * c1 * 9 + c2 + c3 * c2 * 9 + c3 + classes * c3 * 16 + classes
    params = (rng.uniform(-1, 1, n_p) * 0.05).astype(np.float32)
    x = rng.random((batch * steps, 3, 32, 32), dtype=np.float32)
    y = rng.integers(0, classes, batch * steps).astype(np.int64)
    rc = lib.vkml_ref_train_cnn(1, 3, 32, c1, c2, c3, classes, ptr(params, C.c_float), ptr(x, C.c_float),
                                ptr(y, C.c_int64), batch, steps, 0.05, 0.9, ptr(losses, C.c_float))
    report("CNN conv3x3 64-128-256 + Linear 4096->100", rc, batch)
    widths = np.array([784, 128, 10], dtype=np.int64)
    batch = 64
    steps_small = steps
    w = (rng.uniform(-1, 1, 784 * 128 + 128 * 10) * 0.03).astype(np.float32)
    b = np.zeros(138, dtype=np.float32)
    x = rng.random((batch * steps_small, 784), dtype=np.float32)
    y = rng.integers(0, 10, batch * steps_small).astype(np.int64)
    rc = lib.vkml_ref_train_mlp(1, ptr(widths, C.c_int64), 2, ptr(w, C.c_float), ptr(b, C.c_float), ptr(x, C.c_float),
                                ptr(y, C.c_int64), batch, steps_small, 0.1, 0.9, ptr(losses, C.c_float))
    report("MLP 784-128-10", rc, batch)


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.workload == "ops":
        run_ops(args, local_rank)
    elif args.workload == "gemm-sweep":
        run_gemm_sweep(args, local_rank)
    elif args.workload == "adapter-step":
        run_adapter_steps(args)
    elif args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_b200(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
