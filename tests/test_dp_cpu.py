"""Data-parallel host logic on CPU ranks (gloo, world size 2, no GPU):

* sharding a batch over N ranks and averaging the gradients reproduces the single-rank
  run on the whole batch -- this N-rank reference run is the oracle multi-GPU runs are
  held to;
* a rank that leaves before a gradient exchange ends the other rank's collective with an
  error inside the process-group timeout instead of hanging it.
"""
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

import training
from helpers import REF_SO

HERE = os.path.dirname(os.path.abspath(__file__))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(world, args, tmp, extra_env=None, timeout=300):
    port = free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="1")
        env.update(extra_env(rank) if extra_env else {})
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "dp_worker.py"), "--out",
                                       os.path.join(tmp, "run")] + args, env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append((p.returncode, out.decode(errors="replace")))
    return outs


@pytest.mark.skipif(not os.path.exists(REF_SO), reason="oracle/_ref/libvkml_ref.so not built")
def test_two_cpu_ranks_match_the_global_batch(tmp_path):
    steps, b, widths = 12, 16, [32, 64, 64, 10]
    outs = launch(2, ["--mode", "cpu-oracle", "--steps", str(steps), "--batch", str(b), "--widths",
                      ",".join(map(str, widths)), "--lr", "0.05"], str(tmp_path))
    for rc, out in outs:
        assert rc == 0, out
    r0 = np.load(tmp_path / "run.rank0.npz")
    r1 = np.load(tmp_path / "run.rank1.npz")
    assert int(r0["calls"]) == steps * 6  # three Linear layers: weight + bias each
    # both ranks hold the same parameters after every exchange
    np.testing.assert_array_equal(r0["w"], r1["w"])
    np.testing.assert_array_equal(r0["b"], r1["b"])
    # and the run equals one rank on the whole batch (mean loss = mean of the shard means)
    lib = training.load(with_b200=False)
    ws, bs, x, y = training.mlp_problem(widths, 2 * b, steps, data="normal")
    gl, gw, gb = training.train_mlp(lib, training.CPU, widths, ws, bs, x, y, 2 * b, steps, lr=0.05)
    dp_loss = (r0["losses"] + r1["losses"]) / 2
    np.testing.assert_allclose(dp_loss, gl, rtol=2e-5)
    np.testing.assert_allclose(r0["w"], gw, atol=2e-5)
    np.testing.assert_allclose(r0["b"], gb, atol=2e-5)


@pytest.mark.skipif(not os.path.exists(REF_SO), reason="oracle/_ref/libvkml_ref.so not built")
def test_a_rank_that_leaves_ends_the_collective_with_an_error(tmp_path):
    outs = launch(2, ["--mode", "cpu-dropout", "--steps", "1", "--batch", "8", "--widths", "16,16,4"],
                  str(tmp_path), timeout=120)
    assert outs[1][0] == 0  # rank 1 left on purpose
    r0 = np.load(tmp_path / "run.rank0.npz")
    assert str(r0["error"]) != "", "rank 0 should have seen its all-reduce fail"
    assert int(r0["calls"]) == 0
