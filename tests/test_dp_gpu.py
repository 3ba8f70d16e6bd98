"""Data-parallel training on 2 GPUs: each rank replays the recorded step of the wide-MLP
structure on its shard with B200_COMPUTE_GRAD_SYNC (NCCL all-reduce of the backward
span's gradient sinks, on the communication stream, while the span keeps running), and
the mean of the ranks' losses follows the reference CPU run on the whole batch."""
import ctypes as C
import os

import numpy as np
import pytest

import training
from helpers import REF_SO
from test_dp_cpu import launch

pytestmark = pytest.mark.gpu


def gpu_count():
    from vkml_b200 import _abi
    n = C.c_int(0)
    return n.value if _abi.load().b200_device_count(C.byref(n)) == 0 else 0


@pytest.mark.skipif(not os.path.exists(REF_SO), reason="oracle/_ref/libvkml_ref.so not built")
def test_two_gpus_follow_the_cpu_global_batch(tmp_path):
    if gpu_count() < 2:
        pytest.skip("needs 2 GPUs")
    steps, b, widths = 20, 128, [256, 512, 512, 512, 100]
    outs = launch(2, ["--mode", "gpu-replay", "--steps", str(steps), "--batch", str(b), "--lr", "0.02"],
                  str(tmp_path), extra_env=lambda r: {"CUDA_VISIBLE_DEVICES": str(r), "NCCL_NVLS_ENABLE": "0"},
                  timeout=600)
    for rc, out in outs:
        assert rc == 0, out[-3000:]
    r0 = np.load(tmp_path / "run.rank0.npz")
    r1 = np.load(tmp_path / "run.rank1.npz")
    assert int(r0["comm_bytes"]) > 0 and int(r0["comm_bytes"]) == int(r1["comm_bytes"])
    lib = training.load(with_b200=False)
    ws, bs, x, y = training.mlp_problem(widths, 2 * b, steps, data="normal")
    cpu_l, _, _ = training.train_mlp(lib, training.CPU, widths, ws, bs, x, y, 2 * b, steps, lr=0.02)
    dp_loss = (r0["losses"] + r1["losses"]) / 2
    assert len(dp_loss) == steps
    np.testing.assert_allclose(dp_loss, cpu_l, rtol=1e-4)
    # the ranks really exchanged: without it their curves would not add up to the global one,
    # and a single rank's curve differs from the global curve
    assert np.max(np.abs(r0["losses"] - cpu_l) / cpu_l) > 1e-4


def test_a_rank_that_never_joins_ends_init_with_a_timeout():
    """Failure made on the host: rank 0 of a two-rank job starts, rank 1 never does.  The
    communicator is created in NCCL's non-blocking mode and polled against a deadline; when it runs
    out the communicator is aborted and the call returns B200_TIMEOUT (vkML's DeviceError).  No
    kernel or collective is in flight at any point, and the context keeps working afterwards."""
    import time

    import vkml_b200
    from vkml_b200 import DeviceTensor
    from vkml_b200.backend import DeviceError
    b = vkml_b200.Backend(0)
    uid = b.dist_unique_id()
    t0 = time.perf_counter()
    with pytest.raises(DeviceError, match="did not all join"):
        b.dist_init(0, 2, uid, timeout_ms=1500)
    waited = time.perf_counter() - t0
    assert 1.0 < waited < 20.0, waited
    x = DeviceTensor.from_host(b, np.arange(100, dtype=np.float32))
    np.testing.assert_array_equal(x.numpy(), np.arange(100, dtype=np.float32))
    # a one-rank job on the same context still initialises and reduces
    b.dist_init(0, 1, b.dist_unique_id(), timeout_ms=20000)
    b.dist_all_reduce_mean(x.storage.data, 100)
    b.dist_wait()
    np.testing.assert_array_equal(x.numpy(), np.arange(100, dtype=np.float32))
    b.close()
