"""Device-level behaviour of the library: a bounded wait that runs out is reported to the
host and leaves the context usable; a second GPU driven from the same process works."""

import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import assert_bit_equal

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bounded_wait_gives_up_and_is_reported():
    """Failure detection without a GPU fault: a wait nothing will ever satisfy runs into its
    (shortened) time limit, the kernel returns an error status the host reads, the next
    calls work. Runs in a child process because the limit is read from the environment once."""
    env = dict(os.environ, QX_B200_WAIT_LIMIT_MS="5")
    done = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "wait_timeout_worker.py")],
                          env=env, capture_output=True, text=True, timeout=300)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-4000:]
    assert "wait timeout ok" in done.stdout


def test_second_device_from_the_same_process(qx, wl):
    """Kernels that opt in to large dynamic shared memory need the opt-in on every device of
    the process, not once per process."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    results = []
    for device in (0, 1):
        torch.cuda.set_device(device)
        try:
            for fmt, (lo, hi) in ((0, (0.001, 0.02)), (1, (0.002, 0.04))):
                n, k = 512, 2048
                packed = wl.packed_blocks(fmt, n, k, lo, hi, seed=5)
                weights = qx.PackedWeights()
                assert weights.prepare(fmt, packed, n, k) == qx.OK, qx.last_error()
                status, y = weights.qgemm_prepacked(wl.activations_f32(1, k, seed=5), 1)
                assert status == qx.OK, f"device {device}: {qx.last_error()}"
                results.append(y)
                weights.reset()
            w, x, ws, xs = wl.w8a8_inputs(256, 256, 512, seed=5)
            status, y = qx.qgemm_w8a8(w, x, ws, xs, 256, 256, 512)
            assert status == qx.OK, f"device {device}: {qx.last_error()}"
            results.append(y)
        finally:
            torch.cuda.set_device(0)
    half = len(results) // 2
    for a, b in zip(results[:half], results[half:]):
        assert_bit_equal(a, b, "device 0 vs device 1")
