"""The allocation-free decode GEMV entry point (qx_qgemv_prepacked_noalloc_dev).

It exists for hosts that cannot call cudaMalloc while decoding (own memory pool, metered
allocations, no tolerance for the synchronisation an allocation brings): its scratch is a
fixed array inside the library image. The test calls it through the C ABI twice in a row
-- the second call meets the scratch contents the first one left behind -- and compares
both results with the regular entry point, which uses a growable workspace. The two share
the kernel and its summation order, so the outputs must agree bit for bit (and therefore
within the 1e-4 + 1e-5 * |ref| tolerance the other GEMV tests use). Collected last so that
a failure here cannot hide other results in a stop-at-first-failure run.
"""

import numpy as np
import pytest

from conftest import assert_bit_equal, assert_close_f32_path

pytestmark = pytest.mark.gpu
DIST = {0: (0.001, 0.02), 1: (0.002, 0.04)}


@pytest.mark.parametrize("fmt,n,k", [(1, 14336, 4096), (0, 4096, 4096), (1, 300, 1056)])
def test_no_alloc_matches_regular_entry_twice(qx, orc, wl, fmt, n, k):
    import torch
    packed = wl.packed_blocks(fmt, n, k, *DIST[fmt], seed=31)
    weights = qx.PackedWeights()
    assert weights.prepare(fmt, packed, n, k) == qx.OK, qx.last_error()
    xs = [wl.activations_f32(1, k, seed=40 + i) for i in range(2)]
    want = []
    for x in xs:
        y = torch.zeros((1, n), device="cuda")
        assert weights.qgemm_dev(torch.from_numpy(x).cuda(), y, 1, n) == qx.OK, qx.last_error()
        torch.cuda.synchronize()
        want.append(y.cpu().numpy()[0])
    got = []
    for x in xs:  # two calls in a row on the same stream, sharing the static scratch
        y = torch.full((n,), float("nan"), device="cuda")
        assert weights.qgemv_noalloc_dev(torch.from_numpy(x).cuda(), y) == qx.OK, qx.last_error()
        got.append(y)
    torch.cuda.synchronize()
    for i in range(2):
        result = got[i].cpu().numpy()
        assert_bit_equal(result, want[i], f"call {i}")
        _, ref = orc.qgemm(fmt, packed, xs[i], 1, n, k)
        assert_close_f32_path(result, ref[0], f"call {i} vs oracle")


def test_no_alloc_rejects_oversized_matrix(qx, wl):
    import torch
    fmt, n, k = 1, 131072, 4096  # needs 131072 * 16 * 4 B = 8 MiB of unit sums
    packed = np.zeros(n * (k // 32) * 18, np.uint8)
    weights = qx.PackedWeights()
    assert weights.prepare(fmt, packed, n, k) == qx.OK, qx.last_error()
    x = torch.zeros(k, device="cuda")
    y = torch.zeros(n, device="cuda")
    assert weights.qgemv_noalloc_dev(x, y) == qx.INVALID_SHAPE
    assert "static array" in qx.last_error()
    assert qx.lib.qx_qgemv_prepacked_noalloc_dev(None, None, None, None) == qx.INVALID_ARGUMENT
