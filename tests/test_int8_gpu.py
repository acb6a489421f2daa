"""W8A8 int8 GEMM: exact f32 equality with float(int dot) * ws * as, as the reference's own
test demands (tests/correctness/test_int8_gemm.cpp:60-72), and bit-exact int32 accumulators."""

import numpy as np
import pytest

from conftest import assert_bit_equal

pytestmark = pytest.mark.gpu


def test_reference_ladder_exact(qx, orc, golden, gold_inputs):
    """M,N in 1..5, K in {1,15,16,17,63,64,65,100,1408}, full int8 domain with a forced -128."""
    sizes = [1, 15, 16, 17, 63, 64, 65, 100, 1408]
    for m in range(1, 6):
        for n in range(1, 6):
            for k in sizes:
                w, x, ws, xs, row_sum, zp = gold_inputs.int8_inputs(m, n, k)
                for asym in (False, True):
                    status, y = qx.int8_gemm(w, x, ws, xs, m, n, k, row_sum if asym else None,
                                             zp if asym else None, asym)
                    assert status == qx.OK, qx.last_error()
                    _, ref, _ = orc.int8_gemm(w, x, ws, xs, m, n, k, row_sum, zp, asym)
                    assert_bit_equal(y, ref, f"int8 {m}x{n}x{k} asym={asym}")
    for m, n, k in gold_inputs.INT8_SHAPES:
        w, x, ws, xs, row_sum, zp = gold_inputs.int8_inputs(m, n, k)
        _, y = qx.int8_gemm(w, x, ws, xs, m, n, k)
        assert_bit_equal(y, golden["default"][f"int8_{m}x{n}x{k}_y"], f"golden {m}x{n}x{k}")
        _, y = qx.int8_gemm(w, x, ws, xs, m, n, k, row_sum, zp, True)
        assert_bit_equal(y, golden["default"][f"int8_{m}x{n}x{k}_y_azp"], f"golden azp {m}x{n}x{k}")


def test_hand_case(qx):
    # tests/correctness/test_sibling_entrypoints.cpp:270-280
    w8 = np.array([[1, 2, -1, 3], [-2, 1, 0, 2]], np.int8)
    x8 = np.array([[2, -1, 3, 1]], np.int8)
    ws, xs = np.array([0.5, 0.25], np.float32), np.array([2.0], np.float32)
    s1, named = qx.qgemm_w8a8(w8, x8, ws, xs, 1, 2, 4)
    s2, generic = qx.int8_gemm(w8, x8, ws, xs, 1, 2, 4)
    assert s1 == s2 == qx.OK
    assert named.tolist() == generic.tolist() == [[0.0, -1.5]]


@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 384, 512), (512, 1024, 4096),
                                   (300, 200, 1040), (33, 130, 4096), (640, 256, 144),
                                   (1, 4096, 4096), (2048, 128, 256)])
def test_tensor_core_shapes_exact(qx, orc, wl, shape):
    import torch
    m, n, k = shape
    w, x, ws, xs = wl.w8a8_inputs(m, n, k, seed=m + n + k)
    x.reshape(-1)[::97] = -128  # the full int8 domain is legal input
    w.reshape(-1)[::101] = -128
    dev = [torch.from_numpy(a).cuda() for a in (w, x, ws, xs)]
    y = torch.zeros((m, n), device="cuda")
    acc = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    assert qx.int8_gemm_dev(*dev, y, m, n, k, acc=acc) == qx.OK, qx.last_error()
    torch.cuda.synchronize()
    want_acc = x.astype(np.int64) @ w.astype(np.int64).T
    assert np.array_equal(acc.cpu().numpy().astype(np.int64), want_acc), "int32 accumulators"
    want = (want_acc.astype(np.float32) * ws[None, :]) * xs[:, None]
    assert_bit_equal(y.cpu().numpy(), want, f"scaled output {shape}")
    rows = np.linspace(0, m - 1, min(m, 5)).astype(int)
    _, ref, _ = orc.int8_gemm(w, x[rows].copy(), ws, xs[rows].copy(), len(rows), n, k)
    assert_bit_equal(y.cpu().numpy()[rows], ref, "oracle rows")


def test_full_prefill_config(qx, wl):
    """cfg2 at full size: sampled exact outputs + two checksum-of-sums identities that hold
    for every accumulator: sum_o acc[r,o] = X[r,:].colsum(W) and sum_r acc[r,o] = W[o,:].colsum(X)."""
    import torch
    c = wl.CONFIGS["cfg2_w8a8_gemm"]
    m, n, k = c["m"], c["n"], c["k"]
    w, x, ws, xs = wl.w8a8_inputs(m, n, k, seed=0)
    dev = [torch.from_numpy(a).cuda() for a in (w, x, ws, xs)]
    y = torch.zeros((m, n), device="cuda")
    acc = torch.zeros((m, n), dtype=torch.int32, device="cuda")
    assert qx.int8_gemm_dev(*dev, y, m, n, k, acc=acc, check_scales=True) == qx.OK, qx.last_error()
    torch.cuda.synchronize()
    acc_h = acc.cpu().numpy().astype(np.int64)
    assert np.array_equal(acc_h.sum(axis=1), x.astype(np.int64) @ w.astype(np.int64).sum(axis=0))
    assert np.array_equal(acc_h.sum(axis=0), w.astype(np.int64) @ x.astype(np.int64).sum(axis=0))
    rng = np.random.default_rng(0)
    rows, cols = rng.choice(m, 48, replace=False), rng.choice(n, 512, replace=False)
    sub = x[rows].astype(np.int64) @ w[cols].astype(np.int64).T
    assert np.array_equal(acc_h[np.ix_(rows, cols)], sub)
    want = (acc_h.astype(np.float32) * ws[None, :]) * xs[:, None]
    assert_bit_equal(y.cpu().numpy(), want, "cfg2 scaled output")


def test_device_scale_check_and_stride(qx, wl):
    import torch
    m, n, k = 40, 96, 256
    w, x, ws, xs = wl.w8a8_inputs(m, n, k, seed=2)
    ws_bad = ws.copy()
    ws_bad[5] = np.inf
    dev = [torch.from_numpy(a).cuda() for a in (w, x, ws_bad, xs)]
    y = torch.full((m, n + 8), 3.0, device="cuda")
    assert qx.int8_gemm_dev(*dev, y, m, n, k, ldy=n + 8, check_scales=True) == qx.INVALID_ARGUMENT
    dev[2] = torch.from_numpy(ws).cuda()
    assert qx.int8_gemm_dev(*dev, y, m, n, k, ldy=n + 8, check_scales=True) == qx.OK
    torch.cuda.synchronize()
    got = y.cpu().numpy()
    want = ((x.astype(np.int64) @ w.astype(np.int64).T).astype(np.float32) * ws[None, :]) * xs[:, None]
    assert_bit_equal(got[:, :n], want)
    assert np.all(got[:, n:] == 3.0)


@pytest.mark.parametrize("shape,asym", [((512, 1024, 4096), False), ((300, 640, 2048), True),
                                        ((96, 2048, 1024), False)])
def test_stream_k_split_is_exact(qx, orc, wl, shape, asym, monkeypatch):
    """With the K-slab sequence cut into one contiguous range per SM, tiles are finished from
    int32 partial sums of several CTAs: same exact accumulators and f32 bits as whole tiles,
    and stable over repeated launches (the tile counters return to zero)."""
    m, n, k = shape
    w, x, ws, xs = wl.w8a8_inputs(m, n, k, seed=m + n)
    rng = np.random.default_rng(7)
    row_sum = w.astype(np.int64).sum(axis=1).astype(np.int32)
    zp = rng.integers(-20, 21, m).astype(np.int32)
    results = {}
    for mode in ("0", "1"):
        monkeypatch.setenv("QX_B200_INT8_STREAM_K", mode)
        for _ in range(2):
            status, y = qx.int8_gemm(w, x, ws, xs, m, n, k, row_sum if asym else None,
                                     zp if asym else None, asym)
            assert status == qx.OK, qx.last_error()
            results.setdefault(mode, []).append(y)
    _, ref, _ = orc.int8_gemm(w, x, ws, xs, m, n, k, row_sum, zp, asym)
    for mode, ys in results.items():
        for y in ys:
            assert_bit_equal(y, ref, f"stream_k={mode} {shape} asym={asym}")
