"""4-bit prefill GEMM (q4_0 weights x bf16 activations, f32 out) through the C ABI, against
the oracle's f32 path on the same inputs (qgemm = M independent GEMVs,
kernels/quantization/qgemm_ref.cpp:156-162, with the bf16 -> f32 widening of
kernels/utils/float_storage_ref.cpp:195-200).

Tolerance of this path as the benchmark definition states it: 1e-2 relative to the
reference's f32 result; outputs near zero are compared against 1e-2 of their row's rms.
The kernel's own error is far smaller (fp16 weights d * (nibble - 8), exact products, f32
sums), which the rms bound below pins.
"""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

Q4_0 = 1


def _run(qx, wl, packed, xb, n, k, m):
    import torch
    weights = qx.PackedWeights()
    assert weights.prepare(Q4_0, packed, n, k) == qx.OK, qx.last_error()
    y = torch.full((m, n), -7.0, device="cuda")
    x_dev = torch.from_numpy(xb.view(np.int16)).cuda()
    assert weights.qgemm_bf16_dev(x_dev, y, m) == qx.OK, qx.last_error()
    torch.cuda.synchronize()
    return y.cpu().numpy()


def _check(got, ref):
    rms = np.sqrt((ref.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    assert np.all(np.abs(got - ref) <= 1e-2 * np.abs(ref) + 1e-2 * rms)
    err_rms = np.sqrt(((got - ref).astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    assert np.all(err_rms <= 1e-3 * rms + 1e-30), float((err_rms / (rms + 1e-30)).max())


@pytest.mark.parametrize("n,k,m", [(256, 1024, 80), (384, 2048, 300), (200, 544, 64), (128, 256, 257)])
def test_prefill_matches_oracle(qx, orc, wl, n, k, m):
    packed = wl.packed_blocks(Q4_0, n, k, 0.002, 0.04, seed=n + k)
    xb = wl.to_bf16_bits(wl.activations_f32(m, k, seed=m))
    got = _run(qx, wl, packed, xb, n, k, m)
    _, ref = orc.qgemm(Q4_0, packed, wl.bf16_bits_to_f32(xb), m, n, k)
    _check(got, ref)


def test_prefill_row_scaling_and_non_finite_rows(qx, orc, wl):
    """Rows of very different magnitude keep their relative accuracy (the fp16 staging uses an
    exact power-of-two scale per row); a row with a NaN gives NaNs in that row only."""
    n, k, m = 256, 1024, 96
    packed = wl.packed_blocks(Q4_0, n, k, 0.002, 0.04, seed=5)
    x = wl.activations_f32(m, k, seed=6)
    x[3] *= 3.0e7
    x[4] *= 1.0e-20
    x[5] = 0.0
    x[7, 100] = np.nan
    xb = wl.to_bf16_bits(np.nan_to_num(x, nan=0.0))
    xb[7, 100] = 0x7FC0
    got = _run(qx, wl, packed, xb, n, k, m)
    xf = wl.bf16_bits_to_f32(xb)
    finite_rows = [r for r in range(m) if r != 7]
    _, ref = orc.qgemm(Q4_0, packed, xf[finite_rows].copy(), len(finite_rows), n, k)
    _check(got[finite_rows], ref)
    assert np.all(got[5] == 0.0)
    assert np.all(np.isnan(got[7]))


def test_prefill_full_shape_subset(qx, orc, wl):
    """The benchmark shape's weight width and depth at a reduced token count, checked on a
    seeded subset of output channels (every channel is an independent GEMV)."""
    c = wl.CONFIGS["cfg4_q4_0_prefill"]
    n, k, m = 2048, c["k"], 320
    packed = wl.packed_blocks(Q4_0, n, k, c["d_lo"], c["d_hi"], seed=0)
    xb = wl.to_bf16_bits(wl.activations_f32(m, k, seed=4))
    got = _run(qx, wl, packed, xb, n, k, m)
    rows = np.random.default_rng(0).choice(n, 16, replace=False)
    sub = packed.reshape(n, -1)[rows].reshape(-1)
    _, ref = orc.qgemm(Q4_0, sub, wl.bf16_bits_to_f32(xb), m, len(rows), k)
    _check(got[:, rows], ref)


def test_prefill_full_config(qx, orc, wl):
    """The prefill configuration at its full shape (28672 x 8192 q4_0 weights, 2048 bf16
    tokens): 64 seeded output channels x all 2048 tokens against the reference's f32 path on
    the same inputs (every channel is an independent GEMV), at the stated 1e-2 bound."""
    import torch
    c = wl.CONFIGS["cfg4_q4_0_prefill"]
    n, k, m = c["n"], c["k"], c["m"]
    packed = wl.packed_blocks(Q4_0, n, k, c["d_lo"], c["d_hi"], seed=0)
    xb = wl.to_bf16_bits(wl.activations_f32(m, k, seed=4))
    weights = qx.PackedWeights()
    assert weights.prepare(Q4_0, packed, n, k) == qx.OK, qx.last_error()
    y = torch.full((m, n), -7.0, device="cuda")
    x_dev = torch.from_numpy(xb.view(np.int16)).cuda()
    assert weights.qgemm_bf16_dev(x_dev, y, m) == qx.OK, qx.last_error()
    torch.cuda.synchronize()
    rows = np.sort(np.random.default_rng(4).choice(n, 64, replace=False))
    # first and last channel tile, and the tile boundaries in between, are always included
    rows[:4] = (0, 127, 128, n - 1)
    rows = np.unique(rows)
    got = y[:, torch.from_numpy(rows).cuda()].cpu().numpy()
    sub = packed.reshape(n, -1)[rows].reshape(-1).copy()
    _, ref = orc.qgemm(Q4_0, sub, wl.bf16_bits_to_f32(xb), m, len(rows), k)
    _check(got, ref)
    assert qx.lib.qx_check_device_errors() == qx.OK, qx.last_error()
