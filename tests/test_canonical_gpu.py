"""Canonical prepared projections on the GPU (kInt8Symmetric / kInt4Symmetric with typed
input / output, bias and activation), through the C ABI, against the reference's golden
outputs, the oracle and a float64 evaluation of the same operands. The acceptance rule is
the reference's own (|a - e| <= 4e-5 * (1 + |e|),
tests/correctness/test_quant_projection_matrix.cpp:54-57); a 16-bit output may differ by one
unit of its type because it is one rounding of an f32 value that differs in its last bits."""

import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

INT4, INT8 = 0, 2
F32, F16, BF16 = 0, 1, 2
ROW, CHANNEL, GROUP = 2, 3, 4
HERE = os.path.dirname(os.path.abspath(__file__))
OUT_TOLERANCE = {F32: 4e-5, F16: 1.1e-3, BF16: 8.5e-3}


@pytest.fixture(scope="module")
def canon():
    return np.load(os.path.join(HERE, "golden", "golden_canonical.npz"))


def close(actual, expected, tolerance=4e-5):
    actual, expected = np.asarray(actual, np.float64), np.asarray(expected, np.float64)
    return bool(np.all(np.abs(actual - expected) <= tolerance * (1.0 + np.abs(expected))))


def agrees(actual, reference, exact, tolerance=4e-5):
    """Within the reference's tolerance of the reference's output once the reference's own
    distance from the exact value is discounted: its f32 sum (four sequential accumulators)
    drifts from the exact sum as K grows, and that drift is not this kernel's error."""
    actual, reference, exact = (np.asarray(a, np.float64) for a in (actual, reference, exact))
    slack = tolerance * (1.0 + np.abs(reference)) + np.abs(reference - exact)
    return bool(np.all(np.abs(actual - reference) <= slack))


def activation_f64(values, activation):
    from scipy.special import erf
    v = np.asarray(values, np.float64)
    if activation == 1:
        return 0.5 * v * (1.0 + erf(v * 0.7071067811865475))
    if activation == 2:
        return 0.5 * v * (1.0 + np.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))
    if activation == 3:
        return v / (1.0 + np.exp(-v))
    if activation == 4:
        return np.where(v > 0.0, v * v, 0.0)
    return v


def widen(values, storage):
    import torch
    if storage == F32:
        return np.asarray(values, np.float32)
    t = torch.from_numpy(np.ascontiguousarray(values).view(np.int16))
    t = t.view(torch.float16 if storage == F16 else torch.bfloat16)
    return t.float().numpy()


def prepared(qx, layout, mode, n, k, group, data, scales):
    w = qx.CanonicalWeights()
    view = qx.canonical_view(layout, mode, n, k, group, data, scales)
    assert w.prepare(view) == qx.OK, qx.last_error()
    return w


def test_golden_cases_of_the_reference(qx, orc, oracle_mod, canon):
    assert qx.lib.qx_canonical_gemm_variant().decode() == "sm100a_stream_fma_typed"
    for name in canon["names"]:
        name = str(name)
        layout, mode, n, k, group, m = (int(v) for v in canon[name + "/meta"])
        data = np.ascontiguousarray(canon[name + "/data"])
        scales = np.ascontiguousarray(canon[name + "/scales"])
        w = prepared(qx, layout, mode, n, k, group, data, scales)
        t = oracle_mod.CanonicalTensor(layout, mode, n, k, group, data, scales)
        before = qx.launch_count()
        for storage in (F32, F16, BF16):
            x = np.ascontiguousarray(canon[f"{name}/x{storage}"])
            status, y = w.qgemm_storage(x, storage, m)
            assert status == qx.OK, qx.last_error()
            exact = orc.canonical_gemm_f64(t, x, storage, m)
            assert close(y, exact), (name, storage, "f64")
            assert agrees(y, canon[f"{name}/y_x{storage}"], exact), (name, storage, "reference")
            assert agrees(y, orc.canonical_gemm(t, x, storage, m)[1], exact), (name, storage, "oracle")
            if name.startswith("t_"):  # the reference test's own shapes: its literal rule
                assert close(y, canon[f"{name}/y_x{storage}"]), (name, storage)
        # digits of the activations + projection per call; one kernel when a scale group
        # boundary falls inside 16 columns
        if layout == INT8 and mode != GROUP and m >= 5:
            expected = 9  # tensor-core route: row digits, W8A8 GEMM on the digit planes, combine
        else:
            expected = 6 if (group % 16 == 0 or mode != GROUP) else 3
        assert qx.launch_count() - before == expected
        x32 = np.ascontiguousarray(canon[name + "/x0"])
        bias = np.ascontiguousarray(canon[name + "/bias"])
        exact_sum = orc.canonical_gemm_f64(t, x32, F32, m) + bias.astype(np.float64)[None, :]
        for activation in range(5):
            exact = activation_f64(exact_sum, activation)
            for y_type in (F32, F16, BF16):
                status, y = w.qgemm_storage(x32, F32, m, y_type=y_type, bias=bias,
                                            activation=activation)
                assert status == qx.OK, qx.last_error()
                want = widen(canon[f"{name}/y_a{activation}_t{y_type}"], y_type)
                got = widen(y, y_type)
                assert close(got, exact, OUT_TOLERANCE[y_type]), (name, activation, y_type, "f64")
                assert agrees(got, want, exact, OUT_TOLERANCE[y_type]), (name, activation, y_type)
                if name.startswith("t_"):
                    assert close(got, want, OUT_TOLERANCE[y_type]), (name, activation, y_type)
        w.reset()


@pytest.mark.parametrize("case", [(INT8, 0, 4096, 4096, 1), (INT8, 128, 4096, 4096, 4),
                                  (INT4, 128, 4096, 4096, 1), (INT4, 32, 1024, 4096, 16),
                                  (INT8, 0, 1000, 1000, 5), (INT8, 8, 50, 200, 2),
                                  (INT4, 2, 37, 66, 3), (INT8, 0, 14336, 4096, 1)])
def test_seeded_shapes_against_float64(qx, orc, oracle_mod, case):
    layout, group, n, k, m = case
    rng = np.random.Generator(np.random.Philox(key=[n * 7 + k, layout * 100 + group + m]))
    weights = rng.standard_normal((n, k)).astype(np.float32)
    status, t = orc.quantize_canonical(layout, weights, n, k, group)
    assert status == 0
    w = prepared(qx, t.layout, t.scale_mode, n, k, t.group_size, t.data, t.scales)
    x = rng.standard_normal((m, k)).astype(np.float32)
    status, y = w.qgemm_storage(x, F32, m)
    assert status == qx.OK, qx.last_error()
    exact = orc.canonical_gemm_f64(t, x, F32, m)
    assert close(y, exact), case
    # not worse than twice the sequential f32 sum's own error
    if n * k * m <= 1 << 26:
        seq = orc.canonical_gemm(t, x, F32, m)[1]
        assert np.abs(y - exact).max() <= max(2 * np.abs(seq - exact).max(), 1e-6 * np.abs(exact).max())


def test_device_entry_with_typed_tensors(qx, orc, oracle_mod):
    import torch
    n, k, m = 512, 1024, 6
    rng = np.random.Generator(np.random.Philox(key=[11, 12]))
    status, t = orc.quantize_canonical(INT8, rng.standard_normal((n, k)).astype(np.float32), n, k, 0)
    w = prepared(qx, t.layout, CHANNEL, n, k, t.group_size, t.data, t.scales)
    x = torch.from_numpy(rng.standard_normal((m, k)).astype(np.float32)).cuda()
    bias = torch.from_numpy(rng.standard_normal(n).astype(np.float32)).cuda()
    for x_dtype, x_type in ((torch.float32, F32), (torch.float16, F16), (torch.bfloat16, BF16)):
        xt = x.to(x_dtype).contiguous()
        x_exact = xt.float().cpu().numpy()
        for y_dtype, y_type in ((torch.float32, F32), (torch.float16, F16), (torch.bfloat16, BF16)):
            y = torch.zeros((m, n), dtype=y_dtype, device="cuda")
            status = w.qgemm_storage_dev(xt, x_type, y, y_type, m, bias=bias, activation=qx.ACT_SILU)
            assert status == qx.OK, qx.last_error()
            torch.cuda.synchronize()
            want = orc.canonical_gemm(t, np.ascontiguousarray(x_exact), F32, m,
                                      bias=bias.cpu().numpy(), activation=3)[1]
            assert close(y.float().cpu().numpy(), want, OUT_TOLERANCE[y_type]), (x_type, y_type)
    assert qx.lib.qx_check_device_errors() == qx.OK


def test_batch_rows_do_not_depend_on_the_batch(qx, orc):
    # every token is summed in the same order whatever the token tile: rows of a batch are
    # bit-identical to the same rows run in another batch size with the same tile kind
    n, k = 300, 2080
    rng = np.random.Generator(np.random.Philox(key=[21, 22]))
    status, t = orc.quantize_canonical(INT4, rng.standard_normal((n, k)).astype(np.float32), n, k, 32)
    w = prepared(qx, t.layout, t.scale_mode, n, k, t.group_size, t.data, t.scales)
    x = rng.standard_normal((24, k)).astype(np.float32)
    full = w.qgemm_storage(x, F32, 24)[1]
    for m in (1, 3, 5, 8, 13):
        part = w.qgemm_storage(np.ascontiguousarray(x[:m]), F32, m)[1]
        assert np.array_equal(part.view(np.uint32), full[:m].view(np.uint32)), m


def test_entry_point_validation(qx, orc):
    n, k = 8, 64
    rng = np.random.default_rng(2)
    status, t = orc.quantize_canonical(INT8, rng.standard_normal((n, k)).astype(np.float32), n, k, 0)
    w = prepared(qx, t.layout, t.scale_mode, n, k, t.group_size, t.data, t.scales)
    x = np.zeros((2, k), np.float32)
    # order of qgemm_prepacked_storage_impl: activation, handle, shape, storage, pointers
    assert w.qgemm_storage(x, F32, 2, activation=9)[0] == 3
    assert w.qgemm_storage(x, F32, 0)[0] == 1
    assert w.qgemm_storage(x, F32, 2, x_count=5)[0] == 1
    assert w.qgemm_storage(x, F32, 2, y_count=5)[0] == 1
    assert w.qgemm_storage(x, 4, 2)[0] == 2
    assert w.qgemm_storage(x, F32, 2, y_type=3)[0] == 2
    assert w.qgemm_storage(None, F32, 2)[0] == 3
    assert w.qgemm_storage(x, F32, 2)[0] == 0


def test_smoothquant_import_feeds_both_routes(qx, orc, oracle_mod):
    # an imported SmoothQuant tensor runs as a weight-only projection (this file's kernel) and,
    # with its activation scale, as the exact W8A8 GEMM
    rows, cols, m = 96, 256, 4
    rng = np.random.Generator(np.random.Philox(key=[31, 32]))
    codes = rng.integers(-127, 128, rows * cols, dtype=np.int8)
    ws = rng.uniform(0.001, 0.02, rows).astype(np.float32)
    acts = np.array([0.05], np.float32)
    status, view, sums = qx.import_smoothquant_w8a8(codes, ws, acts, rows, cols)
    assert status == qx.OK
    w = qx.CanonicalWeights()
    assert w.prepare(view) == qx.OK, qx.last_error()
    x = rng.standard_normal((m, cols)).astype(np.float32)
    status, y = w.qgemm_storage(x, F32, m)
    assert status == qx.OK
    t = oracle_mod.CanonicalTensor(INT8, CHANNEL, rows, cols, cols, codes.view(np.uint8), ws)
    assert close(y, orc.canonical_gemm_f64(t, x, F32, m))
    xq = np.clip(np.rint(x / acts[0]), -127, 127).astype(np.int8)
    status, y8 = qx.qgemm_w8a8(codes.reshape(rows, cols), xq, ws, np.full(m, acts[0], np.float32),
                               m, rows, cols)
    assert status == qx.OK
    _, want, _ = orc.int8_gemm(codes.reshape(rows, cols), xq, ws, np.full(m, acts[0], np.float32),
                               m, rows, cols)
    assert np.array_equal(y8.view(np.uint32), np.asarray(want, np.float32).view(np.uint32))


# ---- kUInt4Affine, AWQ / GPTQ checkpoints, act-order ------------------------------------------

UINT4 = 1


def test_awq_gptq_checkpoints_through_import_prepare_and_projection(qx, orc, oracle_mod, canon):
    for name in canon["checkpoints"]:
        name = str(name)
        layout, mode, n, k, group, m, symmetric, v2 = (int(v) for v in canon[name + "/meta"])
        extra = {key: np.ascontiguousarray(canon[f"{name}/{key}"]) for key in ("group_index", "act_order")
                 if f"{name}/{key}" in canon}
        qweight, qzeros, qscales = (np.ascontiguousarray(canon[f"{name}/{key}"])
                                    for key in ("qweight", "qzeros", "qscales"))
        if "/awq_" in name:
            status, view, arrays = qx.import_awq_u4(qweight, qzeros, qscales, k, n, group)
        else:
            status, view, arrays = qx.import_gptq_u4(qweight, qzeros, qscales, k, n, group,
                                                     symmetric=bool(symmetric), v2=bool(v2), **extra)
        assert status == qx.OK, name
        w = qx.CanonicalWeights()
        assert w.prepare(view) == qx.OK, qx.last_error()
        zeros = canon[name + "/zeros"]
        t = oracle_mod.CanonicalTensor(layout, mode, n, k, group, canon[name + "/data"],
                                       canon[name + "/scales"], zeros if zeros.size else None,
                                       extra.get("group_index"), extra.get("act_order"))
        x = np.ascontiguousarray(canon[name + "/x0"])
        status, y = w.qgemm_storage(x, F32, m)
        assert status == qx.OK, qx.last_error()
        exact = orc.canonical_gemm_f64(t, x, F32, m)
        assert close(y, exact), (name, "f64")
        assert agrees(y, canon[name + "/y_x0"], exact), (name, "reference")
        # bf16 in, bias + SiLU, bf16 out
        xb = np.ascontiguousarray(canon[name + "/x2"])
        bias = np.ascontiguousarray(canon[name + "/bias"])
        status, yb = w.qgemm_storage(xb, BF16, m, y_type=BF16, bias=bias, activation=3)
        assert status == qx.OK, qx.last_error()
        exact_b = activation_f64(orc.canonical_gemm_f64(t, xb, BF16, m) + bias.astype(np.float64)[None, :], 3)
        assert close(widen(yb, BF16), exact_b, OUT_TOLERANCE[BF16]), (name, "bf16 f64")
        assert agrees(widen(yb, BF16), widen(canon[name + "/y_x2_silu_bf16"], BF16), exact_b,
                      OUT_TOLERANCE[BF16]), (name, "bf16 reference")
        w.reset()


@pytest.mark.parametrize("case", [(4096, 4096, 128, 1), (14336, 4096, 128, 1), (1000, 1056, 32, 5),
                                  (300, 2080, 16, 3), (64, 72, 8, 2), (96, 1024, 1024, 9)])
def test_affine_seeded_shapes_against_float64(qx, orc, oracle_mod, case):
    n, k, group, m = case
    rng = np.random.Generator(np.random.Philox(key=[n + k, group * 10 + m]))
    data = rng.integers(0, 256, n * k // 2, dtype=np.uint8)
    groups = k // group
    scales = rng.uniform(0.002, 0.03, n * groups).astype(np.float32)
    zeros = rng.integers(0, 16, n * groups).astype(np.float32)
    zeros[::7] += 0.5  # fractional zero points take the f32 branch
    t = oracle_mod.CanonicalTensor(UINT4, GROUP, n, k, group, data, scales, zeros)
    w = qx.CanonicalWeights()
    assert w.prepare(qx.canonical_view(UINT4, GROUP, n, k, group, data, scales, zeros=zeros)) == qx.OK, \
        qx.last_error()
    x = rng.standard_normal((m, k)).astype(np.float32)
    status, y = w.qgemm_storage(x, F32, m)
    assert status == qx.OK, qx.last_error()
    exact = orc.canonical_gemm_f64(t, x, F32, m)
    assert close(y, exact), case
    if n * k * m <= 1 << 25:
        seq = orc.canonical_gemm(t, x, F32, m)[1]
        assert np.abs(y - exact).max() <= max(2 * np.abs(seq - exact).max(), 2e-6 * np.abs(exact).max())


def test_affine_prepare_checks(qx):
    n, k, group = 4, 32, 16
    data, scales = np.zeros(n * k // 2, np.uint8), np.ones(n * 2, np.float32)
    zeros = np.ones(n * 2, np.float32)
    w = qx.CanonicalWeights()
    assert w.prepare(qx.canonical_view(UINT4, GROUP, n, k, group, data, scales, zeros=zeros)) == 0
    assert w.prepare(qx.canonical_view(UINT4, GROUP, n, k, group, data, scales)) == 1           # zero points missing
    assert w.prepare(qx.canonical_view(INT4, GROUP, n, k, group, data, scales, zeros=zeros)) == 1  # none expected
    order = np.arange(k, dtype=np.int32)
    assert w.prepare(qx.canonical_view(UINT4, GROUP, n, k, group, data, scales, zeros=zeros,
                                       act_order=order[:-1])) == 1
    order[0] = 1
    assert w.prepare(qx.canonical_view(UINT4, GROUP, n, k, group, data, scales, zeros=zeros,
                                       act_order=order)) == 3
    assert w.prepare(qx.canonical_view(UINT4, GROUP, n, k, group, data, scales, zeros=zeros,
                                       group_index=np.full(k, 2, np.int32))) == 3
    codes8 = np.zeros(n * k, np.uint8)
    assert w.prepare(qx.canonical_view(INT8, ROW, n, k, k, codes8, scales[:n],
                                       act_order=np.arange(k, dtype=np.int32))) == 3
    bad = zeros.copy()
    bad[1] = np.inf
    assert w.prepare(qx.canonical_view(UINT4, GROUP, n, k, group, data, scales, zeros=bad)) == 1


@pytest.mark.parametrize("case", [(4096, 4096, 64), (1000, 1008, 300), (257, 272, 33), (14336, 4096, 512)])
def test_int8_prefill_on_the_tensor_cores(qx, orc, oracle_mod, case):
    # five tokens or more of an int8 tensor with one scale per row: digit planes under a per-token
    # envelope through the W8A8 tensor-core GEMM (300 tokens = a full chunk of 256 and a short one)
    n, k, m = case
    rng = np.random.Generator(np.random.Philox(key=[n, k + m]))
    status, t = orc.quantize_canonical(INT8, rng.standard_normal((n, k)).astype(np.float32), n, k, 0)
    assert status == 0
    w = prepared(qx, t.layout, CHANNEL, n, k, t.group_size, t.data, t.scales)
    x = rng.standard_normal((m, k)).astype(np.float32)
    x[1] *= 1e-6   # a quiet token next to loud ones: the envelope is per token
    x[2, ::3] = 0.0
    bias = rng.standard_normal(n).astype(np.float32)
    before = qx.launch_count()
    status, y = w.qgemm_storage(x, F32, m)
    assert status == qx.OK, qx.last_error()
    assert qx.launch_count() - before >= 3
    # float64 on a sample of rows of the big case, on everything otherwise
    rows = slice(None) if n * k * m <= 1 << 28 else slice(0, 8)
    xs = np.ascontiguousarray(x[rows])
    ms = xs.shape[0]
    exact = orc.canonical_gemm_f64(t, xs, F32, ms)
    assert close(y[rows], exact), case
    # typed: bf16 in, bias + tanh-GELU, f16 out
    import torch
    xb = np.ascontiguousarray(torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16))
    status, yt = w.qgemm_storage(xb, BF16, m, y_type=F16, bias=bias, activation=2)
    assert status == qx.OK, qx.last_error()
    exact_t = activation_f64(orc.canonical_gemm_f64(t, np.ascontiguousarray(xb[rows]), BF16, ms) +
                             bias.astype(np.float64)[None, :], 2)
    assert close(widen(yt, F16)[rows], exact_t, OUT_TOLERANCE[F16]), case
    assert qx.lib.qx_check_device_errors() == qx.OK
