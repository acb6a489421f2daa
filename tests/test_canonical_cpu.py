"""Canonical prepared projections (kInt8Symmetric / kInt4Symmetric), CPU side: the oracle's
restatement against golden vectors produced by the unmodified reference (and against the
reference library when it is built here), and the host-side SmoothQuant importer of the
product against the reference's importer golden row."""

import os

import numpy as np
import pytest

INT4, INT8 = 0, 2
F32, F16, BF16 = 0, 1, 2
ROW, CHANNEL, GROUP = 2, 3, 4
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def canon():
    return np.load(os.path.join(HERE, "golden", "golden_canonical.npz"))


def close(actual, expected, tolerance=4e-5):
    """The acceptance rule of the reference's own projection test
    (tests/correctness/test_quant_projection_matrix.cpp:54-57)."""
    actual, expected = np.asarray(actual, np.float64), np.asarray(expected, np.float64)
    return bool(np.all(np.abs(actual - expected) <= tolerance * (1.0 + np.abs(expected))))


def decode(values, storage, orc):
    if storage == F32:
        return np.asarray(values, np.float32)
    fn = orc.fp16_to_fp32 if storage == F16 else orc.bf16_to_float
    return np.array([fn(int(v)) for v in np.asarray(values).reshape(-1)],
                    np.float32).reshape(np.shape(values))


def tensor_of(oracle_mod, canon, name):
    layout, mode, n, k, group, m = (int(v) for v in canon[name + "/meta"])
    t = oracle_mod.CanonicalTensor(layout, mode, n, k, group, canon[name + "/data"],
                                   canon[name + "/scales"])
    return t, m


def test_quantiser_matches_reference_bits(orc, canon):
    # quantize_canonical of the reference made data and scales of every golden case
    checked = 0
    for name in canon["names"]:
        name = str(name)
        if name + "/w" not in canon:
            continue
        layout, mode, n, k, group, _ = (int(v) for v in canon[name + "/meta"])
        asked = 0 if (layout == INT8 and mode == ROW) else group
        status, t = orc.quantize_canonical(layout, np.ascontiguousarray(canon[name + "/w"]), n, k, asked)
        assert status == 0
        assert (t.scale_mode, t.group_size) == (mode, group)
        assert np.array_equal(t.data, canon[name + "/data"]), name
        assert np.array_equal(t.scales.view(np.uint32), canon[name + "/scales"].view(np.uint32)), name
        checked += 1
    assert checked >= 9


def test_oracle_projection_within_reference_tolerance(orc, oracle_mod, canon):
    for name in canon["names"]:
        name = str(name)
        t, m = tensor_of(oracle_mod, canon, name)
        for storage in (F32, F16, BF16):
            x = np.ascontiguousarray(canon[f"{name}/x{storage}"])
            status, y = orc.canonical_gemm(t, x, storage, m)
            assert status == 0
            assert close(y, canon[f"{name}/y_x{storage}"]), (name, storage)
            # both sit within the same distance of the exact sum
            exact = orc.canonical_gemm_f64(t, x, storage, m)
            assert close(y, exact) and close(canon[f"{name}/y_x{storage}"], exact)
        x32 = np.ascontiguousarray(canon[name + "/x0"])
        bias = np.ascontiguousarray(canon[name + "/bias"])
        for activation in range(5):
            for y_type in (F32, F16, BF16):
                status, y = orc.canonical_gemm(t, x32, F32, m, bias=bias, y_type=y_type,
                                               activation=activation)
                assert status == 0
                want = canon[f"{name}/y_a{activation}_t{y_type}"]
                # a 16-bit output is one rounding of a value that may differ in its last f32
                # bits: allow one unit of the output type on top of the f32 tolerance
                tolerance = 4e-5 if y_type == F32 else (1.1e-3 if y_type == F16 else 8.5e-3)
                assert close(decode(y, y_type, orc), decode(want, y_type, orc), tolerance), \
                    (name, activation, y_type)


def test_oracle_matches_reference_library(orc, ref, oracle_mod):
    rng = np.random.Generator(np.random.Philox(key=[77, 1]))
    for layout, group, n, k, m in ((INT8, 0, 19, 96, 4), (INT8, 32, 7, 256, 1), (INT4, 64, 11, 192, 6)):
        w = rng.standard_normal((n, k)).astype(np.float32)
        so, to = orc.quantize_canonical(layout, w, n, k, group)
        sr, tr = ref.quantize_canonical(layout, w, n, k, group)
        assert so == sr == 0
        assert np.array_equal(to.data, tr.data) and np.array_equal(to.scales, tr.scales)
        assert (to.scale_mode, to.group_size) == (tr.scale_mode, tr.group_size)
        x = rng.standard_normal((m, k)).astype(np.float32)
        bias = rng.standard_normal(n).astype(np.float32)
        for activation in range(5):
            s1, y1 = orc.canonical_gemm(to, x, F32, m, bias=bias, activation=activation)
            s2, y2 = ref.canonical_gemm(tr, x, F32, m, bias=bias, activation=activation)
            assert s1 == s2 == 0 and close(y1, y2)


def test_oracle_validation_order_matches_reference(orc, ref, oracle_mod):
    rng = np.random.default_rng(5)
    n, k = 4, 32
    t = oracle_mod.CanonicalTensor(INT8, ROW, n, k, k, rng.integers(0, 255, n * k, dtype=np.uint8),
                                   np.ones(n, np.float32))
    x = np.zeros((2, k), np.float32)

    assert orc.canonical_gemm(t, x, F32, 2)[0] == ref.canonical_gemm(t, x, F32, 2)[0] == 0
    # wrong element counts, unknown storage, unknown activation, m = 0
    for kw in (dict(x_count=5), dict(y_count=3), dict(y_type=7), dict(activation=9)):
        assert orc.canonical_gemm(t, x, F32, 2, **kw)[0] == ref.canonical_gemm(t, x, F32, 2, **kw)[0] != 0, kw
    assert orc.canonical_gemm(t, x, 5, 2)[0] == ref.canonical_gemm(t, x, 5, 2)[0] == 2
    assert orc.canonical_gemm(t, x, F32, 0)[0] == ref.canonical_gemm(t, x, F32, 0)[0] == 1
    # tensor-level failures: negative scale, wrong byte count, group size that does not divide
    bad = oracle_mod.CanonicalTensor(INT8, ROW, n, k, k, t.data, -np.ones(n, np.float32))
    assert orc.canonical_gemm(bad, x, F32, 2)[0] == ref.canonical_gemm(bad, x, F32, 2)[0] == 1
    bad = oracle_mod.CanonicalTensor(INT8, ROW, n, k, k, t.data[:-1], np.ones(n, np.float32))
    assert orc.canonical_gemm(bad, x, F32, 2)[0] == ref.canonical_gemm(bad, x, F32, 2)[0] == 1
    bad = oracle_mod.CanonicalTensor(INT8, GROUP, n, k, 5, t.data, np.ones(n, np.float32))
    assert orc.canonical_gemm(bad, x, F32, 2)[0] == ref.canonical_gemm(bad, x, F32, 2)[0] == 1
    # a tensor-wide scale: the count is checked first (one scale expected), then the mode
    bad = oracle_mod.CanonicalTensor(INT8, 1, n, k, k, t.data, np.ones(n, np.float32))
    assert orc.canonical_gemm(bad, x, F32, 2)[0] == ref.canonical_gemm(bad, x, F32, 2)[0] == 1
    bad = oracle_mod.CanonicalTensor(INT8, 1, n, k, k, t.data, np.ones(1, np.float32))
    assert orc.canonical_gemm(bad, x, F32, 2)[0] == ref.canonical_gemm(bad, x, F32, 2)[0] == 3


def test_smoothquant_import_golden_row(qx, orc, canon):
    # the reference's importer table: int8 codes pass through unchanged, one scale per
    # output channel, layout int8_symmetric
    assert str(canon["smoothquant/canonical_layout"]) == "int8_symmetric"
    assert str(canon["smoothquant/scale_mode"]) == "channel"
    weights = np.ascontiguousarray(canon["smoothquant/weights"])
    ws = np.array([canon["smoothquant/weight_scale"]], np.float32)
    acts = np.array([canon["smoothquant/activation_scale"]], np.float32)
    status, view, sums = qx.import_smoothquant_w8a8(weights, ws, acts, 1, 4)
    assert status == 0
    layout, mode, group = (int(v) for v in canon["smoothquant/imported_meta"])
    assert (view.layout, view.scale_mode, view.group_size) == (layout, mode, group) == (INT8, CHANNEL, 4)
    assert (view.rows, view.columns, view.data_bytes, view.scale_count) == (1, 4, 4, 1)
    got = np.ctypeslib.as_array((np.ctypeslib.ctypes.c_uint8 * 4).from_address(view.data))
    assert np.array_equal(got, canon["smoothquant/canonical_codes"])
    assert np.array_equal(got, canon["smoothquant/imported_data"])
    assert np.array_equal(sums, canon["smoothquant/imported_row_sums"])
    assert sums[0] == int(weights.astype(np.int32).sum())
    # the oracle's restatement of the same row sums
    status, osums = orc.import_smoothquant_row_sums(weights, ws, acts, 1, 4)
    assert status == 0 and np.array_equal(osums, sums)


def test_smoothquant_import_checks(qx, orc):
    rng = np.random.default_rng(3)
    rows, cols = 6, 40
    w = rng.integers(-128, 128, rows * cols, dtype=np.int8)
    ws = rng.random(rows).astype(np.float32)
    acts = np.array([0.1], np.float32)
    status, view, sums = qx.import_smoothquant_w8a8(w, ws, acts, rows, cols)
    assert status == 0
    assert np.array_equal(sums, w.reshape(rows, cols).astype(np.int32).sum(axis=1))
    assert np.array_equal(sums, orc.import_smoothquant_row_sums(w, ws, acts, rows, cols)[1])
    # supplied row sums are copied, not recomputed
    given = np.arange(rows, dtype=np.int32)
    assert np.array_equal(qx.import_smoothquant_w8a8(w, ws, acts, rows, cols, row_sums=given)[2], given)
    # statuses of the reference's checks (quant_import_ref.cpp:1053-1074)
    assert qx.import_smoothquant_w8a8(None, ws, acts, rows, cols)[0] == 3
    assert qx.import_smoothquant_w8a8(w, ws, acts, 0, cols)[0] == 3
    assert qx.import_smoothquant_w8a8(w[:-1], ws, acts, rows, cols)[0] == 1
    assert qx.import_smoothquant_w8a8(w, ws[:-1], acts, rows, cols)[0] == 1
    assert qx.import_smoothquant_w8a8(w, ws, acts, rows, cols, row_sums=given[:-1])[0] == 1
    bad = ws.copy()
    bad[2] = np.inf
    assert qx.import_smoothquant_w8a8(w, bad, acts, rows, cols)[0] == 1
    bad[2] = -1.0
    assert qx.import_smoothquant_w8a8(w, bad, acts, rows, cols)[0] == 1
    zp = np.zeros(2, np.int32)
    assert qx.import_smoothquant_w8a8(w, ws, acts, rows, cols, zero_points=zp)[0] == 1


def test_smoothquant_import_matches_reference_library(qx, ref):
    rng = np.random.default_rng(9)
    rows, cols = 5, 24
    w = rng.integers(-128, 128, rows * cols, dtype=np.int8)
    ws = rng.random(rows).astype(np.float32)
    acts = rng.random(3).astype(np.float32)
    zp = rng.integers(-5, 5, 3).astype(np.int32)
    s1, view, sums = qx.import_smoothquant_w8a8(w, ws, acts, rows, cols, zero_points=zp)
    s2, t, rsums = ref.import_smoothquant(w, ws, acts, rows, cols, zero_points=zp)
    assert s1 == s2 == 0
    assert (view.layout, view.scale_mode, view.group_size) == (t.layout, t.scale_mode, t.group_size)
    assert np.array_equal(sums, rsums)
    assert np.array_equal(t.data.view(np.int8), w)


def test_prepare_rejects_bad_tensors_without_a_device(qx):
    # argument and shape checks come before any device work
    n, k = 4, 32
    data, scales = np.zeros(n * k, np.uint8), np.ones(n, np.float32)
    w = qx.CanonicalWeights()
    assert w.prepare(qx.canonical_view(7, ROW, n, k, k, data, scales)) == 2
    assert w.prepare(qx.canonical_view(INT8, ROW, 0, k, k, data, scales)) == 1
    assert w.prepare(qx.canonical_view(INT8, ROW, n, k, 5, data, scales)) == 1
    assert w.prepare(qx.canonical_view(INT8, 1, n, k, k, data, scales)) == 1
    assert w.prepare(qx.canonical_view(INT8, 1, n, k, k, data, scales[:1])) == 3
    assert w.prepare(qx.canonical_view(INT8, ROW, n, k, k, data[:-1], scales)) == 1
    assert w.prepare(qx.canonical_view(INT4, GROUP, n, 33, 0, data, scales)) == 1
    assert w.prepare(qx.canonical_view(INT8, GROUP, n, k, 0, data, scales)) == 1
    assert w.prepare(qx.canonical_view(INT8, GROUP, n, k, 16, data, scales)) == 1
    assert w.prepare(qx.canonical_view(INT8, ROW, n, k, k, data, -scales)) == 1
    assert w.prepare(qx.canonical_view(INT8, ROW, n, k, k, None, scales, data_bytes=n * k)) == 3
    assert not w.ready()
    # entry points without a handle
    x = np.zeros(k, np.float32)
    assert qx.lib.qx_qgemm_prepacked_storage(None, x.ctypes.data, F32, k, x.ctypes.data, F32, n, 1) == 3
    assert qx.lib.qx_qgemm_prepacked_epilogue_storage(None, x.ctypes.data, F32, k, None, x.ctypes.data,
                                                      F32, n, 1, 9) == 3


# ---- AWQ / GPTQ importers and the affine layout -----------------------------------------------

UINT4 = 1


def _checkpoint(canon, name):
    meta = [int(v) for v in canon[name + "/meta"]]
    layout, mode, n, k, group, m, symmetric, v2 = meta
    extra = {key: np.ascontiguousarray(canon[f"{name}/{key}"]) for key in ("group_index", "act_order")
             if f"{name}/{key}" in canon}
    return dict(layout=layout, mode=mode, n=n, k=k, group=group, m=m, symmetric=bool(symmetric),
                v2=bool(v2), extra=extra, awq="/awq_" in name,
                qweight=np.ascontiguousarray(canon[name + "/qweight"]),
                qzeros=np.ascontiguousarray(canon[name + "/qzeros"]),
                qscales=np.ascontiguousarray(canon[name + "/qscales"]))


def _import(qx, c):
    if c["awq"]:
        return qx.import_awq_u4(c["qweight"], c["qzeros"], c["qscales"], c["k"], c["n"], c["group"])
    return qx.import_gptq_u4(c["qweight"], c["qzeros"], c["qscales"], c["k"], c["n"], c["group"],
                             symmetric=c["symmetric"], v2=c["v2"], **c["extra"])


def test_awq_gptq_importers_match_reference_bits(qx, canon):
    # the fragments of the reference's importer test, whose codes its golden table lists
    k = n = 8
    status, view, (data, scales, zeros) = qx.import_awq_u4(
        np.full(k, 0x76543210, np.uint32), np.array([0x33333333], np.uint32),
        np.full(n, 0.25, np.float32), k, n, 8)
    assert status == 0 and (view.layout, view.scale_mode, view.group_size) == (UINT4, GROUP, 8)
    assert np.array_equal(data, canon["import_table/awq_u4/group8_reverse_lane/codes"])
    assert np.array_equal(data, canon["fragment/awq/data"])
    assert np.array_equal(zeros, canon["fragment/awq/zeros"]) and np.all(zeros == 3.0)
    assert np.array_equal(scales, canon["fragment/awq/scales"])
    status, view, (data, scales, zeros) = qx.import_gptq_u4(
        np.full(n, 0x76543210, np.uint32), np.array([0x22222222], np.uint32),
        np.full(n, 0.5, np.float32), k, n, 8)
    assert status == 0 and view.layout == UINT4
    assert np.array_equal(data[:4], canon["import_table/gptq_u4/v1_asymmetric/codes"])
    assert np.array_equal(data, canon["fragment/gptq_v1/data"]) and np.all(zeros == 3.0)
    gi = np.array([1, 1, 1, 1, 0, 0, 0, 0], np.int32)
    ao = np.array([4, 5, 6, 7, 0, 1, 2, 3], np.int32)
    status, view, (data, scales, zeros) = qx.import_gptq_u4(
        np.full(n, 0x76543210, np.uint32), np.array([0x88888888] * 2, np.uint32),
        np.concatenate([np.full(n, 1.0, np.float32), np.full(n, 2.0, np.float32)]), k, n, 4,
        symmetric=True, v2=True, group_index=gi, act_order=ao)
    assert status == 0 and view.layout == INT4 and view.zero_point_count == 0
    assert (view.group_index_count, view.act_order_count) == (8, 8)
    assert np.array_equal(data, canon["fragment/gptq_v2_sym/data"])
    assert np.array_equal(scales, canon["fragment/gptq_v2_sym/scales"])
    # seeded checkpoints
    for name in canon["checkpoints"]:
        c = _checkpoint(canon, str(name))
        status, view, (data, scales, zeros) = _import(qx, c)
        assert status == 0, name
        assert (view.layout, view.scale_mode, view.group_size) == (c["layout"], c["mode"], c["group"])
        assert np.array_equal(data, canon[str(name) + "/data"]), name
        assert np.array_equal(scales.view(np.uint32), canon[str(name) + "/scales"].view(np.uint32))
        want_zeros = canon[str(name) + "/zeros"]
        assert view.zero_point_count == want_zeros.size
        if want_zeros.size:
            assert np.array_equal(zeros, want_zeros)


def test_awq_gptq_importer_checks(qx):
    k, n, group = 16, 8, 8
    qw = np.zeros(k * (n // 8), np.uint32)
    qz = np.zeros((k // group) * (n // 8), np.uint32)
    sc = np.ones((k // group) * n, np.float32)
    assert qx.import_awq_u4(qw, qz, sc, k, n, group)[0] == 0
    assert qx.import_awq_u4(None, qz, sc, k, n, group)[0] == 3
    assert qx.import_awq_u4(qw, qz, sc, k, 12, group)[0] == 3          # N not a multiple of 8
    assert qx.import_awq_u4(qw, qz, sc, k, n, 5)[0] == 3               # group does not divide K
    assert qx.import_awq_u4(qw[:-1], qz, sc, k, n, group)[0] == 1
    assert qx.import_awq_u4(qw, qz, sc[:-1], k, n, group)[0] == 1
    bad = sc.copy()
    bad[3] = np.nan
    assert qx.import_awq_u4(qw, qz, bad, k, n, group)[0] == 1
    gq = np.zeros((k // 8) * n, np.uint32)
    assert qx.import_gptq_u4(gq, qz, sc, k, n, group)[0] == 0
    assert qx.import_gptq_u4(gq, qz, sc, 12, n, 4)[0] == 3             # K not a multiple of 8
    assert qx.import_gptq_u4(gq[:-1], qz, sc, k, n, group)[0] == 1
    assert qx.import_gptq_u4(gq, qz, sc, k, n, group, group_index=np.zeros(3, np.int32))[0] == 1
    assert qx.import_gptq_u4(gq, qz, sc, k, n, group, act_order=np.zeros(k, np.int32))[0] == 3  # not a permutation
    assert qx.import_gptq_u4(gq, qz, sc, k, n, group, group_index=np.full(k, 9, np.int32))[0] == 3


def test_importers_match_reference_library(qx, ref):
    rng = np.random.default_rng(21)
    k, n, group = 64, 16, 16
    groups = k // group
    sc = rng.uniform(0.01, 0.1, groups * n).astype(np.float32)
    qz = rng.integers(0, 2 ** 32, groups * (n // 8), dtype=np.uint64).astype(np.uint32)
    qw = rng.integers(0, 2 ** 32, k * (n // 8), dtype=np.uint64).astype(np.uint32)
    s1, view, (data, scales, zeros) = qx.import_awq_u4(qw, qz, sc, k, n, group)
    s2, t = ref.import_awq_u4(qw, qz, sc, k, n, group)
    assert s1 == s2 == 0 and np.array_equal(data, t.data) and np.array_equal(zeros, t.zeros)
    gq = rng.integers(0, 2 ** 32, (k // 8) * n, dtype=np.uint64).astype(np.uint32)
    for symmetric in (False, True):
        for v2 in (False, True):
            s1, view, (data, scales, zeros) = qx.import_gptq_u4(gq, qz, sc, k, n, group, symmetric, v2)
            s2, t = ref.import_gptq_u4(gq, qz, sc, k, n, group, symmetric, v2)
            assert s1 == s2 == 0 and view.layout == t.layout
            assert np.array_equal(data, t.data) and np.array_equal(scales, t.scales)
            if not symmetric:
                assert np.array_equal(zeros, t.zeros)


def test_oracle_affine_and_act_order_within_reference_tolerance(orc, oracle_mod, canon):
    for name in canon["checkpoints"]:
        name = str(name)
        c = _checkpoint(canon, name)
        zeros = canon[name + "/zeros"]
        t = oracle_mod.CanonicalTensor(c["layout"], c["mode"], c["n"], c["k"], c["group"],
                                       canon[name + "/data"], canon[name + "/scales"],
                                       zeros if zeros.size else None, c["extra"].get("group_index"),
                                       c["extra"].get("act_order"))
        x = np.ascontiguousarray(canon[name + "/x0"])
        status, y = orc.canonical_gemm(t, x, F32, c["m"])
        assert status == 0
        exact = orc.canonical_gemm_f64(t, x, F32, c["m"])
        assert close(y, exact) and close(canon[name + "/y_x0"], exact), name
