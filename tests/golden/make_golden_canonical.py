"""Generates golden_canonical.npz by RUNNING THE UNMODIFIED REFERENCE
(oracle/_ref/libqx_ref.so): canonical kInt8Symmetric / kInt4Symmetric tensors made by the
reference's quantize_canonical, and the outputs of its qgemm_prepacked_epilogue_storage for
every storage type and activation; AWQ and GPTQ checkpoints (the fragments of the reference's
importer test and seeded ones: V1, V2, symmetric, act-order) imported by the reference's
import_awq_u4 / import_gptq_u4 and run through the same projection.

    python tests/golden/make_golden_canonical.py

Inputs follow the reference's own test (tests/correctness/test_quant_projection_matrix.cpp):
the make_values formula (:75-87), n = 5, k = 32, m in {1, 16, 128}, group sizes 16 (int8) and
32 (int4), bias = make_values(1, n, 7); plus larger seeded cases. The SmoothQuant row of the
reference's importer golden table (tests/testdata/quant_import_golden.tsv) is parsed from
that file and stored beside the importer's actual output.
"""

from __future__ import annotations

import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

import oracle  # noqa: E402

INT4, INT8 = 0, 2
F32, F16, BF16 = 0, 1, 2


def make_values(rows, columns, salt):
    r = np.arange(rows, dtype=np.int64)[:, None]
    c = np.arange(columns, dtype=np.int64)[None, :]
    code = (r * 29 + c * 17 + salt * 11) % 61
    return ((code - 30).astype(np.float32) / np.float32(13.0) +
            np.float32(0.03125) * ((r + salt) % 5).astype(np.float32)).astype(np.float32)


def encode(ref, values, storage):
    if storage == F32:
        return values.astype(np.float32)
    fn = ref.fp32_to_fp16 if storage == F16 else ref.float_to_bf16
    return np.array([fn(float(v)) for v in values.reshape(-1)], np.uint16).reshape(values.shape)


def main():
    oracle.build()
    ref = oracle.Reference()
    out = {}
    cases = []
    # the reference test's matrix
    for layout, group in ((INT8, 16), (INT4, 32), (INT8, 0)):
        for m in (1, 16, 128):
            cases.append(("t", layout, group, 5, 32, m, None))
    # larger seeded cases: ragged K chunks, rows not a multiple of the CTA tile
    for layout, group, n, k, m, seed in ((INT8, 0, 70, 1040, 3, 1), (INT8, 64, 33, 1536, 9, 2),
                                         (INT4, 32, 70, 1056, 3, 3), (INT4, 128, 40, 1152, 9, 4),
                                         (INT8, 8, 12, 72, 2, 5), (INT4, 2, 9, 34, 2, 6)):
        cases.append(("s", layout, group, n, k, m, seed))
    names = []
    for kind, layout, group, n, k, m, seed in cases:
        if kind == "t":
            w, x, bias = make_values(n, k, 1), make_values(m, k, 3), make_values(1, n, 7).reshape(-1)
        else:
            rng = np.random.Generator(np.random.Philox(key=[seed, 4242]))
            w = rng.standard_normal((n, k)).astype(np.float32)
            x = rng.standard_normal((m, k)).astype(np.float32)
            bias = rng.standard_normal(n).astype(np.float32)
        status, t = ref.quantize_canonical(layout, np.ascontiguousarray(w), n, k, group)
        assert status == 0, (layout, group, n, k, status)
        name = f"{kind}_l{layout}_g{group}_n{n}_k{k}_m{m}"
        names.append(name)
        if w.size <= 4096:
            out[name + "/w"] = w  # small cases also pin the quantiser
        out[name + "/meta"] = np.array([layout, t.scale_mode, n, k, t.group_size, m], np.int64)
        out[name + "/data"] = t.data
        out[name + "/scales"] = t.scales
        out[name + "/bias"] = bias
        for storage in (F32, F16, BF16):
            xe = encode(ref, x, storage)
            out[f"{name}/x{storage}"] = xe
            status, y = ref.canonical_gemm(t, np.ascontiguousarray(xe), storage, m)
            assert status == 0
            out[f"{name}/y_x{storage}"] = y
        # epilogues on f32 input: every activation with bias, into every output type
        x32 = np.ascontiguousarray(x)
        for activation in range(5):
            for y_type in (F32, F16, BF16):
                status, y = ref.canonical_gemm(t, x32, F32, m, bias=bias, y_type=y_type,
                                               activation=activation)
                assert status == 0
                out[f"{name}/y_a{activation}_t{y_type}"] = y
    out["names"] = np.array(names)

    # SmoothQuant row of the reference's importer golden table
    ref_root = oracle.reference_root()
    with open(os.path.join(ref_root, "tests", "testdata", "quant_import_golden.tsv")) as f:
        rows = [line.rstrip("\n").split("\t") for line in f]
    row = next(r for r in rows if r[0] == "smoothquant_w8a8")
    source = dict(item.split("=") for item in row[2].split(";"))
    meta = dict(item.split("=") for item in row[5].split(";"))
    weights = np.array([int(h, 16) for h in source["weights_i8"].split(",")], np.uint8).view(np.int8)
    out["smoothquant/weights"] = weights
    out["smoothquant/weight_scale"] = np.float32(source["weight_scale"])
    out["smoothquant/activation_scale"] = np.float32(source["activation_scale"])
    out["smoothquant/canonical_layout"] = np.array(row[3])
    out["smoothquant/canonical_codes"] = np.frombuffer(bytes.fromhex(row[4]), np.uint8)
    out["smoothquant/scale_mode"] = np.array(meta["scale_mode"])
    # and what the importer itself returns for that source, as one row of four columns
    status, t, sums = ref.import_smoothquant(
        weights, np.array([source["weight_scale"]], np.float32),
        np.array([source["activation_scale"]], np.float32), 1, 4)
    assert status == 0
    out["smoothquant/imported_meta"] = np.array([t.layout, t.scale_mode, t.group_size], np.int64)
    out["smoothquant/imported_data"] = t.data
    out["smoothquant/imported_row_sums"] = sums
    # ---- AWQ / GPTQ: the fragments of the reference's importer test and table
    # (tests/correctness/test_quant_import.cpp:148-247, rows awq_u4 / gptq_u4 of the .tsv), and
    # seeded checkpoints run through the reference's projection
    for row_name in ("awq_u4", "gptq_u4"):
        for r in rows:
            if r[0] == row_name:
                out[f"import_table/{r[0]}/{r[1]}/codes"] = np.frombuffer(bytes.fromhex(r[4]), np.uint8)
    k = n = 8
    frag = {}
    frag["awq"] = ref.import_awq_u4(np.full(k, 0x76543210, np.uint32), np.array([0x33333333], np.uint32),
                                    np.full(n, 0.25, np.float32), k, n, 8)
    frag["gptq_v1"] = ref.import_gptq_u4(np.full(n, 0x76543210, np.uint32), np.array([0x22222222], np.uint32),
                                         np.full(n, 0.5, np.float32), k, n, 8)
    gi = np.array([1, 1, 1, 1, 0, 0, 0, 0], np.int32)
    ao = np.array([4, 5, 6, 7, 0, 1, 2, 3], np.int32)
    frag["gptq_v2_sym"] = ref.import_gptq_u4(
        np.full(n, 0x76543210, np.uint32), np.array([0x88888888] * 2, np.uint32),
        np.concatenate([np.full(n, 1.0, np.float32), np.full(n, 2.0, np.float32)]), k, n, 4,
        symmetric=True, v2=True, group_index=gi, act_order=ao)
    for name, (status, t) in frag.items():
        assert status == 0, name
        out[f"fragment/{name}/meta"] = np.array([t.layout, t.scale_mode, t.group_size], np.int64)
        out[f"fragment/{name}/data"] = t.data
        out[f"fragment/{name}/scales"] = t.scales
        out[f"fragment/{name}/zeros"] = np.zeros(0, np.float32) if t.zeros is None else t.zeros

    seeded = []
    for kind, k, n, group, m, seed in (("awq", 256, 64, 64, 3, 1), ("gptq_v1", 512, 40, 128, 5, 2),
                                      ("gptq_v2", 1024, 24, 32, 2, 3), ("gptq_sym_order", 128, 16, 32, 3, 4),
                                      ("gptq_order", 256, 16, 64, 2, 5)):
        rng = np.random.Generator(np.random.Philox(key=[seed, 777]))
        groups = k // group
        scales = rng.uniform(0.005, 0.05, groups * n).astype(np.float32)
        qzeros = rng.integers(0, 2 ** 32, groups * (n // 8), dtype=np.uint64).astype(np.uint32)
        name = f"checkpoint/{kind}_k{k}_n{n}_g{group}_m{m}"
        if kind == "awq":
            qweight = rng.integers(0, 2 ** 32, k * (n // 8), dtype=np.uint64).astype(np.uint32)
            status, t = ref.import_awq_u4(qweight, qzeros, scales, k, n, group)
            extra = {}
        else:
            qweight = rng.integers(0, 2 ** 32, (k // 8) * n, dtype=np.uint64).astype(np.uint32)
            extra = {}
            if "order" in kind:
                # act-order checkpoint: a permutation of the columns; packed column i belongs to
                # the group of the logical column it came from
                order = rng.permutation(k).astype(np.int32)
                extra = {"act_order": order, "group_index": (order // group).astype(np.int32)}
            status, t = ref.import_gptq_u4(qweight, qzeros, scales, k, n, group,
                                           symmetric="sym" in kind, v2=kind != "gptq_v1", **extra)
        assert status == 0, (kind, status)
        seeded.append(name)
        out[name + "/qweight"], out[name + "/qzeros"], out[name + "/qscales"] = qweight, qzeros, scales
        for key, value in extra.items():
            out[f"{name}/{key}"] = value
        out[name + "/meta"] = np.array([t.layout, t.scale_mode, n, k, t.group_size, m,
                                        int("sym" in kind), int(kind != "gptq_v1")], np.int64)
        out[name + "/data"], out[name + "/scales"] = t.data, t.scales
        out[name + "/zeros"] = np.zeros(0, np.float32) if t.zeros is None else t.zeros
        x = rng.standard_normal((m, k)).astype(np.float32)
        bias = rng.standard_normal(n).astype(np.float32)
        out[name + "/x0"], out[name + "/bias"] = x, bias
        status, y = ref.canonical_gemm_ex(t, x, F32, m)
        assert status == 0
        out[name + "/y_x0"] = y
        xb = encode(ref, x, BF16)
        out[name + "/x2"] = xb
        status, y = ref.canonical_gemm_ex(t, np.ascontiguousarray(xb), BF16, m, bias=bias, y_type=BF16,
                                          activation=3)
        assert status == 0
        out[name + "/y_x2_silu_bf16"] = y
    out["checkpoints"] = np.array(seeded)
    np.savez_compressed(os.path.join(HERE, "golden_canonical.npz"), **out)
    print("wrote golden_canonical.npz:", len(names), "cases")


if __name__ == "__main__":
    main()
