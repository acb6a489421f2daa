"""Generates the golden vectors in this directory by RUNNING THE UNMODIFIED REFERENCE
(oracle/_ref/libqx_ref.so, built by oracle/Makefile from the reference's own sources).

    python tests/golden/make_golden.py

Needs the reference sources (to build the library); the committed .npz files let the
tests run where they are absent. Inputs follow the reference's own tests: the xorshift32
generator and seeds of tests/correctness/test_qgemv.cpp:31-43, :143-175, :229-233, the
integer formulas of tests/correctness/test_w8a32_gemm.cpp:26-36, the hand case of
tests/correctness/test_sibling_entrypoints.cpp:270-280, plus seeded cases drawn with the
benchmark's value distributions.

Two files are written because the reference resolves its kernel variant once per
process: golden_default.npz (runtime-dispatched variants on the generating host) and
golden_forced_ref.npz (QUIXICORE_CPU_*_VARIANT=ref, the portable kernels).
"""

from __future__ import annotations

import hashlib
import importlib.util
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

Q8_0, Q4_0 = 0, 1
Q8_LADDER = [(1, 32), (3, 64), (5, 96), (33, 512), (129, 2048)]
INT8_SHAPES = [(1, 1, 1), (2, 3, 15), (3, 2, 16), (4, 5, 17), (5, 4, 63), (1, 5, 64), (5, 1, 65),
               (3, 3, 100), (5, 5, 1408), (40, 72, 256)]
W8A32_KS = [1, 7, 8, 15, 16, 63, 64, 65, 100, 1408]
FP16_VALUES = [1.0, 0.5, 0.0, -0.0, 65504.0, 65519.996, 65520.0, 1e30, 2.0 ** -14, 2.0 ** -15,
               2.0 ** -24, 2.0 ** -25, -(2.0 ** -24), 0.0123456, 1e-3 / 127.0, 3.0e-5, 6.0e-8,
               5.96e-8 * 1.5, 0.1, -2.7182817, 1024.5, 2049.0]


def _workloads():
    spec = importlib.util.spec_from_file_location(
        "qx_workloads", os.path.join(ROOT, "quixicore-cpu_b200", "workloads.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def int8_inputs(m, n, k):
    rng = np.random.Generator(np.random.Philox(key=[m * 1000003 + n * 1009 + k, 99]))
    w = rng.integers(-128, 128, (n, k), dtype=np.int8)
    x = rng.integers(-128, 128, (m, k), dtype=np.int8)
    w.reshape(-1)[0] = -1
    x.reshape(-1)[0] = -128
    ws = (0.001 * np.arange(1, n + 1)).astype(np.float32)
    xs = (0.002 * np.arange(1, m + 1)).astype(np.float32)
    row_sum = w.astype(np.int32).sum(axis=1).astype(np.int32)
    zp = (np.arange(m) - 2).astype(np.int32)
    return w, x, ws, xs, row_sum, zp


def w8a32_inputs(m, n, k):
    i = np.arange(n * k, dtype=np.int64)
    w = ((i * 37 + 11) % 255 - 127).astype(np.int8).reshape(n, k)
    scales = (np.float32(0.001) * (np.arange(n) + 1).astype(np.float32)).astype(np.float32)
    j = np.arange(m * k, dtype=np.int64)
    x = (((j * 29 + 7) % 101 - 50).astype(np.float32) / np.float32(37.0)).reshape(m, k)
    return w, scales, x


def generate(out_path: str) -> None:
    import oracle as O
    wl = _workloads()
    ref = O.Reference()
    out = {}
    variants = ref.variants()
    for key, value in variants.items():
        out["variant_" + key] = np.array(value)

    out["fp16_values"] = np.array(FP16_VALUES, np.float32)
    out["fp16_bits"] = np.array([ref.fp32_to_fp16(float(v)) for v in np.array(FP16_VALUES, np.float32)],
                                np.uint16)
    out["fp16_all_to_f32"] = np.array([ref.fp16_to_fp32(h) for h in range(65536)],
                                      np.float32).view(np.uint32)
    out["bf16_bits"] = np.array([ref.float_to_bf16(float(v)) for v in np.array(FP16_VALUES, np.float32)],
                                np.uint16)

    # q8_0 ladder (test_qgemv.cpp:229-233)
    for n, k in Q8_LADDER:
        seed = (0x9E3779B9 ^ (n * 131 + k)) & 0xFFFFFFFF
        values = wl.xorshift_uniform(seed, n * k + k)
        w, x = values[:n * k].reshape(n, k).copy(), values[n * k:].copy()
        status, packed = ref.pack(Q8_0, w, n, k)
        assert status == 0
        _, y = ref.qgemv(Q8_0, packed, x, n, k)
        _, dq = ref.unpack(Q8_0, packed, n, k)
        tag = f"q8_{n}x{k}"
        out[tag + "_packed_sha"] = np.array(sha(packed))
        out[tag + "_unpacked_sha"] = np.array(sha(dq))
        out[tag + "_y"] = y
        if n * k <= 33 * 512:
            out[tag + "_packed"] = packed

    # q4_0 33x512 (test_qgemv.cpp:143-175)
    n, k = 33, 512
    values = wl.xorshift_uniform(0xD1B54A32, n * k + k)
    w, x = values[:n * k].reshape(n, k).copy(), values[n * k:].copy()
    status, packed = ref.pack(Q4_0, w, n, k)
    assert status == 0
    _, y = ref.qgemv(Q4_0, packed, x, n, k)
    _, dq = ref.unpack(Q4_0, packed, n, k)
    out["q4_33x512_packed"] = packed
    out["q4_33x512_unpacked_sha"] = np.array(sha(dq))
    out["q4_33x512_y"] = y

    # subnormal-scale block (test_qgemv.cpp:199-216)
    w = np.full((1, 32), 1e-3, np.float32)
    _, packed = ref.pack(Q8_0, w, 1, 32)
    _, y = ref.qgemv(Q8_0, packed, np.ones(32, np.float32), 1, 32)
    out["q8_subnormal_packed"] = packed
    out["q8_subnormal_y"] = y

    # benchmark-distribution cases, small
    for fmt, name, lo, hi in ((Q8_0, "q8", 0.001, 0.02), (Q4_0, "q4", 0.002, 0.04)):
        n, k, m = 48, 4096, 3
        packed = wl.packed_blocks(fmt, n, k, lo, hi, seed=21)
        x = wl.activations_f32(m, k, seed=21)
        _, y = ref.qgemm(fmt, packed, x, m, n, k)
        out[f"{name}_bench_{m}x{n}x{k}_y"] = y
        out[f"{name}_bench_{m}x{n}x{k}_packed_sha"] = np.array(sha(packed))

    # W8A8 (test_int8_gemm.cpp:23-83 ladder subset; test_sibling_entrypoints.cpp:270-280)
    for m, n, k in INT8_SHAPES:
        w, x, ws, xs, row_sum, zp = int8_inputs(m, n, k)
        _, y = ref.int8_gemm(w, x, ws, xs, m, n, k)
        _, y_azp = ref.int8_gemm(w, x, ws, xs, m, n, k, row_sum, zp, True)
        out[f"int8_{m}x{n}x{k}_y"] = y
        out[f"int8_{m}x{n}x{k}_y_azp"] = y_azp
    w8 = np.array([[1, 2, -1, 3], [-2, 1, 0, 2]], np.int8)
    x8 = np.array([[2, -1, 3, 1]], np.int8)
    _, y = ref.qgemm_w8a8(w8, x8, np.array([0.5, 0.25], np.float32), np.array([2.0], np.float32),
                          1, 2, 4)
    out["int8_hand_y"] = y

    # W8A32 (test_w8a32_gemm.cpp:26-36, :86-88)
    for k in W8A32_KS:
        w, scales, x = w8a32_inputs(5, 5, k)
        _, y = ref.qgemm_w8a32(w, scales, x, 5, 5, k)
        out[f"w8a32_5x5x{k}_y"] = y

    # panel layout (src/memory/packed_weights.cpp:253-266), explicit 4-row layout = enum 2
    for fmt, name, lo, hi in ((Q8_0, "q8", 0.001, 0.02), (Q4_0, "q4", 0.002, 0.04)):
        rows, cols = 6, 96
        packed = wl.packed_blocks(fmt, rows, cols, lo, hi, seed=5)
        status, handle = ref.prepacked(fmt, packed, rows, cols, layout=2)
        assert status == 0
        out[f"panel_{name}_6x96_tile4"] = ref.prepacked_panel(handle)
        x = wl.activations_f32(70, cols, seed=5)
        _, y = ref.qgemm_prepacked(handle, x, 70, rows)
        out[f"prepacked_{name}_70x6x96_y"] = y
        ref.prepacked_destroy(handle)

    # ---- callers either side of the GEMV ------------------------------------------------
    # qgemv_w8a8 (block-quantised int8 activations) and the fused decode projections
    for fmt, name, lo, hi in ((Q8_0, "q8", 0.001, 0.02), (Q4_0, "q4", 0.002, 0.04)):
        n, k = 40, 1024
        packed = wl.packed_blocks(fmt, n, k, lo, hi, seed=31)
        gate_w = wl.packed_blocks(fmt, n, k, lo, hi, seed=32)
        x = wl.activations_f32(1, k, seed=31)[0].copy()
        out[f"w8a8_{name}_variant"] = np.array(ref.lib.qxref_qgemv_w8a8_variant(fmt).decode())
        _, y = ref.qgemv_w8a8(fmt, packed, x, n, k)
        out[f"w8a8_{name}_{n}x{k}_y"] = y
        _, up, gate = ref.up_gate(fmt, packed, gate_w, x, n, k)
        out[f"upgate_{name}_{n}x{k}_up"], out[f"upgate_{name}_{n}x{k}_gate"] = up, gate
        for gelu in (1, 0):
            _, act = ref.up_gate_activation(fmt, packed, gate_w, x, n, k, bool(gelu))
            out[f"upgate_{name}_{n}x{k}_act{gelu}"] = act
        kv = 24
        wk_ = wl.packed_blocks(fmt, kv, k, lo, hi, seed=33)
        wv_ = wl.packed_blocks(fmt, kv, k, lo, hi, seed=34)
        _, q, k_out, v_out = ref.qkv(fmt, packed, wk_, wv_, x, n, kv, k)
        out[f"qkv_{name}_q"], out[f"qkv_{name}_k"], out[f"qkv_{name}_v"] = q, k_out, v_out

    # quantize_int8 (kernels/quantization/quantization_ref.cpp:143-168)
    xq = wl.activations_f32(5, 192, seed=41)
    xq[1] = 0.0
    xq[2, 7] = 1e-30
    for group in (0, 32, 64):
        _, codes, scales = ref.quantize_int8(xq, 5, 192, group)
        out[f"quant_int8_g{group}_codes"], out[f"quant_int8_g{group}_scales"] = codes, scales

    # compact int4 rows: authoring, f32 GEMM, W4A8 (tests/correctness/test_lowbit_w8a8.cpp)
    out["lowbit_variant"] = np.array(ref.lib.qxref_lowbit_gemm_variant(2).decode())
    out["lowbit_w8a8_variant"] = np.array(ref.lib.qxref_lowbit_gemm_w8a8_variant().decode())
    for fmt, group, n, k, m in ((2, 0, 19, 200, 3), (3, 64, 17, 256, 2), (2, 0, 9, 33, 4)):
        rng = np.random.Generator(np.random.Philox(key=[fmt * 100 + k, 7]))
        w = (rng.integers(-1000, 1001, (n, k)).astype(np.float32) / np.float32(1000.0)) * np.float32(0.2)
        x = rng.integers(-2000, 2001, (m, k)).astype(np.float32) / np.float32(500.0)
        _, packed, scales = ref.lowbit_pack(fmt, w, n, k, group)
        tag = f"lowbit_f{fmt}_{m}x{n}x{k}"
        out[tag + "_packed"], out[tag + "_scales"] = packed, scales
        _, dq = ref.lowbit_unpack(fmt, packed, scales, n, k, group)
        out[tag + "_unpacked_sha"] = np.array(sha(dq))
        _, y = ref.lowbit_gemm(fmt, packed, scales, x, m, n, k, group)
        out[tag + "_y"] = y
        if fmt == 2:
            _, y8 = ref.lowbit_gemm_w8a8(packed, scales.reshape(-1), x, m, n, k)
            out[tag + "_y_w8a8"] = y8

    np.savez_compressed(out_path, **out)
    print("wrote", out_path, {k: str(v) for k, v in variants.items()})


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "--child":
        generate(sys.argv[2])
    else:
        import oracle as O
        O.build()
        env = dict(os.environ)
        subprocess.check_call([sys.executable, __file__, "--child",
                               os.path.join(HERE, "golden_default.npz")], env=env)
        for name in ("QGEMV", "GGUF_GEMV", "INT8_GEMM", "W8A32", "QGEMV_W8A8", "LOWBIT_W8A8"):
            env[f"QUIXICORE_CPU_{name}_VARIANT"] = "ref"
        subprocess.check_call([sys.executable, __file__, "--child",
                               os.path.join(HERE, "golden_forced_ref.npz")], env=env)
