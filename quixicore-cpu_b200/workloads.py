"""Seeded synthetic inputs for the five benchmark configurations of the quantized-matmul
path (shapes, block formats and value distributions as the benchmark definition states
them; no external dataset is involved). Pure numpy; the same bytes feed the CPU
reference/oracle and the GPU library.
"""

from __future__ import annotations

import numpy as np

Q8_0, Q4_0 = 0, 1

CONFIGS = {
    "cfg0_q8_0_gemv": dict(kind="qgemv", fmt=Q8_0, m=1, n=4096, k=4096, d_lo=0.001, d_hi=0.02),
    "cfg1_q4_0_gemv": dict(kind="qgemv", fmt=Q4_0, m=1, n=14336, k=4096, d_lo=0.002, d_hi=0.04),
    "cfg2_w8a8_gemm": dict(kind="w8a8", m=512, n=14336, k=4096),
    "cfg3_q8_0_batched": dict(kind="qgemv", fmt=Q8_0, m=32, n=28672, k=8192, d_lo=0.001,
                              d_hi=0.02, m_sweep=(1, 4, 8, 16, 32)),
    "cfg4_q4_0_prefill": dict(kind="qgemm_bf16", fmt=Q4_0, m=2048, n=28672, k=8192, d_lo=0.002,
                              d_hi=0.04),
}


def _rng(seed: int, stream: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[seed, stream]))


def packed_blocks(fmt: int, n: int, k: int, d_lo: float, d_hi: float, seed: int = 0,
                  stream: int = 1) -> np.ndarray:
    """Canonical GGUF bytes [n][k/32][34|18]: fp16 scale (|d| ~ U(d_lo, d_hi), random sign)
    followed by 32 int8 codes ~ U{-127..127} (q8_0) or 16 bytes of nibbles ~ U{0..15} (q4_0)."""
    rng = _rng(seed, stream)
    blocks = n * (k // 32)
    d = rng.uniform(d_lo, d_hi, blocks).astype(np.float32)
    d *= rng.integers(0, 2, blocks).astype(np.float32) * 2.0 - 1.0
    d16 = d.astype(np.float16).view(np.uint16)
    code_bytes = 32 if fmt == Q8_0 else 16
    out = np.empty((blocks, 2 + code_bytes), np.uint8)
    out[:, 0] = (d16 & 0xFF).astype(np.uint8)
    out[:, 1] = (d16 >> 8).astype(np.uint8)
    if fmt == Q8_0:
        out[:, 2:] = rng.integers(-127, 128, (blocks, 32), dtype=np.int8).view(np.uint8)
    else:
        out[:, 2:] = rng.integers(0, 256, (blocks, 16), dtype=np.uint8)
    return out.reshape(-1)


def activations_f32(m: int, k: int, seed: int = 0, stream: int = 2) -> np.ndarray:
    return _rng(seed, stream).standard_normal((m, k), dtype=np.float32)


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (finite inputs)."""
    bits = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def w8a8_inputs(m: int, n: int, k: int, seed: int = 0):
    rng_w, rng_x, rng_s = _rng(seed, 11), _rng(seed, 12), _rng(seed, 13)
    w = rng_w.integers(-127, 128, (n, k), dtype=np.int8)
    x = rng_x.integers(-127, 128, (m, k), dtype=np.int8)
    ws = rng_s.uniform(0.001, 0.01, n).astype(np.float32)
    xs = rng_s.uniform(0.005, 0.05, m).astype(np.float32)
    return w, x, ws, xs


def algorithmic_bytes_qgemv(fmt: int, m: int, n: int, k: int) -> int:
    """weights + activations read + outputs written, the reference bench's own convention
    (packed weight bytes + 4*(n + k) per row of x)."""
    return n * (k // 32) * (34 if fmt == Q8_0 else 18) + 4 * m * k + 4 * m * n


def xorshift_uniform(seed: int, count: int) -> np.ndarray:
    """The deterministic generator of the reference's own GEMV tests: xorshift32, top 24
    bits mapped to [-1, 1)."""
    state = np.uint32(seed)
    out = np.empty(count, np.float32)
    s = int(state)
    for i in range(count):
        s ^= (s << 13) & 0xFFFFFFFF
        s ^= s >> 17
        s ^= (s << 5) & 0xFFFFFFFF
        out[i] = np.float32(s >> 8) * np.float32(2.0 / 16777216.0) - np.float32(1.0)
    return out
