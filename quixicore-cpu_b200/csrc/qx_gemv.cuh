// Shared definitions of the decode GEMV / small-batch qgemm kernels: the prepared-weight
// panel geometry, the activation digit images and the dp4a helpers.
//
// Arithmetic. The reference computes, per weight row and per 32-element block b,
//   sum_b = sum_j float(q_j) * x_j   (f32),       y += d_b * sum_b
// (kernels/quantization/qgemv_ref.cpp:62-82, qgemv_w8a8_ref.cpp:95-118). Here each block
// of activations is first written as a 23-bit signed fixed-point number under a
// power-of-two block envelope, x_j ~= scale_b * t_j with |t_j| <= 2^22, and t_j is split
// into balanced base-256 digits, t = 65536*p2 + 256*p1 + p0, each in [-128, 127].
// The 32-term dot product then becomes exact 8-bit integer dot products -- done by the
// tensor core (tcgen05 kind::i8) or by dp4a -- combined once per block in f32:
//   sum_b = scale_b * (2^24*S3 + 65536*S2 + 256*S1 + S0).
// The only rounding on the activation side is the fixed-point step, at most 2^-23 of the
// block envelope per element, the order of one f32 rounding in the reference's own
// 32-term sum; the integer sums are exact.
//
// q4_0 without unpacking the nibbles. Byte i of a block holds element i (low nibble,
// lo_i) and element i + 16 (high nibble, hi_i). With w_i = lo_i + 16*hi_i the raw byte and
// h_i = 16*hi_i = w_i & 0xF0,
//   16 * sum_i (lo_i*t_i + hi_i*t_{i+16}) = sum_i w_i*(16*t_i) + sum_i h_i*(t_{i+16} - 16*t_i),
// so the raw bytes are one unsigned 8-bit operand (against the four digits of 16*t_i,
// i < 16) and the masked bytes a second one (against the four digits of
// z_i = t_{i+16} - 16*t_i, |z_i| < 2^27): one AND per word is all the unpacking there is.
// The factor 16 is folded into the block's power-of-two scale, and the "-8" of the format
// is the per-block constant 16 * 8 * sum_j t_j.
#pragma once

#include "qx_common.cuh"

namespace qx {

constexpr int kTileRows = 128;   // weight rows per panel tile (= MMA M = TMEM lanes)
constexpr int kSlabBlocks = 8;   // 32-element blocks per K-slab (256 elements)
constexpr int kSlabK = kSlabBlocks * kBlockK;
constexpr int kSlabScaleBytes = kTileRows * kSlabBlocks * 2;  // [row][block] fp16 bits

// ---- prepared-weight panel: one contiguous span per (tile of 128 rows, K-slab) ---------
//   q8_0: two code sub-tiles (blocks 0-3, blocks 4-7) of [128 rows][128 bytes], then scales
//   q4_0: one code sub-tile [128 rows][8 blocks x 16 packed bytes], then scales
// Inside a sub-tile the 16-byte chunk c of row r is stored at chunk c ^ (r & 7): the
// 128-byte swizzle the tensor-core operand descriptors expect, already applied in HBM so
// that a stage is filled by one plain bulk copy.
__host__ __device__ constexpr int slab_code_bytes(int format) {
  return format == QX_FORMAT_Q8_0 ? kTileRows * kSlabBlocks * 32 : kTileRows * kSlabBlocks * 16;
}
__host__ __device__ constexpr int slab_span_bytes(int format) {
  return slab_code_bytes(format) + kSlabScaleBytes;
}
// byte offset inside a span of the 16 code bytes `half` (0: elements 0-15, 1: 16-31) of
// block j of row r (q8_0), or of the 16 packed bytes of block j (q4_0)
__host__ __device__ inline int panel_code_offset_q8(int r, int j, int half) {
  return (j >> 2) * (kTileRows * 128) + r * 128 + (((2 * (j & 3) + half) ^ (r & 7)) << 4);
}
__host__ __device__ inline int panel_code_offset_q4(int r, int j) {
  return r * 128 + ((j ^ (r & 7)) << 4);
}
__host__ __device__ inline int panel_scale_offset(int format, int r, int j) {
  return slab_code_bytes(format) + (r * kSlabBlocks + j) * 2;
}

// ---- activation side -------------------------------------------------------------------
// A launch handles mp = 1, 2, 4, 8, 16 or 32 activation rows (m rounded up). The digit
// matrix of a slab has four columns per (block class, activation row): columns
//   n = ((j mod G) * mp + row) * 4 + digit,       G = group_blocks(format, mp),
// and column n is non-zero only in the K range of the blocks j with that class. One MMA
// accumulator of N = 4*mp*G columns therefore holds the digit sums of G consecutive
// blocks side by side (block-diagonal B operand): for mp = 1 a single accumulator of 32
// columns carries a whole slab.
__host__ __device__ constexpr int padded_batch(int m) {
  return m <= 1 ? 1 : (m <= 2 ? 2 : (m <= 4 ? 4 : (m <= 8 ? 8 : (m <= 16 ? 16 : 32))));
}
__host__ __device__ constexpr int group_blocks(int format, int mp) {
  const int g = kSlabBlocks / mp < 1 ? 1 : kSlabBlocks / mp;
  // a q4_0 MMA step spans 32 packed bytes = two blocks
  return format == QX_FORMAT_Q4_0 && g < 2 ? 2 : g;
}
__host__ __device__ constexpr int digit_columns(int format, int mp) {
  return 4 * mp * group_blocks(format, mp);
}
__host__ __device__ inline int digit_row(int format, int mp, int j, int row, int digit) {
  return ((j % group_blocks(format, mp)) * mp + row) * 4 + digit;
}

// Per (block j, activation row) constants, 16 bytes.
struct __align__(16) XConst {
  float scale;  // 2^(e-22): x_j ~= scale * t_j (NaN when the block holds a non-finite value);
                // q4_0: 2^(e-26), the digit sums carry a factor 16
  int k_lo;     // q4_0: 128 * sum_j t_j = 65536 * k_hi + k_lo, 0 <= k_lo < 65536
  int k_hi;
  int pad;
};

// Activation side of one K-slab ("image"), in the form the tensor-core kernel wants in
// shared memory, so one bulk copy brings it in:
//   q8_0: [sub-tile 0 | sub-tile 1], each [N digit rows][128 bytes] (blocks 0-3 | 4-7)
//   q4_0: [digits of 16*t_i, i < 16 | digits of z_i], each [N rows][8 blocks x 16 bytes]
//   then XConst[8 blocks][mp]
// with 16-byte chunks swizzled by the row index like the weight sub-tiles.
__host__ __device__ constexpr int ximage_bytes(int format, int mp) {
  return digit_columns(format, mp) * 256 + 128 * mp;
}
// offset of the 16 digit bytes of (digit row n, chunk cc) in half-image `which`
__host__ __device__ inline int ximage_chunk_offset(int ncols, int which, int n, int cc) {
  return which * ncols * 128 + n * 128 + ((cc ^ (n & 7)) << 4);
}
__host__ __device__ inline int ximage_const_offset(int ncols, int mp, int j, int row) {
  return ncols * 256 + (j * mp + row) * 16;
}

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

// int -> f32 for |s| < 2^22 without the conversion unit (an integer add and a float
// subtract: the int lands in the mantissa of 1.5 * 2^23). Exact.
__device__ __forceinline__ float small_int_to_float(int s) {
  return __int_as_float(s + 0x4B400000) - 12582912.0f;
}
// One block's term from its digit sums (each |s_d| < 2^21): 65536*s2 + 256*s1 + s0 (q8_0) or
// 2^24*s3 + 65536*s2 + 256*s1 + s0 - (65536*k_hi + k_lo) (q4_0), rounded to f32 as
// RN(65536*hi + RN(lo)) with lo = 256*s1 + s0 - k_lo and hi = 256*s3 + s2 - k_hi
// (|hi| < 2^24 is exact).
__device__ __forceinline__ float block_sum(int s0, int s1, int s2) {
  return fmaf(small_int_to_float(s2), 65536.0f,
              fmaf(small_int_to_float(s1), 256.0f, small_int_to_float(s0)));
}
__device__ __forceinline__ float block_sum(int s0, int s1, int s2, int s3, int k_lo, int k_hi) {
  const float lo = fmaf(small_int_to_float(s1), 256.0f, small_int_to_float(s0 - k_lo));
  const float hi = fmaf(small_int_to_float(s3), 256.0f, small_int_to_float(s2 - k_hi));
  return fmaf(hi, 65536.0f, lo);
}

// The same two values with the low parts first combined as integers (exact in 32 bits:
// |256*s1 + s0 - k_lo| < 2^30) and converted by the conversion unit: RN(256*s1 + s0 - k_lo)
// either way, so the bits are identical. Fewer instructions on a slower pipe; measured, the
// epilogues are bound by instruction issue and not by that pipe at any batch size (28672 x
// 8192 q8_0 at 8 / 16 / 32 rows: 69.5 / 111.8 / 208 us against 75.0 / 120.6 / 228 us), so
// the GEMV kernels use these.
__device__ __forceinline__ float block_sum_cvt(int s0, int s1, int s2) {
  return fmaf(small_int_to_float(s2), 65536.0f, __int2float_rn(s0 + (s1 << 8)));
}
__device__ __forceinline__ float block_sum_cvt(int s0, int s1, int s2, int s3, int k_lo, int k_hi) {
  const float lo = __int2float_rn(s0 - k_lo + (s1 << 8));
  const float hi = __int2float_rn(s2 - k_hi + (s3 << 8));  // |hi| < 2^24: exact
  return fmaf(hi, 65536.0f, lo);
}

// The tensor-core kernel and the single-row decode kernel accumulate the two parts of a
// block separately: with ds = d_b * scale_b (one rounded product),
//   L += lo * ds,   H += hi * ds        (one chain each per block parity, ascending blocks)
// and a K unit's sum is (65536 * H_even + L_even) + (65536 * H_odd + L_odd). lo and hi are
// the values of block_sum above: lo = RN(256*s1 + s0 - k_lo), hi = 256*s3 + s2 - k_hi
// (exact), for q8_0 lo = RN(256*s1 + s0), hi = s2. Both conversions give the same bits.
struct BlockParts {
  float lo, hi;
};
__device__ __forceinline__ BlockParts block_parts(int s0, int s1, int s2) {
  return {fmaf(small_int_to_float(s1), 256.0f, small_int_to_float(s0)), small_int_to_float(s2)};
}
__device__ __forceinline__ BlockParts block_parts(int s0, int s1, int s2, int s3, int k_lo, int k_hi) {
  return {fmaf(small_int_to_float(s1), 256.0f, small_int_to_float(s0 - k_lo)),
          fmaf(small_int_to_float(s3), 256.0f, small_int_to_float(s2 - k_hi))};
}
__device__ __forceinline__ BlockParts block_parts_cvt(int s0, int s1, int s2) {
  return {__int2float_rn(s0 + (s1 << 8)), __int2float_rn(s2)};
}
__device__ __forceinline__ BlockParts block_parts_cvt(int s0, int s1, int s2, int s3, int k_lo, int k_hi) {
  return {__int2float_rn(s0 - k_lo + (s1 << 8)), __int2float_rn(s2 - k_hi + (s3 << 8))};
}
__device__ __forceinline__ float unit_sum(float l_even, float h_even, float l_odd, float h_odd) {
  return __fadd_rn(fmaf(h_even, 65536.0f, l_even), fmaf(h_odd, 65536.0f, l_odd));
}

// q4_0 block constants from sum = sum_j t_j (|sum| <= 2^27): 128 * sum split at bit 16
// without leaving 32 bits.
__host__ __device__ inline void q4_offset_constants(int sum, int* k_lo, int* k_hi) {
  *k_lo = (sum & 0x1FF) << 7;
  *k_hi = sum >> 9;
}

// fp16 bits -> f32, identical to kernels/common/fp16.h:11-37 for every finite or
// subnormal bit pattern: the hardware conversion is exact.
__device__ __forceinline__ float half_bits_to_float(unsigned short h) {
  return __half2float(__ushort_as_half(h));
}

}  // namespace qx
