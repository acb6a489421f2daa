// Shared definitions of the decode GEMV / small-batch qgemm kernels: the prepared-weight
// panel geometry, the activation digit tables and the dp4a helpers.
//
// Arithmetic. The reference computes, per weight row and per 32-element block b,
//   sum_b = sum_j float(q_j) * x_j   (f32),       y += d_b * sum_b
// (kernels/quantization/qgemv_ref.cpp:62-82, qgemv_w8a8_ref.cpp:95-118). Here each block
// of activations is first written as a 23-bit signed fixed-point number under a
// power-of-two block envelope, x_j ~= scale_b * t_j with |t_j| <= 2^22, and t_j is split
// into three balanced base-256 digits, t = 65536*p2 + 256*p1 + p0, each in [-128, 127].
// The 32-term dot product then becomes three exact 8-bit integer dot products -- done by
// the tensor core (tcgen05 kind::i8) or by dp4a -- combined once per block in f32:
//   sum_b = scale_b * (65536*S2 + 256*S1 + S0).
// The only rounding on the activation side is the fixed-point step, at most 2^-23 of the
// block envelope per element, the order of one f32 rounding in the reference's own
// 32-term sum; the integer sums are exact.
#pragma once

#include "qx_common.cuh"

namespace qx {

constexpr int kTileRows = 128;   // weight rows per panel tile (= MMA M = TMEM lanes)
constexpr int kSlabBlocks = 4;   // 32-element blocks per K-slab (128 elements)
constexpr int kSlabK = kSlabBlocks * kBlockK;

// Per (activation row m, block b) constants, 16 bytes.
struct __align__(16) XConst {
  float scale;  // 2^(e-22): x_j ~= scale * t_j
  int k01;      // 8 * (256*P1 + P0), P_d = sum_j digit_d(t_j): the q4_0 "-8" offset
  int p2x8;     // 8 * P2
  int pad;
};

// Columns of the digit matrix used by a batch of m activation rows: four per row (three
// digits and one zero column, so a row's digits never straddle a 16-column group),
// rounded up to the sizes the tensor-core kernel is built for.
constexpr int kDigitStride = 4;
__host__ __device__ inline int digit_columns(int m) {
  const int c = kDigitStride * m;
  return c <= 8 ? 8 : (c <= 16 ? 16 : (c <= 32 ? 32 : (c <= 64 ? 64 : 128)));
}

// Activation side of one K-slab as the tensor-core kernel wants it in shared memory, kept
// in that form in scratch memory so that one bulk copy brings it in:
//   [ digit rows: ncols rows x 128 bytes, 16-byte chunks swizzled like a 128B-swizzle TMA
//     tile (chunk c of row r stored at c ^ (r & 7)) | XConst[ncols / 4][4 blocks] ]
__host__ __device__ inline int ximage_bytes(int ncols) { return ncols * 128 + ncols * 16; }
// byte offset, inside a slab image, of the 4 digit bytes of elements 4q..4q+3 of block j
// (0..3) in digit row `col`
__host__ __device__ inline int ximage_digit_offset(int col, int j, int q) {
  const int chunk = 2 * j + (q >> 2);
  return (col >> 3) * 1024 + (col & 7) * 128 + ((chunk ^ (col & 7)) << 4) + (q & 3) * 4;
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

// 65536*v + u rounded once to f32 (|u| < 2^31).
__device__ __forceinline__ float combine_digits(int u, int v) {
  return fmaf((float)v, 65536.0f, (float)u);
}

// fp16 bits -> f32, identical to kernels/common/fp16.h:11-37 for every finite or
// subnormal bit pattern: the hardware conversion is exact.
__device__ __forceinline__ float half_bits_to_float(unsigned short h) {
  return __half2float(__ushort_as_half(h));
}

}  // namespace qx
