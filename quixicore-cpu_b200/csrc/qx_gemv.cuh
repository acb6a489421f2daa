// Device-side building blocks of the decode GEMV: the activation digit table and the
// per-(row, block) integer dot products.
//
// Arithmetic. The reference computes, per weight row and per 32-element block b,
//   sum_b = sum_j float(q_j) * x_j   (f32)        y += d_b * sum_b
// (kernels/quantization/qgemv_ref.cpp:62-82, qgemv_w8a8_ref.cpp:95-118). Here each block
// of activations is first written as a 24-bit two's-complement fixed-point number with a
// power-of-two block scale, x_j ~= scale_b * t_j, |t_j| < 2^23, and t_j is split into its
// three bytes (low and middle unsigned, top signed). The 32-term dot product then becomes
// three exact integer dot products that run on dp4a (four 8-bit products per
// instruction), combined once per block in f32:
//   sum_b = scale_b * (65536 * S2 + 256 * S1 + S0).
// The only rounding on the activation side is the fixed-point step, at most 2^-24 of
// the block's power-of-two envelope per element -- the same order as the rounding of one
// f32 addition in the reference's own 32-term sum -- and the integer sums are exact.
#pragma once

#include "qx_common.cuh"

namespace qx {

// One block of 32 activations, ready for dp4a. dig[d][w] holds byte d of elements
// 4w..4w+3 (little endian within the word). 112 bytes, read as seven 16-byte loads.
struct __align__(16) XBlock {
  uint32_t dig[3][8];
  float scale;     // 2^(e-23): x_j ~= scale * t_j
  int neg8p[3];    // -8 * sum_j byte_d(t_j): the q4_0 "-8" offset, per digit
};
static_assert(sizeof(XBlock) == 112, "XBlock layout");

__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
  uint32_t d;
  asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"((uint32_t)c));
  return (int)d;
}

// streaming 16-byte load: weights are read exactly once
__device__ __forceinline__ uint4 ld_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned short ld_stream_u16(const unsigned short* p) {
  unsigned short v;
  asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return v;
}

// 65536*S2 + 256*S1 + S0 rounded once to f32. |S1|*256 + |S0| < 2^31 for both formats.
__device__ __forceinline__ float combine_digits(int s0, int s1, int s2) {
  return fmaf((float)s2, 65536.0f, (float)(s1 * 256 + s0));
}

// q8_0: w0,w1 = the 32 int8 codes of one block. Returns sum_j q_j * t_j as f32.
__device__ __forceinline__ float block_dot_q8(const uint4& w0, const uint4& w1,
                                              const XBlock& xb) {
  const uint32_t w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
  int s0 = 0, s1 = 0, s2 = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    s0 = dp4a_su(w[i], xb.dig[0][i], s0);
    s1 = dp4a_su(w[i], xb.dig[1][i], s1);
    s2 = dp4a_ss(w[i], xb.dig[2][i], s2);
  }
  return combine_digits(s0, s1, s2);
}

// q4_0: w = the 16 code bytes of one block; byte j = element j (low nibble) and element
// j+16 (high nibble). Returns sum_j (nibble_j - 8) * t_j as f32. The high nibbles are
// used in place (value 16*nibble), so their sums are exact multiples of 16.
__device__ __forceinline__ float block_dot_q4(const uint4& w, const XBlock& xb) {
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
  int l0 = xb.neg8p[0], l1 = xb.neg8p[1], l2 = xb.neg8p[2];
  int h0 = 0, h1 = 0, h2 = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t lo = ww[i] & 0x0F0F0F0Fu;
    const uint32_t hi = ww[i] & 0xF0F0F0F0u;
    l0 = dp4a_uu(lo, xb.dig[0][i], l0);
    l1 = dp4a_uu(lo, xb.dig[1][i], l1);
    l2 = dp4a_us(lo, xb.dig[2][i], l2);
    h0 = dp4a_uu(hi, xb.dig[0][4 + i], h0);
    h1 = dp4a_uu(hi, xb.dig[1][4 + i], h1);
    h2 = dp4a_us(hi, xb.dig[2][4 + i], h2);
  }
  return combine_digits(l0 + (h0 >> 4), l1 + (h1 >> 4), l2 + (h2 >> 4));
}

// fp16 bits -> f32, identical to kernels/common/fp16.h:11-37 for every bit pattern
// (subnormals, infinities and NaN payloads included): the hardware conversion is exact.
__device__ __forceinline__ float half_bits_to_float(unsigned short h) {
  return __half2float(__ushort_as_half(h));
}

}  // namespace qx
