// Internal launch interfaces of the integer / weight-only GEMMs.
#pragma once

#include "qx_common.cuh"

namespace qx {

struct Int8GemmArgs {
  const int8_t* w;      // [n][k]
  const int8_t* x;      // [m][k]
  const float* ws;      // [n]
  const float* as;      // [m]
  const int32_t* row_sum;  // [n] or null
  const int* zp;           // [m] or null
  float* y;             // [m][ldy]
  int32_t* acc;         // optional [m][n]
  long long m, n, k, ldy;
  bool asymmetric;
};

// Tensor-core path (tcgen05 kind::i8, TMA, TMEM). Returns false when the shape or the
// pointers do not meet its alignment rules; the caller then uses the CUDA-core kernel.
bool int8_gemm_tc_supported(const Int8GemmArgs& a);
qx_status launch_int8_gemm_tc(const Int8GemmArgs& a, cudaStream_t stream);

// CUDA-core kernel for any shape and alignment (dp4a on zero-padded shared tiles).
qx_status launch_int8_gemm_simple(const Int8GemmArgs& a, cudaStream_t stream);

qx_status launch_int8_gemm(const Int8GemmArgs& a, cudaStream_t stream);

// flag[0] |= 1 when any of v[0..count) is not finite
qx_status launch_check_finite(const float* v, long long count, int* flag, cudaStream_t stream);

qx_status launch_w8a32(const int8_t* w, const float* ws, const float* x, float* y,
                       long long m, long long n, long long k, long long ldy,
                       qx_workspace* workspace, cudaStream_t stream);

// qgemm_w8a32 from five activation rows on: four exact 8-bit digit planes of the activations
// (31-bit fixed point under one power-of-two envelope per row) through the W8A8 GEMM above,
// combined in f32 (qx_canonical.cu).
bool w8a32_planes_serves(long long m, long long k);
qx_status launch_w8a32_planes(const int8_t* w, const float* ws, const float* x, float* y,
                              long long m, long long n, long long k, long long ldy,
                              qx_workspace* workspace, cudaStream_t stream);

// lowbit_gemm on compact int4 rows through the digit kernels of qx_canonical.cu (exact 8-bit
// activation digits per 16 columns, dp4a): rows of an even number of columns with one scale
// per row or per group of a multiple of 16 columns.
bool int4_offset8_digits_serves(long long m, long long k, long long groups, long long group_size);
qx_status launch_int4_offset8_digits(const uint8_t* packed, const float* scales, const float* x,
                                     float* y, long long m, long long n, long long k,
                                     long long groups, long long group_size, cudaStream_t stream);

const char* int8_gemm_variant_name();

}  // namespace qx
