// CUDA-core kernels of the integer / weight-only GEMMs: the any-shape W8A8 kernel, the
// W8A32 kernel and the finite-scale scan. The tensor-core W8A8 kernel lives in
// qx_int8_gemm_tc.cu; this file serves shapes it cannot take (k not a multiple of 16,
// unaligned pointers, k > 131000 where int32 accumulation could overflow).
//
// Arithmetic follows kernels/quantization/int8_gemm_ref.cpp:9-32 and
// kernels/quantization/w8a32_gemm_ref.cpp:7-24.

#include "qx_gemv.cuh"
#include "qx_int8_gemm.cuh"

namespace qx {
namespace {

constexpr int kTile = 64;     // output tile edge
constexpr int kChunkBytes = 32;

// y[r][o] = float(sum_k W[o,k]*X[r,k] - zp[r]*row_sum[o]) * ws[o] * as[r]
__global__ void __launch_bounds__(256) int8_gemm_simple_kernel(Int8GemmArgs a) {
  __shared__ uint32_t ws_tile[kTile][kChunkBytes / 4 + 1];
  __shared__ uint32_t xs_tile[kTile][kChunkBytes / 4 + 1];
  const int t = threadIdx.x;
  const long long o0 = blockIdx.x * static_cast<long long>(kTile);
  const long long r0 = blockIdx.y * static_cast<long long>(kTile);
  const int tx = t & 15, ty = t >> 4;  // 4 columns (o) x 4 rows (r) per thread

  int acc32[4][4];
  long long acc64[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc32[i][j] = 0;
      acc64[i][j] = 0;
    }

  const int load_row = t >> 2;        // 0..63
  const int load_byte = (t & 3) * 8;  // 0, 8, 16, 24
  int chunks_since_flush = 0;
  for (long long k0 = 0; k0 < a.k; k0 += kChunkBytes) {
    uint32_t wv[2] = {0, 0}, xv[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const long long kk = k0 + load_byte + i;
      if (kk < a.k) {
        if (o0 + load_row < a.n) {
          wv[i >> 2] |= static_cast<uint32_t>(static_cast<uint8_t>(a.w[(o0 + load_row) * a.k + kk]))
                        << (8 * (i & 3));
        }
        if (r0 + load_row < a.m) {
          xv[i >> 2] |= static_cast<uint32_t>(static_cast<uint8_t>(a.x[(r0 + load_row) * a.k + kk]))
                        << (8 * (i & 3));
        }
      }
    }
    __syncthreads();
    ws_tile[load_row][load_byte / 4] = wv[0];
    ws_tile[load_row][load_byte / 4 + 1] = wv[1];
    xs_tile[load_row][load_byte / 4] = xv[0];
    xs_tile[load_row][load_byte / 4 + 1] = xv[1];
    __syncthreads();
#pragma unroll
    for (int kw = 0; kw < kChunkBytes / 4; ++kw) {
      uint32_t wreg[4], xreg[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) wreg[j] = ws_tile[tx * 4 + j][kw];
#pragma unroll
      for (int i = 0; i < 4; ++i) xreg[i] = xs_tile[ty * 4 + i][kw];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc32[i][j] = dp4a_ss(wreg[j], xreg[i], acc32[i][j]);
    }
    // 2048 chunks * 32 products * 2^14 < 2^31: flush before int32 can overflow
    if (++chunks_since_flush == 2048) {
      chunks_since_flush = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc64[i][j] += acc32[i][j];
          acc32[i][j] = 0;
        }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const long long r = r0 + ty * 4 + i;
    if (r >= a.m) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const long long o = o0 + tx * 4 + j;
      if (o >= a.n) continue;
      long long dot = acc64[i][j] + acc32[i][j];
      if (a.asymmetric) dot -= static_cast<long long>(a.zp[r]) * a.row_sum[o];
      const float scaled = __fmul_rn(__ll2float_rn(dot), a.ws[o]);
      a.y[r * a.ldy + o] = __fmul_rn(scaled, a.as[r]);
      if (a.acc != nullptr) a.acc[r * a.n + o] = static_cast<int32_t>(dot);
    }
  }
}

__global__ void __launch_bounds__(256) check_finite_kernel(const float* __restrict__ v,
                                                           long long count, int* flag) {
  bool bad = false;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < count; i += gridDim.x * 256LL) {
    bad |= (__float_as_uint(v[i]) & 0x7F800000u) == 0x7F800000u;
  }
  if (__syncthreads_or(bad) && threadIdx.x == 0) atomicOr(flag, 1);
}

// W8A32, CUDA-core version: one warp per output channel, f32 FMA over k, fixed butterfly.
__global__ void __launch_bounds__(256) w8a32_simple_kernel(const int8_t* __restrict__ w,
                                                           const float* __restrict__ ws,
                                                           const float* __restrict__ x,
                                                           float* __restrict__ y, long long m,
                                                           long long n, long long k,
                                                           long long ldy) {
  const int lane = threadIdx.x & 31;
  const long long o = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (o >= n) return;
  const int8_t* wr = w + o * k;
  const float scale = ws[o];
  for (long long r = 0; r < m; ++r) {
    const float* xr = x + r * k;
    float sum = 0.0f;
    for (long long i = lane; i < k; i += 32) sum = fmaf(xr[i], static_cast<float>(wr[i]), sum);
#pragma unroll
    for (int h = 16; h >= 1; h >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, h);
    if (lane == 0) y[r * ldy + o] = __fmul_rn(sum, scale);
  }
}

}  // namespace

qx_status launch_int8_gemm_simple(const Int8GemmArgs& a, cudaStream_t stream) {
  const long long gx = (a.n + kTile - 1) / kTile, gy = (a.m + kTile - 1) / kTile;
  if (gy > 65535) {
    set_last_error_text("int8_gemm: m too large for the CUDA-core kernel");
    return QX_STATUS_INVALID_SHAPE;
  }
  int8_gemm_simple_kernel<<<dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy)), 256, 0,
                            stream>>>(a);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

qx_status launch_check_finite(const float* v, long long count, int* flag, cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>(min((count + 255) / 256, 1024LL));
  check_finite_kernel<<<grid, 256, 0, stream>>>(v, count, flag);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

qx_status launch_w8a32(const int8_t* w, const float* ws, const float* x, float* y,
                       long long m, long long n, long long k, long long ldy,
                       qx_workspace* /*workspace*/, cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>((n + 7) / 8);
  w8a32_simple_kernel<<<grid, 256, 0, stream>>>(w, ws, x, y, m, n, k, ldy);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

}  // namespace qx
