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

// ------------------------------------------------------------------------------------
// W8A32: Y[r,o] = (sum_k X[r,k] * float(W[o,k])) * scale[o], f32 throughout
// (kernels/quantization/w8a32_gemm_ref.cpp:7-24, w8a32_gemm_avx512.cpp:9-35).
//
// A weight-streaming kernel: the int8 weights are read ONCE for up to MT activation rows
// (the reference re-reads a weight row per activation row), 16 bytes per lane and step, and
// converted to f32 without the conversion unit (byte ^ 0x80 placed into the mantissa of
// 2^23, minus 2^23 + 128: exact). A warp owns C output channels; a CTA (8 warps) stages the
// activations of the current K-chunk (512 columns x MT rows) in shared memory, so one
// 16-byte shared load feeds 4 * C multiply-adds. Per lane the products accumulate in k
// order, the 32 lane sums are added by a fixed butterfly: deterministic, and independent of
// the launch shape. Bound by HBM (the weight bytes) for a handful of rows, by the f32 FMA
// rate from about 8 rows up (MT * 2 flops per weight byte).
// ------------------------------------------------------------------------------------
constexpr int kW8KChunk = 512;  // activation columns staged per step = 32 lanes x 16

__device__ __forceinline__ void int8x4_to_float(uint32_t word, float (&out)[4]) {
  const uint32_t biased = word ^ 0x80808080u;  // b + 128 in every byte
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[i] = __uint_as_float(__byte_perm(biased, 0x4B000000u, 0x7650 + i)) - 8388736.0f;
  }
}

template <int MT, int C>
__global__ void __launch_bounds__(256) w8a32_stream_kernel(const int8_t* __restrict__ w,
                                                           const float* __restrict__ ws,
                                                           const float* __restrict__ x,
                                                           float* __restrict__ y, int m,
                                                           long long n, long long k,
                                                           long long ldy, int w_vector) {
  __shared__ __align__(16) float xs[MT][kW8KChunk];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long o0 = (blockIdx.x * 8LL + warp) * C;
  float acc[C][MT];
#pragma unroll
  for (int c = 0; c < C; ++c) {
#pragma unroll
    for (int r = 0; r < MT; ++r) acc[c][r] = 0.0f;
  }
  for (long long k0 = 0; k0 < k; k0 += kW8KChunk) {
    // this lane's 16 weight bytes of every channel: requested first, so that their latency
    // runs under the staging of the activations
    const long long kl = k0 + lane * 16;
    uint32_t words[C][4];
#pragma unroll
    for (int c = 0; c < C; ++c) {
      const long long o = o0 + c;
      words[c][0] = words[c][1] = words[c][2] = words[c][3] = 0u;
      if (o < n && kl < k) {
        const int8_t* src = w + o * k + kl;
        if (w_vector != 0 && kl + 16 <= k) {
          const uint4 v = __ldg(reinterpret_cast<const uint4*>(src));
          words[c][0] = v.x; words[c][1] = v.y; words[c][2] = v.z; words[c][3] = v.w;
        } else {
          for (int i = 0; i < 16 && kl + i < k; ++i) {
            words[c][i >> 2] |= static_cast<uint32_t>(static_cast<uint8_t>(src[i])) << (8 * (i & 3));
          }
        }
      }
    }
    __syncthreads();  // the previous chunk has been consumed
    // column kk = 16 * lane + 4 * q + i of the chunk goes to position 128 * q + 4 * lane + i:
    // the 32 lanes of a warp then read consecutive 16-byte pieces (no bank conflicts)
    for (int i = threadIdx.x; i < MT * kW8KChunk; i += 256) {
      const int r = i / kW8KChunk, kk = i % kW8KChunk;
      const int at = ((kk >> 2) & 3) * 128 + (kk >> 4) * 4 + (kk & 3);
      xs[r][at] = (r < m && k0 + kk < k) ? x[static_cast<long long>(r) * k + k0 + kk] : 0.0f;
    }
    __syncthreads();
    float wf[C][16];
#pragma unroll
    for (int c = 0; c < C; ++c) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float f[4];
        int8x4_to_float(words[c][q], f);
#pragma unroll
        for (int i = 0; i < 4; ++i) wf[c][4 * q + i] = f[i];
      }
    }
#pragma unroll
    for (int r = 0; r < MT; ++r) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 xv = *reinterpret_cast<const float4*>(&xs[r][q * 128 + lane * 4]);
#pragma unroll
        for (int c = 0; c < C; ++c) {
          acc[c][r] = fmaf(xv.x, wf[c][4 * q], acc[c][r]);
          acc[c][r] = fmaf(xv.y, wf[c][4 * q + 1], acc[c][r]);
          acc[c][r] = fmaf(xv.z, wf[c][4 * q + 2], acc[c][r]);
          acc[c][r] = fmaf(xv.w, wf[c][4 * q + 3], acc[c][r]);
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const long long o = o0 + c;
    const float scale = o < n ? ws[o] : 0.0f;
#pragma unroll
    for (int r = 0; r < MT; ++r) {
      float sum = acc[c][r];
#pragma unroll
      for (int h = 16; h >= 1; h >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, h);
      if (lane == 0 && o < n && r < m) y[r * ldy + o] = __fmul_rn(sum, scale);
    }
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
                       qx_workspace* workspace, cudaStream_t stream) {
  // five rows or more: the tensor cores (digit planes through the W8A8 GEMM); measured on
  // 4096 x 4096 with 16 rows: 17 us against 37 us for the streaming kernel below
  if (w8a32_planes_serves(m, k)) return launch_w8a32_planes(w, ws, x, y, m, n, k, ldy, workspace, stream);
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  // 16-byte weight loads need 16-byte aligned rows
  const int w_vector = (reinterpret_cast<uintptr_t>(w) % 16 == 0 && k % 16 == 0) ? 1 : 0;
  // four channels per warp (each staged activation feeds four multiply-adds) when that still
  // gives at least half of the SMs a CTA, else one
  const bool wide = (n + 31) / 32 >= ctx->prop.multiProcessorCount / 2;
  for (long long r0 = 0; r0 < m; r0 += 16) {
    const int mc = static_cast<int>(m - r0 < 16 ? m - r0 : 16);
    const float* xr = x + r0 * k;
    float* yr = y + r0 * ldy;
    const unsigned grid = static_cast<unsigned>(wide ? (n + 31) / 32 : (n + 7) / 8);
    if (mc <= 4) {
      if (wide) w8a32_stream_kernel<4, 4><<<grid, 256, 0, stream>>>(w, ws, xr, yr, mc, n, k, ldy, w_vector);
      else w8a32_stream_kernel<4, 1><<<grid, 256, 0, stream>>>(w, ws, xr, yr, mc, n, k, ldy, w_vector);
    } else {
      if (wide) w8a32_stream_kernel<16, 4><<<grid, 256, 0, stream>>>(w, ws, xr, yr, mc, n, k, ldy, w_vector);
      else w8a32_stream_kernel<16, 1><<<grid, 256, 0, stream>>>(w, ws, xr, yr, mc, n, k, ldy, w_vector);
    }
    count_launch();
    QX_CUDA_TRY(cudaGetLastError());
  }
  return QX_STATUS_OK;
}

}  // namespace qx
