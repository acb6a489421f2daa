// Decode GEMV / small-batch qgemm over prepared q8_0 and q4_0 weights.
//
// Replaces q8_0_gemv_ref / q4_0_gemv_ref / q4_rows of the reference
// (kernels/quantization/qgemv_ref.cpp:62-92, qgemv_w8a8_ref.cpp:95-118,
// qgemv_gguf_avx2.cpp:295-318) and the per-row loop of qgemm
// (kernels/quantization/qgemm_ref.cpp:156-162).
//
// Kernels
//   quantize_x_kernel   x[m][k] f32 -> XBlock table (workspace scratch), one pass
//   gemv_kslice_kernel  the HBM-bound decode kernel: every thread owns ONE k-block
//                       position for the whole launch (its activation digits stay in
//                       registers) and walks down a contiguous range of weight rows;
//                       a warp therefore reads 32 consecutive blocks of a row = one
//                       contiguous 512 B (q4_0) or 1 KiB (q8_0) span per row, with the
//                       next rows' loads in flight while the current ones are reduced
//   gemv_generic_kernel any k (multiple of 32): one warp per (row, m)
//
// Reduction order (identical in both kernels, so a row's result does not depend on the
// kernel, the batch size or the row partition): per group of 32 consecutive blocks a
// fixed xor-butterfly over the 32 lanes (16, 8, 4, 2, 1), then the groups are added in
// ascending order.

#include "qx_gemv.cuh"
#include "qx_weights.cuh"

namespace qx {
namespace {

// ------------------------------------------------------------------------------------
// activation digits
// ------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) quantize_x_kernel(const float* __restrict__ x,
                                                         XBlock* __restrict__ out,
                                                         long long total_blocks) {
  const long long blk = blockIdx.x * 32LL + (threadIdx.x >> 3);
  const int q = threadIdx.x & 7;
  const bool active = blk < total_blocks;
  float v[4] = {0.f, 0.f, 0.f, 0.f};
  if (active) {
    const float* src = x + blk * 32 + q * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = src[i];
  }
  // max of |bits|: orders finite < inf < NaN, so non-finite inputs are detected
  uint32_t amax_bits = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) amax_bits = max(amax_bits, __float_as_uint(v[i]) & 0x7FFFFFFFu);
#pragma unroll
  for (int s = 1; s < 8; s <<= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, s));
  const uint32_t eb_raw = amax_bits >> 23;
  const bool finite = eb_raw != 255u;
  const uint32_t eb = max(eb_raw, 30u);  // envelope 2^(eb-126) > amax
  const float scale_up = __uint_as_float((276u - eb) << 23);  // 2^(23 - e)
  float scale = __uint_as_float((eb - 22u) << 23);            // 2^(e - 23)
  int t[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    t[i] = finite ? min(__float2int_rn(v[i] * scale_up), 8388607) : 0;
  }
  if (!finite) scale = __uint_as_float(0x7FC00000u);
  uint32_t word[3];
  int psum[3];
#pragma unroll
  for (int d = 0; d < 3; ++d) {
    uint32_t w = 0;
    int p = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t byte = (static_cast<uint32_t>(t[i]) >> (8 * d)) & 255u;
      w |= byte << (8 * i);
      p += d == 2 ? static_cast<int>(static_cast<int8_t>(byte)) : static_cast<int>(byte);
    }
    word[d] = w;
#pragma unroll
    for (int s = 1; s < 8; s <<= 1) p += __shfl_xor_sync(0xffffffffu, p, s);
    psum[d] = p;
  }
  if (active) {
    XBlock* dst = out + blk;
#pragma unroll
    for (int d = 0; d < 3; ++d) dst->dig[d][q] = word[d];
    if (q == 0) {
      dst->scale = scale;
#pragma unroll
      for (int d = 0; d < 3; ++d) dst->neg8p[d] = -8 * psum[d];
    }
  }
}

__device__ __forceinline__ XBlock load_xblock(const XBlock* p) {
  union {
    XBlock xb;
    uint4 raw[7];
  } u;
  const uint4* src = reinterpret_cast<const uint4*>(p);
#pragma unroll
  for (int i = 0; i < 7; ++i) u.raw[i] = __ldg(src + i);
  return u.xb;
}

template <int FMT>
struct Codes;  // the code bytes of one block as 16-byte vectors
template <>
struct Codes<QX_FORMAT_Q8_0> {
  uint4 a, b;
  static constexpr int kVec = 2;
  __device__ __forceinline__ void load(const uint4* plane, long long block) {
    a = ld_stream(plane + 2 * block);
    b = ld_stream(plane + 2 * block + 1);
  }
  __device__ __forceinline__ float dot(const XBlock& xb) const { return block_dot_q8(a, b, xb); }
};
template <>
struct Codes<QX_FORMAT_Q4_0> {
  uint4 a;
  static constexpr int kVec = 1;
  __device__ __forceinline__ void load(const uint4* plane, long long block) {
    a = ld_stream(plane + block);
  }
  __device__ __forceinline__ float dot(const XBlock& xb) const { return block_dot_q4(a, xb); }
};

__device__ __forceinline__ float warp_tree_sum(float v) {
#pragma unroll
  for (int h = 16; h >= 1; h >>= 1) v += __shfl_xor_sync(0xffffffffu, v, h);
  return v;
}

// ------------------------------------------------------------------------------------
// generic kernel: one warp per (row, m)
// ------------------------------------------------------------------------------------
template <int FMT>
__global__ void __launch_bounds__(256) gemv_generic_kernel(
    const uint4* __restrict__ codes, const unsigned short* __restrict__ scales,
    const XBlock* __restrict__ xt, float* __restrict__ y, long long n, long long nb,
    long long ldy) {
  const int lane = threadIdx.x & 31;
  const long long row = blockIdx.x * 8LL + (threadIdx.x >> 5);
  if (row >= n) return;
  const long long m = blockIdx.y;
  const XBlock* xr = xt + m * nb;
  float acc = 0.0f;
  for (long long base = 0; base < nb; base += 32) {
    const long long b = base + lane;
    float v = 0.0f;
    if (b < nb) {
      Codes<FMT> c;
      c.load(codes, row * nb + b);
      const float d = half_bits_to_float(ld_stream_u16(scales + row * nb + b));
      const XBlock xb = load_xblock(xr + b);
      v = __fmul_rn(c.dot(xb), __fmul_rn(d, xb.scale));
    }
    acc += warp_tree_sum(v);
  }
  if (lane == 0) y[m * ldy + row] = acc;
}

// ------------------------------------------------------------------------------------
// k-slice kernel (m == 1, blocks_per_row a multiple of 32 and <= 512)
// ------------------------------------------------------------------------------------
template <int FMT>
struct SliceCfg;
template <>
struct SliceCfg<QX_FORMAT_Q8_0> { static constexpr int kChunk = 2; };
template <>
struct SliceCfg<QX_FORMAT_Q4_0> { static constexpr int kChunk = 4; };

constexpr int kBatchRows = 32;

template <int FMT>
__global__ void __launch_bounds__(512, 1) gemv_kslice_kernel(
    const uint4* __restrict__ codes, const unsigned short* __restrict__ scales,
    const XBlock* __restrict__ xt, float* __restrict__ y, long long n, int nb, int S, int G,
    int total_groups) {
  constexpr int CH = SliceCfg<FMT>::kChunk;
  __shared__ float red[2][16][32];  // [buffer][warp][row-in-batch]

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int grp = warp / S;
  const int slice = warp - grp * S;
  const int gid = blockIdx.x * G + grp;
  const long long r0 = n * gid / total_groups;
  const long long r1 = n * (gid + 1LL) / total_groups;
  const int b = slice * 32 + lane;

  const XBlock xb = load_xblock(xt + b);
  int buf = 0;

  for (long long batch = r0; batch < r1; batch += kBatchRows) {
    float v[kBatchRows];
    Codes<FMT> cur[CH], nxt[CH];
    unsigned short dcur[CH], dnxt[CH];

#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const long long row = batch + i;
      if (row < r1) {
        cur[i].load(codes, row * nb + b);
        dcur[i] = ld_stream_u16(scales + row * nb + b);
      }
    }
#pragma unroll
    for (int c = 0; c < kBatchRows / CH; ++c) {
      if (c + 1 < kBatchRows / CH) {
#pragma unroll
        for (int i = 0; i < CH; ++i) {
          const long long row = batch + (c + 1) * CH + i;
          if (row < r1) {
            nxt[i].load(codes, row * nb + b);
            dnxt[i] = ld_stream_u16(scales + row * nb + b);
          }
        }
      }
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const long long row = batch + c * CH + i;
        float contribution = 0.0f;
        if (row < r1) {
          const float d = half_bits_to_float(dcur[i]);
          contribution = __fmul_rn(cur[i].dot(xb), __fmul_rn(d, xb.scale));
        }
        v[c * CH + i] = contribution;
      }
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        cur[i] = nxt[i];
        dcur[i] = dnxt[i];
      }
    }

    // transpose-reduce: after the five halving steps lane L holds the sum over the
    // warp's 32 blocks for row (batch + L), combined in the order 16, 8, 4, 2, 1.
#pragma unroll
    for (int h = 16; h >= 1; h >>= 1) {
      const bool upper = (lane & h) != 0;
#pragma unroll
      for (int i = 0; i < h; ++i) {
        const float send = upper ? v[i] : v[i + h];
        const float keep = upper ? v[i + h] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, h);
      }
    }

    const long long row = batch + lane;
    if (S == 1) {
      if (row < r1) y[row] = 0.0f + v[0];
    } else {
      red[buf][warp][lane] = v[0];
      asm volatile("bar.sync %0, %1;" ::"r"(1 + grp), "r"(S * 32) : "memory");
      if (slice == 0 && row < r1) {
        float acc = 0.0f;
        for (int s = 0; s < S; ++s) acc += red[buf][warp + s][lane];
        y[row] = acc;
      }
      buf ^= 1;
    }
  }
}

}  // namespace

// ------------------------------------------------------------------------------------
// host launcher
// ------------------------------------------------------------------------------------
qx_status launch_qgemm_f32(const qx_weights* w, const float* x_dev, float* y_dev,
                           long long m, long long ldy, qx_workspace* ws,
                           cudaStream_t stream) {
  const long long nb = w->blocks_per_row;
  const long long n = w->rows;
  const long long total_blocks = m * nb;
  QX_TRY(ws->reserve(static_cast<size_t>(total_blocks) * sizeof(XBlock)));
  XBlock* xt = static_cast<XBlock*>(ws->base);

  const long long qblocks = (total_blocks + 31) / 32;
  quantize_x_kernel<<<static_cast<unsigned>(qblocks), 256, 0, stream>>>(x_dev, xt, total_blocks);
  count_launch();

  const uint4* codes = reinterpret_cast<const uint4*>(w->codes);
  const bool slice_ok = m == 1 && nb % 32 == 0 && nb / 32 <= 16;
  if (slice_ok) {
    DeviceContext* ctx = nullptr;
    QX_TRY(current_context(&ctx));
    const int S = static_cast<int>(nb / 32);
    const int G = 16 / S;
    const int threads = S * G * 32;
    int grid = ctx->prop.multiProcessorCount;
    // no more groups than rows
    if (static_cast<long long>(grid) * G > n) grid = static_cast<int>((n + G - 1) / G);
    const int total_groups = grid * G;
    if (w->format == QX_FORMAT_Q8_0) {
      gemv_kslice_kernel<QX_FORMAT_Q8_0><<<grid, threads, 0, stream>>>(
          codes, w->scales, xt, y_dev, n, static_cast<int>(nb), S, G, total_groups);
    } else {
      gemv_kslice_kernel<QX_FORMAT_Q4_0><<<grid, threads, 0, stream>>>(
          codes, w->scales, xt, y_dev, n, static_cast<int>(nb), S, G, total_groups);
    }
  } else {
    const dim3 grid(static_cast<unsigned>((n + 7) / 8), static_cast<unsigned>(m));
    if (m > 65535) {
      set_last_error_text("qgemm: m > 65535 is not supported by the GEMV path");
      return QX_STATUS_INVALID_SHAPE;
    }
    if (w->format == QX_FORMAT_Q8_0) {
      gemv_generic_kernel<QX_FORMAT_Q8_0><<<grid, 256, 0, stream>>>(codes, w->scales, xt, y_dev,
                                                                   n, nb, ldy);
    } else {
      gemv_generic_kernel<QX_FORMAT_Q4_0><<<grid, 256, 0, stream>>>(codes, w->scales, xt, y_dev,
                                                                   n, nb, ldy);
    }
  }
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

}  // namespace qx
