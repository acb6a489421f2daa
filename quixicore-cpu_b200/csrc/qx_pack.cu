// Authoring kernels: quantise f32 weights into canonical q8_0 / q4_0 blocks and back.
// Bit-exact counterparts of q8_0_pack_ref / q8_0_unpack_ref
// (kernels/quantization/qgemv_ref.cpp:14-57) and q4_0_pack_ref / q4_0_unpack_ref
// (kernels/quantization/qgemv_w8a8_ref.cpp:45-93). Every float operation is an explicitly
// rounded intrinsic so the compiler cannot fuse or reorder it.

#include "qx_common.cuh"

namespace qx {
namespace {

__device__ __forceinline__ bool is_finite_bits(float v) {
  return (__float_as_uint(v) & 0x7F800000u) != 0x7F800000u;
}

// One thread per block; canonical output written as 16-bit words (blocks are only
// 2-byte aligned).
__global__ void __launch_bounds__(256) pack_q8_0_kernel(const float* __restrict__ w,
                                                        long long total_blocks,
                                                        unsigned short* __restrict__ out,
                                                        int* __restrict__ bad) {
  const long long blk = blockIdx.x * 256LL + threadIdx.x;
  if (blk >= total_blocks) return;
  const float* src = w + blk * 32;
  float amax = 0.0f;
  bool finite = true;
  for (int j = 0; j < 32; ++j) {
    finite &= is_finite_bits(src[j]);
    amax = fmaxf(amax, fabsf(src[j]));
  }
  if (!finite) {
    atomicOr(bad, 1);
    return;
  }
  const float d = __fdiv_rn(amax, 127.0f);
  const float inv = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
  unsigned short* dst = out + blk * 17;
  dst[0] = __half_as_ushort(__float2half_rn(d));
  for (int j = 0; j < 32; j += 2) {
    uint32_t pair = 0;
    for (int i = 0; i < 2; ++i) {
      float q = rintf(__fmul_rn(src[j + i], inv));
      q = q < -127.0f ? -127.0f : (q > 127.0f ? 127.0f : q);
      pair |= static_cast<uint32_t>(static_cast<uint8_t>(static_cast<int8_t>(q))) << (8 * i);
    }
    dst[1 + j / 2] = static_cast<unsigned short>(pair);
  }
}

__global__ void __launch_bounds__(256) pack_q4_0_kernel(const float* __restrict__ w,
                                                        long long total_blocks,
                                                        unsigned short* __restrict__ out,
                                                        int* __restrict__ bad) {
  const long long blk = blockIdx.x * 256LL + threadIdx.x;
  if (blk >= total_blocks) return;
  const float* src = w + blk * 32;
  float amax = 0.0f, vmax = 0.0f;
  bool finite = true;
  for (int j = 0; j < 32; ++j) {
    const float v = src[j];
    finite &= is_finite_bits(v);
    if (fabsf(v) > amax) {
      amax = fabsf(v);
      vmax = v;
    }
  }
  if (!finite) {
    atomicOr(bad, 1);
    return;
  }
  const float d = __fdiv_rn(vmax, -8.0f);
  const float inv = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
  unsigned short* dst = out + blk * 9;
  dst[0] = __half_as_ushort(__float2half_rn(d));
  for (int j = 0; j < 16; j += 2) {
    uint32_t pair = 0;
    for (int i = 0; i < 2; ++i) {
      // lround: nearest, halves away from zero
      int lo = static_cast<int>(roundf(__fmul_rn(src[j + i], inv))) + 8;
      int hi = static_cast<int>(roundf(__fmul_rn(src[j + i + 16], inv))) + 8;
      lo = lo < 0 ? 0 : (lo > 15 ? 15 : lo);
      hi = hi < 0 ? 0 : (hi > 15 ? 15 : hi);
      pair |= static_cast<uint32_t>(lo | (hi << 4)) << (8 * i);
    }
    dst[1 + j / 2] = static_cast<unsigned short>(pair);
  }
}

template <int FMT>
__global__ void __launch_bounds__(256) unpack_kernel(const unsigned short* __restrict__ in,
                                                     long long total_blocks,
                                                     float* __restrict__ w) {
  constexpr int kWords = FMT == QX_FORMAT_Q8_0 ? 17 : 9;
  const long long blk = blockIdx.x * 256LL + threadIdx.x;
  if (blk >= total_blocks) return;
  const unsigned short* src = in + blk * kWords;
  const float d = __half2float(__ushort_as_half(src[0]));
  float* dst = w + blk * 32;
  if (FMT == QX_FORMAT_Q8_0) {
    for (int j = 0; j < 32; ++j) {
      const int q = static_cast<int8_t>((src[1 + j / 2] >> (8 * (j & 1))) & 255);
      dst[j] = __fmul_rn(d, static_cast<float>(q));
    }
  } else {
    for (int j = 0; j < 16; ++j) {
      const int byte = (src[1 + j / 2] >> (8 * (j & 1))) & 255;
      dst[j] = __fmul_rn(static_cast<float>((byte & 15) - 8), d);
      dst[j + 16] = __fmul_rn(static_cast<float>((byte >> 4) - 8), d);
    }
  }
}

}  // namespace

// out_bad: device int set to 1 when a non-finite weight was met (pack only)
qx_status launch_pack(int format, const float* w_dev, long long total_blocks, void* packed_dev,
                      int* bad_dev, cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>((total_blocks + 255) / 256);
  if (format == QX_FORMAT_Q8_0) {
    pack_q8_0_kernel<<<grid, 256, 0, stream>>>(w_dev, total_blocks,
                                               static_cast<unsigned short*>(packed_dev), bad_dev);
  } else {
    pack_q4_0_kernel<<<grid, 256, 0, stream>>>(w_dev, total_blocks,
                                               static_cast<unsigned short*>(packed_dev), bad_dev);
  }
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

qx_status launch_unpack(int format, const void* packed_dev, long long total_blocks, float* w_dev,
                        cudaStream_t stream) {
  const unsigned grid = static_cast<unsigned>((total_blocks + 255) / 256);
  if (format == QX_FORMAT_Q8_0) {
    unpack_kernel<QX_FORMAT_Q8_0><<<grid, 256, 0, stream>>>(
        static_cast<const unsigned short*>(packed_dev), total_blocks, w_dev);
  } else {
    unpack_kernel<QX_FORMAT_Q4_0><<<grid, 256, 0, stream>>>(
        static_cast<const unsigned short*>(packed_dev), total_blocks, w_dev);
  }
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

}  // namespace qx
