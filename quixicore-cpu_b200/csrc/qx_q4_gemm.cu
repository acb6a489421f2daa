// Prefill GEMM over prepared q4_0 weights with bf16 activations:
//   Y[m, rows] = bf16_to_f32(X)[m, k] . dequant(W)^T,   f32 accumulate and output.
// Counterpart of qgemm_prepacked for m >= 64 (kernels/quantization/qgemm_panel.cpp:242-287)
// with the bf16 -> f32 input conversion of float_storage
// (kernels/utils/float_storage_ref.cpp:195-200).
//
// A dense contraction on the tensor cores (tcgen05 kind::f16, fp16 x fp16 -> f32 in TMEM).
// A pre-pass rewrites every activation row as fp16 under a power-of-two row scale (exact:
// bf16 has fewer mantissa bits than fp16, and the scale puts the row's largest value just
// below 2^15, so nothing within 2^-29 of it leaves the normal range); the epilogue undoes
// the scale. The weights stay 4-bit in HBM; every CTA dequantises the K-slab it is about
// to multiply tile-wise into shared memory:
//   producer  (1 thread)  bulk copies of packed slabs (18 KiB = 128 rows x 256 K) into a
//                         2-slot ring; TMA tiles of the activations (bn tokens x 64 K,
//                         128-byte swizzle) into a 3-slot ring
//   dequant   (8 warps)   one (row, block) item per lane and K-step: 16 packed bytes ->
//                         32 fp16 values d * (nibble - 8), written as the A operand
//                         (128 rows x 64 K, 128-byte swizzle) into a 4-slot ring
//   MMA       (1 thread)  four tcgen05.mma (K = 16) per K-step into one of two TMEM
//                         accumulators of 128 channels x bn tokens
//   epilogue  (8 warps)   TMEM -> registers -> row scale -> coalesced f32 stores,
//                         overlapped with the next tile's MMAs through the second accumulator
// Rounding: the weight d * (nibble - 8) is one fp16 multiply of the block's own fp16 scale
// (relative error at most 2^-12 per weight); products are exact and sums f32 in the tensor
// core. This is the stated 1e-2 tolerance class of the 4-bit prefill path (measured: about
// 2e-4 of a row's rms); batches below 64 rows and q8_0 weights take the exact digit
// kernels instead.

#include <cuda.h>
#include <cuda_fp16.h>

#include "qx_gemv.cuh"
#include "qx_gemv_tc.cuh"
#include "qx_sm100.cuh"
#include "qx_weights.cuh"

namespace qx {
namespace {

using namespace sm100;

constexpr int kRows = 128;           // weight rows per tile (MMA M, TMEM lanes)
constexpr int kStepK = 64;           // K elements per MMA step group (128 bytes of bf16)
constexpr int kStepsPerSlab = kSlabK / kStepK;  // 4
constexpr int kRawSlots = 2, kASlots = 4, kBSlots = 3;
constexpr int kRawBytes = 18 * 1024;  // packed q4_0 slab span: codes 16 KiB + scales 2 KiB
constexpr int kABytes = kRows * 128;  // 16 KiB
constexpr int kMaxTokens = 256;       // tokens per tile (MMA N)
constexpr int kDequantWarps = 8, kEpiWarps = 8;
constexpr int kThreads = 32 * (2 + kEpiWarps + kDequantWarps);

struct Q4GemmParams {
  const uint8_t* panel;
  const float* row_unscale;  // [m]: what a token's sums are multiplied by (undoes the row scale)
  float* y;
  long long m, rows, ldy;
  int slabs;      // K-slabs per row
  int bn;         // tokens per tile
  int o_tiles, r_tiles;
  int* error;
};

struct __align__(16) Q4GemmBarriers {
  uint64_t raw_full[kRawSlots], raw_empty[kRawSlots];
  uint64_t a_full[kASlots], a_empty[kASlots];
  uint64_t b_full[kBSlots], b_empty[kBSlots];
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

__device__ __forceinline__ void bulk_copy_g2s(void* smem_dst, const void* gsrc, uint32_t bytes,
                                              uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes),
      "r"(smem_u32(bar))
      : "memory");
}

struct Ring {
  uint32_t slot = 0, phase = 0;
  __device__ __forceinline__ void advance(uint32_t slots) {
    if (++slot == slots) {
      slot = 0;
      phase ^= 1u;
    }
  }
};

// Two nibbles (two bytes of `nib`, picked by `selector`) -> fp16x2 of d * (nibble - 8):
// 0x6400 | n is the fp16 value 1024 + n, so the subtraction is exact.
__device__ __forceinline__ uint32_t dequant_pair(uint32_t nib, uint32_t selector, __half2 d2) {
  const uint32_t bits = __byte_perm(nib, 0x64646464u, selector);
  __half2 v = *reinterpret_cast<const __half2*>(&bits);
  v = __hsub2(v, __floats2half2_rn(1032.0f, 1032.0f));
  v = __hmul2(v, d2);
  return *reinterpret_cast<const uint32_t*>(&v);
}
// Four nibbles held as the bytes of `nib` -> 4 fp16 values (two words), element order kept.
__device__ __forceinline__ void dequant_word(uint32_t nib, __half2 d2, uint32_t* out) {
  out[0] = dequant_pair(nib, 0x4140u, d2);  // bytes 0, 1
  out[1] = dequant_pair(nib, 0x4342u, d2);  // bytes 2, 3
}

__global__ void __launch_bounds__(kThreads, 1)
q4_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const Q4GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t b_bytes = static_cast<uint32_t>(p.bn) * 128u;
  uint8_t* a_ring = smem;                               // kASlots x 16 KiB
  uint8_t* b_ring = a_ring + kASlots * kABytes;         // kBSlots x bn x 128 B (1024-aligned)
  uint8_t* raw_ring = b_ring + kBSlots * kMaxTokens * 128;
  auto* bars = reinterpret_cast<Q4GemmBarriers*>(raw_ring + kRawSlots * kRawBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kRawSlots; ++s) {
      mbar_init(&bars->raw_full[s], 1);
      mbar_init(&bars->raw_empty[s], kDequantWarps);
    }
    for (int s = 0; s < kASlots; ++s) {
      mbar_init(&bars->a_full[s], kDequantWarps);
      mbar_init(&bars->a_empty[s], 1);
    }
    for (int s = 0; s < kBSlots; ++s) {
      mbar_init(&bars->b_full[s], 1);
      mbar_init(&bars->b_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], kEpiWarps);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_x);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  const int total_tiles = p.o_tiles * p.r_tiles;
  // tiles of this CTA: blockIdx.x, blockIdx.x + gridDim.x, ...; o-tile major so that CTAs
  // running at the same time share weight slabs in L2
  if (warp == 0) {
    // ------------------------------ producer ----------------------------------
    if (lane == 0) {
      bool ok = true;
      Ring raw, b;
      // packed slabs run one slab ahead of the activation tiles
      int next_tile = blockIdx.x, next_slab = 0;
      auto issue_raw = [&]() -> bool {
        if (next_tile >= total_tiles) return true;
        if (!mbar_wait(&bars->raw_empty[raw.slot], raw.phase ^ 1u, abort_flag)) return false;
        const long long span = static_cast<long long>(next_tile / p.r_tiles) * p.slabs + next_slab;
        mbar_arrive_expect_tx(&bars->raw_full[raw.slot], kRawBytes);
        bulk_copy_g2s(raw_ring + raw.slot * kRawBytes, p.panel + span * kRawBytes, kRawBytes,
                      &bars->raw_full[raw.slot]);
        raw.advance(kRawSlots);
        if (++next_slab == p.slabs) {
          next_slab = 0;
          next_tile += gridDim.x;
        }
        return true;
      };
      ok = issue_raw();
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int r0 = (tile % p.r_tiles) * p.bn;
        for (int s = 0; s < p.slabs && ok; ++s) {
          ok = issue_raw();
          for (int t = 0; t < kStepsPerSlab && ok; ++t) {
            if (!mbar_wait(&bars->b_empty[b.slot], b.phase ^ 1u, abort_flag)) {
              ok = false;
              break;
            }
            mbar_arrive_expect_tx(&bars->b_full[b.slot], b_bytes);
            tma_load_2d(b_ring + b.slot * (kMaxTokens * 128), &map_x, &bars->b_full[b.slot],
                        (s * kStepsPerSlab + t) * kStepK, r0);
            b.advance(kBSlots);
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        report_error(p.error, 21);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (elect_one()) {
      // f32 accumulate, fp16 x fp16 (format fields 0), N = bn, M = 128
      const uint32_t idesc = (1u << 4) |
                             (static_cast<uint32_t>(p.bn >> 3) << 17) |
                             (static_cast<uint32_t>(kRows >> 4) << 24);
      Ring a, b;
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * 256u;
        const int steps = p.slabs * kStepsPerSlab;
        for (int ks = 0; ks < steps; ++ks) {
          if (!mbar_wait(&bars->a_full[a.slot], a.phase, abort_flag) ||
              !mbar_wait(&bars->b_full[b.slot], b.phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint64_t a_desc = make_sw128_kmajor_desc(smem_u32(a_ring + a.slot * kABytes));
          const uint64_t b_desc =
              make_sw128_kmajor_desc(smem_u32(b_ring + b.slot * (kMaxTokens * 128)));
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            // 16 fp16 = 32 bytes of K inside the swizzle atom: +2 in the (addr >> 4) field
            mma_f16_ss(d_tmem, a_desc + static_cast<uint64_t>(2 * kk),
                       b_desc + static_cast<uint64_t>(2 * kk), idesc, (ks | kk) != 0 ? 1u : 0u);
          }
          tc_commit(&bars->a_empty[a.slot]);
          tc_commit(&bars->b_empty[b.slot]);
          a.advance(kASlots);
          b.advance(kBSlots);
        }
        if (!ok) break;
        tc_commit(&bars->tmem_full[acc]);
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        report_error(p.error, 22);
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // ------------------------------ epilogue ----------------------------------
    // Warp w reads TMEM lanes 32*(w & 3).. (its channel quarter) and takes the 32-token
    // column chunks c with (c & 1) == half. A thread owns one output channel, so for a
    // fixed token the 32 lanes store 32 consecutive floats of Y.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const long long o = static_cast<long long>(tile / p.r_tiles) * kRows + quarter * 32 + lane;
      const long long r0 = static_cast<long long>(tile % p.r_tiles) * p.bn;
      if (!mbar_wait(&bars->tmem_full[acc], acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int chunks = p.bn / 32;
      for (int c = half; c < chunks; c += 2) {
        uint32_t v[32];
        const uint32_t taddr = tmem_base + acc * 256u + static_cast<uint32_t>(c * 32) +
                               (static_cast<uint32_t>(quarter * 32) << 16);
        tmem_ld_32x32(taddr, v);
        tmem_ld_wait();
        if (o >= p.rows) continue;
        const long long rc = r0 + c * 32;
        float* yp = p.y + rc * p.ldy + o;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          if (rc + j < p.m) {
            yp[j * p.ldy] = __fmul_rn(__uint_as_float(v[j]), __ldg(p.row_unscale + rc + j));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (!ok) {
      *abort_flag = 1;
      report_error(p.error, 23);
    }
  } else {
    // ------------------------------ dequantisers ------------------------------
    // Item of a lane in K-step t of a slab: row r = item / 2, block j = 2t + item % 2. The
    // packed tile is [128 rows][8 blocks x 16 bytes], the A tile [128 rows][128 bytes],
    // both with the 16-byte chunk c of row r stored at chunk c ^ (r & 7).
    const int item = (warp - 2 - kEpiWarps) * 32 + lane;
    const int r = item >> 1, jb = item & 1;
    Ring raw, a;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      for (int s = 0; s < p.slabs && ok; ++s) {
        if (!mbar_wait(&bars->raw_full[raw.slot], raw.phase, abort_flag)) {
          ok = false;
          break;
        }
        const uint8_t* packed = raw_ring + raw.slot * kRawBytes;
        for (int t = 0; t < kStepsPerSlab; ++t) {
          const int j = 2 * t + jb;
          const uint4 w = *reinterpret_cast<const uint4*>(packed + r * 128 + ((j ^ (r & 7)) << 4));
          const unsigned short d_bits = *reinterpret_cast<const unsigned short*>(
              packed + kRows * 128 + (r * kSlabBlocks + j) * 2);
          const __half d = __ushort_as_half(d_bits);
          const __half2 d2 = __halves2half2(d, d);
          // elements 0..15 are the low nibbles of bytes 0..15, elements 16..31 the high ones
          uint32_t out[16];
          const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            dequant_word(words[i] & 0x0F0F0F0Fu, d2, out + 2 * i);
            dequant_word((words[i] >> 4) & 0x0F0F0F0Fu, d2, out + 8 + 2 * i);
          }
          if (!mbar_wait(&bars->a_empty[a.slot], a.phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* row = a_ring + a.slot * kABytes + r * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            *reinterpret_cast<uint4*>(row + (((4 * jb + c) ^ (r & 7)) << 4)) =
                make_uint4(out[4 * c], out[4 * c + 1], out[4 * c + 2], out[4 * c + 3]);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&bars->a_full[a.slot]);
          a.advance(kASlots);
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->raw_empty[raw.slot]);  // packed slab consumed
        raw.advance(kRawSlots);
      }
    }
    if (!ok) {
      *abort_flag = 1;
      report_error(p.error, 24);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

constexpr size_t kQ4GemmSmem = 1024 + kASlots * kABytes + kBSlots * kMaxTokens * 128 +
                               kRawSlots * kRawBytes + sizeof(Q4GemmBarriers) + 64;

__global__ void __launch_bounds__(256) bf16_to_f32_kernel(const uint16_t* __restrict__ in,
                                                          float* __restrict__ out,
                                                          long long count) {
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < count; i += gridDim.x * 256LL) {
    out[i] = __uint_as_float(static_cast<uint32_t>(in[i]) << 16);
  }
}

// One CTA per activation row: bf16 -> fp16 under a power-of-two scale that puts the row's
// largest magnitude in [2^14, 2^15) (exact), and the factor that undoes it. Rows holding a
// NaN or an infinity are converted unscaled, so the result is non-finite as well.
__global__ void __launch_bounds__(256) scale_rows_to_fp16_kernel(const uint16_t* __restrict__ x,
                                                                 __half* __restrict__ out,
                                                                 float* __restrict__ row_unscale,
                                                                 long long k) {
  __shared__ uint32_t warp_max[8];
  const uint16_t* row = x + blockIdx.x * k;
  uint32_t amax = 0;  // of the bf16 bit patterns without sign: monotonic in magnitude
  for (long long i = threadIdx.x; i < k; i += 256) amax = max(amax, static_cast<uint32_t>(row[i] & 0x7FFFu));
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) amax = max(amax, __shfl_xor_sync(0xffffffffu, amax, s));
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax;
  __syncthreads();
  amax = warp_max[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) amax = max(amax, warp_max[i]);
  const uint32_t exponent = amax >> 7;  // biased, 8 bits
  // finite and non-zero rows: scale 2^(141 - exponent) maps [2^(e-127), 2^(e-126)) to [2^14, 2^15)
  const bool scaled = exponent != 255u && exponent != 0u && exponent >= 15u && exponent <= 253u;
  const float scale = scaled ? __uint_as_float((268u - exponent) << 23) : 1.0f;
  const float unscale = scaled ? __uint_as_float((exponent - 14u) << 23) : 1.0f;
  for (long long i = threadIdx.x; i < k; i += 256) {
    const float v = __uint_as_float(static_cast<uint32_t>(row[i]) << 16);
    out[blockIdx.x * k + i] = __float2half_rn(v * scale);
  }
  if (threadIdx.x == 0) row_unscale[blockIdx.x] = unscale;
}

qx_status launch_tc(const qx_weights* w, const uint16_t* x_bf16_dev, float* y_dev, long long m,
                    long long ldy, qx_workspace* ws, cudaStream_t stream) {
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  // workspace: [row factors | fp16 activations]
  const size_t factor_bytes = align_up(static_cast<size_t>(m) * sizeof(float), 256);
  QX_TRY(ws->reserve(kWorkspaceCounterBytes + factor_bytes +
                     static_cast<size_t>(m) * w->columns * sizeof(__half)));
  uint8_t* base = static_cast<uint8_t*>(ws->base) + kWorkspaceCounterBytes;
  float* row_unscale = reinterpret_cast<float*>(base);
  __half* x_half = reinterpret_cast<__half*>(base + factor_bytes);
  scale_rows_to_fp16_kernel<<<static_cast<unsigned>(m), 256, 0, stream>>>(x_bf16_dev, x_half,
                                                                           row_unscale, w->columns);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());

  const int bn = m >= kMaxTokens ? kMaxTokens : static_cast<int>((m + 31) / 32 * 32);
  CUtensorMap map_x;
  if (!encode_tma_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x_half,
                     static_cast<uint64_t>(w->columns), static_cast<uint64_t>(m),
                     static_cast<uint64_t>(w->columns) * 2, kStepK, static_cast<uint32_t>(bn))) {
    set_last_error_text("cuTensorMapEncodeTiled failed for the prefill activations");
    return QX_STATUS_DEVICE_ERROR;
  }
  Q4GemmParams p{};
  p.panel = w->panel;
  p.row_unscale = row_unscale;
  p.y = y_dev;
  p.m = m;
  p.rows = w->rows;
  p.ldy = ldy;
  p.slabs = static_cast<int>(w->slabs);
  p.bn = bn;
  p.o_tiles = static_cast<int>(w->tiles);
  p.r_tiles = static_cast<int>((m + bn - 1) / bn);
  p.error = ctx->error_dev;
  static SmemOptIn opt_in;
  QX_TRY(opt_in.ensure(q4_gemm_tc_kernel, kQ4GemmSmem));
  const long long tiles = static_cast<long long>(p.o_tiles) * p.r_tiles;
  const int grid = static_cast<int>(tiles < ctx->prop.multiProcessorCount
                                        ? tiles
                                        : ctx->prop.multiProcessorCount);
  q4_gemm_tc_kernel<<<grid, kThreads, kQ4GemmSmem, stream>>>(map_x, p);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

}  // namespace

const char* q4_gemm_variant_name() { return "sm100a_tcgen05_f16_dequant"; }

qx_status launch_q4_gemm_bf16(const qx_weights* w, const uint16_t* x_bf16_dev, float* y_dev,
                              long long m, long long ldy, qx_workspace* ws, cudaStream_t stream) {
  if (w->format == QX_FORMAT_Q4_0 && m >= 64 && w->tiles < (1LL << 20) && m < (1LL << 30) &&
      m * w->columns < (1LL << 40)) {
    return launch_tc(w, x_bf16_dev, y_dev, m, ldy, ws, stream);
  }
  // Exact path: widen the activations to f32 (bf16 -> f32 is exact) and reuse the f32
  // batched kernel; its scratch sits at the start of the workspace and the widened copy
  // behind it.
  const long long count = m * w->columns;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  GemvScratch scratch;
  QX_TRY(gemv_scratch_layout(w, static_cast<int>(m < kGemvMaxBatch ? m : kGemvMaxBatch),
                             ctx->prop.multiProcessorCount, &scratch));
  const size_t table_bytes = align_up(scratch.total_bytes, 256);
  QX_TRY(ws->reserve(table_bytes + static_cast<size_t>(count) * sizeof(float)));
  float* x_f32 = reinterpret_cast<float*>(static_cast<uint8_t*>(ws->base) + table_bytes);
  const unsigned grid = static_cast<unsigned>(min((count + 255) / 256, 4096LL));
  bf16_to_f32_kernel<<<grid, 256, 0, stream>>>(x_bf16_dev, x_f32, count);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return launch_qgemm_f32(w, x_f32, y_dev, m, ldy, ws, stream);
}

}  // namespace qx
