// W8A8 prefill GEMM on the 5th-generation tensor cores.
//
// Replaces int8_gemm_{ref,avx2,avx512_vnni}_kernel of the reference
// (kernels/quantization/int8_gemm_ref.cpp:9-32, int8_gemm_avx512.cpp:77-100):
//   acc[r,o] = sum_k W[o,k] * X[r,k]   (exact, int32 in TMEM)
//   Y[r,o]   = float(acc - zp[r]*row_sum[o]) * ws[o] * as[r]     (two rounded multiplies,
//              left to right, as int8_gemm_ref.cpp:28-29)
//
// Mapping. Both operands are K-contiguous, so both are "K-major" MMA operands and need
// no transposition. The WEIGHT tile is the MMA's A operand (128 output channels = 128
// TMEM lanes) and the ACTIVATION tile is B (up to 256 tokens = TMEM columns). With that
// orientation an epilogue thread owns one output channel and walks over tokens, so for a
// fixed token the 32 lanes of a warp store 32 consecutive floats of Y: fully coalesced
// stores without a shared-memory transpose.
//
// Pipeline (persistent CTAs, one per SM, 320 threads):
//   warp 0      TMA producer: 128-byte-swizzled K-slabs of W (128 x 128 B) and X
//               (BN x 128 B) into a 4-stage shared-memory ring (full/empty mbarriers)
//   warp 1      MMA issuer: one thread issues tcgen05.mma kind::i8 (K = 32 per
//               instruction, four per slab) into one of two TMEM accumulators
//   warps 2-9   epilogue: tcgen05.ld -> int->f32 -> scale -> global stores, overlapped
//               with the next tile's MMAs through the second accumulator
// No cluster launch and no multicast: every CTA loads its own operands.
//
// Work split. Whole tiles, round robin over the persistent CTAs. Optionally (see
// choose_stream_k) the (tile, K-slab) sequence is cut into equal contiguous ranges, one per
// CTA ("stream-K", 128-channel tiles), which keeps every SM busy when there are few tiles: a CTA whose range covers only part
// of a tile's K writes its exact int32 partial sums to scratch memory and counts itself
// in on the tile's counter; the CTA that completes the count adds the partial sums (an
// integer sum: the result does not depend on who finishes) and runs the scaling epilogue.
// Nobody waits for another CTA.

#include <cuda.h>

#include <cstdlib>
#include <mutex>

#include "qx_int8_gemm.cuh"
#include "qx_sm100.cuh"

namespace qx {

// ---- host: tensor-map encoding ------------------------------------------------------
namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = []() -> EncodeFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) !=
            cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return nullptr;
    }
    return reinterpret_cast<EncodeFn>(ptr);
  }();
  return fn;
}
}  // namespace

bool encode_tma_2d(CUtensorMap* map, CUtensorMapDataType dtype, int elem_bytes, const void* base,
                   uint64_t inner_elems, uint64_t rows, uint64_t row_stride_bytes,
                   uint32_t box_inner_elems, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  if (fn == nullptr) return false;
  (void)elem_bytes;
  const cuuint64_t dims[2] = {inner_elems, rows};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner_elems, box_rows};
  const cuuint32_t elem_strides[2] = {1, 1};
  return fn(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

namespace {

constexpr int kBM = 128;        // output channels per tile (MMA M, TMEM lanes)
constexpr int kBK = 128;        // bytes of K per pipeline stage (one swizzle atom)
constexpr int kMaxStages = 4;
__host__ __device__ constexpr int stages_for(int na) { return na == 1 ? 4 : 3; }
constexpr int kEpiWarps = 8;  // two per TMEM lane quarter, splitting the token columns
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kTmemCols = 512;  // two accumulators of up to 256 columns

struct TcParams {
  const float* ws;
  const float* as;
  const int32_t* row_sum;
  const int* zp;
  float* y;
  int32_t* acc;
  long long m, n, ldy;
  int k_slabs;   // ceil(k / 128)
  int bn;        // tokens per tile: multiple of 32, <= 256
  int o_tiles, r_tiles;
  int asymmetric;
  int stream_k;        // 1: contiguous (tile, K-slab) ranges per CTA; 0: whole tiles round robin
  int32_t* partial;    // [cta][2][bn][128] partial accumulators of split tiles (stream-K)
  int* tile_counters;  // [tiles], zero between launches (stream-K)
  int* error;    // device word, set non-zero when a bounded wait gave up
};

// One contiguous piece of work: K-slabs [ks0, ks1) of a tile.
struct Segment {
  int tile, ks0, ks1;
};
// The segments of one CTA, in order; every role walks the same sequence.
struct WorkIter {
  int stream_k, k_slabs, total_tiles, tile, stride;
  long long u, u_end;
  __device__ WorkIter(const TcParams& p) {
    stream_k = p.stream_k;
    k_slabs = p.k_slabs;
    total_tiles = p.o_tiles * p.r_tiles;
    tile = blockIdx.x;
    stride = gridDim.x;
    const long long units = static_cast<long long>(total_tiles) * k_slabs;
    u = blockIdx.x * units / gridDim.x;
    u_end = (blockIdx.x + 1LL) * units / gridDim.x;
  }
  __device__ bool next(Segment* s) {
    if (stream_k == 0) {
      if (tile >= total_tiles) return false;
      *s = Segment{tile, 0, k_slabs};
      tile += stride;
      return true;
    }
    if (u >= u_end) return false;
    s->tile = static_cast<int>(u / k_slabs);
    s->ks0 = static_cast<int>(u - static_cast<long long>(s->tile) * k_slabs);
    const long long rest = u_end - u;
    s->ks1 = rest < k_slabs - s->ks0 ? s->ks0 + static_cast<int>(rest) : k_slabs;
    u += s->ks1 - s->ks0;
    return true;
  }
};
// first unit of CTA c's stream-K range
__device__ __forceinline__ long long sk_range_start(long long c, long long units, long long ctas) {
  return c * units / ctas;
}

// 16-byte aligned and sized: the activation-scale tile behind it is read as float4
struct __align__(16) TcBarriers {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};

// NA = weight tiles of 128 channels per CTA tile. NA = 1: 128 x bn outputs, two TMEM
// accumulators (epilogue overlaps the next tile). NA = 2: 256 x bn outputs from one
// activation slab per step -- a third less operand traffic from L2 per MAC, which is what
// bounds this shape -- at the price of a single accumulator set (all 512 TMEM columns).
template <int NA>
__global__ void __launch_bounds__(kThreads, 1) int8_gemm_tc_kernel(
    const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
    const TcParams p) {
  constexpr uint32_t kAccBuffers = NA == 1 ? 2 : 1;
  constexpr int kStages = stages_for(NA);
  using namespace sm100;
  extern __shared__ uint8_t smem_raw[];
  // stage ring, 1024-byte aligned for the 128-byte swizzle
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t a_bytes = NA * kBM * kBK;
  const uint32_t b_bytes = static_cast<uint32_t>(p.bn) * kBK;
  const uint32_t stage_bytes = a_bytes + b_bytes;
  TcBarriers* bars = reinterpret_cast<TcBarriers*>(smem + kStages * stage_bytes);
  float* as_tile = reinterpret_cast<float*>(bars + 1);  // [2][256] activation scales
  int* zp_tile = reinterpret_cast<int*>(as_tile + 2 * 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &bars->abort_flag;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&bars->tmem_full[a], 1);
      mbar_init(&bars->tmem_empty[a], kEpiWarps);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_x);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  const int total_tiles = p.o_tiles * p.r_tiles;
  const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) |
                         (static_cast<uint32_t>(p.bn >> 3) << 17) |
                         (static_cast<uint32_t>(kBM >> 4) << 24);

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one()) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      WorkIter work(p);
      Segment seg;
      while (ok && work.next(&seg)) {
        const int tile = seg.tile;
        const int o0 = (tile / p.r_tiles) * (NA * kBM);
        const int r0 = (tile % p.r_tiles) * p.bn;
        for (int ks = seg.ks0; ks < seg.ks1; ++ks) {
          if (!mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * stage_bytes;
          mbar_arrive_expect_tx(&bars->full[stage], stage_bytes);
          tma_load_2d(sa, &map_w, &bars->full[stage], ks * kBK, o0);
          tma_load_2d(sa + a_bytes, &map_x, &bars->full[stage], ks * kBK, r0);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        *abort_flag = 1;
        report_error(p.error, 1);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (elect_one()) {
      uint32_t stage = 0, phase = 0, acc = 0, acc_phase = 0;
      bool ok = true;
      WorkIter work(p);
      Segment seg;
      while (ok && work.next(&seg)) {
        if (!mbar_wait(&bars->tmem_empty[acc], acc_phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * (NA * 256u);
        for (int ks = seg.ks0; ks < seg.ks1; ++ks) {
          if (!mbar_wait(&bars->full[stage], phase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t sa = smem_u32(smem + stage * stage_bytes);
          const uint64_t a_desc = make_sw128_kmajor_desc(sa);
          const uint64_t b_desc = make_sw128_kmajor_desc(sa + a_bytes);
#pragma unroll
          for (int kk = 0; kk < kBK / 32; ++kk) {
            // advance 32 bytes of K inside the swizzle atom: +2 in the (addr >> 4) field
#pragma unroll
            for (int na = 0; na < NA; ++na) {
              // weight tile `na` starts kBM rows (16 KiB) further into the slab
              mma_i8_ss(d_tmem + na * 256u,
                        a_desc + static_cast<uint64_t>(kk * 2 + na * ((kBM * kBK) >> 4)),
                        b_desc + static_cast<uint64_t>(kk * 2), idesc,
                        (ks != seg.ks0 || kk != 0) ? 1u : 0u);
            }
          }
          tc_commit(&bars->empty[stage]);  // frees the slab once the MMAs have read it
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tc_commit(&bars->tmem_full[acc]);
        if (++acc == kAccBuffers) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        report_error(p.error, 2);
      }
    }
  } else {
    // ------------------------------ epilogue ----------------------------------
    // Eight warps: warp w reads TMEM lanes 32*(w & 3).. (its channel quarter) and takes the
    // 32-token column chunks c with (c & 1) == half. A thread owns one output channel, so
    // for a fixed token the 32 lanes store 32 consecutive floats of Y.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int epi_thread = threadIdx.x - 64;  // 0..255
    uint32_t acc = 0, acc_phase = 0;
    bool ok = true;
    int* last_flag = zp_tile + 2 * 256;  // one word behind the staged tables
    // Scales one 32-token chunk of exact accumulators v[] (channel o, tokens rc..rc+31)
    // and stores it.
    auto store_chunk = [&](const uint32_t (&v)[32], long long o, long long rc, float wscale,
                           long long rsum, const float* sc, const int* zpc) {
      float* yp = p.y + rc * p.ldy + o;
      if (!p.asymmetric && p.acc == nullptr && rc + 32 <= p.m) {
        // common case: whole chunk in range, symmetric, no accumulator dump
#pragma unroll
        for (int j4 = 0; j4 < 32; j4 += 4) {
          const float4 s4 = *reinterpret_cast<const float4*>(sc + j4);
          const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const float f = __int2float_rn(static_cast<int>(v[j4 + jj]));
            *yp = __fmul_rn(__fmul_rn(f, wscale), sv[jj]);
            yp += p.ldy;
          }
        }
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const long long r = rc + j;
          if (r < p.m) {
            const int raw = static_cast<int>(v[j]);
            float f;
            if (p.asymmetric) {
              const long long dot = static_cast<long long>(raw) - zpc[j] * rsum;
              f = __ll2float_rn(dot);
              if (p.acc != nullptr) p.acc[r * p.n + o] = static_cast<int32_t>(dot);
            } else {
              f = __int2float_rn(raw);
              if (p.acc != nullptr) p.acc[r * p.n + o] = raw;
            }
            p.y[r * p.ldy + o] = __fmul_rn(__fmul_rn(f, wscale), sc[j]);
          }
        }
      }
    };
    WorkIter work(p);
    Segment seg;
    const long long units = static_cast<long long>(total_tiles) * p.k_slabs;
    while (ok && work.next(&seg)) {
      const int tile = seg.tile;
      const bool whole = seg.ks0 == 0 && seg.ks1 == p.k_slabs;
      const long long o_base = static_cast<long long>(tile / p.r_tiles) * (NA * kBM) + quarter * 32 + lane;
      const long long r0 = static_cast<long long>(tile % p.r_tiles) * p.bn;
      // stage this tile's activation scales (and zero points) for broadcast reads
      float* as_s = as_tile + acc * 256;
      int* zp_s = zp_tile + acc * 256;
      for (int i = epi_thread; i < p.bn; i += 32 * kEpiWarps) {
        const long long r = r0 + i;
        as_s[i] = r < p.m ? p.as[r] : 0.0f;
        zp_s[i] = (p.asymmetric && r < p.m) ? p.zp[r] : 0;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");  // epilogue warps only

      if (!mbar_wait(&bars->tmem_full[acc], acc_phase, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const int chunks = p.bn / 32;
      if (whole) {
#pragma unroll
        for (int na = 0; na < NA; ++na) {
          const long long o = o_base + na * kBM;
          const bool o_ok = o < p.n;
          const float wscale = o_ok ? p.ws[o] : 0.0f;
          const long long rsum = (p.asymmetric && o_ok) ? p.row_sum[o] : 0;
          for (int c = half; c < chunks; c += 2) {
            uint32_t v[32];
            const uint32_t taddr = tmem_base + (acc * NA + na) * 256u + static_cast<uint32_t>(c * 32) +
                                   (static_cast<uint32_t>(quarter * 32) << 16);
            tmem_ld_32x32(taddr, v);
            tmem_ld_wait();
            if (!o_ok) continue;
            store_chunk(v, o, r0 + c * 32, wscale, rsum, as_s + c * 32, zp_s + c * 32);
          }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);
      } else {
        // Part of a tile's K range (stream-K, NA == 1): publish the partial sums, count in,
        // and finish the tile if every other part has been counted in already.
        const int ch = quarter * 32 + lane;  // channel within the tile
        const int my_slot = seg.ks0 != 0 ? 0 : 1;
        int32_t* mine = p.partial + (static_cast<long long>(blockIdx.x) * 2 + my_slot) * (256 * kBM);
        for (int c = half; c < chunks; c += 2) {
          uint32_t v[32];
          const uint32_t taddr = tmem_base + acc * 256u + static_cast<uint32_t>(c * 32) +
                                 (static_cast<uint32_t>(quarter * 32) << 16);
          tmem_ld_32x32(taddr, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) mine[(c * 32 + j) * kBM + ch] = static_cast<int32_t>(v[j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bars->tmem_empty[acc]);  // accumulator no longer needed
        __threadfence();
        asm volatile("bar.sync 1, 256;" ::: "memory");
        // the CTAs whose ranges touch this tile: first..last
        const long long tile_first = static_cast<long long>(tile) * p.k_slabs;
        const long long tile_last = tile_first + p.k_slabs - 1;
        int c_first = static_cast<int>(tile_first * gridDim.x / units);
        while (sk_range_start(c_first + 1LL, units, gridDim.x) <= tile_first) ++c_first;
        while (sk_range_start(c_first, units, gridDim.x) > tile_first) --c_first;
        int c_last = static_cast<int>(tile_last * gridDim.x / units);
        while (sk_range_start(c_last + 1LL, units, gridDim.x) <= tile_last) ++c_last;
        while (sk_range_start(c_last, units, gridDim.x) > tile_last) --c_last;
        if (epi_thread == 0) {
          const int old = atomicAdd(p.tile_counters + tile, 1);
          const int last = old + 1 == c_last - c_first + 1 ? 1 : 0;
          if (last) p.tile_counters[tile] = 0;  // for the next launch
          __threadfence();
          *last_flag = last;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (*last_flag != 0) {
          const long long o = o_base;
          const bool o_ok = o < p.n;
          const float wscale = o_ok ? p.ws[o] : 0.0f;
          const long long rsum = (p.asymmetric && o_ok) ? p.row_sum[o] : 0;
          for (int c = half; c < chunks && o_ok; c += 2) {
            uint32_t v[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
            for (int cta = c_first; cta <= c_last; ++cta) {
              // that CTA's piece of this tile starts mid-tile (slot 0) or at K = 0 (slot 1)
              const int slot = sk_range_start(cta, units, gridDim.x) > tile_first ? 0 : 1;
              const int32_t* part = p.partial + (static_cast<long long>(cta) * 2 + slot) * (256 * kBM);
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                v[j] += static_cast<uint32_t>(__ldcg(part + (c * 32 + j) * kBM + ch));
              }
            }
            store_chunk(v, o, r0 + c * 32, wscale, rsum, as_s + c * 32, zp_s + c * 32);
          }
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");  // last_flag is reused by the next part
      }
      if (++acc == kAccBuffers) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (!ok) {
      *abort_flag = 1;
      report_error(p.error, 3);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

size_t tc_smem_bytes(int na, int bn) {
  return 1024 + static_cast<size_t>(stages_for(na)) * (na * kBM * kBK + bn * kBK) + sizeof(TcBarriers) +
         2 * 256 * sizeof(float) + 2 * 256 * sizeof(int) + 16 + 64;
}

}  // namespace

bool int8_gemm_tc_supported(const Int8GemmArgs& a) {
  if (a.k % 16 != 0 || a.k > 131000) return false;  // TMA row stride; int32 exactness
  if ((reinterpret_cast<uintptr_t>(a.w) | reinterpret_cast<uintptr_t>(a.x)) & 15u) return false;
  if (a.m > (1LL << 30) || a.n > (1LL << 30)) return false;
  return encode_fn() != nullptr;
}

namespace {
template <int NA>
qx_status launch_tc_na(const CUtensorMap& map_w, const CUtensorMap& map_x, const TcParams& p,
                       int grid, cudaStream_t stream) {
  static SmemOptIn opt_in;
  QX_TRY(opt_in.ensure(int8_gemm_tc_kernel<NA>, tc_smem_bytes(NA, 256)));
  int8_gemm_tc_kernel<NA><<<grid, kThreads, tc_smem_bytes(NA, p.bn), stream>>>(map_w, map_x, p);
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

// Scratch of the stream-K split, one per device, kept for the life of the process:
// partial accumulators of 2 pieces per CTA and the tile counters (zero between launches).
constexpr int kStreamKMaxCtas = 256;
constexpr long long kStreamKMaxTiles = 1 << 20;
struct StreamKScratch {
  int32_t* partial = nullptr;
  int* counters = nullptr;
};
StreamKScratch g_stream_k[64];
std::mutex g_stream_k_mutex;

qx_status stream_k_scratch(int device, StreamKScratch* out) {
  if (device < 0 || device >= 64) return QX_STATUS_DEVICE_ERROR;
  std::lock_guard<std::mutex> lock(g_stream_k_mutex);
  StreamKScratch& s = g_stream_k[device];
  if (s.partial == nullptr) {
    const size_t partial_bytes = static_cast<size_t>(kStreamKMaxCtas) * 2 * 256 * kBM * sizeof(int32_t);
    const size_t counter_bytes = static_cast<size_t>(kStreamKMaxTiles) * sizeof(int);
    void* block = nullptr;
    cudaError_t err = cudaMalloc(&block, partial_bytes + counter_bytes);
    if (err != cudaSuccess) {
      set_last_error("cudaMalloc(stream-K scratch)", err);
      return err == cudaErrorMemoryAllocation ? QX_STATUS_OUT_OF_MEMORY : QX_STATUS_DEVICE_ERROR;
    }
    err = cudaMemset(static_cast<uint8_t*>(block) + partial_bytes, 0, counter_bytes);
    if (err != cudaSuccess) {
      set_last_error("cudaMemset(stream-K counters)", err);
      (void)cudaFree(block);
      return QX_STATUS_DEVICE_ERROR;
    }
    s.partial = static_cast<int32_t*>(block);
    s.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(block) + partial_bytes);
  }
  *out = s;
  return QX_STATUS_OK;
}

// The stream-K split is opt-in (QX_B200_INT8_STREAM_K=1). On the benchmark's prefill shape
// (112 tiles of 256 channels, 148 SMs, 28 us) publishing and re-reading 128 KiB partial sums
// per split tile costs more than the idle last wave it removes (43 us against 27.5 us), so
// whole tiles stay the default; it pays only when a tile's K loop is long against that.
bool choose_stream_k(long long tiles128, int k_slabs, int sm_count) {
  const char* forced = std::getenv("QX_B200_INT8_STREAM_K");
  if (forced == nullptr || forced[0] != '1') return false;
  return tiles128 * k_slabs >= sm_count && tiles128 <= kStreamKMaxTiles;
}

// weight tiles per CTA tile: 2 (256 channels) when that still gives most SMs a tile
int choose_weight_tiles(long long n, long long r_tiles, int sm_count) {
  if (const char* forced = std::getenv("QX_B200_INT8_WEIGHT_TILES")) {
    if (forced[0] == '1') return 1;
    if (forced[0] == '2') return 2;
  }
  const long long tiles2 = (n + 2 * kBM - 1) / (2 * kBM) * r_tiles;
  return tiles2 * 10 >= static_cast<long long>(sm_count) * 6 ? 2 : 1;
}
}  // namespace

qx_status launch_int8_gemm_tc(const Int8GemmArgs& a, cudaStream_t stream) {
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  int bn = 256;
  if (a.m < 256) bn = static_cast<int>((a.m + 31) / 32 * 32);
  const long long r_tiles = (a.m + bn - 1) / bn;
  const int k_slabs = static_cast<int>((a.k + kBK - 1) / kBK);
  const int sm_count = ctx->prop.multiProcessorCount;
  const bool stream_k = sm_count <= kStreamKMaxCtas &&
                        choose_stream_k((a.n + kBM - 1) / kBM * r_tiles, k_slabs, sm_count);
  const int na = stream_k ? 1 : choose_weight_tiles(a.n, r_tiles, sm_count);
  CUtensorMap map_w, map_x;
  if (!encode_tma_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.w, static_cast<uint64_t>(a.k),
                     static_cast<uint64_t>(a.n), static_cast<uint64_t>(a.k), kBK,
                     static_cast<uint32_t>(na * kBM)) ||
      !encode_tma_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, a.x, static_cast<uint64_t>(a.k),
                     static_cast<uint64_t>(a.m), static_cast<uint64_t>(a.k), kBK,
                     static_cast<uint32_t>(bn))) {
    set_last_error_text("cuTensorMapEncodeTiled failed for the W8A8 operands");
    return QX_STATUS_DEVICE_ERROR;
  }
  TcParams p{};
  p.ws = a.ws;
  p.as = a.as;
  p.row_sum = a.row_sum;
  p.zp = a.zp;
  p.y = a.y;
  p.acc = a.acc;
  p.m = a.m;
  p.n = a.n;
  p.ldy = a.ldy;
  p.k_slabs = static_cast<int>((a.k + kBK - 1) / kBK);
  p.bn = bn;
  p.o_tiles = static_cast<int>((a.n + na * kBM - 1) / (na * kBM));
  p.r_tiles = static_cast<int>(r_tiles);
  p.asymmetric = a.asymmetric ? 1 : 0;
  p.error = ctx->error_dev;
  const long long tiles = static_cast<long long>(p.o_tiles) * p.r_tiles;
  p.stream_k = stream_k ? 1 : 0;
  if (stream_k) {
    StreamKScratch scratch;
    QX_TRY(stream_k_scratch(ctx->device, &scratch));
    p.partial = scratch.partial;
    p.tile_counters = scratch.counters;
  }
  const int grid = static_cast<int>(stream_k || tiles >= sm_count ? sm_count : tiles);
  return na == 2 ? launch_tc_na<2>(map_w, map_x, p, grid, stream)
                 : launch_tc_na<1>(map_w, map_x, p, grid, stream);
}

}  // namespace qx
