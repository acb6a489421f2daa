// Decode GEMV / small-batch qgemm on the tensor cores (tcgen05 kind::i8 + TMEM).
//
// Why tensor cores for a GEMV: at HBM speed one SM must consume ~22 bytes of packed
// weights per clock, i.e. 1.2 q4_0 blocks of 32 weights. Dequantising and multiplying
// those on the CUDA cores needs ~90 instructions per block -- the whole issue budget.
// Here the 8-bit products run on the tensor core instead: the weight codes are the MMA's
// A operand (128 weight rows x 32 codes of one block), the activation digits (three
// balanced base-256 digits per activation, see qx_gemv.cuh) are the B operand (8..128
// digit columns), and one MMA per block leaves the three exact integer block sums of 128
// rows in TMEM. The CUDA cores only combine the digits and apply the fp16 block scale:
// ~10 instructions per block.
//
// One K-slab (4 blocks = 128 elements of 128 rows) per pipeline stage:
//   q8_0  the 16 KiB code slab is one TMA tile (128-byte swizzle) straight from the panel
//   q4_0  the 8 KiB packed slab is one bulk copy into a deep ring of packed slabs (the
//         bytes in flight); eight producer warps read it back, split the nibbles and store
//         the unsigned codes into the same swizzled layout the TMA tile would have
//   both  the activation digit slab (TMA) and the slab's 512 fp16 scales (bulk copy)
// Warp roles: 0 = TMA producer, 1 = MMA issuer (one thread), 2-9 = epilogue (thread =
// weight row, accumulators in registers; two sets of four warps take alternate K units),
// then for q4_0 one unpack warp per stage and a packed-slab loader warp (its own warp: a
// waiting lane would stall the other lanes of its warp).
//
// Work split and summation order. K is cut into units of `unit_slabs` slabs, a function of
// K alone. A row's result is defined as the sum, in ascending order, of its unit sums,
// each accumulated block by block from zero -- so it does not depend on the number of
// rows, on how rows are sharded over GPUs, on the batch size or on the SM count. The
// (row tile, unit) sequence is cut into equal contiguous ranges, one per persistent CTA,
// so every SM streams the same number of bytes. A row's even and odd units are summed
// separately (two sets of epilogue warps take alternate units) and added at the end. A
// CTA that owns all units of a tile sums them in registers; a tile shared by several CTAs
// goes through per-unit partial sums in scratch memory. Either way each thread counts
// its share in on a per-row counter and the thread that completes the count adds the
// pieces in the fixed order: no thread waits for another one.

#include <cuda.h>

#include "qx_gemv_tc.cuh"
#include "qx_sm100.cuh"

namespace qx {
namespace {

using namespace sm100;

constexpr int kABytes = kTileRows * 128;  // unpacked code slab in shared memory
constexpr int kSBytes = kSlabBlocks * kTileRows * 2;
constexpr int kEpilogueWarps = 8;   // two sets of four (one warp per TMEM lane quarter)
constexpr int kFirstUnpackWarp = 2 + kEpilogueWarps;
constexpr int kRawBytes = kTileRows * kSlabBlocks * 16 + kSBytes;  // packed q4_0 slab + scales (9 KiB)
constexpr int kQ8SpanRows = (kABytes + kSBytes) / 128;              // q8_0 slab span as 128-byte rows

template <int FMT, int NMMA>
struct TcGeom {
  static constexpr int kBBytes = NMMA * 128;
  static constexpr int kMaxM = NMMA / kDigitStride;
  static constexpr int kXBytes = NMMA * 144;  // activation slab image: digit rows + constants
  // stage: [codes 16 KiB][scales 1 KiB][activation image], padded to the swizzle atom
  static constexpr int kStageBytes = (kABytes + kSBytes + kXBytes + 1023) / 1024 * 1024;
  // q8_0: the stage ring itself holds the bytes in flight. q4_0: every stage is paired with
  // a packed-slab buffer filled by a bulk copy (the bytes in flight) and owned by one
  // unpack warp, so up to eight slabs are being unpacked at the same time.
  static constexpr int kBudget = FMT == QX_FORMAT_Q4_0 ? 224 * 1024 : 200 * 1024;
  static constexpr int kPerStage = kStageBytes + (FMT == QX_FORMAT_Q4_0 ? kRawBytes : 0);
  static constexpr int kStages = kBudget / kPerStage > 8 ? 8 : kBudget / kPerStage;
  static constexpr int kRawStages = FMT == QX_FORMAT_Q4_0 ? kStages : 0;
  // warps: TMA, MMA, 8 epilogue, then for q4_0 one unpack warp per stage and the loader
  static constexpr int kThreads = 32 * (2 + kEpilogueWarps + (FMT == QX_FORMAT_Q4_0 ? kStages + 1 : 0));
  static constexpr int kColStride = NMMA <= 32 ? 32 : NMMA;  // TMEM columns per block
  static constexpr int kBlocksPerT = NMMA <= 64 ? 4 : 2;   // blocks per TMEM stage
  static constexpr int kTCols = kBlocksPerT * kColStride;  // 128 or 256
  static constexpr int kTStages = 512 / kTCols;            // 4 or 2
  // Each epilogue set has its own ring of TMEM stages, so every TMEM barrier is used by
  // one set only (a parity wait cannot tell apart phases two steps apart).
  static constexpr int kTPerSet = kTStages / 2;           // 2 or 1
  // blocks whose TMEM loads are issued before one wait (register budget: 64 values)
  static constexpr int kLdBatch = NMMA <= 16 ? 4 : (NMMA == 32 ? 2 : 1);
};

struct GemvTcParams {
  const uint8_t* panel;          // [tile][slab]{codes, scales}; q4_0 is read by bulk copies
  const uint8_t* ximg;           // [slab] activation images (ximage_bytes(NMMA) each)
  float* y;
  float* partial;                // [tile][slot][m][128], slot = K unit (or even/odd sum)
  int* counters;                 // [tile][128], one per weight row
  int* error;
  long long ldy, rows;
  int m, nbpad, slabs, tiles;
  int unit_slabs, units_per_tile;  // K split: units of unit_slabs slabs
  int slots_per_tile;              // max(units_per_tile, 2)
  long long total_units;
  long long* debug;  // [ctas][16] cycle counters, profiling builds only
};

template <int FMT, int NMMA>
struct __align__(8) GemvBarriers {
  uint64_t full[TcGeom<FMT, NMMA>::kStages];
  uint64_t empty[TcGeom<FMT, NMMA>::kStages];
  uint64_t tmem_full[TcGeom<FMT, NMMA>::kTStages];
  uint64_t tmem_empty[TcGeom<FMT, NMMA>::kTStages];
  uint64_t raw_full[12];
  uint64_t raw_empty[12];
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
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&v)[N]);
template <>
__device__ __forceinline__ void tmem_ld_cols<8>(uint32_t taddr, uint32_t (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
                 "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_cols<16>(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
template <>
__device__ __forceinline__ void tmem_ld_cols<32>(uint32_t taddr, uint32_t (&v)[32]) {
  tmem_ld_32x32(taddr, v);
}

// start of CTA c's slab range
__device__ __forceinline__ long long range_start(long long c, long long total, long long ctas) {
  return c * total / ctas;
}
template <int FMT, int NMMA>
__global__ void __launch_bounds__((TcGeom<FMT, NMMA>::kThreads), 1)
gemv_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const GemvTcParams p) {
  using G = TcGeom<FMT, NMMA>;
  constexpr bool kQ4 = FMT == QX_FORMAT_Q4_0;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* raw_ring = smem + G::kStages * G::kStageBytes;  // q4_0 only
  auto* bars = reinterpret_cast<GemvBarriers<FMT, NMMA>*>(raw_ring + G::kRawStages * kRawBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &bars->abort_flag;
  // kernels queued behind this one may be scheduled as soon as SMs free up; whatever they
  // touch of this kernel's data they guard with their own griddepcontrol.wait
  asm volatile("griddepcontrol.launch_dependents;");

  if (threadIdx.x == 0) {
    for (int s = 0; s < G::kStages; ++s) {
      mbar_init(&bars->full[s], kQ4 ? 2 : 1);  // TMA bytes (+ the stage's unpack warp)
      mbar_init(&bars->empty[s], 1 + 4);  // MMA commit + four epilogue warps (scales read)
    }
    for (int t = 0; t < G::kTStages; ++t) {
      mbar_init(&bars->tmem_full[t], 1);
      mbar_init(&bars->tmem_empty[t], 4);
    }
    for (int r = 0; r < G::kRawStages; ++r) {
      mbar_init(&bars->raw_full[r], 1);
      mbar_init(&bars->raw_empty[r], 1);
    }
    bars->abort_flag = 0;
    mbar_fence_init();
    if (!kQ4) prefetch_tensormap(&map_a);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  const long long u_begin = range_start(blockIdx.x, p.total_units, gridDim.x);
  const long long u_end = range_start(blockIdx.x + 1LL, p.total_units, gridDim.x);
  // units tile every row tile's slabs contiguously, so a CTA's units are one contiguous
  // range of global slabs (tile * slabs + slab)
  long long s_begin = 0, s_end = 0;
  if (u_end > u_begin) {
    const long long last = u_end - 1;
    const int last_end = static_cast<int>(last % p.units_per_tile + 1) * p.unit_slabs;
    s_begin = (u_begin / p.units_per_tile) * p.slabs + (u_begin % p.units_per_tile) * p.unit_slabs;
    s_end = (last / p.units_per_tile) * p.slabs + (last_end < p.slabs ? last_end : p.slabs);
  }

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      QX_PROF_DECL(w_empty);
      const long long t_start = QX_PROF_NOW();
      int slab = static_cast<int>(s_begin % p.slabs);
      // the activation images are written by the preceding kernel in the stream
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (long long gs = s_begin; gs < s_end; ++gs, slab = slab + 1 == p.slabs ? 0 : slab + 1) {
        if (!QX_PROF_WAIT(w_empty, mbar_wait(&bars->empty[stage], phase ^ 1u, abort_flag))) {
          ok = false;
          break;
        }
        uint8_t* st = smem + stage * G::kStageBytes;
        mbar_arrive_expect_tx(&bars->full[stage], (kQ4 ? 0 : kABytes + kSBytes) + G::kXBytes);
        if (!kQ4) {
          // codes and scales of the slab: one tile of 136 rows x 128 bytes
          tma_load_2d(st, &map_a, &bars->full[stage], 0, static_cast<int>(gs * kQ8SpanRows));
        }
        bulk_copy_g2s(st + kABytes + kSBytes, p.ximg + static_cast<long long>(slab) * G::kXBytes,
                      G::kXBytes, &bars->full[stage]);
        if (++stage == G::kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      QX_PROF_STORE(0, w_empty);
      QX_PROF_STORE(1, QX_PROF_NOW() - t_start);
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error, 11);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (elect_one()) {
      const uint32_t idesc = (2u << 4) | ((kQ4 ? 0u : 1u) << 7) | (1u << 10) |
                             (static_cast<uint32_t>(NMMA >> 3) << 17) |
                             (static_cast<uint32_t>(kTileRows >> 4) << 24);
      uint32_t stage = 0, phase = 0;
      uint32_t ring_pos[2] = {0, 0}, ring_phase[2] = {0, 0};  // per epilogue set
      bool ok = true;
      QX_PROF_DECL(w_full);
      QX_PROF_DECL(w_tempty);
      int slab = static_cast<int>(s_begin % p.slabs);
      int unit = slab / p.unit_slabs;
      int slab_in_unit = slab - unit * p.unit_slabs;
      for (long long gs = s_begin; gs < s_end && ok; ++gs) {
        const int eset = unit & 1;
        uint32_t ts = eset * G::kTPerSet + ring_pos[eset];
        uint32_t tphase = ring_phase[eset];
        if (!QX_PROF_WAIT(w_full, mbar_wait(&bars->full[stage], phase, abort_flag))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + stage * G::kStageBytes);
        const uint64_t a_desc = make_sw128_kmajor_desc(sa);
        const uint64_t b_desc = make_sw128_kmajor_desc(sa + kABytes + kSBytes);
#pragma unroll
        for (int j = 0; j < kSlabBlocks; ++j) {
          if (j % G::kBlocksPerT == 0) {
            if (!QX_PROF_WAIT(w_tempty, mbar_wait(&bars->tmem_empty[ts], tphase ^ 1u, abort_flag))) {
              ok = false;
              break;
            }
            tc_fence_after_sync();
          }
          const uint32_t d_tmem = tmem_base + ts * G::kTCols + (j % G::kBlocksPerT) * G::kColStride;
          // one block = 32 bytes of K inside the swizzle atom: +2 in the (addr >> 4) field
          mma_i8_ss(d_tmem, a_desc + static_cast<uint64_t>(2 * j),
                    b_desc + static_cast<uint64_t>(2 * j), idesc, 0u);
          if (j % G::kBlocksPerT == G::kBlocksPerT - 1) {
            tc_commit(&bars->tmem_full[ts]);
            if (++ring_pos[eset] == G::kTPerSet) {
              ring_pos[eset] = 0;
              ring_phase[eset] ^= 1u;
            }
            ts = eset * G::kTPerSet + ring_pos[eset];
            tphase = ring_phase[eset];
          }
        }
        if (!ok) break;
        tc_commit(&bars->empty[stage]);
        if (++stage == G::kStages) {
          stage = 0;
          phase ^= 1u;
        }
        if (++slab == p.slabs) {
          slab = 0;
          unit = 0;
          slab_in_unit = 0;
        } else if (++slab_in_unit == p.unit_slabs) {
          slab_in_unit = 0;
          ++unit;
        }
      }
      QX_PROF_STORE(2, w_full);
      QX_PROF_STORE(3, w_tempty);
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error, 12);
      }
    }
  } else if (warp < 2 + kEpilogueWarps) {
    // ------------------------------ epilogue ----------------------------------
    // Two sets of four warps; set e takes the K units with (unit & 1) == e, so while one
    // set waits on barriers, TMEM loads and conversions the other one issues. A row's
    // result is (sum of even units, ascending) + (sum of odd units, ascending).
    const int eset = (warp - 2) >> 2;
    const int quarter = warp & 3;
    const int row_in_tile = quarter * 32 + lane;
    const int epi_thread = threadIdx.x - 64;
    float acc[G::kMaxM], total[G::kMaxM];  // current unit; units of a tile this CTA owns
#pragma unroll
    for (int m = 0; m < G::kMaxM; ++m) acc[m] = total[m] = 0.0f;
    // byte offset of this row's scale of block j inside the stage's 1 KiB scale area. q4_0:
    // linear [block][row] (copied by the unpack warp). q8_0: the area arrived as rows
    // 128..135 of the swizzled TMA tile, so 16-byte chunks are permuted by the row index.
    auto scale_offset = [&](int j) {
      const int linear = (j * kTileRows + row_in_tile) * 2;
      if (kQ4) return linear;
      const int r128 = linear >> 7, chunk = (linear >> 4) & 7;
      return r128 * 128 + ((chunk ^ (r128 & 7)) << 4) + (linear & 15);
    };
    int units_mine = 0;  // units of the current split tile this thread has written
    // deferred completion check of the last published share
    int pend_old = 0, pend_add = 0, pend_tile = 0, pend_target = 0;
    bool pend_owned = false;
    auto resolve_pending = [&]() {
      if (pend_add > 0 && pend_old + pend_add == pend_target) {
        const long long row = static_cast<long long>(pend_tile) * kTileRows + row_in_tile;
        const float* slots = p.partial + (static_cast<long long>(pend_tile) * p.slots_per_tile *
                                          p.m) * kTileRows;
        const int count = pend_owned ? 2 : p.units_per_tile;
#pragma unroll
        for (int m = 0; m < G::kMaxM; ++m) {
          if (m < p.m) {
            // owned tiles hold (even sum, odd sum); split tiles hold one sum per unit
            float even = 0.0f, odd = 0.0f;
            for (int u = 0; u < count; u += 2) {
              even += __ldcg(slots + (static_cast<long long>(u) * p.m + m) * kTileRows + row_in_tile);
            }
            for (int u = 1; u < count; u += 2) {
              odd += __ldcg(slots + (static_cast<long long>(u) * p.m + m) * kTileRows + row_in_tile);
            }
            if (row < p.rows) p.y[m * p.ldy + row] = even + odd;
          }
        }
        p.counters[static_cast<long long>(pend_tile) * kTileRows + row_in_tile] = 0;  // next launch
      }
      pend_add = 0;
    };
    uint32_t stage = 0, phase = 0, ring_pos = 0, tphase = 0;
    uint32_t ts = eset * G::kTPerSet;
    bool ok = true;
    QX_PROF_DECL(w_tfull);
    QX_PROF_DECL(w_sfull);
    const long long t_start = QX_PROF_NOW();
    int tile = static_cast<int>(s_begin / p.slabs);
    int slab = static_cast<int>(s_begin - static_cast<long long>(tile) * p.slabs);
    int unit = slab / p.unit_slabs;
    int slab_in_unit = slab - unit * p.unit_slabs;
    for (long long gs = s_begin; gs < s_end && ok; ++gs) {
      const bool mine = (unit & 1) == eset;
      if (mine) {
      const uint8_t* stage_base = smem + stage * G::kStageBytes;
      const int4* xcs = reinterpret_cast<const int4*>(stage_base + kABytes + kSBytes + G::kBBytes);
      constexpr int kChunk = NMMA <= 32 ? NMMA : 32;
      constexpr int kChunksPerBlock = NMMA / kChunk;
      float dsc[kSlabBlocks];
#pragma unroll
      for (int jb = 0; jb < kSlabBlocks; jb += G::kLdBatch) {
        if (jb % G::kBlocksPerT == 0) {
          if (!QX_PROF_WAIT(w_tfull, mbar_wait(&bars->tmem_full[ts], tphase, abort_flag))) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (jb == 0) {
            // the stage's barrier completed before the MMAs ran; waiting on it here makes
            // the bulk-copied scales and block constants visible to this thread
            if (!QX_PROF_WAIT(w_sfull, mbar_wait(&bars->full[stage], phase, abort_flag))) {
              ok = false;
              break;
            }
#pragma unroll
            for (int j = 0; j < kSlabBlocks; ++j) {
              dsc[j] = half_bits_to_float(*reinterpret_cast<const unsigned short*>(
                  stage_base + kABytes + scale_offset(j)));
            }
          }
        }
#pragma unroll
        for (int ch = 0; ch < kChunksPerBlock; ch += 2) {
          // issue the loads of this batch (up to 64 values), then wait once
          uint32_t v[G::kLdBatch * (kChunksPerBlock > 1 ? 2 : 1)][kChunk];
#pragma unroll
          for (int jj = 0; jj < G::kLdBatch; ++jj) {
            const int j = jb + jj;
            const uint32_t taddr = tmem_base + ts * G::kTCols +
                                   (j % G::kBlocksPerT) * G::kColStride +
                                   (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
            for (int c = 0; c < (kChunksPerBlock > 1 ? 2 : 1); ++c) {
              const int c0 = (ch + c) * kChunk;
              if (c0 < kDigitStride * p.m) {  // warp-uniform: later columns are unused
                tmem_ld_cols<kChunk>(taddr + c0, v[jj * (kChunksPerBlock > 1 ? 2 : 1) + c]);
              }
            }
          }
          tmem_ld_wait();
          const bool last_of_tstage =
              (jb + G::kLdBatch) % G::kBlocksPerT == 0 && ch + 2 >= kChunksPerBlock;
          if (last_of_tstage) {  // values are in registers: hand the TMEM stage back now
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->tmem_empty[ts]);
          }
#pragma unroll
          for (int jj = 0; jj < G::kLdBatch; ++jj) {
            const int j = jb + jj;
#pragma unroll
            for (int c = 0; c < (kChunksPerBlock > 1 ? 2 : 1); ++c) {
              const int c0 = (ch + c) * kChunk;
#pragma unroll
              for (int mm = 0; mm < kChunk / kDigitStride; ++mm) {
                const int m = c0 / kDigitStride + mm;  // columns 4m..4m+2 hold its digits
                if (m < p.m) {
                  const int4 raw = xcs[m * kSlabBlocks + j];
                  const uint32_t* vv4 = v[jj * (kChunksPerBlock > 1 ? 2 : 1) + c];
                  const int s0 = static_cast<int>(vv4[kDigitStride * mm]);
                  const int s1 = static_cast<int>(vv4[kDigitStride * mm + 1]);
                  const int s2 = static_cast<int>(vv4[kDigitStride * mm + 2]);
                  const int u = s1 * 256 + s0 - (kQ4 ? raw.y : 0);
                  const int hi = s2 - (kQ4 ? raw.z : 0);
                  acc[m] = fmaf(combine_digits(u, hi), __fmul_rn(dsc[j], __int_as_float(raw.x)),
                                acc[m]);
                }
              }
            }
          }
          if (last_of_tstage) {
            if (++ring_pos == G::kTPerSet) {
              ring_pos = 0;
              tphase ^= 1u;
            }
            ts = eset * G::kTPerSet + ring_pos;
          }
        }
      }
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->empty[stage]);  // scales / constants consumed
      }
      if (++stage == G::kStages) {
        stage = 0;
        phase ^= 1u;
      }

      // ---- unit / tile boundaries ----
      const bool unit_end = slab_in_unit + 1 == p.unit_slabs || slab == p.slabs - 1;
      if (unit_end) {
        const long long tile_first = gs - slab;
        const bool owns_tile = s_begin <= tile_first && s_end >= tile_first + p.slabs;
        float* tile_slots = p.partial + (static_cast<long long>(tile) * p.slots_per_tile * p.m) *
                                            kTileRows;
        if (mine) {
          if (owns_tile) {
#pragma unroll
            for (int m = 0; m < G::kMaxM; ++m) {
              total[m] += acc[m];
              acc[m] = 0.0f;
            }
          } else {
            float* part = tile_slots + static_cast<long long>(unit) * p.m * kTileRows;
#pragma unroll
            for (int m = 0; m < G::kMaxM; ++m) {
              if (m < p.m) part[m * kTileRows + row_in_tile] = acc[m];
              acc[m] = 0.0f;
            }
            ++units_mine;
          }
        }
        const bool share_end = slab == p.slabs - 1 || gs == s_end - 1;
        if (share_end) {
          // Publish this thread's share of the row and count it in on the row's counter
          // (release); whoever completes the count finishes the row (acquire). Rows are
          // independent, so no thread ever waits for another one here, and the result of
          // the atomic is only looked at one share later (or after the loop).
          resolve_pending();
          int add = units_mine;
          if (owns_tile) {
            // the sums of the even and of the odd units go to slots 0 and 1
            float* slot = tile_slots + static_cast<long long>(eset) * p.m * kTileRows;
#pragma unroll
            for (int m = 0; m < G::kMaxM; ++m)
              if (m < p.m) slot[m * kTileRows + row_in_tile] = total[m];
            add = 1;
          }
          if (add > 0) {
            int* counter = p.counters + static_cast<long long>(tile) * kTileRows + row_in_tile;
            asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], %2;"
                         : "=r"(pend_old)
                         : "l"(counter), "r"(add)
                         : "memory");
            pend_add = add;
            pend_tile = tile;
            pend_target = owns_tile ? 2 : p.units_per_tile;
            pend_owned = owns_tile;
          }
          units_mine = 0;
#pragma unroll
          for (int m = 0; m < G::kMaxM; ++m) total[m] = 0.0f;
        }
      }
      // advance (tile, slab, unit) without divisions
      if (++slab == p.slabs) {
        slab = 0;
        ++tile;
        unit = 0;
        slab_in_unit = 0;
      } else if (++slab_in_unit == p.unit_slabs) {
        slab_in_unit = 0;
        ++unit;
      }
    }
    resolve_pending();
    if (epi_thread == 0) {
      QX_PROF_STORE(4, w_tfull);
      QX_PROF_STORE(5, w_sfull);
      QX_PROF_STORE(6, QX_PROF_NOW() - t_start);
    }
    if (!ok) {
      *abort_flag = 1;
      atomicExch(p.error, 13);
    }
  } else if (kQ4 && warp == kFirstUnpackWarp + G::kStages) {
    // ------------------------------ q4_0 packed-slab loader ------------------
    if (lane == 0) {
      // packed q4_0 slab + its scales: one 9 KiB bulk copy, as far ahead as the ring allows
      uint32_t rs = 0, rphase = 0;
      bool ok = true;
      for (long long gs = s_begin; gs < s_end; ++gs) {
        if (!mbar_wait(&bars->raw_empty[rs], rphase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&bars->raw_full[rs], kRawBytes);
        bulk_copy_g2s(raw_ring + rs * kRawBytes, p.panel + gs * kRawBytes, kRawBytes,
                      &bars->raw_full[rs]);
        if (++rs == G::kRawStages) {
          rs = 0;
          rphase ^= 1u;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        atomicExch(p.error, 15);
      }
    }
  } else if (kQ4) {
    // ------------------------------ q4_0 unpack producers ---------------------
    // Unpack warp u owns stage u and packed buffer u: it handles every kStages-th slab on
    // its own, so the waits and fences of different slabs overlap across warps.
    const int u = warp - kFirstUnpackWarp;
    const int pt = threadIdx.x - kFirstUnpackWarp * 32;
    bool ok = true;
    QX_PROF_DECL(w_empty);
    QX_PROF_DECL(w_raw);
    const long long t_start = QX_PROF_NOW();
    if (u < G::kStages) {
      uint32_t phase = 0;
      const uint4* raw = reinterpret_cast<const uint4*>(raw_ring + u * kRawBytes);
      uint8_t* a_smem = smem + u * G::kStageBytes;
      for (long long gs = s_begin + u; gs < s_end; gs += G::kStages, phase ^= 1u) {
        if (!QX_PROF_WAIT(w_raw, mbar_wait(&bars->raw_full[u], phase, abort_flag)) ||
            !QX_PROF_WAIT(w_empty, mbar_wait(&bars->empty[u], phase ^ 1u, abort_flag))) {
          ok = false;
          break;
        }
#pragma unroll
        for (int it = 0; it < 16; it += 4) {
          uint4 packed[4];
#pragma unroll
          for (int h = 0; h < 4; ++h) packed[h] = raw[(it + h) * 32 + lane];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const int item = (it + h) * 32 + lane;
            const int r = item >> 2, j = item & 3;
            const uint4 w = packed[h];
            uint4 lo, hi;
            lo.x = w.x & 0x0F0F0F0Fu; hi.x = (w.x >> 4) & 0x0F0F0F0Fu;
            lo.y = w.y & 0x0F0F0F0Fu; hi.y = (w.y >> 4) & 0x0F0F0F0Fu;
            lo.z = w.z & 0x0F0F0F0Fu; hi.z = (w.z >> 4) & 0x0F0F0F0Fu;
            lo.w = w.w & 0x0F0F0F0Fu; hi.w = (w.w >> 4) & 0x0F0F0F0Fu;
            // row r of the slab: 128 bytes, 16-byte chunk c stored at c ^ (r & 7)
            uint8_t* rowp = a_smem + r * 128;
            *reinterpret_cast<uint4*>(rowp + (((2 * j) ^ (r & 7)) << 4)) = lo;      // elements 0..15
            *reinterpret_cast<uint4*>(rowp + (((2 * j + 1) ^ (r & 7)) << 4)) = hi;  // 16..31
          }
        }
        // the slab's 512 fp16 scales ride behind the codes: move them next to the stage
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          reinterpret_cast<uint4*>(a_smem + kABytes)[h * 32 + lane] = raw[512 + h * 32 + lane];
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->raw_empty[u]);  // packed buffer may be refilled
          mbar_arrive(&bars->full[u]);       // unpacked codes are in place
        }
      }
    }
    if (pt == 0) {
      QX_PROF_STORE(7, w_empty);
      QX_PROF_STORE(9, w_raw);
      QX_PROF_STORE(8, QX_PROF_NOW() - t_start);
    }
    if (!ok) {
      *abort_flag = 1;
      atomicExch(p.error, 14);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int FMT, int NMMA>
constexpr size_t gemv_smem_bytes() {
  return 1024 + static_cast<size_t>(TcGeom<FMT, NMMA>::kStages) * TcGeom<FMT, NMMA>::kStageBytes +
         static_cast<size_t>(TcGeom<FMT, NMMA>::kRawStages) * kRawBytes +
         sizeof(GemvBarriers<FMT, NMMA>) + 64;
}

template <int FMT, int NMMA>
qx_status launch_one(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemvTcParams& p,
                     int grid, cudaStream_t stream) {
  constexpr size_t smem = gemv_smem_bytes<FMT, NMMA>();
  static bool attr_set = false;
  if (!attr_set) {
    QX_CUDA_TRY(cudaFuncSetAttribute(gemv_tc_kernel<FMT, NMMA>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)));
    attr_set = true;
  }
  // Programmatic dependent launch: this kernel may start while the activation quantizer
  // in front of it is still running. Everything that does not depend on the activations
  // (barrier set-up, TMEM allocation, the weight pipeline) proceeds; the thread that
  // copies the activation images waits for the quantizer's results (griddepcontrol.wait).
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>(grid));
  config.blockDim = dim3(TcGeom<FMT, NMMA>::kThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  QX_CUDA_TRY(cudaLaunchKernelEx(&config, gemv_tc_kernel<FMT, NMMA>, map_a, map_b, p));
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

template <int FMT>
qx_status launch_fmt(int ncols, const CUtensorMap& map_a, const CUtensorMap& map_b,
                     const GemvTcParams& p, int grid, cudaStream_t stream) {
  switch (ncols) {
    case 8: return launch_one<FMT, 8>(map_a, map_b, p, grid, stream);
    case 16: return launch_one<FMT, 16>(map_a, map_b, p, grid, stream);
    case 32: return launch_one<FMT, 32>(map_a, map_b, p, grid, stream);
    case 64: return launch_one<FMT, 64>(map_a, map_b, p, grid, stream);
    case 128: return launch_one<FMT, 128>(map_a, map_b, p, grid, stream);
    default: break;
  }
  set_last_error_text("gemv: unsupported digit column count");
  return QX_STATUS_DEVICE_ERROR;
}

}  // namespace

// Device buffer the profiling build writes its cycle counters to (null otherwise).
long long* gemv_profile_buffer() {
#ifdef QX_GEMV_PROFILE
  static long long* buffer = []() {
    long long* ptr = nullptr;
    if (cudaMalloc(&ptr, 1024 * 16 * sizeof(long long)) != cudaSuccess) return static_cast<long long*>(nullptr);
    (void)cudaMemset(ptr, 0, 1024 * 16 * sizeof(long long));
    return ptr;
  }();
  return buffer;
#else
  return nullptr;
#endif
}

// K split: units of U slabs with at most 32 units per row; a function of K alone.
static int unit_slabs_for(long long slabs) { return static_cast<int>((slabs + 31) / 32); }

qx_status gemv_scratch_layout(const qx_weights* w, int m, int sm_count, GemvScratch* out) {
  if (w->tiles > kMaxCounterTiles) {
    set_last_error_text("qgemm: more than 262144 weight rows per prepared handle are not supported");
    return QX_STATUS_INVALID_SHAPE;
  }
  const int unit_slabs = unit_slabs_for(w->slabs);
  const int units_per_tile = static_cast<int>((w->slabs + unit_slabs - 1) / unit_slabs);
  const long long total_units = w->tiles * units_per_tile;
  const int ncols = digit_columns(m);
  const long long kpad = w->slabs * kSlabK;
  size_t off = kCounterBytes;
  out->ximg_offset = off;
  off += align_up(static_cast<size_t>(w->slabs) * ximage_bytes(ncols), 256);
  out->partial_offset = off;
  const int slots = units_per_tile > 2 ? units_per_tile : 2;
  off += align_up(static_cast<size_t>(w->tiles) * slots * m * kTileRows * sizeof(float), 256);
  out->total_bytes = off;
  out->ctas = static_cast<int>(total_units < sm_count ? total_units : sm_count);
  out->unit_slabs = unit_slabs;
  out->units_per_tile = units_per_tile;
  return QX_STATUS_OK;
}

qx_status launch_gemv_tc(const qx_weights* w, const uint8_t* ximg, float* y, int m,
                         long long ldy, uint8_t* ws_base, const GemvScratch& scratch,
                         cudaStream_t stream) {
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  return launch_gemv_tc_at(w, ximg, y, m, ldy, ws_base, scratch, ctx->flag + 1, stream);
}

qx_status launch_gemv_tc_at(const qx_weights* w, const uint8_t* ximg, float* y, int m,
                            long long ldy, uint8_t* ws_base, const GemvScratch& scratch,
                            int* error_word, cudaStream_t stream) {
  const int ncols = digit_columns(m);
  const long long kpad = w->slabs * kSlabK;
  CUtensorMap map_a{}, map_b{};  // map_b is unused (kept for the kernel signature)
  if (w->format == QX_FORMAT_Q8_0) {
    const uint64_t span_rows = static_cast<uint64_t>(w->tiles) * w->slabs * kQ8SpanRows;
    if (!encode_tma_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w->panel, 128, span_rows, 128, 128,
                       kQ8SpanRows)) {
      set_last_error_text("cuTensorMapEncodeTiled failed for the GEMV weight panel");
      return QX_STATUS_DEVICE_ERROR;
    }
  }
  GemvTcParams p{};
  p.panel = w->panel;
  p.ximg = ximg;
  p.y = y;
  p.partial = reinterpret_cast<float*>(ws_base + scratch.partial_offset);
  p.counters = reinterpret_cast<int*>(ws_base);
  p.error = error_word;
  p.ldy = ldy;
  p.rows = w->rows;
  p.m = m;
  p.nbpad = static_cast<int>(w->slabs) * kSlabBlocks;
  p.slabs = static_cast<int>(w->slabs);
  p.tiles = static_cast<int>(w->tiles);
  p.unit_slabs = scratch.unit_slabs;
  p.units_per_tile = scratch.units_per_tile;
  p.slots_per_tile = scratch.units_per_tile > 2 ? scratch.units_per_tile : 2;
  p.total_units = w->tiles * scratch.units_per_tile;
  p.debug = gemv_profile_buffer();
  if (w->format == QX_FORMAT_Q8_0) {
    return launch_fmt<QX_FORMAT_Q8_0>(ncols, map_a, map_b, p, scratch.ctas, stream);
  }
  return launch_fmt<QX_FORMAT_Q4_0>(ncols, map_a, map_b, p, scratch.ctas, stream);
}

}  // namespace qx

#ifdef QX_GEMV_PROFILE
// Profiling builds only: copies the per-CTA cycle counters of the last launches to the
// host (16 values per CTA) and clears them.
extern "C" QX_API int qx_debug_gemv_profile(long long* host_out, int ctas) {
  long long* buffer = qx::gemv_profile_buffer();
  if (buffer == nullptr || ctas > 1024) return -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  if (cudaMemcpy(host_out, buffer, sizeof(long long) * 16 * ctas, cudaMemcpyDeviceToHost) !=
      cudaSuccess) {
    return -3;
  }
  (void)cudaMemset(buffer, 0, 1024 * 16 * sizeof(long long));
  return 0;
}
#endif
