// Decode GEMV / small-batch qgemm on the tensor cores (tcgen05 kind::i8 + TMEM).
//
// Why tensor cores for a GEMV: at HBM speed one SM must consume ~22 bytes of packed
// weights per clock, i.e. 1.2 q4_0 blocks of 32 weights. Dequantising and multiplying
// those on the CUDA cores needs ~90 instructions per block -- the whole issue budget.
// Here the 8-bit products run on the tensor core instead: the weight codes are the MMA's
// A operand (128 weight rows x 32 code bytes), the activation digits (balanced base-256
// digits, see qx_gemv.cuh) are the B operand, and the exact integer digit sums of 128
// rows land in TMEM. The CUDA cores only combine the digits and apply the fp16 block
// scale: ~10 instructions per block and row.
//
// One K-slab (8 blocks = 256 elements of 128 rows) per pipeline step. Its span of the
// prepared panel (codes already in the operand's swizzled layout, then the fp16 scales)
// arrives by one bulk copy into a deep ring of weight slots; its activation image is
// either built in place by a quantizer warp (one or two activation rows: no second
// kernel, nothing between this kernel and the weights) or copied from the images the
// quantizer kernel wrote. The B operand is block
// diagonal: its N = 32..256 columns are (block class, activation row, digit), so one
// accumulator holds the sums of several blocks side by side and, for one or two
// activation rows, a single TMEM load brings a whole slab to the epilogue thread.
//   q8_0  8 MMAs per slab (one per block, K = 32 code bytes)
//   q4_0  the raw packed bytes are an unsigned operand as they are (4 MMAs against the
//         digits of 16*t[i]); four warps mask out the high nibbles into a second tile (4
//         more MMAs against the digits of t[i+16] - 16*t[i]): see qx_gemv.cuh
// Warp roles: 0 = copy producer (one thread), 1 = MMA issuer (one thread), 2-9 = epilogue
// (thread = weight row, accumulators in registers; two sets of four warps take alternate
// K units), then for q4_0 four warps for the high nibbles (a quarter of every slab each)
// and, for decode batches, three activation quantizer warps (one per work slot).
//
// Work split and summation order. K is cut into units of `unit_slabs` slabs, a function of
// K alone. A row's result is defined as (sum of its even units) + (sum of its odd units),
// each in ascending order; a unit's sum comes from four chains over its blocks in ascending
// order -- the low and the high part of the even blocks and of the odd blocks, qx_gemv.cuh
// -- so it does not depend on the number of rows, on how rows are sharded over GPUs, on the
// batch size, on the SM count or on which of the two GEMV kernels ran (a single activation
// row on a small matrix goes to qx_gemv_decode.cu). The (row tile, unit) sequence is cut into equal contiguous ranges,
// one per persistent CTA, so every SM streams the same number of bytes. Unit sums go to
// scratch memory; each thread counts the units it wrote in on a per-row counter and the
// thread that completes the count adds them in the fixed order: no thread waits for
// another one.

#include <cuda.h>

#include "qx_gemv_tc.cuh"
#include "qx_sm100.cuh"

namespace qx {
namespace {

using namespace sm100;

constexpr int kSmemLimit = 227 * 1024;
constexpr int kMaxPushPeers = 7;

// weight slots (at most 8) that fit beside `work_slots` work slots
constexpr int weight_slots_fit(int budget, int work_bytes, int weight_bytes, int work_slots) {
  return (budget - work_slots * work_bytes) / weight_bytes > 8
             ? 8
             : (budget - work_slots * work_bytes) / weight_bytes;
}

template <int FMT, int MP>
struct TcGeom {
  static constexpr bool kQ4 = FMT == QX_FORMAT_Q4_0;
  // Decode batches (one or two activation rows) quantize the activations inside the kernel
  // (one more warp); larger batches read images written by the quantizer kernel.
  static constexpr bool kFused = MP <= 2;
  static constexpr int kG = group_blocks(FMT, MP);     // blocks per accumulator
  static constexpr int kN = digit_columns(FMT, MP);    // MMA N = accumulator columns
  static constexpr int kGroups = kSlabBlocks / kG;     // accumulators per slab
  // Two rings in shared memory. Weight slots hold a slab's span of the panel as copied
  // (the bytes in flight: as many slots as fit). Work slots hold what exists only around
  // the MMAs of a slab: the q4_0 masked-byte tile and the digits built in the kernel.
  static constexpr int kWBytes = slab_span_bytes(FMT);   // 34 KiB | 18 KiB
  static constexpr int kScaleOffset = slab_code_bytes(FMT);
  static constexpr int kHBytes = kQ4 ? kTileRows * 128 : 0;
  static constexpr int kBBytes = kN * 256;
  static constexpr int kXBytes = ximage_bytes(FMT, MP);  // digit rows + constants
  // When the kernel quantizes itself the block constants live in their own small ring,
  // one entry per weight slot, because they are needed longer (until the epilogue has
  // read them) than the operands of the MMAs.
  static constexpr int kConstBytes = 128 * MP;
  // ... a ring indexed by the CTA-local slab number, deep enough that the quantizer warps
  // (at most kWorkSlots slabs ahead of the MMAs) never lap the epilogue (at most the
  // accumulator ring behind the MMAs); checked below
  static constexpr int kConstSlots = kFused ? (MP == 1 ? 32 : 16) : 0;
  static constexpr int kConstRing = kConstSlots > 0 ? kConstSlots : 1;  // divisor (never 0)
  // Images that come from the quantizer kernel travel with the weights (copied as far
  // ahead); images built in the kernel sit in the work slot.
  static constexpr int kSlotBytes = kWBytes + (kFused ? 0 : (kXBytes + 1023) / 1024 * 1024);
  static constexpr int kWorkBytes = (kHBytes + (kFused ? kBBytes : 0) + 1023) / 1024 * 1024;
  // ... and the activations of the next slabs wait in a small ring of their own (copied
  // there asynchronously a few slabs ahead: a load from L2 takes longer than a slab).
  static constexpr int kQuantWarps = 3;  // == kWorkSlots when the kernel quantizes itself
  static constexpr int kXRingSlots = 4;  // per quantizer warp
  static constexpr int kXRingBytes = kFused ? kQuantWarps * kXRingSlots * MP * kSlabK * 4 : 0;
  static constexpr int kBudget = kSmemLimit - 1024 - 2048 - kConstSlots * kConstBytes -
                                 kXRingBytes;  // slack, barriers, constants, activation ring
  // the in-kernel quantizer has one work slot per quantizer warp; otherwise three work slots
  // unless that costs more than one weight slot
  static constexpr int kWorkSlots =
      kFused ? kQuantWarps
             : (weight_slots_fit(kBudget, kWorkBytes, kSlotBytes, 3) + 1 >=
                        weight_slots_fit(kBudget, kWorkBytes, kSlotBytes, 2)
                    ? 3
                    : 2);
  static constexpr int kSlots = weight_slots_fit(kBudget, kWorkBytes, kSlotBytes, kWorkSlots);
  // One TMEM stage (the unit handed from the MMA issuer to the epilogue) holds several
  // accumulators when they are narrow: up to 128 columns (a whole slab per hand-over for
  // decode batches).
  static constexpr int kStageTarget = 128;
  static constexpr int kGroupsPerStage =
      kN >= kStageTarget ? 1 : (kStageTarget / kN < kGroups ? kStageTarget / kN : kGroups);
  static constexpr int kStagesPerSlab = kGroups / kGroupsPerStage;
  static constexpr int kTCols = kN * kGroupsPerStage;  // TMEM columns per stage
  static constexpr int kTStages = 512 / kTCols > 16 ? 16 : 512 / kTCols;
  // Epilogue sets take the K units in turn (unit mod kSets); which set sums a unit does not
  // matter for the result (unit sums meet in scratch memory and are added in a fixed order).
  // Decode batches are bound by the per-slab latency of an epilogue thread (barrier waits,
  // TMEM load, a dependent chain per block), so a single activation row gets three sets,
  // two to four rows two. From eight rows on the epilogue is bound by its work per item and
  // by how far the MMAs can run ahead in TMEM (a slab then fills half of it or more): ONE
  // set whose warps all work on the same stage, each on a share of the activation rows.
  static constexpr int kSets = MP == 1 ? 3 : (MP >= 8 ? 1 : 2);
  // Each epilogue set has its own ring of accumulators, so every TMEM barrier is used by
  // one set only (a parity wait cannot tell apart phases two steps apart).
  static constexpr int kTPerSet = kTStages / kSets;
  // Epilogue: per set four warps (one per TMEM lane quarter) times kEpiSplit: from eight
  // activation rows on, the kEpiSplit warps of a lane quarter take four (at 32 rows: eight)
  // activation rows each, so a thread handles 32 (64) items per slab instead of 64 - 256.
  static constexpr int kEpiSplit = MP >= 16 ? 4 : (MP == 8 ? 2 : 1);
  static constexpr int kEpiWarps = 4 * kSets * kEpiSplit;
  static constexpr int kRowsPerThread = MP / kEpiSplit;  // activation rows per epilogue thread
  // (two instead of four from 16 activation rows on: the CTA then has 640 threads, which
  // leaves the epilogue 96 registers instead of 80 and its digit sums and accumulators
  // unspilled)
  static constexpr int kUnpackWarps = kQ4 ? (MP >= 16 ? 2 : 4) : 0;
  static constexpr int kFirstUnpackWarp = 2 + kEpiWarps;
  static constexpr int kQuantWarp = kFirstUnpackWarp + kUnpackWarps;  // fused only
  static constexpr int kThreads = 32 * (2 + kEpiWarps + kUnpackWarps + (kFused ? kQuantWarps : 0));
  static constexpr int kColsPerWarp = kTCols / kEpiSplit;  // a warp's share of a stage
  // arrivals on a slot's `ready` barrier (0: the MMA issuer waits for the copies themselves)
  static constexpr int kReadyCount = (kFused ? 1 : 0) + kUnpackWarps;
  static constexpr int kLdCols = kColsPerWarp >= 64 ? 64 : 32;  // columns fetched per TMEM wait
  static constexpr int kShareCols = 4 * kRowsPerThread;  // columns of (one block, a warp's rows)
  static_assert(kEpiSplit == 1 || kShareCols == 16 || kShareCols == 32, "TMEM load widths");
  static constexpr bool kRollGroups = MP >= 8 && kEpiSplit == 1;
  static_assert(kSlots + kWorkSlots + kTStages + kConstSlots <= kThreads - 64, "one barrier group per thread");
  static_assert(kSlots >= 2 && kTPerSet >= 1 && kTPerSet <= 15 && kN >= 32 && kN <= 256, "geometry");
  static_assert(!kFused || kSlots > kWorkSlots, "a work slot's previous slab is newer than a weight slot's");
  static_assert(!kFused || kWorkSlots == kQuantWarps, "one quantizer warp per work slot");
  // (depth only matters for speed: an entry is rewritten after the epilogue has released it)
  static_assert(!kFused || kConstSlots >= kWorkSlots + kTStages / kStagesPerSlab + 4,
                "constants ring deeper than quantizer lead + epilogue lag");
  static_assert(kScaleOffset + kSlabScaleBytes == kWBytes && kWBytes % 1024 == 0, "span");
};

struct GemvTcParams {
  const uint8_t* panel;          // [tile][slab] spans
  const uint8_t* ximg;           // [slab] activation images (batches above two rows)
  const float* x;                // [m][ldx] activations (decode batches)
  float* y;
  float* partial;                // [tile][unit][m][128] unit sums
  int* counters;                 // [tile][128], one per weight row
  int* error;
  long long ldy, ldx, rows;
  int m, slabs, tiles, nb;
  int x_vector;                  // x and ldx allow 16-byte loads
  int unit_slabs, units_per_tile;  // K split: units of unit_slabs slabs
  // unit ranges of the CTAs: CTA c takes units_per_cta units, the first units_rem CTAs one more
  uint32_t units_per_cta, units_rem;
  // Row-sharded runs (one process per GPU): every finished output is also stored into the
  // other ranks' inboxes over NVLink as an 8-byte {value, valid} cell (an all-gather fused
  // into the epilogue; the receiving side is allgather_unpack_kernel in qx_peer.cu).
  // Fused handles (several matrices back to back): segment s starts at tile
  // seg_tile_begin[s], has seg_rows[s] rows and writes dense [m][seg_rows[s]] outputs at
  // seg_y[s]. One segment for ordinary handles: {0, rows, y with row stride ldy}.
  int segments;
  int seg_tile_begin[qx_weights::kMaxSegments];
  long long seg_rows[qx_weights::kMaxSegments];
  float* seg_y[qx_weights::kMaxSegments];
  int int8_activations;               // in-kernel quantizer: the rule of qgemv_w8a8
  int peers;                          // other ranks (0: no push)
  uint32_t push_tag;                  // tag of this step's cells
  PushCell* push_cells[kMaxPushPeers];  // the other ranks' inboxes, at this rank's slice
};

template <int FMT, int MP>
struct __align__(8) GemvBarriers {
  uint64_t raw_full[TcGeom<FMT, MP>::kSlots];    // the slab's span landed in its weight slot
  uint64_t done[TcGeom<FMT, MP>::kSlots];        // the slab's epilogue is through (so are its MMAs)
  // everything the slab's MMAs read is in place: the span has landed (the warps below wait
  // for that first) and the in-kernel quantizer warp / the four masking warps have written
  // their parts. One barrier for the MMA issuer instead of one per producer.
  uint64_t ready[TcGeom<FMT, MP>::kSlots];
  uint64_t mma_done[TcGeom<FMT, MP>::kWorkSlots];   // the slab's MMAs have read the work slot
  // the block constants of CTA-local slab i are written (entry i mod kConstSlots)
  uint64_t const_ready[TcGeom<FMT, MP>::kConstSlots > 0 ? TcGeom<FMT, MP>::kConstSlots : 1];
  // ... and the epilogue set that used them is through with them
  uint64_t const_free[TcGeom<FMT, MP>::kConstSlots > 0 ? TcGeom<FMT, MP>::kConstSlots : 1];
  uint64_t tmem_full[TcGeom<FMT, MP>::kTStages];
  uint64_t tmem_empty[TcGeom<FMT, MP>::kTStages];
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

// Ring position i mod `slots` with the parity of i / slots.
struct RingPos {
  uint32_t slot = 0, phase = 0;
  __device__ __forceinline__ void advance(uint32_t slots) {
    if (++slot == slots) {
      slot = 0;
      phase ^= 1u;
    }
  }
  __device__ __forceinline__ void advance_by(uint32_t steps, uint32_t slots) {
    slot += steps;
    while (slot >= slots) {
      slot -= slots;
      phase ^= 1u;
    }
  }
};

// The low bytes of four values, packed into a word.
__device__ __forceinline__ uint32_t pack_low_bytes(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
// word[d] = the balanced base-256 digits d (as signed bytes) of t[0..3], d < ND. The digit
// is the low byte of the running quotient, and removing it is (t + 128) >> 8.
template <int ND>
__device__ __forceinline__ void pack_digits(int (&t)[4], uint32_t (&word)[4]) {
#pragma unroll
  for (int d = 0; d < ND; ++d) {
    word[d] = pack_low_bytes(t[0], t[1], t[2], t[3]);
    if (d + 1 < ND) {
#pragma unroll
      for (int i = 0; i < 4; ++i) t[i] = (t[i] + 128) >> 8;
    }
  }
}

// In-kernel activation quantizer (decode batches): writes a slab's digits into a work slot
// whose digit area is zero outside the block-diagonal positions, and its block constants.
// Lane (b = lane / 4, q = lane % 4) handles elements 4q..4q+3 and 16+4q..16+4q+3 of block
// b of every row: `lo` / `hi` are those values (zeros past the end of the row);
// digit_offset[m][d] is the lane's byte offset in the digit area for digit d of row m.
template <int FMT, int MP>
__device__ __forceinline__ void write_slab_image(uint8_t* digits, XConst* consts,
                                                 const int (&digit_offset)[MP][4],
                                                 const float4 (&lo)[MP], const float4 (&hi)[MP],
                                                 bool block_valid, int lane, bool int8_activations) {
  using G = TcGeom<FMT, MP>;
  const int b = lane >> 2, q = lane & 3;
#pragma unroll
  for (int m = 0; m < MP; ++m) {
    const float v[8] = {lo[m].x, lo[m].y, lo[m].z, lo[m].w, hi[m].x, hi[m].y, hi[m].z, hi[m].w};
    // max of |bits|: orders finite < inf < NaN, so non-finite inputs are detected
    uint32_t amax_bits = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) amax_bits = max(amax_bits, __float_as_uint(v[i]) & 0x7FFFFFFFu);
    amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 1));
    amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 2));
    const uint32_t eb_raw = amax_bits >> 23;
    const bool finite = eb_raw != 255u;
    const uint32_t eb = max(eb_raw, 30u);                       // envelope 2^(eb-126) > amax
    float scale_up = finite ? __uint_as_float((275u - eb) << 23) : 0.0f;  // 2^(22 - e)
    // 2^(e - 22); q4_0: 2^(e - 26), its digit sums carry a factor 16
    float scale = __uint_as_float((eb - (FMT == QX_FORMAT_Q4_0 ? 25u : 21u)) << 23);
    if (int8_activations) {
      // qgemv_w8a8 (kernels/quantization/qgemv_w8a8_ref.cpp:18-41): scale = amax / 127,
      // codes nearbyint(x * (1 / scale)) clamped to +-127, both divisions IEEE
      const float block_scale = __fdiv_rn(__uint_as_float(amax_bits), 127.0f);
      scale_up = (finite && block_scale != 0.0f) ? __fdiv_rn(1.0f, block_scale) : 0.0f;
      scale = FMT == QX_FORMAT_Q4_0 ? block_scale * 0.0625f : block_scale;
    }
    if (!finite) scale = __uint_as_float(0x7FC00000u);  // NaN/inf in -> NaN out
    if (!block_valid) scale = 0.0f;
    int t_lo[4], t_hi[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // |t| <= 2^22 (a non-finite block has scale_up = 0; 0 * inf = NaN converts to 0)
      t_lo[i] = __float2int_rn(v[i] * scale_up);
      t_hi[i] = __float2int_rn(v[4 + i] * scale_up);
      if (int8_activations) {
        t_lo[i] = max(-127, min(127, t_lo[i]));
        t_hi[i] = max(-127, min(127, t_hi[i]));
      }
    }
    uint32_t w_lo[4], w_hi[4];
    if (FMT == QX_FORMAT_Q8_0) {
      pack_digits<3>(t_lo, w_lo);
      pack_digits<3>(t_hi, w_hi);
#pragma unroll
      for (int d = 0; d < 3; ++d) {
        // the second half of the block is the neighbouring 16-byte chunk
        *reinterpret_cast<uint32_t*>(digits + digit_offset[m][d]) = w_lo[d];
        *reinterpret_cast<uint32_t*>(digits + (digit_offset[m][d] ^ 16)) = w_hi[d];
      }
    } else {
      int sum = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) sum += t_lo[i] + t_hi[i];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        t_lo[i] *= 16;
        t_hi[i] -= t_lo[i];  // z_i
      }
      pack_digits<4>(t_lo, w_lo);
      pack_digits<4>(t_hi, w_hi);
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        *reinterpret_cast<uint32_t*>(digits + digit_offset[m][d]) = w_lo[d];
        *reinterpret_cast<uint32_t*>(digits + G::kN * 128 + digit_offset[m][d]) = w_hi[d];
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      if (q == 0) q4_offset_constants(sum, &consts[b * MP + m].k_lo, &consts[b * MP + m].k_hi);
    }
    if (q == 0) consts[b * MP + m].scale = scale;
  }
}

template <int FMT, int MP>
__global__ void __launch_bounds__((TcGeom<FMT, MP>::kThreads), 1)
gemv_tc_kernel(const GemvTcParams p) {
  using G = TcGeom<FMT, MP>;
  constexpr bool kQ4 = G::kQ4;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* work_ring = smem + G::kSlots * G::kSlotBytes;  // slot: [masked bytes (q4_0) | digits]
  // block constants of the slab in each weight slot (only when the kernel quantizes itself)
  uint8_t* const_ring = work_ring + G::kWorkSlots * G::kWorkBytes;
  uint8_t* x_ring = const_ring + G::kConstSlots * G::kConstBytes;
  auto* bars = reinterpret_cast<GemvBarriers<FMT, MP>*>(x_ring + G::kXRingBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  volatile int* abort_flag = &bars->abort_flag;
  // kernels queued behind this one may be scheduled as soon as SMs free up; whatever they
  // touch of this kernel's data they guard with their own griddepcontrol.wait
  asm volatile("griddepcontrol.launch_dependents;");

  // This CTA's contiguous range of K units (32-bit arithmetic only: it sits in front of the
  // first weight copy). Units tile every row tile's slabs contiguously, so the range is one
  // contiguous range of global slabs (tile * slabs + slab).
  const uint32_t cta = blockIdx.x;
  const uint32_t u_begin = cta * p.units_per_cta + (cta < p.units_rem ? cta : p.units_rem);
  const uint32_t u_end = u_begin + p.units_per_cta + (cta < p.units_rem ? 1u : 0u);
  long long s_begin = 0, s_end = 0;
  int tile0 = 0, slab0 = 0;  // row tile and K-slab (within the tile) of the range's first slab
  if (u_end > u_begin) {
    const uint32_t upt = static_cast<uint32_t>(p.units_per_tile);
    const uint32_t tile_b = u_begin / upt, last = u_end - 1, tile_l = last / upt;
    const int last_end = static_cast<int>(last - tile_l * upt + 1) * p.unit_slabs;
    tile0 = static_cast<int>(tile_b);
    slab0 = static_cast<int>(u_begin - tile_b * upt) * p.unit_slabs;
    s_begin = static_cast<long long>(tile_b) * p.slabs + slab0;
    s_end = static_cast<long long>(tile_l) * p.slabs + (last_end < p.slabs ? last_end : p.slabs);
  }
  const int count = static_cast<int>(s_end - s_begin);  // slabs of this CTA

  // copy producer state (thread 0): next span to copy and the activation image that goes with it
  constexpr uint32_t kTxBytes = G::kWBytes + (G::kFused ? 0 : G::kXBytes);
  const uint8_t* wsrc = p.panel + s_begin * G::kWBytes;
  const int ahead = count < G::kSlots ? count : G::kSlots;
  if (threadIdx.x == 0) {
    // The weights depend on nothing in front of this kernel: the first copies leave before
    // the rest of the CTA is set up (the other barriers, TMEM allocation, zero fill, the
    // block-wide barrier). Initialising a barrier costs tens of cycles, so this thread does
    // only the ones its copies complete on.
    for (int s = 0; s < G::kSlots; ++s) mbar_init(&bars->raw_full[s], 1);  // expect_tx arrival
    bars->abort_flag = 0;
    mbar_fence_init();
    for (int i = 0; i < ahead; ++i) {
      mbar_arrive_expect_tx(&bars->raw_full[i], kTxBytes);
      bulk_copy_g2s(smem + i * G::kSlotBytes, wsrc, G::kWBytes, &bars->raw_full[i]);
      wsrc += G::kWBytes;
    }
  } else if (threadIdx.x >= 64) {
    // every other barrier, one per thread
    const int b = threadIdx.x - 64;
    constexpr uint32_t kSetArrivals = 4 * G::kEpiSplit;  // the warps of one epilogue set
    if (b < G::kSlots) {
      // one epilogue set: it has seen the slab's last accumulator, so the MMAs are done too
      mbar_init(&bars->done[b], kSetArrivals);
      mbar_init(&bars->ready[b], G::kReadyCount > 0 ? G::kReadyCount : 1);
    } else if (b < G::kSlots + G::kWorkSlots) {
      mbar_init(&bars->mma_done[b - G::kSlots], 1);
    } else if (b < G::kSlots + G::kWorkSlots + G::kTStages) {
      const int t = b - G::kSlots - G::kWorkSlots;
      mbar_init(&bars->tmem_full[t], 1);
      mbar_init(&bars->tmem_empty[t], kSetArrivals);
    } else if (b < G::kSlots + G::kWorkSlots + G::kTStages + G::kConstSlots) {
      const int c = b - G::kSlots - G::kWorkSlots - G::kTStages;
      mbar_init(&bars->const_ready[c], 1);
      mbar_init(&bars->const_free[c], kSetArrivals);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  if (G::kFused) {
    // the quantizer warp only ever writes the block-diagonal positions of the digit areas
    for (int s = 0; s < G::kWorkSlots; ++s) {
      uint4* area = reinterpret_cast<uint4*>(work_ring + s * G::kWorkBytes + G::kHBytes);
      for (int i = threadIdx.x; i < G::kBBytes / 16; i += G::kThreads) area[i] = make_uint4(0u, 0u, 0u, 0u);
    }
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------ copy producer -----------------------------
    // Slab i uses weight slot i mod kSlots, free again when slab i - kSlots is done.
    if (lane == 0) {
      bool ok = true;
      int xslab = slab0;
      if (!G::kFused) {
        // the activation images are the output of the kernel in front of this one
        asm volatile("griddepcontrol.wait;" ::: "memory");
        for (int i = 0; i < ahead; ++i) {
          bulk_copy_g2s(smem + i * G::kSlotBytes + G::kWBytes,
                        p.ximg + static_cast<long long>(xslab) * G::kXBytes, G::kXBytes,
                        &bars->raw_full[i]);
          xslab = xslab + 1 == p.slabs ? 0 : xslab + 1;
        }
      }
      RingPos freed;  // slab i - kSlots
      for (int i = G::kSlots; i < count; ++i) {
        if (!mbar_wait(&bars->done[freed.slot], freed.phase, abort_flag)) {
          ok = false;
          break;
        }
        uint8_t* slot = smem + freed.slot * G::kSlotBytes;
        mbar_arrive_expect_tx(&bars->raw_full[freed.slot], kTxBytes);
        bulk_copy_g2s(slot, wsrc, G::kWBytes, &bars->raw_full[freed.slot]);
        wsrc += G::kWBytes;
        if (!G::kFused) {
          bulk_copy_g2s(slot + G::kWBytes, p.ximg + static_cast<long long>(xslab) * G::kXBytes,
                        G::kXBytes, &bars->raw_full[freed.slot]);
          xslab = xslab + 1 == p.slabs ? 0 : xslab + 1;
        }
        freed.advance(G::kSlots);
      }
      if (!ok) {
        *abort_flag = 1;
        report_error(p.error, 11);
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (elect_one()) {
      const uint32_t idesc = (2u << 4) | ((kQ4 ? 0u : 1u) << 7) | (1u << 10) |
                             (static_cast<uint32_t>(G::kN >> 3) << 17) |
                             (static_cast<uint32_t>(kTileRows >> 4) << 24);
      RingPos raw, work;
      uint32_t ring_pos_all = 0, ring_par_all = 0;  // accumulator ring of each epilogue set: 4 bits each
      bool ok = true;
      int gave_up = 12;  // which wait ran out: 12 weights, 15 image, 16 accumulator, 17 high nibbles
      int slab = slab0;
      int unit = slab / p.unit_slabs;
      int slab_in_unit = slab - unit * p.unit_slabs;
      for (int i = 0; i < count && ok; ++i) {
        const uint32_t eset = static_cast<uint32_t>(unit % G::kSets);
        // `ready` covers the span only where the masking warps (which wait for it) arrive on
        // it; the quantizer warps run ahead of the copies
        if ((G::kUnpackWarps == 0 &&
             !mbar_wait(&bars->raw_full[raw.slot], raw.phase, abort_flag)) ||
            (G::kReadyCount > 0 &&
             !mbar_wait(&bars->ready[raw.slot], raw.phase, abort_flag))) {
          ok = false;
          break;
        }
        tc_fence_after_sync();
        const uint32_t sa = smem_u32(smem + raw.slot * G::kSlotBytes);
        const uint32_t sw = smem_u32(work_ring + work.slot * G::kWorkBytes);
        const uint32_t sb = G::kFused ? sw + G::kHBytes : sa + G::kWBytes;  // digit rows
#pragma unroll
        for (int g = 0; g < G::kGroups; ++g) {
          const uint32_t pos = (ring_pos_all >> (4u * eset)) & 15u;
          const uint32_t par = (ring_par_all >> (4u * eset)) & 1u;
          const uint32_t ts = eset * G::kTPerSet + pos;
          if (g % G::kGroupsPerStage == 0) {
            if (!mbar_wait(&bars->tmem_empty[ts], par ^ 1u, abort_flag)) {
              ok = false;
              gave_up = 16;
              break;
            }
            tc_fence_after_sync();
          }
          const uint32_t d_tmem = tmem_base + ts * G::kTCols + (g % G::kGroupsPerStage) * G::kN;
          if (!kQ4) {
            // one MMA per block: 32 code bytes inside the swizzle atom = +2 in (addr >> 4)
#pragma unroll
            for (int b = 0; b < G::kG; ++b) {
              const int j = g * G::kG + b;
              const uint64_t a_desc = make_sw128_kmajor_desc(sa + (j >> 2) * (kTileRows * 128));
              const uint64_t b_desc = make_sw128_kmajor_desc(sb + (j >> 2) * (G::kN * 128));
              mma_i8_ss(d_tmem, a_desc + static_cast<uint64_t>(2 * (j & 3)),
                        b_desc + static_cast<uint64_t>(2 * (j & 3)), idesc, b > 0 ? 1u : 0u);
            }
          } else {
            // one MMA step = 32 packed bytes = two blocks; raw bytes first, then the high
            // nibbles once their tile is written
            constexpr int kSteps = G::kG / 2;
            const uint64_t a_raw = make_sw128_kmajor_desc(sa);
            const uint64_t b_low = make_sw128_kmajor_desc(sb);
#pragma unroll
            for (int t = 0; t < kSteps; ++t) {
              const uint64_t k = static_cast<uint64_t>(2 * (g * kSteps + t));
              mma_i8_ss(d_tmem, a_raw + k, b_low + k, idesc, t > 0 ? 1u : 0u);
            }
            const uint64_t a_high = make_sw128_kmajor_desc(sw);
            const uint64_t b_high = make_sw128_kmajor_desc(sb + G::kN * 128);
#pragma unroll
            for (int t = 0; t < kSteps; ++t) {
              const uint64_t k = static_cast<uint64_t>(2 * (g * kSteps + t));
              mma_i8_ss(d_tmem, a_high + k, b_high + k, idesc, 1u);
            }
          }
          if (g % G::kGroupsPerStage == G::kGroupsPerStage - 1) {
            tc_commit(&bars->tmem_full[ts]);
            const uint32_t next = pos + 1 == G::kTPerSet ? 0u : pos + 1;
            const uint32_t flip = pos + 1 == G::kTPerSet ? 1u : 0u;
            ring_pos_all = (ring_pos_all & ~(15u << (4u * eset))) | (next << (4u * eset));
            ring_par_all ^= flip << (4u * eset);
          }
        }
        if (!ok) break;
        tc_commit(&bars->mma_done[work.slot]);
        raw.advance(G::kSlots);
        work.advance(G::kWorkSlots);
        if (++slab == p.slabs) {
          slab = 0;
          unit = 0;
          slab_in_unit = 0;
        } else if (++slab_in_unit == p.unit_slabs) {
          slab_in_unit = 0;
          ++unit;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        report_error(p.error, gave_up);
      }
    }
  } else if (warp < 2 + G::kEpiWarps) {
    // ------------------------------ epilogue ----------------------------------
    // kSets sets of four warps; set e takes the K units with unit mod kSets == e, so while one
    // set waits on barriers, TMEM loads and conversions the others issue.
    const int eset = (warp - 2) / (4 * G::kEpiSplit);
    const int split = ((warp - 2) >> 2) % G::kEpiSplit;  // which share of the activation rows
    const int quarter = warp & 3;  // TMEM lanes 32*quarter .. +31 are this warp's
    constexpr int kMine = G::kRowsPerThread;
    const int row_in_tile = quarter * 32 + lane;
    // Current unit, activation rows split * kMine ..: four chains per row (qx_gemv.cuh:
    // low and high part of the blocks, even and odd blocks, ascending block order each) that
    // meet at the end of the unit. The single-row decode kernel (qx_gemv_decode.cu) sums in
    // exactly this order, so a row of a batch and the same row alone give the same bits.
    float acc[4][kMine];  // [2 * block parity + part]
#pragma unroll
    for (int m = 0; m < kMine; ++m) acc[0][m] = acc[1][m] = acc[2][m] = acc[3][m] = 0.0f;
    int units_mine = 0;  // units of the current tile this thread has written
    // A share of a row = this thread's units of one tile. Counting a share in on the row's
    // counter needs a fence (the unit sums must be visible before the count), and a fence
    // waits for the thread's outstanding stores: right after the last unit sum was stored
    // that is a microsecond, a slab later it is nearly free. So a finished share stays
    // "open" until the end of this thread's next slab, is counted in there (the atomic's
    // result is not looked at yet) and resolved another slab later -- only the last share of
    // the CTA's range pays the full latency, after the loop.
    int open_tile = 0, open_add = 0;              // written, not counted in
    int cnt_tile = 0, cnt_add = 0, cnt_old = 0;   // counted in, result not looked at
    // this thread completed the row's count in `tile`: add its unit sums in the fixed order
    auto finish_row = [&](int done_tile) {
      int seg = 0;
#pragma unroll
      for (int q = 1; q < qx_weights::kMaxSegments; ++q) {
        if (q < p.segments && done_tile >= p.seg_tile_begin[q]) seg = q;
      }
      const long long row =
          static_cast<long long>(done_tile - p.seg_tile_begin[seg]) * kTileRows + row_in_tile;
      const long long seg_rows = p.seg_rows[seg];
      const long long ldy = p.segments > 1 ? seg_rows : p.ldy;
      float* y_out = p.seg_y[seg];
      const float* slots = p.partial +
                           static_cast<long long>(done_tile) * p.units_per_tile * p.m * kTileRows +
                           row_in_tile;
      for (int m = 0; m < p.m; ++m) {
        // units_per_tile <= 16: fetch all unit sums first (independent loads), then add
        // the even and the odd ones in ascending order
        float v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          v[u] = u < p.units_per_tile
                     ? __ldcg(slots + (static_cast<long long>(u) * p.m + m) * kTileRows)
                     : 0.0f;
        }
        float even = 0.0f, odd = 0.0f;
#pragma unroll
        for (int u = 0; u < 16; u += 2) {
          if (u < p.units_per_tile) even += v[u];
          if (u + 1 < p.units_per_tile) odd += v[u + 1];
        }
        if (row < seg_rows) {
          const float value = even + odd;
          const long long at = m * ldy + row;
          y_out[at] = value;
          for (int r = 0; r < p.peers; ++r) {
            // value and tag in ONE 8-byte store: whoever sees the tag sees the value
            asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(p.push_cells[r] + at),
                         "r"(__float_as_uint(value)), "r"(p.push_tag)
                         : "memory");
          }
        }
      }
      p.counters[static_cast<long long>(done_tile) * kTileRows + row_in_tile] = 0;  // next launch
    };
    // Whoever completes a row's count adds its unit sums (acquire). Rows are independent,
    // so no thread ever waits for another one.
    auto resolve_counted = [&]() {
      if (cnt_add > 0 && cnt_old + cnt_add == p.units_per_tile * G::kEpiSplit) {
        asm volatile("fence.acq_rel.gpu;" ::: "memory");
        finish_row(cnt_tile);
      }
      cnt_add = 0;
    };
    auto count_open = [&]() {
      if (open_add == 0) return;
      resolve_counted();
      int* counter = p.counters + static_cast<long long>(open_tile) * kTileRows + row_in_tile;
      asm volatile("fence.acq_rel.gpu;" ::: "memory");  // release: the share's unit sums
      asm volatile("atom.add.relaxed.gpu.global.s32 %0, [%1], %2;"
                   : "=r"(cnt_old)
                   : "l"(counter), "r"(open_add)
                   : "memory");
      cnt_tile = open_tile;
      cnt_add = open_add;
      open_add = 0;
    };
    RingPos raw, work;
    uint32_t ring_pos = 0, tphase = 0;
    bool ok = true;
    int tile = tile0;
    int slab = slab0;
    int unit = slab / p.unit_slabs;
    int slab_in_unit = slab - unit * p.unit_slabs;
    for (int i = 0; i < count && ok; ++i) {
      const bool mine = unit % G::kSets == eset;
      if (mine) {
        const uint8_t* raw_base = smem + raw.slot * G::kSlotBytes;
        const int4* xcs = reinterpret_cast<const int4*>(
            G::kFused ? const_ring + (i % G::kConstRing) * G::kConstBytes
                      : raw_base + G::kWBytes + G::kBBytes);
        uint32_t scw[4] = {0u, 0u, 0u, 0u};  // this row's eight fp16 block scales
        // (large batches keep the loop over accumulators rolled: unrolled, the loop body
        // would not fit the instruction cache)
#pragma unroll(G::kRollGroups ? 1 : G::kStagesPerSlab)
        for (int st = 0; st < G::kStagesPerSlab; ++st) {
          const uint32_t ts = eset * G::kTPerSet + ring_pos;
          if (!mbar_wait(&bars->tmem_full[ts], tphase, abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (st == 0) {
            // these barriers completed before the MMAs ran; waiting on them here makes the
            // copied scales and the block constants visible to this thread (the constants
            // of the in-kernel quantizer have a ring and barriers of their own, indexed by
            // the slab number: no other barrier of theirs is safe to wait on this late)
            if (!mbar_wait(&bars->raw_full[raw.slot], raw.phase, abort_flag) ||
                (G::kFused &&
                 !mbar_wait(&bars->const_ready[i % G::kConstRing],
                            static_cast<uint32_t>(i / G::kConstRing) & 1u,
                            abort_flag))) {
              ok = false;
              break;
            }
            if (!G::kRollGroups) {
              const uint4 s4 = *reinterpret_cast<const uint4*>(raw_base + G::kScaleOffset +
                                                               row_in_tile * (kSlabBlocks * 2));
              scw[0] = s4.x; scw[1] = s4.y; scw[2] = s4.z; scw[3] = s4.w;
            }
          }
          if constexpr (G::kEpiSplit > 1) {
            // Row-split stages: this warp's share of every block of the stage (accumulator
            // b / kG, block class b % kG, activation rows split * kMine ..) is fetched at
            // once, the stage handed back, then the items are combined.
            constexpr int kShares = G::kGroupsPerStage * G::kG;
            // With 32 activation rows the CTA has so many threads that 64 registers of digit
            // sums would spill: the shares are then fetched and combined one after the other
            // (the stage is handed back after the last fetch either way).
            constexpr bool kSerial = MP >= 32 && kShares > 1;
            constexpr int kHeld = kSerial ? 1 : kShares;
            uint32_t v[kHeld][G::kShareCols];
            auto fetch = [&](int b) {
              const uint32_t taddr = tmem_base + ts * G::kTCols + (b / G::kG) * G::kN +
                                     (b % G::kG) * (4 * MP) + split * G::kShareCols +
                                     (static_cast<uint32_t>(quarter * 32) << 16);
              tmem_ld_cols(taddr, v[kSerial ? 0 : b]);
            };
            auto hand_back = [&]() {
              tmem_ld_wait();
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&bars->tmem_empty[ts]);
            };
            if (!kSerial) {
#pragma unroll
              for (int b = 0; b < kShares; ++b) fetch(b);
              hand_back();
            }
#pragma unroll
            for (int b = 0; b < kShares; ++b) {
              if (kSerial) {
                fetch(b);
                if (b == kShares - 1) {
                  hand_back();
                } else {
                  tmem_ld_wait();
                }
              }
              const int j = (st * G::kGroupsPerStage + b / G::kG) * G::kG + b % G::kG;
              const float d = half_bits_to_float(
                  static_cast<unsigned short>((scw[j >> 1] >> (16 * (j & 1))) & 0xFFFFu));
#pragma unroll
              for (int lm = 0; lm < kMine; ++lm) {
                const int m = split * kMine + lm;
                {  // (rows past the batch have zero digits and a zero scale: no guard needed)
                  const int4 xc = xcs[j * MP + m];  // {scale, k_lo, k_hi, -}
                  const uint32_t* sums = v[kSerial ? 0 : b];
                  const int s0 = static_cast<int>(sums[4 * lm]);
                  const int s1 = static_cast<int>(sums[4 * lm + 1]);
                  const int s2 = static_cast<int>(sums[4 * lm + 2]);
                  const int s3 = static_cast<int>(sums[4 * lm + 3]);
                  const BlockParts parts =
                      kQ4 ? block_parts_cvt(s0, s1, s2, s3, xc.y, xc.z) : block_parts_cvt(s0, s1, s2);
                  const float term_scale = __fmul_rn(d, __int_as_float(xc.x));
                  acc[2 * (j & 1)][lm] = fmaf(parts.lo, term_scale, acc[2 * (j & 1)][lm]);
                  acc[2 * (j & 1) + 1][lm] = fmaf(parts.hi, term_scale, acc[2 * (j & 1) + 1][lm]);
                }
              }
            }
          } else {
#pragma unroll
          for (int c0 = 0; c0 < G::kColsPerWarp; c0 += G::kLdCols) {
            uint32_t v[G::kLdCols / 32][32];
            const uint32_t taddr = tmem_base + ts * G::kTCols + split * G::kColsPerWarp + c0 +
                                   (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll
            for (int h = 0; h < G::kLdCols / 32; ++h) tmem_ld_32x32(taddr + 32 * h, v[h]);
            tmem_ld_wait();
            if (c0 + G::kLdCols == G::kColsPerWarp) {  // all values in registers: hand the stage back
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(&bars->tmem_empty[ts]);
            }
#pragma unroll
            for (int q = 0; q < G::kLdCols / 4; ++q) {
              // columns 4*idx .. 4*idx+3: the four digit sums of (block class, activation row)
              // column in this warp's share of the stage: accumulator, then (class, row)
              const int column = c0 + 4 * q;
              const int idx = (column % G::kN) / 4;
              const int lm = G::kEpiSplit == 1 ? idx % MP : idx;  // row within this thread's share
              const int m = split * kMine + lm;
              const int j = (st * G::kGroupsPerStage + column / G::kN) * G::kG +
                            (G::kEpiSplit == 1 ? idx / MP : 0);
              {  // (rows past the batch have zero digits: their sums are zero, never stored)
                const int4 xc = xcs[j * MP + m];  // {scale, k_lo, k_hi, -}
                const int s0 = static_cast<int>(v[(4 * q) >> 5][(4 * q) & 31]);
                const int s1 = static_cast<int>(v[(4 * q) >> 5][(4 * q + 1) & 31]);
                const int s2 = static_cast<int>(v[(4 * q) >> 5][(4 * q + 2) & 31]);
                const int s3 = static_cast<int>(v[(4 * q) >> 5][(4 * q + 3) & 31]);
                const BlockParts parts =
                    G::kFused ? (kQ4 ? block_parts_cvt(s0, s1, s2, s3, xc.y, xc.z) : block_parts_cvt(s0, s1, s2))
                              : (kQ4 ? block_parts_cvt(s0, s1, s2, s3, xc.y, xc.z) : block_parts_cvt(s0, s1, s2));
                const float d = half_bits_to_float(
                    G::kRollGroups
                        ? *reinterpret_cast<const unsigned short*>(
                              raw_base + G::kScaleOffset + (row_in_tile * kSlabBlocks + j) * 2)
                        : static_cast<unsigned short>((scw[j >> 1] >> (16 * (j & 1))) & 0xFFFFu));
                const float term_scale = __fmul_rn(d, __int_as_float(xc.x));
                if (j & 1) {
                  acc[2][lm] = fmaf(parts.lo, term_scale, acc[2][lm]);
                  acc[3][lm] = fmaf(parts.hi, term_scale, acc[3][lm]);
                } else {
                  acc[0][lm] = fmaf(parts.lo, term_scale, acc[0][lm]);
                  acc[1][lm] = fmaf(parts.hi, term_scale, acc[1][lm]);
                }
              }
            }
          }
          }
          if (++ring_pos == G::kTPerSet) {
            ring_pos = 0;
            tphase ^= 1u;
          }
        }
        if (!ok) break;
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&bars->done[raw.slot]);  // scales consumed
          if (G::kFused) mbar_arrive(&bars->const_free[i % G::kConstRing]);
        }
      }
      raw.advance(G::kSlots);
      work.advance(G::kWorkSlots);

      // ---- unit / tile boundaries ----
      const bool unit_end = slab_in_unit + 1 == p.unit_slabs || slab == p.slabs - 1;
      if (unit_end) {
        if (mine) {
          count_open();  // an older share: its unit sums were stored a slab or more ago
          float* part = p.partial +
                        (static_cast<long long>(tile) * p.units_per_tile + unit) * p.m * kTileRows +
                        row_in_tile;
#pragma unroll
          for (int lm = 0; lm < kMine; ++lm) {
            const int m = split * kMine + lm;
            if (m < p.m) part[m * kTileRows] = unit_sum(acc[0][lm], acc[1][lm], acc[2][lm], acc[3][lm]);
            acc[0][lm] = acc[1][lm] = acc[2][lm] = acc[3][lm] = 0.0f;
          }
          ++units_mine;
        }
        const bool share_end = slab == p.slabs - 1 || i == count - 1;
        if (share_end) {
          // this thread's units of the row are written: the share is counted in a slab later
          if (units_mine > 0) {
            count_open();  // (only if this slab was not `mine`: at most one share stays open)
            open_tile = tile;
            open_add = units_mine;
          }
          units_mine = 0;
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
    count_open();
    resolve_counted();
    if (!ok) {
      *abort_flag = 1;
      report_error(p.error, 13);
    }
  } else if (kQ4 && warp < G::kFirstUnpackWarp + G::kUnpackWarps) {
    // ------------------------------ q4_0 high nibbles -------------------------
    // The raw tile is [128 rows][8 blocks x 16 bytes] with swizzled chunks; the tile of the
    // masked bytes (16 * high nibble) has the same layout, so the extraction is position by
    // position. The warps take an equal share of every slab each.
    const int u = warp - G::kFirstUnpackWarp;
    bool ok = true;
    RingPos raw, work;
    for (int i = 0; i < count; ++i) {
      if (!mbar_wait(&bars->raw_full[raw.slot], raw.phase, abort_flag)) {
        ok = false;
        break;
      }
      if (i >= G::kWorkSlots) {  // the work slot's previous tile has been consumed
        if (!mbar_wait(&bars->mma_done[work.slot], work.phase ^ 1u, abort_flag)) {
          ok = false;
          break;
        }
      }
      // 1024 16-byte chunks per tile, an equal share per warp, eight chunks per lane at a time
      constexpr int kChunksPerWarp = 1024 / (G::kUnpackWarps > 0 ? G::kUnpackWarps : 1);
      const uint4* packed =
          reinterpret_cast<const uint4*>(smem + raw.slot * G::kSlotBytes) + u * kChunksPerWarp;
      uint4* high =
          reinterpret_cast<uint4*>(work_ring + work.slot * G::kWorkBytes) + u * kChunksPerWarp;
#pragma unroll
      for (int batch = 0; batch < kChunksPerWarp / 256; ++batch) {
        uint4 w[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) w[h] = packed[batch * 256 + h * 32 + lane];
#pragma unroll
        for (int h = 0; h < 8; ++h) {
          high[batch * 256 + h * 32 + lane] =
              make_uint4(w[h].x & 0xF0F0F0F0u, w[h].y & 0xF0F0F0F0u, w[h].z & 0xF0F0F0F0u,
                         w[h].w & 0xF0F0F0F0u);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bars->ready[raw.slot]);
      raw.advance(G::kSlots);
      work.advance(G::kWorkSlots);
    }
    if (!ok) {
      *abort_flag = 1;
      report_error(p.error, 14);
    }
  } else if (G::kFused && warp >= G::kQuantWarp) {
    // ------------------------------ activation quantizers ---------------------
    // Quantizer warp w builds the images of slabs w, w + 3, ... in work slot w (one warp
    // per work slot: building an image is a long dependent chain, three of them overlap).
    // Lane (b, q): elements 4q..4q+3 and 16+4q..16+4q+3 of block b. Every lane copies its
    // own values into a ring in shared memory kAhead of its slabs before it needs them
    // (cp.async: no registers held meanwhile; a load from L2 takes longer than a slab).
    constexpr int kW = G::kQuantWarps;
    constexpr int kAhead = G::kXRingSlots - 1;
    const int qw = warp - G::kQuantWarp;
    bool ok = true;
    const int b = lane >> 2, q = lane & 3;
    const int first_slab = (slab0 + qw) % p.slabs;
    const int step = kW % p.slabs;  // slabs wrap around at the end of a row tile
    int copy_slab = first_slab, use_slab = first_slab;
    int copy_i = qw;  // CTA-local index of the next slab to copy
    RingPos raw;
    raw.advance_by(static_cast<uint32_t>(qw), G::kSlots);
    uint32_t slot_uses = 0;  // images built in this warp's work slot so far
    float* lane_ring = reinterpret_cast<float*>(x_ring) + qw * (G::kXRingSlots * MP * kSlabK) +
                       b * 32 + 4 * q;
    uint32_t copy_entry = 0, use_entry = 0;
    auto copy_ahead = [&]() {
      if (copy_i < count) {
        const int block = copy_slab * kSlabBlocks + b;
        if (block < p.nb) {
          float* entry = lane_ring + copy_entry * (MP * kSlabK);
#pragma unroll
          for (int m = 0; m < MP; ++m) {
            if (m < p.m) {
              const float* src = p.x + static_cast<long long>(m) * p.ldx + block * 32 + 4 * q;
              if (p.x_vector != 0) {
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(
                                 smem_u32(entry + m * kSlabK)),
                             "l"(src)
                             : "memory");
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(
                                 smem_u32(entry + m * kSlabK + 16)),
                             "l"(src + 16)
                             : "memory");
              } else {  // activations not on a 16-byte boundary
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  entry[m * kSlabK + e] = __ldg(src + e);
                  entry[m * kSlabK + 16 + e] = __ldg(src + 16 + e);
                }
              }
            }
          }
        }
        copy_slab += step;
        if (copy_slab >= p.slabs) copy_slab -= p.slabs;
        copy_i += kW;
        copy_entry = copy_entry + 1 == G::kXRingSlots ? 0 : copy_entry + 1;
      }
      asm volatile("cp.async.commit_group;" ::: "memory");  // one group per call, even if empty
    };
    int digit_offset[MP][4];
#pragma unroll
    for (int m = 0; m < MP; ++m) {
#pragma unroll
      for (int d = 0; d < 4; ++d) {
        const int row = ((b % G::kG) * MP + m) * 4 + d;
        digit_offset[m][d] =
            kQ4 ? row * 128 + ((b ^ (row & 7)) << 4) + 4 * q
                : (b >> 2) * (G::kN * 128) + row * 128 + (((2 * (b & 3)) ^ (row & 7)) << 4) + 4 * q;
      }
    }
    uint8_t* digits = work_ring + qw * G::kWorkBytes + G::kHBytes;
    // the activations may be the output of the kernel in front of this one
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int k = 0; k < kAhead; ++k) copy_ahead();
    for (int i = qw; i < count; i += kW) {
      copy_ahead();
      // all but the newest kAhead groups have landed: slab i's values are in the ring
      asm volatile("cp.async.wait_group %0;" ::"n"(kAhead) : "memory");
      float4 cur_lo[MP], cur_hi[MP];
      const bool cur_valid = use_slab * kSlabBlocks + b < p.nb;
      const float* entry = lane_ring + use_entry * (MP * kSlabK);
#pragma unroll
      for (int m = 0; m < MP; ++m) {
        cur_lo[m] = cur_hi[m] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (cur_valid && m < p.m) {
          cur_lo[m] = *reinterpret_cast<const float4*>(entry + m * kSlabK);
          cur_hi[m] = *reinterpret_cast<const float4*>(entry + m * kSlabK + 16);
        }
      }
      use_slab += step;
      if (use_slab >= p.slabs) use_slab -= p.slabs;
      use_entry = use_entry + 1 == G::kXRingSlots ? 0 : use_entry + 1;
      // The MMAs of this work slot's previous slab have read its digits. Nothing here waits
      // for the weights: the images are built up to kWorkSlots slabs ahead of the MMAs. That
      // previous slab is i - kWorkSlots > i - kSlots, so the `ready` barrier of slab i's
      // weight slot has long moved on to this slab's phase; the constants go to entry
      // i mod kConstSlots once the epilogue has released its previous user.
      if ((slot_uses > 0 &&
           !mbar_wait(&bars->mma_done[qw], (slot_uses - 1u) & 1u, abort_flag)) ||
          (i >= G::kConstRing &&
           !mbar_wait(&bars->const_free[i % G::kConstRing],
                      (static_cast<uint32_t>(i / G::kConstRing) - 1u) & 1u, abort_flag))) {
        ok = false;
        break;
      }
      {
        write_slab_image<FMT, MP>(
            digits, reinterpret_cast<XConst*>(const_ring + (i % G::kConstRing) * G::kConstBytes),
            digit_offset, cur_lo, cur_hi, cur_valid, lane, p.int8_activations != 0);
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&bars->const_ready[i % G::kConstRing]);
        mbar_arrive(&bars->ready[raw.slot]);
      }
      raw.advance_by(kW, G::kSlots);
      ++slot_uses;
    }
    if (!ok) {
      *abort_flag = 1;
      report_error(p.error, 18);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int FMT, int MP>
constexpr size_t gemv_smem_bytes() {
  return 1024 + static_cast<size_t>(TcGeom<FMT, MP>::kSlots) * TcGeom<FMT, MP>::kSlotBytes +
         static_cast<size_t>(TcGeom<FMT, MP>::kWorkSlots) * TcGeom<FMT, MP>::kWorkBytes +
         TcGeom<FMT, MP>::kConstSlots * TcGeom<FMT, MP>::kConstBytes +
         TcGeom<FMT, MP>::kXRingBytes + sizeof(GemvBarriers<FMT, MP>) + 64;
}

template <int FMT, int MP>
qx_status launch_one(const GemvTcParams& p, int grid, cudaStream_t stream) {
  constexpr size_t smem = gemv_smem_bytes<FMT, MP>();
  static_assert(smem <= kSmemLimit, "shared memory budget");
  static SmemOptIn opt_in;
  QX_TRY(opt_in.ensure(gemv_tc_kernel<FMT, MP>, smem));
  // Programmatic dependent launch: this kernel may start while the kernel in front of it
  // (the activation quantizer, or whatever produces the activations) is still running.
  // Everything that does not depend on the activations (barrier set-up, TMEM allocation,
  // the first weight copies) proceeds; the thread or warp that reads the activations or
  // their images waits for that kernel's results (griddepcontrol.wait).
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>(grid));
  config.blockDim = dim3(TcGeom<FMT, MP>::kThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  QX_CUDA_TRY(cudaLaunchKernelEx(&config, gemv_tc_kernel<FMT, MP>, p));
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

template <int FMT>
qx_status launch_fmt(int mp, const GemvTcParams& p, int grid, cudaStream_t stream) {
  switch (mp) {
    case 1: return launch_one<FMT, 1>(p, grid, stream);
    case 2: return launch_one<FMT, 2>(p, grid, stream);
    case 4: return launch_one<FMT, 4>(p, grid, stream);
    case 8: return launch_one<FMT, 8>(p, grid, stream);
    case 16: return launch_one<FMT, 16>(p, grid, stream);
    case 32: return launch_one<FMT, 32>(p, grid, stream);
    default: break;
  }
  set_last_error_text("gemv: unsupported batch size");
  return QX_STATUS_DEVICE_ERROR;
}

}  // namespace

static bool int8_rule_absent(const GemvOptions* options) {
  return options == nullptr || !options->int8_activations;
}

// K split: units of U slabs with at most 16 units per row; a function of K alone.
static int unit_slabs_for(long long slabs) { return static_cast<int>((slabs + 15) / 16); }

qx_status gemv_scratch_layout(const qx_weights* w, int m, int sm_count, GemvScratch* out) {
  if (w->tiles > kMaxCounterTiles) {
    set_last_error_text("qgemm: more than 262144 weight rows per prepared handle are not supported");
    return QX_STATUS_INVALID_SHAPE;
  }
  const int unit_slabs = unit_slabs_for(w->slabs);
  const int units_per_tile = static_cast<int>((w->slabs + unit_slabs - 1) / unit_slabs);
  const long long total_units = w->tiles * units_per_tile;
  size_t off = kCounterBytes;
  out->ximg_offset = off;
  off += align_up(static_cast<size_t>(w->slabs) * ximage_bytes(w->format, padded_batch(m)), 256);
  out->partial_offset = off;
  off += align_up(static_cast<size_t>(w->tiles) * units_per_tile * m * kTileRows * sizeof(float), 256);
  out->total_bytes = off;
  out->ctas = static_cast<int>(total_units < sm_count ? total_units : sm_count);
  out->unit_slabs = unit_slabs;
  out->units_per_tile = units_per_tile;
  return QX_STATUS_OK;
}

bool gemv_tc_quantizes_in_kernel(int m) { return padded_batch(m) <= 2; }

qx_status launch_gemv_tc(const qx_weights* w, const float* x, const uint8_t* ximg, float* y, int m,
                         long long ldy, uint8_t* ws_base, const GemvScratch& scratch,
                         cudaStream_t stream, const GemvPush* push, const GemvOptions* options) {
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  if (w->segments > 1) {
    for (int s = 0; s < w->segments; ++s) {
      if (options == nullptr || options->segment_y[s] == nullptr) {
        set_last_error_text("gemv: a fused handle needs one output pointer per segment");
        return QX_STATUS_INVALID_ARGUMENT;
      }
    }
    if (push != nullptr) {
      set_last_error_text("gemv: fused handles cannot push to other ranks");
      return QX_STATUS_INVALID_ARGUMENT;
    }
  }
  if (push != nullptr && push->peers > kMaxPushPeers) {
    set_last_error_text("gemv: more than 7 peer ranks");
    return QX_STATUS_INVALID_ARGUMENT;
  }
  // a single activation row goes to the streaming decode kernel (same bits, see there)
  const int sms = ctx->prop.multiProcessorCount;
  if (gemv_decode_enabled() && gemv_decode_serves(w, 1, scratch, sms)) {
    if (m == 1) {
      return launch_gemv_decode(w, x, y, scratch, sms, ctx->error_dev, stream, push, options);
    }
    // Two q4_0 rows on a small matrix: two launches of that kernel, one behind the other
    // (they overlap like any two steps), beat the persistent kernel's two-row variant
    // (14336 x 4096: 17 us against 21 us); from three rows on, and for q8_0, they do not.
    if (m == 2 && w->format == QX_FORMAT_Q4_0 && int8_rule_absent(options)) {
      for (int row = 0; row < 2; ++row) {
        GemvPush row_push;
        GemvOptions row_options;
        if (push != nullptr) {
          row_push = *push;
          for (int r = 0; r < push->peers; ++r) row_push.cells[r] = push->cells[r] + row * ldy;
        }
        if (options != nullptr) {
          row_options = *options;
          for (int q = 0; q < w->segments; ++q) {
            if (options->segment_y[q] != nullptr) {
              row_options.segment_y[q] = options->segment_y[q] + row * w->seg_rows[q];
            }
          }
        }
        QX_TRY(launch_gemv_decode(w, x + row * w->columns, y + row * ldy, scratch, sms,
                                  ctx->error_dev, stream, push != nullptr ? &row_push : nullptr,
                                  options != nullptr ? &row_options : nullptr));
      }
      return QX_STATUS_OK;
    }
  }
  return launch_gemv_tc_at(w, x, ximg, y, m, ldy, ws_base, scratch, ctx->error_dev, stream, push,
                           options);
}

qx_status launch_gemv_tc_at(const qx_weights* w, const float* x, const uint8_t* ximg, float* y,
                            int m, long long ldy, uint8_t* ws_base, const GemvScratch& scratch,
                            int* error_word, cudaStream_t stream, const GemvPush* push,
                            const GemvOptions* options) {
  GemvTcParams p{};
  p.segments = w->segments;
  for (int s = 0; s < qx_weights::kMaxSegments; ++s) {
    p.seg_tile_begin[s] = static_cast<int>(w->seg_tile_begin[s]);
    p.seg_rows[s] = w->seg_rows[s];
    p.seg_y[s] = (options != nullptr && options->segment_y[s] != nullptr) ? options->segment_y[s] : y;
  }
  if (w->segments > 1) {
    for (int s = 0; s < w->segments; ++s) {
      if (options == nullptr || options->segment_y[s] == nullptr) {
        set_last_error_text("gemv: a fused handle needs one output pointer per segment");
        return QX_STATUS_INVALID_ARGUMENT;
      }
    }
    if (push != nullptr) {
      set_last_error_text("gemv: fused handles cannot push to other ranks");
      return QX_STATUS_INVALID_ARGUMENT;
    }
  }
  p.int8_activations = (options != nullptr && options->int8_activations) ? 1 : 0;
  if (p.int8_activations != 0 && m != 1) {
    set_last_error_text("gemv: the int8 activation rule serves one activation row");
    return QX_STATUS_INVALID_SHAPE;
  }
  p.panel = w->panel;
  p.ximg = ximg;
  p.x = x;
  p.ldx = w->columns;
  p.nb = static_cast<int>(w->blocks_per_row);
  p.x_vector = reinterpret_cast<uintptr_t>(x) % 16 == 0 ? 1 : 0;
  p.y = y;
  p.partial = reinterpret_cast<float*>(ws_base + scratch.partial_offset);
  p.counters = reinterpret_cast<int*>(ws_base);
  p.error = error_word;
  p.ldy = ldy;
  p.rows = w->rows;
  p.m = m;
  p.slabs = static_cast<int>(w->slabs);
  p.tiles = static_cast<int>(w->tiles);
  p.unit_slabs = scratch.unit_slabs;
  p.units_per_tile = scratch.units_per_tile;
  const long long total_units = w->tiles * scratch.units_per_tile;  // < 2^23 (gemv_scratch_layout)
  p.units_per_cta = static_cast<uint32_t>(total_units / scratch.ctas);
  p.units_rem = static_cast<uint32_t>(total_units % scratch.ctas);
  if (push != nullptr && push->peers > 0) {
    if (push->peers > kMaxPushPeers) {
      set_last_error_text("gemv: more than 7 peer ranks");
      return QX_STATUS_INVALID_ARGUMENT;
    }
    p.peers = push->peers;
    p.push_tag = push->tag;
    for (int r = 0; r < push->peers; ++r) p.push_cells[r] = push->cells[r];
  }
  if (w->format == QX_FORMAT_Q8_0) {
    return launch_fmt<QX_FORMAT_Q8_0>(padded_batch(m), p, scratch.ctas, stream);
  }
  return launch_fmt<QX_FORMAT_Q4_0>(padded_batch(m), p, scratch.ctas, stream);
}

}  // namespace qx
