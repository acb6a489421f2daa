// Single-row decode GEMV (M = 1): small CTAs that stream the prepared panel.
//
// A decode GEMV over a few tens of megabytes lasts a handful of microseconds, of the order
// of the costs at a kernel boundary (the grid has to drain, the next grid has to start, the
// first bytes have to come from HBM). One persistent CTA per SM with all of the SM's shared
// memory cannot overlap with its neighbours in the stream: the next kernel's CTA only gets
// on the SM when this one has left, and its first copy only leaves then. This kernel is
// built the other way round: many small CTAs (a row tile of 128 weight rows x a quarter or
// an eighth of K each, three or four resident per SM), each of which sends off the copies
// of its first slabs of weights BEFORE it waits for the kernel in front of it
// (griddepcontrol.wait). CTAs of the next launch take the places CTAs of this launch free
// one by one, so while one launch drains and the next has its activations quantized, HBM
// keeps delivering the next launch's weights.
//
// Arithmetic: identical to the tensor-core kernel (qx_gemv_tc.cu, qx_gemv.cuh): activation
// blocks as balanced base-256 digits under a power-of-two envelope, exact 8-bit integer
// digit sums, one f32 combination per block, blocks of a K unit accumulated in two chains
// (even and odd blocks, ascending), a row = (sum of even units) + (sum of odd units). The
// bits of a row do not depend on which of the two kernels computed it. The integer sums
// come from the warp-level MMA (mma.sync m16n8k32, u8/s8 x s8): with 32 products per
// instruction and lane the CUDA cores are left with the per-block combination only, which
// is what keeps the kernel on the memory side of its roofline.
//
// One MMA pair per (16 weight rows, two neighbouring blocks): the K = 32 slots of the MMA
// hold 16 code bytes of block A and 16 of block B, columns 0-3 of the B operand the four
// digits against block A (zero in B's slots), columns 4-7 the digits against block B. For
// q4_0 the first MMA takes the raw bytes (low nibble + 16 * high nibble) against the digits
// of 16 * t[i], the second the masked bytes (16 * high nibble) against the digits of
// t[i + 16] - 16 * t[i]; for q8_0 the two MMAs take the two halves of the blocks. Lane
// (g, t) of a warp then holds, for weight rows g and g + 8, digit sums (s0, s1) of block A
// (t = 0), (s2, s3) of A (t = 1), (s0, s1) of B (t = 2), (s2, s3) of B (t = 3).
//
// A CTA: eight warps of 16 weight rows each. A slab's span of the panel (codes in the
// tensor-core kernel's swizzled layout, then the fp16 scales) arrives by one bulk copy into
// a ring of two stages; the lanes read their eight code bytes per row and block pair
// straight from there, and the last warp to have taken a slab out of a stage sends off the
// copy of the slab that uses the stage next (no copy warp, nobody waits for a free stage).
// All CTAs of a launch are meant to be resident at once (four per SM for q4_0), with room
// left for the first CTAs of the next launch. The CTAs of a row tile form a thread-
// block cluster: unit sums go into the shared memory of the cluster's first CTA, which adds
// them in the fixed order after a cluster barrier -- no scratch memory, no atomics, no
// memory fences.

#include <cuda.h>
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>

#include "qx_gemv_tc.cuh"
#include "qx_sm100.cuh"

namespace qx {
namespace {

using namespace sm100;

constexpr int kDecodeWarps = kTileRows / 16;
constexpr int kDecodeThreads = 32 * kDecodeWarps;
constexpr int kDecodeStages = 2;         // ring depth (spans of one slab)
constexpr int kMaxCtaSlabs = 8;          // slabs of K per CTA (their digits stay in shared memory)
constexpr int kMaxUnits = 16;            // units per row (gemv_scratch_layout)
// B-operand fragments of a slab: per block pair 16 entries {first b0, b1, second b0, b1} for
// the lanes whose fragment is not zero by construction (column block == K-slot block), then
// zero entries for all other lanes: two of them (entries 16 and 20), so that the zero entry
// a quarter warp reads lies in the other half of the banks than its four real entries
constexpr int kFragPairBytes = 21 * 16;
constexpr int kFragBytes = 4 * kFragPairBytes;
constexpr int kLaneConstBytes = 4 * 4 * 8;  // per slab: [block pair][lane % 4]{scale, -k}
constexpr int kMaxPushPeers = 7;
constexpr int kSmemPerSm = 227 * 1024;

struct DecodeParams {
  const uint8_t* panel;
  const float* x;
  int* error;
  int slabs, nb, x_vector;
  int unit_slabs, units_per_tile;
  int ksplit;         // CTAs per row tile = cluster size
  int cta_slabs;      // most slabs any CTA handles (sizes the digit area)
  int segments;
  int seg_tile_begin[qx_weights::kMaxSegments];
  long long seg_rows[qx_weights::kMaxSegments];
  float* seg_y[qx_weights::kMaxSegments];
  int int8_activations;
  int peers;
  uint32_t push_tag;
  PushCell* push_cells[kMaxPushPeers];
  unsigned prefetch_stride;  // 0: a CTA calls only its own slabs into L2
};

struct __align__(8) DecodeBarriers {
  uint64_t full[2];   // the slab's span has landed in the stage
  int released[2];    // warps that have taken a slab out of the stage, counted over all its uses
  int abort_flag;
};

__device__ __forceinline__ void bulk_copy_g2s(uint32_t smem_dst, const void* gsrc, uint32_t bytes,
                                              uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(gsrc)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* gsrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(reinterpret_cast<uint64_t>(gsrc)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void cluster_arrive() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of `local` (a shared-memory address of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ void cluster_store(uint32_t remote, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
// shared-memory loads by 32-bit address (the lanes' addresses are built with XORs on it)
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ unsigned short lds16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}

// D = A * B + C: 16 weight rows x 32 code bytes (u8 for q4_0, s8 for q8_0) against 32 x 8
// digit bytes.
template <bool UNSIGNED_A>
__device__ __forceinline__ void mma_m16n8k32(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1, int c0, int c1,
                                             int c2, int c3) {
  if (UNSIGNED_A) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c0), "r"(c1), "r"(c2), "r"(c3));
  }
}

__device__ __forceinline__ uint32_t pack_low_bytes(int a, int b, int c, int d) {
  return __byte_perm(__byte_perm(a, b, 0x0040), __byte_perm(c, d, 0x0040), 0x5410);
}
// word[d] = the balanced base-256 digits d (signed bytes) of t[0..3]
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

struct __align__(8) LaneConst {
  float scale;  // the block's power-of-two scale (qx_gemv.cuh: XConst::scale)
  int neg_k;    // minus the q4_0 offset constant of this lane's part: -k_lo (low) or -k_hi
};

// The activation digits of one slab in MMA B-operand order, and its block constants. Lane
// (b = lane / 4, q = lane % 4) handles elements 4q..4q+3 (`lo`) and 16+4q..16+4q+3 (`hi`) of
// block b -- the same values, rounded the same way, as the quantizer of the tensor-core
// kernel. In the MMA pair of block pair b / 2 these are the K slots of lane t' =
// 2 * (b % 2) + q / 2, register q % 2, and digit d is column g' = 4 * (b % 2) + d; all
// other lanes' fragments are zero. The constants go where the consuming lanes
// look for them: entry [b / 2][2 * (b % 2) + part].
template <int FMT>
__device__ __forceinline__ void write_slab_fragments(uint8_t* frags, LaneConst* consts, float4 lo,
                                                     float4 hi, bool block_valid, int lane,
                                                     bool int8_activations) {
  const int b = lane >> 2, q = lane & 3;
  const float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
  uint32_t amax_bits = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) amax_bits = max(amax_bits, __float_as_uint(v[i]) & 0x7FFFFFFFu);
  amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 1));
  amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, 2));
  const uint32_t eb_raw = amax_bits >> 23;
  const bool finite = eb_raw != 255u;
  const uint32_t eb = max(eb_raw, 30u);  // envelope 2^(eb-126) > amax
  float scale_up = finite ? __uint_as_float((275u - eb) << 23) : 0.0f;  // 2^(22 - e)
  float scale = __uint_as_float((eb - (FMT == QX_FORMAT_Q4_0 ? 25u : 21u)) << 23);
  if (int8_activations) {
    // qgemv_w8a8 (kernels/quantization/qgemv_w8a8_ref.cpp:18-41)
    const float block_scale = __fdiv_rn(__uint_as_float(amax_bits), 127.0f);
    scale_up = (finite && block_scale != 0.0f) ? __fdiv_rn(1.0f, block_scale) : 0.0f;
    scale = FMT == QX_FORMAT_Q4_0 ? block_scale * 0.0625f : block_scale;
  }
  if (!finite) scale = __uint_as_float(0x7FC00000u);  // NaN/inf in -> NaN out
  if (!block_valid) scale = 0.0f;
  int t_lo[4], t_hi[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    t_lo[i] = __float2int_rn(v[i] * scale_up);
    t_hi[i] = __float2int_rn(v[4 + i] * scale_up);
    if (int8_activations) {
      t_lo[i] = max(-127, min(127, t_lo[i]));
      t_hi[i] = max(-127, min(127, t_hi[i]));
    }
  }
  int sum = 0;
  uint32_t w_lo[4] = {0u, 0u, 0u, 0u}, w_hi[4] = {0u, 0u, 0u, 0u};
  if (FMT == QX_FORMAT_Q8_0) {
    pack_digits<3>(t_lo, w_lo);
    pack_digits<3>(t_hi, w_hi);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) sum += t_lo[i] + t_hi[i];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      t_lo[i] *= 16;
      t_hi[i] -= t_lo[i];  // z_i
    }
    pack_digits<4>(t_lo, w_lo);
    pack_digits<4>(t_hi, w_hi);
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  }
  const int cb = b & 1;
  const int reg = q & 1;
  // entry of lane (g' = 4 * cb + d, t' = 2 * cb + q / 2): ((cb * 4 + d) * 2 + q / 2)
  uint32_t* pair = reinterpret_cast<uint32_t*>(frags + (b >> 1) * kFragPairBytes);
#pragma unroll
  for (int d = 0; d < 4; ++d) {  // (q8_0: the fourth digit is zero)
    uint32_t* entry = pair + ((cb * 4 + d) * 2 + (q >> 1)) * 4;
    entry[reg] = w_lo[d];
    entry[2 + reg] = w_hi[d];
  }
  // the pair's two zero entries: one word each from the eight lanes of the pair
  pair[(cb == 0 ? 16 : 20) * 4 + q] = 0u;
  if (q == 0) {
    int k_lo = 0, k_hi = 0;
    if (FMT == QX_FORMAT_Q4_0) q4_offset_constants(sum, &k_lo, &k_hi);
    LaneConst* mine = consts + (b >> 1) * 4 + 2 * cb;
    mine[0] = {scale, -k_lo};
    mine[1] = {scale, -k_hi};
  }
}

// CS: slabs per CTA when every CTA of the launch has the same number (the loops over slabs
// then unroll and the ring positions are constants), 0: read from the parameters.
template <int FMT, int CS>
__global__ void __launch_bounds__(kDecodeThreads, FMT == QX_FORMAT_Q4_0 ? 4 : 2)
gemv_decode_kernel(const DecodeParams p) {
  constexpr bool kQ4 = FMT == QX_FORMAT_Q4_0;
  constexpr int kSpan = slab_span_bytes(FMT);
  constexpr int kScaleOffset = slab_code_bytes(FMT);
  constexpr int kCodeSets = kQ4 ? 1 : 2;  // q8_0: the two halves of a block are separate bytes
  constexpr int kStages = kDecodeStages;
  static_assert(kSpan % 2048 == 0, "the lanes' XOR addressing needs stages on 2 KiB boundaries");
  // [ring: stages x span][fragments: cta_slabs x kFragBytes][constants][unit sums][barriers]
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* frags = smem + kStages * kSpan;
  LaneConst* consts = reinterpret_cast<LaneConst*>(frags + p.cta_slabs * kFragBytes);
  float* sums = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(consts) +
                                         p.cta_slabs * kLaneConstBytes);
  auto* bars = reinterpret_cast<DecodeBarriers*>(sums + kMaxUnits * kTileRows);
  volatile int* abort_flag = &bars->abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t ring = smem_u32(smem);

  asm volatile("griddepcontrol.launch_dependents;");
  // every CTA of the cluster is running before anyone stores into a neighbour's shared
  // memory: arrive now, wait after the set-up
  cluster_arrive();

  const int tile = static_cast<int>(blockIdx.x) / p.ksplit;
  const int part = static_cast<int>(blockIdx.x) - tile * p.ksplit;  // == cluster rank
  // the tile's units in `ksplit` nearly equal consecutive shares
  const int unit_begin = part * p.units_per_tile / p.ksplit;
  const int unit_end = (part + 1) * p.units_per_tile / p.ksplit;
  const int slab_begin = unit_begin * p.unit_slabs;
  const int slab_end = min(unit_end * p.unit_slabs, p.slabs);
  const int count = CS > 0 ? CS : max(slab_end - slab_begin, 0);
  const uint8_t* wsrc = p.panel + (static_cast<long long>(tile) * p.slabs + slab_begin) * kSpan;

  if (threadIdx.x == 0) {
    // the weights depend on nothing in front of this kernel: the first copies leave at once
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      bars->released[s] = 0;
    }
    bars->abort_flag = 0;
    mbar_fence_init();
    const int ahead = min(count, kStages);
    for (int i = 0; i < ahead; ++i) {
      mbar_arrive_expect_tx(&bars->full[i], kSpan);
      bulk_copy_g2s(ring + i * kSpan, wsrc + static_cast<long long>(i) * kSpan, kSpan, &bars->full[i]);
    }
    // ... and the CTA's other slabs are called into L2, so that they are near when the
    // stages come free
    for (int i = ahead; i < count; ++i) prefetch_l2(wsrc + static_cast<long long>(i) * kSpan, kSpan);
    // Only about `prefetch_stride` CTAs of a launch find room on the SMs while the launch
    // in front of it is still computing; the others start when that one leaves and would
    // all ask HBM for their first slabs at once, with every SM waiting. So each CTA also
    // calls into L2 what the CTAs `prefetch_stride`, 2 * `prefetch_stride`, ... further on
    // will copy: the early CTAs between them fetch the whole matrix while the launch in
    // front computes (a line that is in L2 already costs nothing).
    if (p.prefetch_stride > 0) {
      for (unsigned other = blockIdx.x + p.prefetch_stride; other < gridDim.x; other += p.prefetch_stride) {
        const int o_tile = static_cast<int>(other) / p.ksplit;
        const int o_part = static_cast<int>(other) - o_tile * p.ksplit;
        const int o_begin = (o_part * p.units_per_tile / p.ksplit) * p.unit_slabs;
        const int o_end = min(((o_part + 1) * p.units_per_tile / p.ksplit) * p.unit_slabs, p.slabs);
        const uint8_t* src = p.panel + (static_cast<long long>(o_tile) * p.slabs + o_begin) * kSpan;
        for (int i = 0; i < o_end - o_begin; ++i) prefetch_l2(src + static_cast<long long>(i) * kSpan, kSpan);
      }
    }
  }
  __syncthreads();
  cluster_wait();

  const int g = lane >> 2, t = lane & 3, hi = t >> 1;
  const int r0 = 16 * warp + g;  // rows r0 and r0 + 8 of the tile; (r0 & 7) == g for both
  // This lane's eight code bytes of (row r0, block pair pr) inside a stage. The panel stores
  // the 16-byte chunk c of a row at position c ^ (row & 7); with the pair index in the upper
  // bits of the chunk number that XOR comes down to one XOR of the address with a constant:
  //   q4_0  chunk = 2 * pr + hi:            address = code_base ^ (pr << 5)
  //   q8_0  chunk = 4 * (pr & 1) + 2 * hi + half (sub-tile pr / 2):
  //                                         address = code_base ^ (half << 4) ^ ((pr & 1) << 6)
  const uint32_t code_base =
      kQ4 ? r0 * 128 + ((g >> 1) << 5) + ((hi ^ (g & 1)) << 4) + (t & 1) * 8
          : r0 * 128 + ((g >> 2) << 6) + (((2 * hi) ^ (g & 3)) << 4) + (t & 1) * 8;
  const uint32_t scale_base = kScaleOffset + (r0 * kSlabBlocks + hi) * 2;  // blocks 2 * pr + hi
  // [pair][MMA][K half]{row r0, row r0 + 8}: this lane's code bytes of the current slab
  uint2 code[4][kCodeSets][2];
  uint32_t scale_bits[4];  // fp16 scales of this lane's block of each pair: row r0 | row r0 + 8
  bool ok = true;
  // Takes slab i (stage i % 2, its use number i / 2) out of the ring into registers -- the
  // weights depend on nothing in front of this kernel -- and frees the stage: the last warp
  // through sends off the copy of the slab that uses the stage next (the count runs over
  // all uses of a stage: nothing is reset).
  auto take_slab = [&](int i) -> bool {
    const uint32_t stage = static_cast<uint32_t>(i) & 1u, use = static_cast<uint32_t>(i) >> 1;
    // (the outcome is made uniform: the lanes of a warp run MMAs and shuffles together)
    if (!__all_sync(0xffffffffu, mbar_wait(&bars->full[stage], use & 1u, abort_flag))) return false;
    const uint32_t base = ring + stage * kSpan;
#pragma unroll
    for (int pr = 0; pr < 4; ++pr) {
#pragma unroll
      for (int half = 0; half < kCodeSets; ++half) {
        const uint32_t at = kQ4 ? base + (code_base ^ (pr << 5))
                                : base + (pr >> 1) * (kTileRows * 128) +
                                      (code_base ^ (half << 4) ^ ((pr & 1) << 6));
        // four 32-bit loads, in the order the MMA wants its A registers (row g | row g + 8)
        code[pr][half][0] = make_uint2(lds32(at), lds32(at + 8 * 128));
        code[pr][half][1] = make_uint2(lds32(at + 4), lds32(at + 8 * 128 + 4));
      }
      scale_bits[pr] = static_cast<uint32_t>(lds16(base + scale_base + pr * 4)) |
                       (static_cast<uint32_t>(lds16(base + scale_base + pr * 4 + 8 * kSlabBlocks * 2)) << 16);
    }
    __syncwarp();
    if (lane == 0) {
      const int before = atomicAdd(&bars->released[stage], 1);
      if (before == static_cast<int>(kDecodeWarps * (use + 1) - 1) && i + kStages < count) {
        mbar_arrive_expect_tx(&bars->full[stage], kSpan);
        bulk_copy_g2s(base, wsrc + static_cast<long long>(i + kStages) * kSpan, kSpan,
                      &bars->full[stage]);
      }
    }
    return true;
  };
  // the first slab before the activations are there: its stage is refilled that early
  if (count > 0) ok = take_slab(0);

  // the activations may be the output of the kernel in front of this one
  asm volatile("griddepcontrol.wait;" ::: "memory");
  for (int s = warp; s < count; s += kDecodeWarps) {
    const int block = (slab_begin + s) * kSlabBlocks + (lane >> 2);
    const bool valid = block < p.nb;
    float4 lo = make_float4(0.0f, 0.0f, 0.0f, 0.0f), hi4 = lo;
    if (valid) {
      const float* src = p.x + static_cast<long long>(block) * 32 + 4 * (lane & 3);
      if (p.x_vector != 0) {
        lo = __ldg(reinterpret_cast<const float4*>(src));
        hi4 = __ldg(reinterpret_cast<const float4*>(src + 16));
      } else {
        lo = make_float4(__ldg(src), __ldg(src + 1), __ldg(src + 2), __ldg(src + 3));
        hi4 = make_float4(__ldg(src + 16), __ldg(src + 17), __ldg(src + 18), __ldg(src + 19));
      }
    }
    write_slab_fragments<FMT>(frags + s * kFragBytes, consts + s * 16, lo, hi4, valid, lane,
                              p.int8_activations != 0);
  }
  __syncthreads();

  const uint32_t leader_sums = cluster_map(smem_u32(sums), 0);
  // (lanes whose fragment is zero by construction read the pair's zero entry)
  // (real entries of quarter warp q = lane / 8: 4 * q .. 4 * q + 3)
  uint32_t frag_at = smem_u32(frags) +
                     ((g >> 2) == hi ? ((hi * 4 + (g & 3)) * 2 + (t & 1)) : ((lane >> 3) & 1 ? 16 : 20)) * 16;
  uint32_t const_at = smem_u32(consts) + t * 8;
  // This lane's chain for its two rows: blocks of parity t / 2, low (t even) or high part.
  float acc0 = 0.0f, acc1 = 0.0f;
  int unit = unit_begin, slab_in_unit = 0;
#pragma unroll
  for (int i = 0; i < (CS > 0 ? CS : count); ++i) {
    if (!ok) break;
#pragma unroll
    for (int pr = 0; pr < 4; ++pr) {
      const uint4 b = lds128(frag_at + pr * kFragPairBytes);
      const uint2 lc = lds64(const_at + pr * 32);  // {scale, -k of this lane's part}
      const int nk = static_cast<int>(lc.y);
      int c[4];
      const uint2 lo = code[pr][0][0], up = code[pr][0][1];  // K slots 4t.. | 16 + 4t.., two rows each
      if (kQ4) {
        mma_m16n8k32<true>(c, lo.x, lo.y, up.x, up.y, b.x, b.y, 0, 0, 0, 0);
        mma_m16n8k32<true>(c, lo.x & 0xF0F0F0F0u, lo.y & 0xF0F0F0F0u, up.x & 0xF0F0F0F0u,
                           up.y & 0xF0F0F0F0u, b.z, b.w, c[0], c[1], c[2], c[3]);
      } else {
        const uint2 lo2 = code[pr][kCodeSets - 1][0], up2 = code[pr][kCodeSets - 1][1];
        mma_m16n8k32<false>(c, lo.x, lo.y, up.x, up.y, b.x, b.y, 0, 0, 0, 0);
        mma_m16n8k32<false>(c, lo2.x, lo2.y, up2.x, up2.y, b.z, b.w, c[0], c[1], c[2], c[3]);
      }
      // this lane's part of its block (low: s0 - k_lo + 256 s1; high: s2 - k_hi + 256 s3)
      const float f0 = __int2float_rn(c[0] + nk + (c[1] << 8));
      const float f1 = __int2float_rn(c[2] + nk + (c[3] << 8));
      const float scale = __uint_as_float(lc.x);
      const __half2 d = *reinterpret_cast<const __half2*>(&scale_bits[pr]);  // exact conversions
      acc0 = fmaf(f0, __fmul_rn(__low2float(d), scale), acc0);
      acc1 = fmaf(f1, __fmul_rn(__high2float(d), scale), acc1);
    }
    frag_at += kFragBytes;
    const_at += kLaneConstBytes;
    if (++slab_in_unit == p.unit_slabs || i == count - 1) {
      // the unit's sum from its four chains, into the first CTA of the cluster
      const float h0 = __shfl_down_sync(0xffffffffu, acc0, 1);
      const float h1 = __shfl_down_sync(0xffffffffu, acc1, 1);
      const float class0 = fmaf(h0, 65536.0f, acc0), class1 = fmaf(h1, 65536.0f, acc1);
      const float odd0 = __shfl_down_sync(0xffffffffu, class0, 2);
      const float odd1 = __shfl_down_sync(0xffffffffu, class1, 2);
      if (t == 0) {
        cluster_store(leader_sums + (unit * kTileRows + r0) * 4, __fadd_rn(class0, odd0));
        cluster_store(leader_sums + (unit * kTileRows + r0 + 8) * 4, __fadd_rn(class1, odd1));
      }
      acc0 = acc1 = 0.0f;
      slab_in_unit = 0;
      ++unit;
    }
    if (i + 1 < count) ok = take_slab(i + 1);
  }
  if (!ok) {
    *abort_flag = 1;
    report_error(p.error, 22);
  }
  __syncwarp();
  cluster_arrive();
  cluster_wait();

  if (part == 0 && threadIdx.x < kTileRows) {
    // ------------------------------ the row's sum ------------------------------
    const int row_in_tile = threadIdx.x;
    int seg = 0;
#pragma unroll
    for (int q = 1; q < qx_weights::kMaxSegments; ++q) {
      if (q < p.segments && tile >= p.seg_tile_begin[q]) seg = q;
    }
    const long long row = static_cast<long long>(tile - p.seg_tile_begin[seg]) * kTileRows + row_in_tile;
    if (row < p.seg_rows[seg]) {
      float even = 0.0f, odd = 0.0f;
#pragma unroll
      for (int u = 0; u < kMaxUnits; u += 2) {
        if (u < p.units_per_tile) even += sums[u * kTileRows + row_in_tile];
        if (u + 1 < p.units_per_tile) odd += sums[(u + 1) * kTileRows + row_in_tile];
      }
      const float value = even + odd;
      p.seg_y[seg][row] = value;
      for (int r = 0; r < p.peers; ++r) {
        // value and tag in ONE 8-byte store: whoever sees the tag sees the value
        asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %2};" ::"l"(p.push_cells[r] + row),
                     "r"(__float_as_uint(value)), "r"(p.push_tag)
                     : "memory");
      }
    }
  }
}

struct DecodePlan {
  int ksplit, cta_slabs;
  long long free_slots;  // CTAs that fit on the device beside one launch
  size_t smem;
};

template <int FMT>
constexpr size_t decode_smem_bytes(int cta_slabs) {
  return static_cast<size_t>(kDecodeStages) * slab_span_bytes(FMT) +
         static_cast<size_t>(cta_slabs) * (kFragBytes + kLaneConstBytes) +
         kMaxUnits * kTileRows * sizeof(float) + sizeof(DecodeBarriers) + 64;
}

// How a handle is cut into CTAs: `ksplit` CTAs (a cluster) per row tile, each with at most
// kMaxCtaSlabs slabs of K; a whole launch has to be resident at once (the next launch's CTAs
// then move in as this launch's leave). Among the splits that allow that, measured on
// matrices of 17 - 66 MB:
//  - at most four slabs per CTA first: the ring has two stages, every further slab is a
//    refill at L2 latency in the CTA's critical path (3584 x 8192 q8_0: 6.8 us with four
//    slabs per CTA, 10.0 us with eight); q8_0 with more than four is left to the persistent
//    kernel, q4_0 (four CTAs per SM to hide the refills) still wins with eight;
//  - then a split that leaves room for a whole second launch beside this one (4096 x 4096
//    q8_0: 5.4 us with 128 CTAs of four slabs, 6.8 us with 256 of two, which fill the SMs);
//  - then the finest one: more CTAs are more warps per SM (4096 x 4096 q4_0: 4.3 us with
//    256 CTAs of two slabs, 7.5 us with 128 of four).
// Larger matrices stay with the persistent tensor-core kernel.
template <int FMT>
bool plan_decode(const qx_weights* w, const GemvScratch& scratch, int sm_count, DecodePlan* plan) {
  const int units = scratch.units_per_tile, unit_slabs = scratch.unit_slabs;
  if (units > kMaxUnits) return false;
  constexpr int kCtasByRegisters = FMT == QX_FORMAT_Q4_0 ? 4 : 2;  // __launch_bounds__
  bool found = false;
  int best_deep = 0, best_single = 0;  // of the plan found so far: > 4 slabs, no room for a second launch
  for (int ks = 1; ks <= 8; ks *= 2) {
    if (ks > 1 && ks > units) break;
    const int upc = (units + ks - 1) / ks;
    const int cta_slabs = upc * unit_slabs;
    if (cta_slabs > kMaxCtaSlabs) continue;
    const int deep = cta_slabs > 4 ? 1 : 0;
    if (deep != 0 && FMT != QX_FORMAT_Q4_0) continue;
    const size_t smem = decode_smem_bytes<FMT>(cta_slabs);
    int per_sm = static_cast<int>(kSmemPerSm / (smem + 1024));
    if (per_sm > kCtasByRegisters) per_sm = kCtasByRegisters;
    const long long grid = w->tiles * ks, slots = static_cast<long long>(per_sm) * sm_count;
    if (grid > slots) continue;
    const int single = 2 * grid > slots ? 1 : 0;
    // ks ascends, so among equals the later (finer) split wins
    if (found && (deep > best_deep || (deep == best_deep && single > best_single))) continue;
    plan->ksplit = ks;
    plan->cta_slabs = cta_slabs;
    plan->smem = smem;
    plan->free_slots = slots - grid;
    found = true;
    best_deep = deep;
    best_single = single;
  }
  return found;
}

template <int FMT, int CS>
qx_status launch_decode_one(const DecodeParams& p, const DecodePlan& plan, long long tiles,
                            cudaStream_t stream) {
  static SmemOptIn opt_in;
  QX_TRY(opt_in.ensure(gemv_decode_kernel<FMT, CS>, decode_smem_bytes<FMT>(kMaxCtaSlabs)));
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>(tiles * plan.ksplit));
  config.blockDim = dim3(kDecodeThreads);
  config.dynamicSmemBytes = plan.smem;
  config.stream = stream;
  // Programmatic dependent launch (the CTAs start while the kernel in front is still
  // running and wait for its results themselves) and one cluster per row tile.
  cudaLaunchAttribute attributes[2]{};
  attributes[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attributes[0].val.programmaticStreamSerializationAllowed = 1;
  attributes[1].id = cudaLaunchAttributeClusterDimension;
  attributes[1].val.clusterDim.x = static_cast<unsigned>(plan.ksplit);
  attributes[1].val.clusterDim.y = 1;
  attributes[1].val.clusterDim.z = 1;
  config.attrs = attributes;
  config.numAttrs = 2;
  QX_CUDA_TRY(cudaLaunchKernelEx(&config, gemv_decode_kernel<FMT, CS>, p));
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  return QX_STATUS_OK;
}

template <int FMT>
qx_status launch_decode_fmt(const DecodeParams& p, const DecodePlan& plan, long long tiles,
                            cudaStream_t stream) {
  // every CTA has plan.cta_slabs slabs when K divides evenly
  const bool even = static_cast<long long>(plan.ksplit) * plan.cta_slabs == p.slabs;
  if (even && plan.cta_slabs == 2) return launch_decode_one<FMT, 2>(p, plan, tiles, stream);
  if (even && plan.cta_slabs == 4) return launch_decode_one<FMT, 4>(p, plan, tiles, stream);
  if (even && plan.cta_slabs == 8) return launch_decode_one<FMT, 8>(p, plan, tiles, stream);
  return launch_decode_one<FMT, 0>(p, plan, tiles, stream);
}

}  // namespace

bool gemv_decode_enabled() {
  static const bool enabled = []() {
    const char* v = std::getenv("QX_B200_DECODE_KERNEL");
    return v == nullptr || std::strcmp(v, "0") != 0;
  }();
  return enabled;
}

bool gemv_decode_serves(const qx_weights* w, int m, const GemvScratch& scratch, int sm_count) {
  if (m != 1) return false;
  DecodePlan plan{};
  return w->format == QX_FORMAT_Q4_0 ? plan_decode<QX_FORMAT_Q4_0>(w, scratch, sm_count, &plan)
                                     : plan_decode<QX_FORMAT_Q8_0>(w, scratch, sm_count, &plan);
}

qx_status launch_gemv_decode(const qx_weights* w, const float* x, float* y,
                             const GemvScratch& scratch, int sm_count, int* error_word,
                             cudaStream_t stream, const GemvPush* push,
                             const GemvOptions* options) {
  DecodePlan plan{};
  const bool q4 = w->format == QX_FORMAT_Q4_0;
  if (!(q4 ? plan_decode<QX_FORMAT_Q4_0>(w, scratch, sm_count, &plan)
           : plan_decode<QX_FORMAT_Q8_0>(w, scratch, sm_count, &plan))) {
    set_last_error_text("gemv: shape not served by the decode kernel");
    return QX_STATUS_INVALID_SHAPE;
  }
  DecodeParams p{};
  p.segments = w->segments;
  for (int s = 0; s < qx_weights::kMaxSegments; ++s) {
    p.seg_tile_begin[s] = static_cast<int>(w->seg_tile_begin[s]);
    p.seg_rows[s] = w->seg_rows[s];
    p.seg_y[s] = (options != nullptr && options->segment_y[s] != nullptr) ? options->segment_y[s] : y;
  }
  p.int8_activations = (options != nullptr && options->int8_activations) ? 1 : 0;
  p.panel = w->panel;
  p.x = x;
  p.error = error_word;
  p.slabs = static_cast<int>(w->slabs);
  p.nb = static_cast<int>(w->blocks_per_row);
  p.x_vector = reinterpret_cast<uintptr_t>(x) % 16 == 0 ? 1 : 0;
  p.unit_slabs = scratch.unit_slabs;
  p.units_per_tile = scratch.units_per_tile;
  p.ksplit = plan.ksplit;
  p.cta_slabs = plan.cta_slabs;
  // (not when a CTA would have to call for more than eight others: few free places)
  p.prefetch_stride = plan.free_slots * 8 >= w->tiles * plan.ksplit
                          ? static_cast<unsigned>(plan.free_slots)
                          : 0u;
  if (push != nullptr && push->peers > 0) {
    p.peers = push->peers;
    p.push_tag = push->tag;
    for (int r = 0; r < push->peers; ++r) p.push_cells[r] = push->cells[r];
  }
  return q4 ? launch_decode_fmt<QX_FORMAT_Q4_0>(p, plan, w->tiles, stream)
            : launch_decode_fmt<QX_FORMAT_Q8_0>(p, plan, w->tiles, stream);
}

}  // namespace qx
