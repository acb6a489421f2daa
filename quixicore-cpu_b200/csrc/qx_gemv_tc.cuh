// Launch interface of the tensor-core decode GEMV (qx_gemv_tc.cu).
#pragma once

#include "qx_gemv.cuh"
#include "qx_weights.cuh"

namespace qx {

constexpr int kGemvMaxBatch = 32;          // activation rows per launch (128 digit columns)
constexpr size_t kCounterBytes = kWorkspaceCounterBytes;  // tile arrival counters
constexpr long long kMaxCounterTiles = kCounterBytes / 4 / kTileRows;  // one counter per row

struct GemvScratch {
  size_t ximg_offset, partial_offset, total_bytes;
  int ctas;             // persistent CTAs of the launch
  int unit_slabs;       // slabs per K unit (a function of K alone)
  int units_per_tile;
};

// Scratch of one launch with `m` activation rows on a device with `sm_count` SMs. The
// first kCounterBytes of every workspace hold the per-tile arrival counters (zero
// between launches); the rest is laid out per call.
qx_status gemv_scratch_layout(const qx_weights* w, int m, int sm_count, GemvScratch* out);

// Row-sharded runs: where the kernel also delivers its results to the other ranks. Every
// finished output is stored as one 8-byte cell {value bits, tag of the step} into each
// peer's inbox (peer-mapped device pointers, already offset to this rank's slice of the
// step's parity buffer). Data and tag travel in one store, so the receiver needs no flag and
// the sender no fence: a cell that carries the step's tag holds the step's value.
struct PushCell {
  uint32_t value_bits;
  uint32_t tag;  // push_tag(step); the receiver of that step clears it when it takes the value
};
// Never zero, and different for steps that can be in flight at the same time: with small
// kernels and programmatic dependent launch the receive kernels of several steps can be
// resident at once and poll the same cells (steps two apart share a parity buffer); each
// takes only the cells of its own step.
inline uint32_t push_tag(long long step) {
  return static_cast<uint32_t>(static_cast<unsigned long long>(step) & 0x7FFFFFFFull) | 0x80000000u;
}
struct GemvPush {
  int peers = 0;
  uint32_t tag = 0;
  PushCell* cells[7] = {};
};

// Batches of one or two activation rows are quantized inside the GEMV kernel (it reads x);
// larger ones need the slab images written by the quantizer kernel first (qx_gemv.cu).
bool gemv_tc_quantizes_in_kernel(int m);

// x: activations [m][columns] f32; ximg: activation slab images (unused when the kernel
// quantizes itself)
qx_status launch_gemv_tc(const qx_weights* w, const float* x, const uint8_t* ximg, float* y, int m,
                         long long ldy, uint8_t* ws_base, const GemvScratch& scratch,
                         cudaStream_t stream, const GemvPush* push = nullptr,
                         const GemvOptions* options = nullptr);

// Same, with the device word that receives a non-zero role code when a bounded wait gives
// up passed in by the caller instead of taken from the per-device context.
qx_status launch_gemv_tc_at(const qx_weights* w, const float* x, const uint8_t* ximg, float* y,
                            int m, long long ldy, uint8_t* ws_base, const GemvScratch& scratch,
                            int* error_word, cudaStream_t stream, const GemvPush* push = nullptr,
                            const GemvOptions* options = nullptr);

// ---- single-row decode kernel (qx_gemv_decode.cu) ----------------------------------------
// Whether launch_gemv_tc hands single-row launches to it (on unless the environment says
// QX_B200_DECODE_KERNEL=0), and whether it serves this handle: one activation row and a K
// that splits into at most eight CTAs of at most eight slabs per row tile.
bool gemv_decode_enabled();
bool gemv_decode_serves(const qx_weights* w, int m, const GemvScratch& scratch, int sm_count);
// Same results, bit for bit, as launch_gemv_tc_at with m = 1; needs no scratch memory.
qx_status launch_gemv_decode(const qx_weights* w, const float* x, float* y,
                             const GemvScratch& scratch, int sm_count, int* error_word,
                             cudaStream_t stream, const GemvPush* push = nullptr,
                             const GemvOptions* options = nullptr);

const char* gemv_variant_name();

}  // namespace qx
