/*
 * qx_b200 -- C ABI of the B200 (sm_100a) implementation of the QuixiCore-CPU quantized
 * matmul hot path: q8_0 / q4_0 GEMV and batched qgemm, W8A8 int8 GEMM, W8A32 GEMM and
 * prepared (device-resident) packed weights.
 *
 * Every entry point below is the binding target for one public function of the
 * reference's `quixicore_cpu::` namespace; the comment above each declaration names the
 * reference declaration (file:line inside the reference project) it replaces. Argument
 * order, meaning, validation order and returned status values follow the reference.
 * Plain pointers and sizes only; no C++ or torch types cross this boundary.
 *
 * Pointer conventions
 *   - entry points WITHOUT a suffix take HOST pointers, copy inputs to the GPU, run the
 *     kernel on the library's own stream and copy the result back before returning
 *     (drop-in semantics of the reference: synchronous, caller owns every buffer);
 *   - entry points ending in `_dev` take DEVICE pointers and a `cudaStream_t` passed as
 *     `void*`; they enqueue work and return without waiting for it. One exception: a call
 *     whose scratch does not fit the workspace it was given (or the library's default one)
 *     grows that workspace first, which synchronises the device, frees and allocates. To
 *     keep `_dev` calls purely asynchronous (and legal inside stream capture), create the
 *     workspace up front with qx_workspace_create(reserve_bytes) large enough for the
 *     biggest call, or run each shape once before capturing.
 *
 * There is no CPU fallback: without a usable sm_100 device every compute entry point
 * returns QX_STATUS_DEVICE_ERROR.
 */
#ifndef QX_B200_H_
#define QX_B200_H_

#include <stddef.h>
#include <stdint.h>

/* Every entry point is exported with default visibility; the library itself is built
 * with hidden visibility so nothing else leaks. */
#if defined(_WIN32)
#define QX_API __declspec(dllexport)
#else
#define QX_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* quixicore_cpu::Status, include/quixicore_cpu/status.h:5-11 (values 0..4 identical).
 * QX_STATUS_DEVICE_ERROR is additive: a CUDA runtime / driver call failed or no
 * sm_100 device is present. qx_last_error_string() describes the failure. */
typedef enum qx_status {
  QX_STATUS_OK = 0,
  QX_STATUS_INVALID_SHAPE = 1,
  QX_STATUS_UNSUPPORTED_FORMAT = 2,
  QX_STATUS_INVALID_ARGUMENT = 3,
  QX_STATUS_OUT_OF_MEMORY = 4,
  QX_STATUS_DEVICE_ERROR = 5
} qx_status;

/* quixicore_cpu::QuantFormat, include/quixicore_cpu/qgemv.h:10-51. Numeric values are
 * stable; this path implements kQ8_0 (0) and kQ4_0 (1). Every other value is reported
 * as QX_STATUS_UNSUPPORTED_FORMAT by every entry point. */
enum { QX_FORMAT_Q8_0 = 0, QX_FORMAT_Q4_0 = 1 };

/* ---- device discovery: replaces quixicore_cpu::cpu_features(),
 * include/quixicore_cpu/cpu_features.h:13-41 (CPUID probing becomes device / NVLink
 * discovery). Fills *info for the current CUDA device. */
typedef struct qx_device_info {
  int device;               /* CUDA ordinal */
  int sm_major, sm_minor;   /* compute capability */
  int sm_count;
  int max_smem_per_block;   /* opt-in bytes */
  int l2_bytes;
  size_t hbm_bytes;
  int visible_devices;      /* CUDA devices visible to this process */
  int peer_access_mask;     /* bit i set: this device can map device i's memory */
  char name[64];
  /* NVLink discovery (read-only driver queries per visible peer) */
  int nvlink_peer_mask;     /* bit i set: peer i is reached over NVLink / NVSwitch (the pair
                               supports native atomics over the link; PCIe paths do not) */
  int nvlink_peers;         /* number of bits set in nvlink_peer_mask */
  int nvlink_uniform;       /* 1: every NVLink peer has the best performance rank, i.e. a
                               switched fabric with the same bandwidth to every peer */
  signed char peer_performance_rank[16]; /* driver's link ranking of peer i (0 = best), -1: none */
} qx_device_info;
QX_API qx_status qx_device_query(qx_device_info* info);
QX_API const char* qx_last_error_string(void);
/* Reports and clears the current device's pipeline error word: QX_STATUS_DEVICE_ERROR (and
 * a message naming the role code) if a kernel enqueued through a `_dev` entry point gave up
 * one of its bounded waits since the last report, else QX_STATUS_OK. It does not wait for
 * the GPU: synchronise the stream first. The host-pointer entry points make the same check
 * before they return. No counterpart in the reference (its kernels cannot stall). */
QX_API qx_status qx_check_device_errors(void);

/* ---- sizes, authoring ---------------------------------------------------------- */

/* qgemv_packed_size, include/quixicore_cpu/qgemv.h:70-71 (src/dispatch/qgemv.cpp:198-208) */
QX_API qx_status qx_qgemv_packed_size(int format, long long n, long long k, size_t* size);
/* qgemv_pack, include/quixicore_cpu/qgemv.h:77-78 (src/dispatch/qgemv.cpp:210-275):
 * quantise row-major f32 weights [n,k] into packed blocks. Host pointers. */
QX_API qx_status qx_qgemv_pack(int format, const float* weights, long long n, long long k,
                        void* packed);
/* qgemv_unpack, include/quixicore_cpu/qgemv.h:89-90 (src/dispatch/qgemv.cpp:277-300) */
QX_API qx_status qx_qgemv_unpack(int format, const void* packed, long long n, long long k,
                          float* weights);

/* ---- GEMV / batched GEMM over canonical packed bytes (host pointers) ---------------- */

/* qgemv, include/quixicore_cpu/qgemv.h:108-109 (src/dispatch/qgemv.cpp:337-365) */
QX_API qx_status qx_qgemv(int format, const void* packed, const float* x, float* y,
                   long long n, long long k);
/* qgemm, include/quixicore_cpu/qgemm.h:19-20 (kernels/quantization/qgemm_ref.cpp:141-164) */
QX_API qx_status qx_qgemm(int format, const void* packed_weights, const float* x, float* y,
                   long long m, long long n, long long k);
/* ---- qgemv_w8a8: the activation-quantising GEMV, include/quixicore_cpu/qgemv_w8a8.h:17-29
 * (src/dispatch/qgemv_w8a8.cpp:109-153; kernels/quantization/qgemv_w8a8_ref.cpp:18-41,
 * 120-177). The activations are quantised per 32-element block to int8 (scale amax / 127,
 * codes nearbyint(x / scale) clamped to +-127), the block dots are exact integers and each is
 * scaled by d_block * scale_block in f32. Non-finite activations: QX_STATUS_INVALID_ARGUMENT
 * (host-pointer form; the device form propagates NaN). */
QX_API qx_status qx_qgemv_w8a8(int format, const void* packed_weights, const float* x, float* y,
                        long long n, long long k);
QX_API qx_status qx_qgemv_w8a8_packed_size(int format, long long n, long long k, long long* bytes);
QX_API qx_status qx_qgemv_w8a8_pack(int format, const float* weights, long long n, long long k,
                             void* packed);
QX_API const char* qx_qgemv_w8a8_variant(int format);

/* ---- fused decode projections, include/quixicore_cpu/qgemv.h:143-154
 * (kernels/quantization/qgemv_fused_ref.cpp:195-340): several weight matrices over the same
 * activation vector. Here they are ONE launch over a fused handle (the matrices laid out back
 * to back on the device), which is what makes a decode layer's small GEMVs worth their fixed
 * launch cost. HOST pointers; `gelu_tanh` non-zero selects tanh-GELU, zero SiLU. */
QX_API qx_status qx_qgemv_up_gate(int format, const void* packed_up, const void* packed_gate,
                           const float* x, float* up, float* gate, long long n, long long k);
QX_API qx_status qx_qgemv_up_gate_activation(int format, const void* packed_up,
                                      const void* packed_gate, const float* x, float* out,
                                      long long n, long long k, int gelu_tanh);
QX_API qx_status qx_qgemv_qkv(int format, const void* packed_q, const void* packed_k,
                       const void* packed_v, const float* x, float* q, float* k_out,
                       float* v_out, long long query_dim, long long kv_dim,
                       long long input_dim);

/* qgemv_variant, include/quixicore_cpu/qgemv.h (src/dispatch/qgemv.cpp:392-405): name of
 * the kernel family that serves the format, "unsupported" otherwise. */
QX_API const char* qx_qgemv_variant(int format);

/* ---- prepared weights: replaces quixicore_cpu::CpuPackedWeights,
 * include/quixicore_cpu/packed_weights.h:72-97 (src/memory/packed_weights.cpp:197-278).
 * The handle owns a device-resident, re-laid-out copy of the canonical bytes (split
 * planes: block codes and fp16 scales; same total size as the canonical bytes). */
typedef struct qx_weights qx_weights;

/* CpuPackedWeightsInfo, include/quixicore_cpu/packed_weights.h:36-67 (the fields that
 * have a device meaning). */
typedef struct qx_weights_info {
  int format;
  long long rows, columns;
  long long block_size, blocks_per_row;
  size_t block_bytes;
  size_t contract_bytes;      /* canonical packed size */
  size_t prepared_bytes;      /* device bytes held by the handle */
  double memory_amplification;
  uint64_t preparation_ns;
  int device;
  int has_dense_bf16;         /* 1 after the first prefill GEMM built its fp16 tile cache */
  long long row_tile;         /* rows per panel tile on the device (128) */
  size_t panel_bytes;         /* bytes of the device panel (padded tiles included) */
} qx_weights_info;

/* CpuPackedWeights::prepare(format, contract_packed, rows, columns, layout),
 * packed_weights.h:82-84. `contract_packed` is a HOST pointer to canonical bytes; they
 * are copied (the caller may free them). Row range [row_begin, row_begin+row_count) of
 * the [rows, columns] matrix is kept on the current device: pass 0 / rows for the whole
 * matrix, or one shard's range when weights are sharded by output row over GPUs. */
QX_API qx_status qx_weights_prepare(int format, const void* contract_packed, long long rows,
                             long long columns, long long row_begin, long long row_count,
                             qx_weights** out);
/* Several matrices with the same column count in one handle (up + gate, q + k + v), each a
 * HOST pointer to canonical bytes of rows[i] x columns; count <= 4. One GEMV launch streams
 * all of them (qx_qgemm_fused_dev). Additive: the reference fuses per call instead
 * (kernels/quantization/qgemv_fused_ref.cpp:195-340). */
QX_API qx_status qx_weights_prepare_fused(int format, const void* const* contract_packed,
                                   const long long* rows, int count, long long columns,
                                   qx_weights** out);
/* Same, from canonical bytes already resident on the device (no host copy). */
QX_API qx_status qx_weights_prepare_dev(int format, const void* contract_packed_dev,
                                 long long rows, long long columns, long long row_begin,
                                 long long row_count, void* stream, qx_weights** out);
/* CpuPackedWeights::info(), packed_weights.h:88 */
QX_API qx_status qx_weights_get_info(const qx_weights* weights, qx_weights_info* info);
/* CpuPackedWeights::panel_data(), packed_weights.h:90: the re-laid-out panel. Here a DEVICE
 * pointer ([tile][K-slab] spans, see qx_weights_info.row_tile / panel_bytes); NULL for a
 * NULL handle. */
QX_API const void* qx_weights_panel_dev(const qx_weights* weights);
/* CpuPackedWeights::reset() / destructor, packed_weights.h:75,86 */
QX_API void qx_weights_destroy(qx_weights* weights);

/* Workspace, include/quixicore_cpu/workspace.h:19-58: reusable scratch arena, here in
 * device memory. NULL in the calls below selects a per-device default workspace owned
 * by the library (grown on demand, never shrunk). Calls that share a workspace must be
 * ordered on one stream. */
typedef struct qx_workspace qx_workspace;
QX_API qx_status qx_workspace_create(size_t reserve_bytes, qx_workspace** out);
QX_API size_t qx_workspace_capacity(const qx_workspace* workspace);
QX_API void qx_workspace_destroy(qx_workspace* workspace);

/* qgemm_prepacked(weights, x, y, m, workspace), include/quixicore_cpu/qgemm.h:26-27
 * (kernels/quantization/qgemm_panel.cpp:214-287). x [m, columns] f32, y [m, rows_kept]
 * f32, HOST pointers; m == 1 is the decode GEMV. */
QX_API qx_status qx_qgemm_prepacked(const qx_weights* weights, const float* x, float* y,
                             long long m, qx_workspace* workspace);
/* Same with DEVICE pointers on `stream`. ldy is the row stride of y in floats (>= rows
 * kept); pass the full N and an offset pointer to write a shard's slice in place. */
QX_API qx_status qx_qgemm_prepacked_dev(const qx_weights* weights, const float* x_dev,
                                 float* y_dev, long long m, long long ldy,
                                 qx_workspace* workspace, void* stream);
/* All matrices of a fused handle against the same activations: y_dev[i] (device pointers,
 * one per matrix, dense [m][rows_i]) = x . dequant(W_i)^T, m <= 32, one launch. */
QX_API qx_status qx_qgemm_fused_dev(const qx_weights* weights, const float* x_dev,
                             float* const* y_dev, long long m, qx_workspace* workspace,
                             void* stream);
/* qgemv_up_gate_activation on a fused {up, gate} handle: out_dev[n] = act(gate) * up;
 * scratch_dev holds 2 n floats (the two projections). */
QX_API qx_status qx_qgemv_up_gate_activation_dev(const qx_weights* up_gate, const float* x_dev,
                                          float* out_dev, float* scratch_dev, int gelu_tanh,
                                          qx_workspace* workspace, void* stream);
/* qgemv_w8a8 on a prepared handle, device pointers (m = 1). */
QX_API qx_status qx_qgemv_w8a8_prepacked_dev(const qx_weights* weights, const float* x_dev,
                                      float* y_dev, qx_workspace* workspace, void* stream);
/* qgemm_prepacked_storage with bf16 input, include/quixicore_cpu/qgemm.h:32-34 restricted
 * to FloatStorageType::kBF16 input and f32 output: the M >= 64 prefill GEMM. x_bf16_dev
 * [m, columns] bf16 bits, device pointers. */
QX_API qx_status qx_qgemm_prepacked_bf16_dev(const qx_weights* weights, const uint16_t* x_bf16_dev,
                                      float* y_dev, long long m, long long ldy,
                                      qx_workspace* workspace, void* stream);

/* ---- row-sharded decode with the all-gather fused into the GEMV -------------------------
 * One process per GPU; rank r keeps a contiguous row range of W (qx_weights_prepare with
 * row_begin / row_count) and every rank ends up with the full output, the semantics of
 * all_gather in kernels/collectives/collectives_ref.cpp:26-37. No counterpart in the
 * reference's quantized-matmul API (its row partition is over threads of one process).
 *
 * Instead of a collective after the GEMV, the kernel's row finishers store each result
 * into every other rank's INBOX over NVLink as one 8-byte cell {value, tag of the step}
 * (plain peer stores; data and tag travel together, so there are no flags and no fences),
 * and qx_allgather_wait_dev enqueues the receiving kernel: it takes every cell as soon as it
 * carries the step's tag, writes the value into this rank's plain result buffer and clears
 * the cell (kernels of several steps can be resident at once; each takes only its own).
 * It polls while this rank's own GEMV is still running and is through a moment after the
 * last slice has arrived; every wait is bounded (2 s). Steps alternate between two halves
 * of the buffers by the parity of `step`, so a rank may be one step ahead of a peer; `step`
 * counts from 1 and must advance by one per push / wait pair on every rank. Nothing about
 * a step lives in device memory, so both calls can be captured in a CUDA graph (a captured
 * sequence that is replayed must hold an even number of steps).
 *
 * The inbox must be peer-mappable: allocate it with qx_peer_alloc
 * (qx_push_inbox_bytes(world, m, rows) bytes, zero-initialised), pass the 64-byte handle to
 * the other processes (any channel) and map it there with qx_peer_open. Layouts:
 * results [2 parities][world][m][rows_per_rank] floats (ordinary device memory),
 * inbox   [2 parities][world][m][rows_per_rank] 8-byte cells. */
typedef struct qx_push_plan {
  int world;                 /* ranks, 2..8 */
  int rank;                  /* this rank */
  long long rows_per_rank;   /* rows of every shard (the handle's row count) */
  float* results_local;      /* this rank's result buffer (device pointer) */
  void* inbox_local;         /* this rank's inbox (device pointer) */
  void* inbox_peer[8];       /* inbox_peer[r]: rank r's inbox mapped here (r != rank) */
} qx_push_plan;

QX_API size_t qx_push_inbox_bytes(int world, long long m, long long rows_per_rank);
QX_API qx_status qx_peer_alloc(size_t bytes, void** dev_ptr, unsigned char handle[64]);
QX_API qx_status qx_peer_open(const unsigned char handle[64], void** dev_ptr);
QX_API qx_status qx_peer_close(void* dev_ptr);
QX_API qx_status qx_peer_free(void* dev_ptr);
/* y = x . dequant(W_shard)^T for m <= 32 activation rows, written to this rank's slice of
 * the step's result buffer and to every other rank's inbox. Only enqueues. */
QX_API qx_status qx_qgemm_prepacked_push_dev(const qx_weights* weights, const float* x_dev,
                                             long long m, const qx_push_plan* plan,
                                             long long step, qx_workspace* workspace,
                                             void* stream);
/* Enqueues the receive of all other ranks' slices of step `step`; *results_dev (host
 * variable, optional) receives the device address of that step's [world][m][rows_per_rank]
 * results in this rank's buffer, complete once this kernel has completed. A cell that does
 * not arrive in time (2 s; QX_B200_WAIT_LIMIT_MS in the environment overrides it) sets the
 * error word reported by qx_check_device_errors() or the next host-pointer call
 * (QX_STATUS_DEVICE_ERROR, role code 31); the kernel then returns. After such an error the
 * inbox may hold cells of the abandoned step: clear it before the plan is used again. */
QX_API qx_status qx_allgather_wait_dev(const qx_push_plan* plan, long long m, long long step,
                                       const float** results_dev, void* stream);

/* Decode GEMV (m = 1) that never allocates device memory. No counterpart in the
 * reference (its scratch is ordinary host memory).
 *
 * Who needs it: hosts that run the decode step where cudaMalloc / cudaFree are not
 * available to them -- a serving loop whose device memory is handed out once by the
 * application's own pool, a process whose GPU allocations are metered by an external
 * broker, or a latency-critical thread that cannot afford the device-wide synchronisation
 * an allocation implies. qx_qgemm_prepacked_dev grows a workspace on demand; this entry
 * point instead keeps all of its scratch (activation images, partial sums, row counters)
 * in one 6 MiB array that is part of the library image on every GPU that loads it, from
 * load until process exit. `weights` is a handle prepared earlier (preparing allocates;
 * do it at load time); x_dev [columns] and y_dev [rows] are device pointers.
 *
 * Limits and rules:
 *  - the matrix must fit the array: about rows * min(16, columns/256) * 4 bytes <= 5 MiB
 *    (every benchmark shape fits, e.g. 28672 x 8192); larger ones are rejected with
 *    QX_STATUS_INVALID_SHAPE and a message from qx_last_error_string();
 *  - the first call on a device looks up the array's device address (no allocation, but a
 *    runtime query): make that call before starting any stream capture;
 *  - all calls on a GPU share the array and it keeps the previous call's contents; each
 *    call clears the counters it needs on `stream` first. Calls that could overlap on the
 *    GPU (different streams, no ordering) race on it: keep them on one stream or order
 *    them with events;
 *  - a stalled pipeline is reported like everywhere else: the kernel leaves its role code in
 *    the device's error word (host memory mapped when the weights were prepared, so nothing
 *    is allocated here) and qx_check_device_errors() or the next host-pointer call on the
 *    device returns QX_STATUS_DEVICE_ERROR.
 * Results are bit-identical to qx_qgemm_prepacked_dev with m = 1. */
QX_API qx_status qx_qgemv_prepacked_noalloc_dev(const qx_weights* weights, const float* x_dev,
                                                float* y_dev, void* stream);

/* ---- W8A8 ---------------------------------------------------------------------- */

/* int8_gemm, include/quixicore_cpu/qgemm.h:235-239 (src/dispatch/int8_gemm.cpp:67-94).
 * W [n,k] int8, X [m,k] int8, Y [m,n] f32 = float(acc) * weight_scale[o] *
 * activation_scale[r], acc exact. HOST pointers. */
QX_API qx_status qx_int8_gemm(const int8_t* weights, const int8_t* x, const float* weight_scale,
                       const float* activation_scale, const int32_t* weight_row_sum,
                       const int* activation_zero_point, float* y, long long m,
                       long long n, long long k, int asymmetric);
/* qgemm_w8a8, include/quixicore_cpu/qgemm.h:250-252 */
QX_API qx_status qx_qgemm_w8a8(const int8_t* weights, const int8_t* x, const float* weight_scale,
                        const float* activation_scale, float* y, long long m,
                        long long n, long long k);
/* qgemm_w8a8_azp, include/quixicore_cpu/qgemm.h:253-257 */
QX_API qx_status qx_qgemm_w8a8_azp(const int8_t* weights, const int8_t* x,
                            const float* weight_scale, const float* activation_scale,
                            const int32_t* weight_row_sum, const int* activation_zero_point,
                            float* y, long long m, long long n, long long k);
/* int8_gemm_variant, include/quixicore_cpu/qgemm.h:240 */
QX_API const char* qx_int8_gemm_variant(void);
/* Device-pointer form. The reference validates that every scale is finite on each call
 * (src/dispatch/int8_gemm.cpp:78-85); here that scan runs on the device and a non-finite
 * scale makes the call return QX_STATUS_INVALID_ARGUMENT only when `check_scales` is
 * non-zero (it costs one small kernel and a 4-byte read-back, i.e. a synchronisation).
 * ldy: row stride of y in floats. acc_i32_dev (optional, may be NULL) receives the raw
 * int32 accumulators [m,n] (after the zero-point correction) for bit-exact checks. */
QX_API qx_status qx_int8_gemm_dev(const int8_t* weights_dev, const int8_t* x_dev,
                           const float* weight_scale_dev, const float* activation_scale_dev,
                           const int32_t* weight_row_sum_dev,
                           const int* activation_zero_point_dev, float* y_dev,
                           int32_t* acc_i32_dev, long long m, long long n, long long k,
                           long long ldy, int asymmetric, int check_scales, void* stream);

/* ---- W8A32 --------------------------------------------------------------------- */

/* qgemm_w8a32, include/quixicore_cpu/qgemm.h:244-246 (src/dispatch/w8a32_gemm.cpp:61-73).
 * HOST pointers. */
QX_API qx_status qx_qgemm_w8a32(const int8_t* weights, const float* weight_scale, const float* x,
                         float* y, long long m, long long n, long long k);
/* qgemm_w8a32_variant, include/quixicore_cpu/qgemm.h:247 */
QX_API const char* qx_qgemm_w8a32_variant(void);
QX_API qx_status qx_qgemm_w8a32_dev(const int8_t* weights_dev, const float* weight_scale_dev,
                             const float* x_dev, float* y_dev, long long m, long long n,
                             long long k, long long ldy, int check_scales,
                             qx_workspace* workspace, void* stream);

/* ---- compact 4-bit rows (LowBitFormat) and the int8 activation quantiser -----------------
 * quixicore_cpu::LowBitFormat, include/quixicore_cpu/lowbit.h:15-20: rows of ADJACENT 4-bit
 * codes (element 2i in the low nibble, value = nibble - 8) with separate f32 scales, one per
 * row (kInt4Row) or per group of group_size inputs (kInt4Group). The 2- and 3-bit formats of
 * the enum are sized correctly by qx_lowbit_packed_size but not served by the kernels
 * (QX_STATUS_UNSUPPORTED_FORMAT). */
enum { QX_LOWBIT_INT2_ROW = 0, QX_LOWBIT_INT3_GROUP64 = 1, QX_LOWBIT_INT4_ROW = 2, QX_LOWBIT_INT4_GROUP = 3 };
/* lowbit_packed_size, include/quixicore_cpu/lowbit.h:24-26 */
QX_API qx_status qx_lowbit_packed_size(int format, long long rows, long long dim,
                                long long group_size, size_t* weight_bytes,
                                size_t* scale_count);
/* lowbit_pack / lowbit_unpack, include/quixicore_cpu/lowbit.h:28-33. HOST pointers. */
QX_API qx_status qx_lowbit_pack(int format, const float* weights, uint8_t* packed, float* scales,
                         long long rows, long long dim, long long group_size);
QX_API qx_status qx_lowbit_unpack(int format, const uint8_t* packed, const float* scales,
                           float* weights, long long rows, long long dim, long long group_size);
/* lowbit_gemm, include/quixicore_cpu/lowbit.h:36-39: Y[m,n] = X[m,k] . dequant(W[n,k])^T in
 * f32. HOST pointers; the _dev form takes device pointers and a stream. */
QX_API qx_status qx_lowbit_gemm(int format, const uint8_t* packed_weights, const float* weight_scales,
                         const float* x, float* y, long long m, long long n, long long k,
                         long long group_size);
QX_API qx_status qx_lowbit_gemm_dev(int format, const uint8_t* packed_dev,
                             const float* weight_scales_dev, const float* x_dev, float* y_dev,
                             long long m, long long n, long long k, long long group_size,
                             void* stream);
QX_API const char* qx_lowbit_gemm_variant(int format);
/* lowbit_gemm_w8a8, include/quixicore_cpu/lowbit.h:44-47 (src/dispatch/lowbit_w8a8.cpp:68-101):
 * W4A8 for kInt4Row. Every activation row is quantised to int8 (quantize_int8 with one group
 * per row), the dot is an exact integer, Y = float(dot) * weight_scale[o] * activation_scale[r]
 * -- bit-identical to the reference. HOST pointers; the _dev form takes device pointers plus
 * qx_lowbit_w8a8_scratch_bytes(m, k) bytes of device scratch (it allocates nothing). */
QX_API qx_status qx_lowbit_gemm_w8a8(const uint8_t* packed_weights, const float* weight_scales,
                              const float* x, float* y, long long m, long long n, long long k);
QX_API size_t qx_lowbit_w8a8_scratch_bytes(long long m, long long k);
QX_API qx_status qx_lowbit_gemm_w8a8_dev(const uint8_t* packed_dev, const float* weight_scales_dev,
                                  const float* x_dev, float* y_dev, void* scratch_dev,
                                  long long m, long long n, long long k, void* stream);
QX_API const char* qx_lowbit_gemm_w8a8_variant(void);
/* quantize_int8, include/quixicore_cpu/quantization.h (kernels/quantization/
 * quantization_ref.cpp:143-168): per (row, group) scale = amax / 127, codes =
 * clamp(nearbyint(x / scale), -127, 127); group_size 0 = one group per row. Bit-identical to
 * the reference. HOST pointers; the _dev form takes device pointers (code_sums_dev optional:
 * the sum of every group's codes). */
QX_API qx_status qx_quantize_int8(const float* x, int8_t* codes, float* scales, long long rows,
                           long long dim, long long group_size);
QX_API qx_status qx_quantize_int8_dev(const float* x_dev, int8_t* codes_dev, float* scales_dev,
                               int* code_sums_dev, long long rows, long long dim,
                               long long group_size, void* stream);

/* ---- canonical prepared projections (CanonicalQuantTensor -> prepared weights) ------------
 * The reference prepares a CanonicalQuantTensor (include/quixicore_cpu/quant_import.h:24-36)
 * with CpuPackedWeights::prepare(tensor) (src/memory/packed_weights.cpp:280-398) and runs
 * typed projections on it (include/quixicore_cpu/qgemm.h:29-42). This library serves the two
 * integer layouts of that contract:
 *   kInt8Symmetric  one signed byte per element, rows of `columns` bytes;
 *   kInt4Symmetric  two elements per byte, the lower K index in the low nibble, a nibble
 *                   n >= 8 meaning n - 16 (kernels/quantization/qgemm_canonical.cpp:81-84,
 *                   160-163);
 *   kUInt4Affine    the same nibbles read as 0..15 with an f32 zero point beside every scale:
 *                   value = scale * (nibble - zero) (qgemm_canonical.cpp:164-167) -- the layout
 *                   the AWQ and GPTQ importers produce;
 * with f32 scales per row / output channel or per (row, group of group_size columns)
 * (scale_index, qgemm_canonical.cpp:86-115). GPTQ act-order tensors carry two optional maps of
 * `columns` ints: group_index (packed column -> scale group) and act_order (packed column ->
 * column of the activations), both honoured as in canonical_storage_panels
 * (qgemm_canonical.cpp:2823-2840). Enum values are the reference's
 * (include/quixicore_cpu/quant_contract.h:12-38); every other layout is reported as
 * QX_STATUS_UNSUPPORTED_FORMAT. */
enum { QX_CANONICAL_INT4_SYMMETRIC = 0, QX_CANONICAL_UINT4_AFFINE = 1, QX_CANONICAL_INT8_SYMMETRIC = 2 };
enum { QX_SCALE_NONE = 0, QX_SCALE_TENSOR = 1, QX_SCALE_ROW = 2, QX_SCALE_CHANNEL = 3, QX_SCALE_GROUP = 4 };
/* FloatStorageType, include/quixicore_cpu/float_storage.h:18 */
enum { QX_STORAGE_F32 = 0, QX_STORAGE_F16 = 1, QX_STORAGE_BF16 = 2 };
/* LinearActivation, include/quixicore_cpu/ops.h:56 */
enum { QX_ACTIVATION_NONE = 0, QX_ACTIVATION_GELU_ERF = 1, QX_ACTIVATION_GELU_TANH = 2,
       QX_ACTIVATION_SILU = 3, QX_ACTIVATION_RELU2 = 4 };

/* The fields of CanonicalQuantTensor this path reads, as a view over caller-owned HOST
 * arrays: metadata.layout / scale_mode / logical_rows / logical_columns / group_size,
 * data, scales. */
typedef struct qx_canonical_tensor {
  int layout;             /* QX_CANONICAL_* */
  int scale_mode;         /* QX_SCALE_ROW, QX_SCALE_CHANNEL or QX_SCALE_GROUP */
  long long rows;         /* output channels N */
  long long columns;      /* input features K */
  long long group_size;   /* columns per scale for QX_SCALE_GROUP; 0 or `columns` otherwise */
  const uint8_t* data;    /* canonical bytes: rows * columns (int8) or rows * columns / 2 */
  size_t data_bytes;
  const float* scales;    /* rows (row / channel) or rows * (columns / group_size) */
  size_t scale_count;
  const float* zero_points;   /* kUInt4Affine: one per scale; NULL / 0 otherwise */
  size_t zero_point_count;
  const int* group_index;     /* optional, `columns` entries (4-bit layouts only) */
  size_t group_index_count;
  const int* act_order;       /* optional, a permutation of 0 .. columns-1 */
  size_t act_order_count;
} qx_canonical_tensor;

typedef struct qx_canonical_weights qx_canonical_weights;

/* CpuPackedWeights::prepare(const CanonicalQuantTensor&), include/quixicore_cpu/
 * packed_weights.h (src/memory/packed_weights.cpp:280-398), with the checks of
 * validate_canonical_quant_tensor (kernels/quantization/quant_import_ref.cpp:401-476) for
 * these layouts. Uploads codes and scales once; the handle owns its device memory. */
QX_API qx_status qx_canonical_prepare(const qx_canonical_tensor* tensor,
                                      qx_canonical_weights** out);
QX_API void qx_canonical_destroy(qx_canonical_weights* weights);

/* qgemm_prepacked_storage, include/quixicore_cpu/qgemm.h:32-34: Y[m,rows] =
 * X[m,columns] . dequantize(W)^T with x and y stored as f32, f16 or bf16 (converted at the
 * kernel boundary, f32 arithmetic in between). x_count / y_count are the element counts of
 * FloatStorageInput / FloatStorageOutput and must equal m * columns / m * rows. HOST
 * pointers. Results agree with the reference within the tolerance of its own test
 * (|a - e| <= 4e-5 * (1 + |e|), tests/correctness/test_quant_projection_matrix.cpp:54-57):
 * the reference's summation order differs between its ISA variants, so there is no single
 * bit pattern to match. */
QX_API qx_status qx_qgemm_prepacked_storage(const qx_canonical_weights* weights, const void* x,
                                            int x_type, long long x_count, void* y, int y_type,
                                            long long y_count, long long m);
/* qgemm_prepacked_epilogue_storage, include/quixicore_cpu/qgemm.h:37-42: the same with an
 * output-channel bias (may be NULL) added and the activation applied before the store
 * (store_projection_output, qgemm_canonical.cpp:2570-2581). */
QX_API qx_status qx_qgemm_prepacked_epilogue_storage(const qx_canonical_weights* weights,
                                                     const void* x, int x_type, long long x_count,
                                                     const float* bias, void* y, int y_type,
                                                     long long y_count, long long m,
                                                     int activation);
/* DEVICE pointers and a stream. Enqueues two kernels (the digits of the activations, then the
 * projection; one more when the tensor has an act-order map; three per 256 tokens on the
 * tensor-core route that int8 tensors with one scale per row take from five tokens on) and
 * returns without waiting. The digit images (1792 bytes per token and 512 columns; on the
 * tensor-core route 4 * min(m, 256) * (columns + 4 * rows) bytes) live in `workspace` (NULL:
 * the library's default one), which grows -- and then synchronises the device -- the first time a larger call
 * arrives; calls that may run concurrently on different streams need workspaces of their own. */
QX_API qx_status qx_qgemm_prepacked_epilogue_storage_dev(const qx_canonical_weights* weights,
                                                         const void* x_dev, int x_type,
                                                         const float* bias_dev, void* y_dev,
                                                         int y_type, long long m, int activation,
                                                         qx_workspace* workspace, void* stream);
QX_API const char* qx_canonical_gemm_variant(void);

/* import_smoothquant_w8a8, include/quixicore_cpu/quant_import.h:117-133
 * (kernels/quantization/quant_import_ref.cpp:1051-1116): signed int8 weights [rows,columns]
 * with one f32 scale per output channel become a kInt8Symmetric tensor with channel scales
 * and group_size = columns; the per-row sums of the codes (the correction term of the
 * asymmetric W8A8 route) are copied when supplied and computed otherwise. Host-side format
 * conversion, no device work: *tensor becomes a view of the source arrays and
 * row_sums_out[rows] is filled. */
typedef struct qx_smoothquant_source {
  const int8_t* weights;
  size_t weight_count;
  const float* weight_scales;
  size_t weight_scale_count;
  const float* activation_scales;
  size_t activation_scale_count;
  const int* activation_zero_points;
  size_t activation_zero_point_count;
  const int32_t* row_sums;
  size_t row_sum_count;
  long long rows;
  long long columns;
} qx_smoothquant_source;
QX_API qx_status qx_import_smoothquant_w8a8(const qx_smoothquant_source* source,
                                            qx_canonical_tensor* tensor, int32_t* row_sums_out);

/* import_awq_u4, include/quixicore_cpu/quant_import.h:56-69 (quant_import_ref.cpp:840-903):
 * AWQ GEMM checkpoints -- qweight[K, N/8] words of eight 4-bit codes in the lane order
 * {0,4,1,5,2,6,3,7}, qzeros[K/group, N/8], scales[K/group, N] -- become a kUInt4Affine tensor
 * [N rows, K columns] with group scales and zero points. Host-side format conversion: the
 * caller provides data_out[N*K/2], scales_out[N*K/group] and zero_points_out[N*K/group];
 * *tensor becomes a view of them. */
typedef struct qx_awq_u4_source {
  const uint32_t* qweight;
  size_t qweight_words;
  const uint32_t* qzeros;
  size_t qzero_words;
  const float* scales;
  size_t scale_count;
  long long input_features;
  long long output_features;
  long long group_size;
} qx_awq_u4_source;
QX_API qx_status qx_import_awq_u4(const qx_awq_u4_source* source, qx_canonical_tensor* tensor,
                                  uint8_t* data_out, float* scales_out, float* zero_points_out);

/* import_gptq_u4, include/quixicore_cpu/quant_import.h:71-92 (quant_import_ref.cpp:905-999):
 * qweight[K/8, N], qzeros[G, N/8], scales[G, N]; V1 checkpoints store zero - 1; `symmetric`
 * folds the zero point into signed codes (kInt4Symmetric), otherwise kUInt4Affine; group_index
 * and act_order are passed through (the tensor view points at the source's arrays).
 * zero_points_out may be NULL for symmetric sources. */
typedef struct qx_gptq_u4_source {
  const uint32_t* qweight;
  size_t qweight_words;
  const uint32_t* qzeros;
  size_t qzero_words;
  const float* scales;
  size_t scale_count;
  const int* group_index;
  size_t group_index_count;
  const int* act_order;
  size_t act_order_count;
  long long input_features;
  long long output_features;
  long long group_size;
  int symmetric;
  int gptq_v2;
} qx_gptq_u4_source;
QX_API qx_status qx_import_gptq_u4(const qx_gptq_u4_source* source, qx_canonical_tensor* tensor,
                                   uint8_t* data_out, float* scales_out, float* zero_points_out);

/* ---- threading: set_num_threads / num_threads, include/quixicore_cpu/threading.h:11-12.
 * The fork-join pool is replaced by CUDA streams; these are kept so callers link. The
 * value is stored and returned, results never depend on it. */
QX_API void qx_set_num_threads(int n);
QX_API int qx_num_threads(void);

/* Number of kernels this library has launched in the calling process (all streams). */
QX_API unsigned long long qx_kernel_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* QX_B200_H_ */
