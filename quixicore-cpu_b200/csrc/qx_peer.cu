// Row-sharded decode across the GPUs of one node with the all-gather fused into the GEMV:
// peer-mappable buffers (CUDA IPC, one process per GPU), the pushing GEMV entry point and
// the kernel that receives the other ranks' slices. Semantics of all_gather in
// kernels/collectives/collectives_ref.cpp:26-37; the transport is plain 8-byte peer stores
// from the GEMV's row finishers (qx_gemv_tc.cu), no cluster multicast and no remote loads.

#include <cstdlib>
#include <cstring>

#include "qx_gemv_tc.cuh"
#include "qx_sm100.cuh"
#include "qx_weights.cuh"

namespace qx {
namespace {

// Receiving side of the fused all-gather. The inbox of a rank holds, per step parity, one
// 8-byte cell per (sending rank, activation row, weight row): {value bits, tag of the step}.
// The senders (the GEMV kernels of the other ranks) store value and tag together; this
// kernel takes every cell of the other ranks' slices as soon as it carries this step's tag,
// writes the value into the plain result buffer and clears the cell. No flags, no fences,
// no step counter in device memory: the tag travels with the data.
//
// It is launched programmatically, so it polls while this rank's own GEMV still runs (its
// blocks fit beside the GEMV's on the SMs) and is through a moment after the last slice
// has arrived. Before it exits, every thread waits for the kernels in front of it: when
// this kernel has completed, this rank's own slice (written by its GEMV) is complete too,
// which is what the kernel behind it relies on when it reads the gathered results.
//
// Why the tag is the step and not a valid bit: the kernels of a step are small, and with
// programmatic dependent launch the kernels of the following steps start as soon as there
// is room -- the receive kernels of steps s and s + 2, which share a parity buffer, can be
// resident at the same time. With a plain valid bit the later one took cells of the
// earlier step (and the earlier one then waited for them until its limit). Why a cell is
// never overwritten before it is taken: a rank pushes step s + 2 into the parity buffer of
// step s only after its own receive of step s + 1 has completed; that needed the
// receiver's push of step s + 1, which the receiver's GEMV only makes after its receive of
// step s has completed (it waits for the kernel in front before it reads its activations).
// Every wait is bounded: a cell that does not arrive within the limit makes the thread
// record role code 31 and stop polling.
__global__ void __launch_bounds__(256) allgather_unpack_kernel(PushCell* inbox, float* results,
                                                               long long slice, int world, int rank,
                                                               uint32_t step_tag, int* error,
                                                               unsigned long long limit_ns) {
  asm volatile("griddepcontrol.launch_dependents;");
  const long long total = static_cast<long long>(world) * slice;
  const unsigned long long start = sm100::global_timer_ns();
  bool ok = true;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total && ok; i += gridDim.x * 256LL) {
    if (i / slice == rank) continue;  // this rank's own slice comes straight from its GEMV
    uint32_t bits = 0, tag = 0;
    for (uint32_t spin = 0;; ++spin) {
      asm volatile("ld.relaxed.sys.global.v2.b32 {%0, %1}, [%2];"
                   : "=r"(bits), "=r"(tag)
                   : "l"(inbox + i)
                   : "memory");
      if (tag == step_tag) break;  // (cells of other steps are not this kernel's to take)
      if ((spin & 15u) == 15u) {
        const unsigned long long waited = sm100::global_timer_ns() - start;
        if (waited > limit_ns) {
          ok = false;
          break;
        }
        // poll tightly while the slices are expected any moment, back off afterwards
        if (waited > 20000ull) __nanosleep(200);
      }
    }
    if (!ok) break;
    results[i] = __uint_as_float(bits);
    asm volatile("st.relaxed.sys.global.v2.b32 [%0], {%1, %1};" ::"l"(inbox + i), "r"(0u) : "memory");
  }
  if (!ok) sm100::report_error(error, 31);
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

// Time limit of the receive kernel: 2 s, or QX_B200_WAIT_LIMIT_MS milliseconds (1..10000)
// when that is set in the environment (tests of the give-up path use a few milliseconds).
unsigned long long wait_limit_ns() {
  static const unsigned long long limit = []() -> unsigned long long {
    const char* text = std::getenv("QX_B200_WAIT_LIMIT_MS");
    if (text != nullptr) {
      const long ms = std::strtol(text, nullptr, 10);
      if (ms >= 1 && ms <= 10000) return static_cast<unsigned long long>(ms) * 1000000ull;
    }
    return sm100::kWaitLimitNs;
  }();
  return limit;
}

qx_status check_plan(const qx_push_plan* plan) {
  if (plan == nullptr || plan->world < 2 || plan->world > 8 || plan->rank < 0 ||
      plan->rank >= plan->world || plan->rows_per_rank <= 0 || plan->results_local == nullptr ||
      plan->inbox_local == nullptr) {
    return QX_STATUS_INVALID_ARGUMENT;
  }
  return QX_STATUS_OK;
}

}  // namespace
}  // namespace qx

extern "C" {

size_t qx_push_inbox_bytes(int world, long long m, long long rows_per_rank) {
  if (world < 1 || m < 1 || rows_per_rank < 1) return 0;
  return 2 * static_cast<size_t>(world) * static_cast<size_t>(m) * static_cast<size_t>(rows_per_rank) *
         sizeof(qx::PushCell);
}

qx_status qx_peer_alloc(size_t bytes, void** dev_ptr, unsigned char handle[64]) {
  using namespace qx;
  if (dev_ptr == nullptr || handle == nullptr || bytes == 0) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void* ptr = nullptr;
  cudaError_t err = cudaMalloc(&ptr, align_up(bytes, 256));
  if (err != cudaSuccess) {
    set_last_error("cudaMalloc(peer buffer)", err);
    return err == cudaErrorMemoryAllocation ? QX_STATUS_OUT_OF_MEMORY : QX_STATUS_DEVICE_ERROR;
  }
  cudaIpcMemHandle_t ipc;
  if ((err = cudaMemset(ptr, 0, align_up(bytes, 256))) != cudaSuccess ||
      (err = cudaIpcGetMemHandle(&ipc, ptr)) != cudaSuccess) {
    set_last_error("cudaIpcGetMemHandle", err);
    (void)cudaFree(ptr);
    return QX_STATUS_DEVICE_ERROR;
  }
  memcpy(handle, &ipc, 64);
  *dev_ptr = ptr;
  return QX_STATUS_OK;
}

qx_status qx_peer_open(const unsigned char handle[64], void** dev_ptr) {
  using namespace qx;
  if (dev_ptr == nullptr || handle == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  cudaIpcMemHandle_t ipc;
  memcpy(&ipc, handle, 64);
  void* ptr = nullptr;
  const cudaError_t err = cudaIpcOpenMemHandle(&ptr, ipc, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) {
    set_last_error("cudaIpcOpenMemHandle", err);
    return QX_STATUS_DEVICE_ERROR;
  }
  *dev_ptr = ptr;
  return QX_STATUS_OK;
}

qx_status qx_peer_close(void* dev_ptr) {
  if (dev_ptr == nullptr) return QX_STATUS_OK;
  const cudaError_t err = cudaIpcCloseMemHandle(dev_ptr);
  if (err != cudaSuccess) {
    qx::set_last_error("cudaIpcCloseMemHandle", err);
    return QX_STATUS_DEVICE_ERROR;
  }
  return QX_STATUS_OK;
}

qx_status qx_peer_free(void* dev_ptr) {
  if (dev_ptr == nullptr) return QX_STATUS_OK;
  const cudaError_t err = cudaFree(dev_ptr);
  if (err != cudaSuccess) {
    qx::set_last_error("cudaFree(peer buffer)", err);
    return QX_STATUS_DEVICE_ERROR;
  }
  return QX_STATUS_OK;
}

qx_status qx_qgemm_prepacked_push_dev(const qx_weights* weights, const float* x_dev, long long m,
                                      const qx_push_plan* plan, long long step,
                                      qx_workspace* workspace, void* stream) {
  using namespace qx;
  if (weights == nullptr || x_dev == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  QX_TRY(check_plan(plan));
  for (int r = 0; r < plan->world; ++r) {
    if (r != plan->rank && plan->inbox_peer[r] == nullptr) return QX_STATUS_INVALID_ARGUMENT;
  }
  if (step <= 0) return QX_STATUS_INVALID_ARGUMENT;
  if (m <= 0 || m > kGemvMaxBatch || weights->rows != plan->rows_per_rank) return QX_STATUS_INVALID_SHAPE;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  // result buffer and inboxes: [parity][world][m][rows_per_rank]; this rank writes slice `rank`
  const long long slice = m * plan->rows_per_rank;
  const long long offset = (step & 1) * plan->world * slice + static_cast<long long>(plan->rank) * slice;
  GemvPush push;
  push.peers = plan->world - 1;
  push.tag = push_tag(step);
  int slot = 0;
  for (int r = 0; r < plan->world; ++r) {
    if (r == plan->rank) continue;
    push.cells[slot++] = static_cast<PushCell*>(plan->inbox_peer[r]) + offset;
  }
  return launch_qgemm_f32(weights, x_dev, plan->results_local + offset, m, plan->rows_per_rank,
                          workspace != nullptr ? workspace : &ctx->workspace,
                          static_cast<cudaStream_t>(stream), &push);
}

qx_status qx_allgather_wait_dev(const qx_push_plan* plan, long long m, long long step,
                                const float** results_dev, void* stream) {
  using namespace qx;
  QX_TRY(check_plan(plan));
  if (m <= 0 || m > kGemvMaxBatch || step <= 0) return QX_STATUS_INVALID_ARGUMENT;
  DeviceContext* ctx = nullptr;
  QX_TRY(current_context(&ctx));
  const long long slice = m * plan->rows_per_rank;
  const long long parity_offset = (step & 1) * plan->world * slice;
  const long long cells = static_cast<long long>(plan->world - 1) * slice;
  long long blocks = (cells + 1023) / 1024;  // about four cells per thread
  blocks = blocks < 1 ? 1 : (blocks > 64 ? 64 : blocks);
  cudaLaunchConfig_t config{};
  config.gridDim = dim3(static_cast<unsigned>(blocks));
  config.blockDim = dim3(256);
  config.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  QX_CUDA_TRY(cudaLaunchKernelEx(&config, allgather_unpack_kernel,
                                 static_cast<PushCell*>(plan->inbox_local) + parity_offset,
                                 plan->results_local + parity_offset, slice, plan->world, plan->rank,
                                 push_tag(step), ctx->error_dev, wait_limit_ns()));
  count_launch();
  QX_CUDA_TRY(cudaGetLastError());
  if (results_dev != nullptr) *results_dev = plan->results_local + parity_offset;
  return QX_STATUS_OK;
}

}  // extern "C"
