// W8A8 dispatch: picks the tensor-core kernel when the operands meet its alignment rules,
// otherwise the any-shape CUDA-core kernel. Mirrors the variant table of the reference
// (src/dispatch/int8_gemm.cpp:20-63): the choice is resolved once per process and
// QX_B200_INT8_GEMM_VARIANT=dp4a forces the CUDA-core kernel for A/B checks, as
// QUIXICORE_CPU_INT8_GEMM_VARIANT does there. Both are GPU kernels; there is no CPU path.

#include <cstdlib>
#include <cstring>

#include "qx_int8_gemm.cuh"

namespace qx {
namespace {
bool force_simple() {
  static const bool forced = []() {
    const char* v = std::getenv("QX_B200_INT8_GEMM_VARIANT");
    return v != nullptr && std::strcmp(v, "dp4a") == 0;
  }();
  return forced;
}
}  // namespace

const char* int8_gemm_variant_name() {
  return force_simple() ? "sm100a_dp4a" : "sm100a_tcgen05_i8";
}

qx_status launch_int8_gemm(const Int8GemmArgs& a, cudaStream_t stream) {
  if (!force_simple() && int8_gemm_tc_supported(a)) return launch_int8_gemm_tc(a, stream);
  return launch_int8_gemm_simple(a, stream);
}

}  // namespace qx
