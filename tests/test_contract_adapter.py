"""The KernelCall adapter (include/qx_b200_contract.hpp): the umbrella contract ABI of the
reference (include/quixicore/contract/kernel_abi.hpp:53-107) wired to this library's entry
points. On CPU: it compiles as plain C++17 (against its own restatement of the ABI and, when
the reference's headers are present, against those), validates tensor views and reports a
missing device as runtime_error. On a GPU: host and device tensors reach the kernels and the
results equal the typed entry points' bit for bit."""

import os
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "quixicore-cpu_b200")
REFERENCE_INCLUDE = os.path.join(os.environ.get("QX_REFERENCE_ROOT") or
                                 os.path.join(os.path.dirname(ROOT), "reference"), "include")

COMMON = r"""
    #include <cstdio>
    #include <cstdlib>
    #include <cstring>
    #include <vector>
    #include "qx_b200_contract.hpp"
    namespace qc = quixicore::contract;
    namespace api = quixicore::b200::contract_api;
    #define CHECK(cond) do { if (!(cond)) { std::printf("FAILED: %s (line %d)\n", #cond, __LINE__); return 1; } } while (0)
    static qc::TensorView view(void* data, const std::int64_t* shape, std::size_t rank, qc::DType dtype,
                               qc::MemorySpace space) {
      return qc::TensorView{data, shape, nullptr, rank, dtype, space, qc::tensor_contiguous};
    }
"""

CPU_PROGRAM = textwrap.dedent(COMMON + r"""
    int main() {
      const std::int64_t wshape[2] = {4, 64}, xshape[1] = {64}, yshape[1] = {4}, bad[1] = {5};
      std::vector<unsigned char> w(4 * 2 * 34, 0);
      std::vector<float> x(64, 1.0f), y(4, 0.0f);
      qc::TensorView in[2] = {view(w.data(), wshape, 2, qc::DType::packed, qc::MemorySpace::host),
                              view(x.data(), xshape, 1, qc::DType::f32, qc::MemorySpace::host)};
      qc::TensorView out[1] = {view(y.data(), yshape, 1, qc::DType::f32, qc::MemorySpace::host)};
      qc::Attribute format{"format", qc::AttributeKind::i64, nullptr, 0, 0, 0.0};
      qc::KernelCall call{in, 2, out, 1, &format, 1, nullptr, nullptr, nullptr, 0};
      CHECK(api::dispatch("rms_norm", call).code == qc::StatusCode::adapter_not_wired);
      qc::KernelCall no_format = call;
      no_format.attribute_count = 0;
      CHECK(api::dispatch("qgemv", no_format).code == qc::StatusCode::invalid_argument);
      qc::KernelCall one_input = call;
      one_input.input_count = 1;
      CHECK(api::dispatch("qgemv", one_input).code == qc::StatusCode::invalid_argument);
      out[0] = view(y.data(), bad, 1, qc::DType::f32, qc::MemorySpace::host);
      CHECK(api::dispatch("qgemv", call).code == qc::StatusCode::invalid_shape);
      out[0] = view(y.data(), yshape, 1, qc::DType::f16, qc::MemorySpace::host);
      CHECK(api::dispatch("qgemv", call).code == qc::StatusCode::invalid_shape);
      out[0] = view(y.data(), yshape, 1, qc::DType::f32, qc::MemorySpace::host);
      in[1] = view(x.data(), xshape, 1, qc::DType::f64, qc::MemorySpace::host);
      CHECK(api::dispatch("qgemv", call).code == qc::StatusCode::unsupported_dtype);
      in[1] = view(x.data(), xshape, 1, qc::DType::f32, qc::MemorySpace::device);
      CHECK(api::dispatch("qgemv", call).code == qc::StatusCode::invalid_argument);  // mixed spaces
      in[1] = view(x.data(), xshape, 1, qc::DType::f32, qc::MemorySpace::host);
      format.i64 = 9;  // not a format of this path: the entry point's own status comes back
      CHECK(api::dispatch("qgemv", call).code == qc::StatusCode::unsupported_format);
      format.i64 = 0;
      const qc::Status status = api::dispatch("qgemv", call);
      // with a device the call computes; without one it must fail loudly, never fall back
      CHECK(status.code == qc::StatusCode::ok || status.code == qc::StatusCode::runtime_error);
      std::printf("contract adapter ok %d\n", static_cast<int>(status.code));
      return 0;
    }
""")

GPU_PROGRAM = textwrap.dedent(COMMON + r"""
    #include <cuda_runtime.h>
    int main() {
      const long long n = 384, k = 2048, m = 3;
      std::vector<unsigned char> w(n * (k / 32) * 18);
      unsigned state = 12345u;
      for (auto& b : w) { state = state * 1664525u + 1013904223u; b = static_cast<unsigned char>(state >> 24); }
      for (long long blk = 0; blk < n * (k / 32); ++blk) { w[blk * 18] = 0x66; w[blk * 18 + 1] = 0x1E; }  // d ~ 0.006
      std::vector<float> x(m * k), y_adapter(m * n), y_typed(m * n);
      for (auto& v : x) { state = state * 1664525u + 1013904223u; v = static_cast<float>(static_cast<int>(state >> 16) - 32768) / 8192.0f; }
      const std::int64_t wshape[2] = {n, k}, xshape[2] = {m, k}, yshape[2] = {m, n};
      qc::Attribute attrs[2] = {{"format", qc::AttributeKind::i64, nullptr, 0, 1, 0.0},
                                {"prepared", qc::AttributeKind::bytes, nullptr, 0, 0, 0.0}};
      // host tensors
      qc::TensorView in[2] = {view(w.data(), wshape, 2, qc::DType::packed, qc::MemorySpace::host),
                              view(x.data(), xshape, 2, qc::DType::f32, qc::MemorySpace::host)};
      qc::TensorView out[1] = {view(y_adapter.data(), yshape, 2, qc::DType::f32, qc::MemorySpace::host)};
      qc::KernelCall call{in, 2, out, 1, attrs, 1, nullptr, nullptr, nullptr, 0};
      CHECK(api::dispatch("qgemm", call).is_ok());
      CHECK(qx_qgemm(1, w.data(), x.data(), y_typed.data(), m, n, k) == QX_STATUS_OK);
      CHECK(std::memcmp(y_adapter.data(), y_typed.data(), sizeof(float) * m * n) == 0);
      // device tensors on a stream, weights through a prepared handle
      qx_weights* handle = nullptr;
      CHECK(qx_weights_prepare(1, w.data(), n, k, 0, n, &handle) == QX_STATUS_OK);
      float *x_dev = nullptr, *y_dev = nullptr;
      cudaStream_t stream;
      CHECK(cudaStreamCreate(&stream) == cudaSuccess);
      CHECK(cudaMalloc(&x_dev, sizeof(float) * m * k) == cudaSuccess && cudaMalloc(&y_dev, sizeof(float) * m * n) == cudaSuccess);
      CHECK(cudaMemcpyAsync(x_dev, x.data(), sizeof(float) * m * k, cudaMemcpyHostToDevice, stream) == cudaSuccess);
      qc::TensorView din[2] = {view(x_dev /* canonical bytes are not read */, wshape, 2, qc::DType::packed, qc::MemorySpace::device),
                               view(x_dev, xshape, 2, qc::DType::f32, qc::MemorySpace::device)};
      qc::TensorView dout[1] = {view(y_dev, yshape, 2, qc::DType::f32, qc::MemorySpace::device)};
      qc::KernelCall dcall{din, 2, dout, 1, attrs, 1, nullptr, stream, nullptr, 0};
      CHECK(api::dispatch("qgemm", dcall).code == qc::StatusCode::invalid_argument);  // no handle
      attrs[1].data = handle;
      dcall.attribute_count = 2;
      CHECK(api::dispatch("qgemm", dcall).is_ok());
      std::vector<float> y_back(m * n);
      CHECK(cudaMemcpyAsync(y_back.data(), y_dev, sizeof(float) * m * n, cudaMemcpyDeviceToHost, stream) == cudaSuccess);
      CHECK(cudaStreamSynchronize(stream) == cudaSuccess);
      CHECK(std::memcmp(y_back.data(), y_typed.data(), sizeof(float) * m * n) == 0);
      CHECK(qx_check_device_errors() == QX_STATUS_OK);
      // int8_gemm with host tensors against the typed entry point
      const long long im = 40, in_ = 72, ik = 256;
      std::vector<signed char> wi(in_ * ik), xi(im * ik);
      for (auto& v : wi) { state = state * 1664525u + 1013904223u; v = static_cast<signed char>(state >> 24); }
      for (auto& v : xi) { state = state * 1664525u + 1013904223u; v = static_cast<signed char>(state >> 24); }
      std::vector<float> ws(in_, 0.003f), as(im, 0.02f), yi(im * in_), yt(im * in_);
      const std::int64_t s_w[2] = {in_, ik}, s_x[2] = {im, ik}, s_ws[1] = {in_}, s_as[1] = {im}, s_y[2] = {im, in_};
      qc::TensorView iin[4] = {view(wi.data(), s_w, 2, qc::DType::i8, qc::MemorySpace::host),
                               view(xi.data(), s_x, 2, qc::DType::i8, qc::MemorySpace::host),
                               view(ws.data(), s_ws, 1, qc::DType::f32, qc::MemorySpace::host),
                               view(as.data(), s_as, 1, qc::DType::f32, qc::MemorySpace::host)};
      qc::TensorView iout[1] = {view(yi.data(), s_y, 2, qc::DType::f32, qc::MemorySpace::host)};
      qc::KernelCall icall{iin, 4, iout, 1, nullptr, 0, nullptr, nullptr, nullptr, 0};
      CHECK(api::dispatch("int8_gemm", icall).is_ok());
      CHECK(qx_int8_gemm(reinterpret_cast<const int8_t*>(wi.data()), reinterpret_cast<const int8_t*>(xi.data()),
                         ws.data(), as.data(), nullptr, nullptr, yt.data(), im, in_, ik, 0) == QX_STATUS_OK);
      CHECK(std::memcmp(yi.data(), yt.data(), sizeof(float) * im * in_) == 0);
      qx_weights_destroy(handle);
      std::printf("contract adapter gpu ok\n");
      return 0;
    }
""")


def _build(tmp_path, source_text, name, compiler, extra=()):
    source = tmp_path / f"{name}.cpp"
    source.write_text(source_text)
    exe = tmp_path / name
    cmd = [compiler, "-std=c++17", "-I", os.path.join(ROOT, "include"), *extra, str(source), "-o", str(exe),
           "-L", PKG, "-lqx_b200"]
    cmd += ["-Xlinker", f"-rpath={PKG}"] if compiler.endswith("nvcc") else [f"-Wl,-rpath,{PKG}"]
    build = subprocess.run(cmd, capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    return exe


def test_adapter_compiles_and_validates(qx, tmp_path):
    variants = [("own", [])]
    if os.path.exists(os.path.join(REFERENCE_INCLUDE, "quixicore", "contract", "kernel_abi.hpp")):
        variants.append(("reference_abi", ["-I", REFERENCE_INCLUDE]))
    for name, extra in variants:
        exe = _build(tmp_path, CPU_PROGRAM, "adapter_" + name, "g++", ["-Wall", "-Wextra", "-Werror", *extra])
        run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
        assert run.returncode == 0, run.stdout + run.stderr
        assert "contract adapter ok" in run.stdout


@pytest.mark.gpu
def test_adapter_reaches_the_kernels(qx, tmp_path):
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    exe = _build(tmp_path, GPU_PROGRAM, "adapter_gpu", nvcc, ["-x", "cu"])
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "contract adapter gpu ok" in run.stdout
