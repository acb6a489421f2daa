"""The C++ face of the C ABI (include/qx_b200.hpp, namespace quixicore_cpu) compiles as plain
C++17, links against the library and reproduces the reference's host-side contract without
a GPU: packed sizes (tests/correctness/test_qgemv.cpp:116-122) and the validation order of
qgemv / qgemm / int8_gemm (format -> shape -> pointers; test_qgemv.cpp:106-107,
src/dispatch/int8_gemm.cpp:72-85), all of which return before any device is touched."""

import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "quixicore-cpu_b200")

PROGRAM = textwrap.dedent(r"""
    #include <cstdio>
    #include <cstdlib>
    #include "qx_b200.hpp"
    using namespace quixicore_cpu;
    #define CHECK(cond) do { if (!(cond)) { std::printf("FAILED: %s (line %d)\n", #cond, __LINE__); return 1; } } while (0)
    int main() {
      std::size_t size = 0;
      CHECK(qgemv_packed_size(QuantFormat::kQ8_0, 1, 32, &size) == Status::kOk && size == 34);
      CHECK(qgemv_packed_size(QuantFormat::kQ4_0, 1, 32, &size) == Status::kOk && size == 18);
      CHECK(qgemv_packed_size(QuantFormat::kQ8_0, 4096, 4096, &size) == Status::kOk && size == 17825792u);
      CHECK(qgemv_packed_size(QuantFormat::kQ8_0, 3, 33, &size) == Status::kInvalidShape);
      CHECK(qgemv_packed_size(static_cast<QuantFormat>(7), 1, 32, &size) == Status::kUnsupportedFormat);
      float x[32] = {0}, y[1] = {0};
      unsigned char packed[34] = {0};
      // a null pointer together with a bad shape reports the shape
      CHECK(qgemv(QuantFormat::kQ8_0, nullptr, x, y, 1, 31) == Status::kInvalidShape);
      CHECK(qgemv(QuantFormat::kQ8_0, nullptr, x, y, 1, 32) == Status::kInvalidArgument);
      CHECK(qgemv(QuantFormat::kQ8_0, packed, x, nullptr, 1, 32) == Status::kInvalidArgument);
      CHECK(qgemv(static_cast<QuantFormat>(9), packed, x, y, 1, 32) == Status::kUnsupportedFormat);
      CHECK(qgemm(QuantFormat::kQ4_0, packed, x, y, 0, 1, 32) == Status::kInvalidShape);
      CHECK(int8_gemm(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, y, 0, 1, 4) == Status::kInvalidShape);
      CHECK(int8_gemm(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, y, 1, 1, 4) == Status::kInvalidArgument);
      CHECK(qgemm_w8a32(nullptr, nullptr, x, y, 1, 1, 0) == Status::kInvalidShape);
      CpuPackedWeights weights;
      CHECK(!weights.ready());
      CHECK(weights.prepare(QuantFormat::kQ8_0, nullptr, 1, 32) == Status::kInvalidArgument);
      CHECK(weights.prepare(QuantFormat::kQ8_0, packed, 1, 31) == Status::kInvalidShape);
      CHECK(qgemm_prepacked(weights, x, y, 1) == Status::kInvalidArgument);  // not ready
      // the reference's layout enumerators (include/quixicore_cpu/packed_weights.h:14-20) and
      // the info fields a caller may name
      static_assert(static_cast<int>(CpuPanelLayout::kAuto) == 0 &&
                    static_cast<int>(CpuPanelLayout::kPortableRows1) == 1 &&
                    static_cast<int>(CpuPanelLayout::kNeonRows4) == 2 &&
                    static_cast<int>(CpuPanelLayout::kAvx2Rows8) == 3 &&
                    static_cast<int>(CpuPanelLayout::kAvx512Rows16) == 4, "layout values");
      CHECK(weights.prepare(QuantFormat::kQ8_0, nullptr, 1, 32, CpuPanelLayout::kAvx512Rows16) ==
            Status::kInvalidArgument);
      const CpuPackedWeightsInfo blank = weights.info();
      CHECK(blank.layout == CpuPanelLayout::kAuto && blank.row_tile == 0 && blank.panel_bytes == 0);
      CHECK(weights.contract_data() == nullptr && weights.panel_data() == nullptr);
      // callers either side of the GEMV: same names, same checks before any data is touched
      CHECK(qgemv_w8a8(QuantFormat::kQ8_0, nullptr, x, y, 1, 31) == Status::kInvalidShape);
      CHECK(qgemv_w8a8(QuantFormat::kQ8_0, nullptr, x, y, 1, 32) == Status::kInvalidArgument);
      CHECK(qgemv_up_gate(QuantFormat::kQ4_0, packed, packed, x, nullptr, y, 1, 32) == Status::kInvalidArgument);
      CHECK(qgemv_up_gate_activation(QuantFormat::kQ4_0, packed, packed, x, y, 0, 32) == Status::kInvalidShape);
      CHECK(qgemv_qkv(QuantFormat::kQ8_0, packed, packed, packed, x, y, y, y, 1, 1, 33) == Status::kInvalidShape);
      std::size_t wb = 0, sc = 0;
      CHECK(lowbit_packed_size(LowBitFormat::kInt4Row, 3, 33, 0, &wb, &sc) == Status::kOk && wb == 51 && sc == 3);
      CHECK(static_cast<int>(LowBitFormat::kInt4Group) == 3);
      std::int8_t codes[32];
      float scale[1];
      CHECK(quantize_int8(nullptr, codes, scale, 1, 32, 0) == Status::kInvalidArgument);
      CHECK(lowbit_gemm_w8a8(nullptr, scale, x, y, 1, 1, 32) == Status::kInvalidArgument);
      // canonical tensors: checks of validate_canonical_quant_tensor before any device work,
      // and the SmoothQuant importer (host only)
      std::uint8_t cdata[64] = {0};
      float cscales[2] = {0.5f, 0.25f};
      CanonicalQuantTensorView view;
      view.layout = CanonicalQuantLayout::kInt8Symmetric;
      view.scale_mode = QuantScaleMode::kRow;
      view.logical_rows = 2; view.logical_columns = 32; view.group_size = 32;
      view.data = cdata; view.data_bytes = 64; view.scales = cscales; view.scale_count = 2;
      CanonicalPackedWeights canonical;
      view.data_bytes = 63;
      CHECK(canonical.prepare(view) == Status::kInvalidShape);
      view.data_bytes = 64;
      view.scale_mode = QuantScaleMode::kTensor;
      CHECK(canonical.prepare(view) == Status::kInvalidShape);     // one scale expected
      view.scale_count = 1;
      CHECK(canonical.prepare(view) == Status::kInvalidArgument);  // mode not served by this layout
      view.layout = static_cast<CanonicalQuantLayout>(5);
      CHECK(canonical.prepare(view) == Status::kUnsupportedFormat);
      CHECK(!canonical.ready());
      CHECK(qgemm_prepacked_storage(canonical, {x, FloatStorageType::kF32, 32}, {y, FloatStorageType::kF32, 1}, 1) ==
            Status::kInvalidArgument);
      CHECK(qgemm_prepacked_epilogue_storage(canonical, {x, FloatStorageType::kBF16, 32}, nullptr,
                                             {y, FloatStorageType::kF16, 1}, 1, static_cast<LinearActivation>(7)) ==
            Status::kInvalidArgument);
      const std::int8_t sq_weights[4] = {-127, -64, 0, 127};
      const float sq_scale[1] = {0.25f}, sq_act[1] = {0.125f};
      SmoothQuantW8A8Source sq{};
      sq.weights = sq_weights; sq.weight_count = 4; sq.weight_scales = sq_scale; sq.weight_scale_count = 1;
      sq.activation_scales = sq_act; sq.activation_scale_count = 1; sq.rows = 1; sq.columns = 4;
      CanonicalQuantTensorView imported;
      std::int32_t row_sum[1] = {0};
      CHECK(import_smoothquant_w8a8(sq, &imported, row_sum) == Status::kOk);
      CHECK(imported.layout == CanonicalQuantLayout::kInt8Symmetric && imported.scale_mode == QuantScaleMode::kChannel);
      CHECK(imported.group_size == 4 && imported.data_bytes == 4 && row_sum[0] == -64);
      sq.weight_count = 3;
      CHECK(import_smoothquant_w8a8(sq, &imported, row_sum) == Status::kInvalidShape);
      // the AWQ fragment of the reference's importer test (test_quant_import.cpp:148-185)
      std::uint32_t awq_weight[8], awq_zero[1] = {0x33333333u};
      float awq_scale[8], awq_out_scale[8], awq_out_zero[8];
      for (int i = 0; i < 8; ++i) { awq_weight[i] = 0x76543210u; awq_scale[i] = 0.25f; }
      std::uint8_t awq_data[32];
      AwqU4Source awq{};
      awq.qweight = awq_weight; awq.qweight_words = 8; awq.qzeros = awq_zero; awq.qzero_words = 1;
      awq.scales = awq_scale; awq.scale_count = 8; awq.input_features = 8; awq.output_features = 8; awq.group_size = 8;
      CHECK(import_awq_u4(awq, &imported, awq_data, awq_out_scale, awq_out_zero) == Status::kOk);
      CHECK(imported.layout == CanonicalQuantLayout::kUInt4Affine && imported.zero_point_count == 8);
      CHECK(awq_data[0] == 0x00 && awq_data[4] == 0x44 && awq_data[28] == 0x77 && awq_out_zero[5] == 3.0f);
      awq.output_features = 12;
      CHECK(import_awq_u4(awq, &imported, awq_data, awq_out_scale, awq_out_zero) == Status::kInvalidArgument);
      GptqU4Source gptq{};
      CHECK(import_gptq_u4(gptq, &imported, awq_data, awq_out_scale, awq_out_zero) == Status::kInvalidArgument);
      CpuPackedWeights moved = std::move(weights);
      CHECK(!moved.ready() && moved.info().rows == 0);
      set_num_threads(4);
      CHECK(num_threads() == 4);
      CHECK(qgemv_variant(QuantFormat::kQ8_0) != nullptr && int8_gemm_variant() != nullptr);
      std::printf("cpp mirror ok\n");
      return 0;
    }
""")


def test_cpp_mirror_compiles_links_and_validates(tmp_path):
    source = tmp_path / "mirror.cpp"
    source.write_text(PROGRAM)
    exe = tmp_path / "mirror"
    build = subprocess.run(
        ["g++", "-std=c++17", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
         str(source), "-o", str(exe), "-L", PKG, "-lqx_b200", f"-Wl,-rpath,{PKG}"],
        capture_output=True, text=True)
    assert build.returncode == 0, build.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=60)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "cpp mirror ok" in run.stdout
