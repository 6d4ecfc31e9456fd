// Registration shim for the reference's CPU (AMX) kernels on this path.  TEST / BASELINE
// INFRASTRUCTURE ONLY.  It only DECLARES the reference's entry points (defined in
// sgl-kernel/csrc/cpu/gemm.cpp, gemm_fp8.cpp, moe.cpp, moe_fp8.cpp of the reference tree, which
// oracle/build_ref.py compiles in place) and registers them under a private namespace with the
// schemas of sgl-kernel/csrc/cpu/torch_extension_cpu.cpp:286-325.
#include <ATen/ATen.h>
#include <torch/extension.h>
#include <torch/library.h>

at::Tensor convert_weight_packed(at::Tensor& weight);
at::Tensor fp8_scaled_mm_cpu(at::Tensor& mat1, at::Tensor& mat2, at::Tensor& scales2, std::vector<int64_t> block_size,
                             const std::optional<at::Tensor>& bias, at::ScalarType out_dtype, bool is_vnni);
at::Tensor fused_experts_cpu(at::Tensor& hidden_states, at::Tensor& w1, at::Tensor& w2, at::Tensor& topk_weights,
                             at::Tensor& topk_ids, bool inplace, bool use_int8_w8a8, bool use_fp8_w8a16,
                             const std::optional<at::Tensor>& w1_scale, const std::optional<at::Tensor>& w2_scale,
                             const std::optional<std::vector<int64_t>> block_size,
                             const std::optional<at::Tensor>& a1_scale, const std::optional<at::Tensor>& a2_scale,
                             bool is_vnni);

TORCH_LIBRARY_FRAGMENT(sglb200_ref, m) {
  m.def("convert_weight_packed(Tensor weight) -> Tensor");
  m.impl("convert_weight_packed", torch::kCPU, &convert_weight_packed);
  m.def(
      "fp8_scaled_mm_cpu(Tensor mat1, Tensor mat2, Tensor scales2, int[] block_size, Tensor? bias, ScalarType "
      "out_dtype, bool is_vnni) -> Tensor");
  m.impl("fp8_scaled_mm_cpu", torch::kCPU, &fp8_scaled_mm_cpu);
  m.def(
      "fused_experts_cpu(Tensor hidden_states, Tensor w1, Tensor w2, Tensor topk_weights, Tensor topk_ids, bool "
      "inplace, bool use_int8_w8a8, bool use_fp8_w8a16, Tensor? w1_scale, Tensor? w2_scale, int[]? block_size, "
      "Tensor? a1_scale, Tensor? a2_scale, bool is_vnni) -> Tensor");
  m.impl("fused_experts_cpu", torch::kCPU, &fused_experts_cpu);
}
