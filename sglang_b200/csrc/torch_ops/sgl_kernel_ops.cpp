// torch op registration over the C ABI of libsglb200.so: the ops of namespace `sgl_kernel` on the block-FP8 path,
// with the schemas of the reference's sgl-kernel/csrc/common_extension.cc (lines cited per op).  This file holds no
// kernel: every op validates like the reference (TORCH_CHECK -> RuntimeError before any launch), allocates with torch
// where the reference op allocates, takes the current CUDA stream and calls one sglb200_* entry point.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/types.h>

#include "../../../include/sglb200.h"

namespace {

void* stream_of(const torch::Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

int dtype_code(at::ScalarType t) {
  if (t == at::kBFloat16) return SGLB200_BF16;
  if (t == at::kHalf) return SGLB200_F16;
  if (t == at::kFloat) return SGLB200_F32;
  TORCH_CHECK(false, "unsupported dtype ", t, ": expected bfloat16, float16 or float32");
  return -1;
}

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == 0, what, ": ", sglb200_status_string(rc), " (", sglb200_last_error_detail(), ")");
}

// common_extension.cc:168-171; checks as sgl-kernel/csrc/gemm/fp8_blockwise_gemm_kernel.cu:374-406
torch::Tensor fp8_blockwise_scaled_mm(const torch::Tensor& mat_a, const torch::Tensor& mat_b, const torch::Tensor& scales_a,
                                      const torch::Tensor& scales_b, at::ScalarType out_dtype) {
  TORCH_CHECK(mat_a.is_cuda(), "mat_a must be a CUDA tensor");
  TORCH_CHECK(mat_b.is_cuda(), "mat_b must be a CUDA tensor");
  TORCH_CHECK(mat_a.dim() == 2, "mat_a must be a 2D tensor");
  TORCH_CHECK(mat_b.dim() == 2, "mat_b must be a 2D tensor");
  TORCH_CHECK(mat_a.stride(1) == 1, "mat_a must be a row major tensor");
  TORCH_CHECK(mat_b.stride(0) == 1, "mat_b must be a column major tensor");
  TORCH_CHECK(mat_a.size(1) == mat_b.size(0), "mat_a and mat_b shapes cannot be multiplied");
  TORCH_CHECK(mat_a.size(1) % 16 == 0, "mat_a must be multiple of 16 bytes for memory alignment");
  TORCH_CHECK(mat_a.scalar_type() == at::kFloat8_e4m3fn, "mat_a must be Float8_e4m3fn");
  TORCH_CHECK(mat_b.scalar_type() == at::kFloat8_e4m3fn, "mat_b must be Float8_e4m3fn");
  TORCH_CHECK(out_dtype == at::kHalf || out_dtype == at::kBFloat16, "out_dtype must be Half or BFloat16");
  const int64_t M = mat_a.size(0), K = mat_a.size(1), N = mat_b.size(1);
  const int64_t kt = (K + 127) / 128, nt = (N + 127) / 128;
  TORCH_CHECK(scales_a.dim() == 2 && scales_a.size(0) == M && scales_a.size(1) == kt, "size of scales_a is not matched");
  TORCH_CHECK(scales_b.dim() == 2 && scales_b.size(0) == kt && scales_b.size(1) == nt, "size of scales_b is not matched");
  TORCH_CHECK(scales_a.scalar_type() == at::kFloat, "scales_a must be Float32");
  TORCH_CHECK(scales_b.scalar_type() == at::kFloat, "scales_b must be Float32");
  TORCH_CHECK((N * 2) % 16 == 0, "out must be multiple of 16 bytes for memory alignment");
  const c10::cuda::CUDAGuard guard(mat_a.device());
  auto out = torch::empty({M, N}, mat_a.options().dtype(out_dtype));
  if (M == 0 || N == 0) return out;
  const int64_t lda = M > 1 ? mat_a.stride(0) : std::max<int64_t>(mat_a.stride(0), K);
  const int64_t ldb = N > 1 ? mat_b.stride(1) : std::max<int64_t>(mat_b.stride(1), K);
  const int64_t ws_bytes = sglb200_fp8_blockwise_scaled_mm_workspace_bytes(M, N, K);
  if (ws_bytes > 0) {  // few rows: split-K scratch from torch's caching allocator
    auto ws = torch::empty({ws_bytes}, mat_a.options().dtype(at::kByte));
    check_rc(sglb200_fp8_blockwise_scaled_mm_ws(mat_a.data_ptr(), mat_b.data_ptr(), scales_a.data_ptr<float>(),
                                                scales_b.data_ptr<float>(), out.data_ptr(), M, N, K, lda, ldb,
                                                out.stride(0), scales_a.stride(0), scales_a.stride(1), scales_b.stride(1),
                                                scales_b.stride(0), dtype_code(out_dtype), ws.data_ptr(), ws_bytes,
                                                stream_of(mat_a)),
             "fp8_blockwise_scaled_mm");
  } else {
    check_rc(sglb200_fp8_blockwise_scaled_mm(mat_a.data_ptr(), mat_b.data_ptr(), scales_a.data_ptr<float>(),
                                             scales_b.data_ptr<float>(), out.data_ptr(), M, N, K, lda, ldb, out.stride(0),
                                             scales_a.stride(0), scales_a.stride(1), scales_b.stride(1), scales_b.stride(0),
                                             dtype_code(out_dtype), stream_of(mat_a)),
             "fp8_blockwise_scaled_mm");
  }
  return out;
}

// common_extension.cc:173-181 (v2 adds fuse_silu_and_mul and masked_m); checks as per_token_group_quant_8bit.cu:125-131
void quant_impl(const torch::Tensor& input, const torch::Tensor& output_q, const torch::Tensor& output_s, int64_t group_size,
                double eps, double fp8_min, double fp8_max, bool scale_ue8m0, bool fuse_silu_and_mul,
                const c10::optional<torch::Tensor>& masked_m) {
  TORCH_CHECK(input.is_cuda() && output_q.is_cuda() && output_s.is_cuda(), "tensors must be CUDA tensors");
  TORCH_CHECK(input.is_contiguous(), "input must be contiguous");
  TORCH_CHECK(output_q.is_contiguous(), "output_q must be contiguous");
  TORCH_CHECK(output_q.scalar_type() == at::kFloat8_e4m3fn,
              "output_q must be Float8_e4m3fn (the int8 destination is not implemented)");
  const c10::cuda::CUDAGuard guard(input.device());
  // eps in the input dtype, as the torch-native reference clamps (python/sglang/test/test_block_fp8.py:43)
  float eps_eff = (float)eps;
  if (input.scalar_type() == at::kBFloat16) eps_eff = static_cast<float>(c10::BFloat16((float)eps));
  const int64_t hidden_in = input.size(-1);
  const int64_t hidden = fuse_silu_and_mul ? hidden_in / 2 : hidden_in;
  TORCH_CHECK(group_size > 0 && hidden % group_size == 0, "the last dimension of `x` cannot be divisible by `group_size`");
  if (input.dim() == 3) {
    const int64_t E = input.size(0), max_m = input.size(1);
    TORCH_CHECK(output_s.dim() == 3, "output_s must be 3D for the [E, max_m, K] layout");
    const int32_t* mptr = nullptr;
    if (masked_m.has_value()) {
      TORCH_CHECK(masked_m->scalar_type() == at::kInt && masked_m->is_contiguous() && masked_m->numel() == E,
                  "masked_m must be a contiguous int32 tensor with one entry per expert");
      mptr = masked_m->data_ptr<int32_t>();
    }
    if (E == 0 || max_m == 0 || hidden == 0) return;
    check_rc(sglb200_group_quant_fp8_batched(input.data_ptr(), dtype_code(input.scalar_type()), output_q.data_ptr(),
                                             output_s.data_ptr(), E, max_m, hidden, (int)group_size, eps_eff,
                                             (float)fp8_min, (float)fp8_max, scale_ue8m0 ? 1 : 0,
                                             fuse_silu_and_mul ? 1 : 0, mptr, output_s.stride(0), output_s.stride(1),
                                             output_s.stride(2), stream_of(input)),
             "sgl_per_token_group_quant_8bit(masked)");
    return;
  }
  TORCH_CHECK(!masked_m.has_value(), "masked_m needs the 3-D [E, max_m, K] layout");
  TORCH_CHECK(output_s.dim() == 2, "output_s must be 2D");
  const int64_t rows = hidden_in ? input.numel() / hidden_in : 0;
  TORCH_CHECK(output_q.numel() == rows * hidden, "output_q has the wrong number of elements");
  if (rows == 0 || hidden == 0) return;
  if (fuse_silu_and_mul) {
    check_rc(sglb200_silu_mul_group_quant_fp8(input.data_ptr(), dtype_code(input.scalar_type()), output_q.data_ptr(),
                                              output_s.data_ptr(), nullptr, rows, hidden, (int)group_size, eps_eff,
                                              (float)fp8_min, (float)fp8_max, scale_ue8m0 ? 1 : 0, output_s.stride(0),
                                              output_s.stride(1), stream_of(input)),
             "sgl_per_token_group_quant_8bit(fuse_silu_and_mul)");
  } else {
    check_rc(sglb200_per_token_group_quant_fp8(input.data_ptr(), dtype_code(input.scalar_type()), output_q.data_ptr(),
                                               output_s.data_ptr(), rows, hidden, (int)group_size, eps_eff, (float)fp8_min,
                                               (float)fp8_max, scale_ue8m0 ? 1 : 0, output_s.stride(0), output_s.stride(1),
                                               stream_of(input)),
             "sgl_per_token_group_quant_8bit");
  }
}

void sgl_per_token_group_quant_8bit(const torch::Tensor& input, const torch::Tensor& output_q, const torch::Tensor& output_s,
                                    int64_t group_size, double eps, double fp8_min, double fp8_max, bool scale_ue8m0) {
  quant_impl(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, false, c10::nullopt);
}

void sgl_per_token_group_quant_8bit_v2(const torch::Tensor& input, const torch::Tensor& output_q,
                                       const torch::Tensor& output_s, int64_t group_size, double eps, double fp8_min,
                                       double fp8_max, bool scale_ue8m0, bool fuse_silu_and_mul,
                                       const c10::optional<torch::Tensor>& masked_m) {
  quant_impl(input, output_q, output_s, group_size, eps, fp8_min, fp8_max, scale_ue8m0, fuse_silu_and_mul, masked_m);
}

// common_extension.cc:274-279.  a [rows, K] e4m3; b [E, K, N] = weight[E, N, K].transpose(1, 2); scales_a [rows, K/128];
// scales_b [E, K/128, N/128] = weight_scale[E, N/128, K/128].transpose(1, 2); problem_sizes [E, 3]; expert_offsets
// [E] or [E + 1].  The pointer, stride, layout and workspace tensors of the schema are accepted and not read.
void fp8_blockwise_scaled_grouped_mm(torch::Tensor& output, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&,
                                     const torch::Tensor&, const torch::Tensor&, const torch::Tensor& a,
                                     const torch::Tensor& b, const torch::Tensor& scales_a, const torch::Tensor& scales_b,
                                     const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&,
                                     const torch::Tensor&, const torch::Tensor& problem_sizes,
                                     const torch::Tensor& expert_offsets, const torch::Tensor&) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && output.is_cuda(), "tensors must be CUDA tensors");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 3, "a must be [rows, K] and b [E, K, N]");
  TORCH_CHECK(a.scalar_type() == at::kFloat8_e4m3fn && b.scalar_type() == at::kFloat8_e4m3fn, "a and b must be Float8_e4m3fn");
  TORCH_CHECK(b.stride(1) == 1, "b must be the transposed view of weights stored [E, N, K]");
  TORCH_CHECK(scales_a.scalar_type() == at::kFloat && scales_b.scalar_type() == at::kFloat, "scales must be Float32");
  TORCH_CHECK(problem_sizes.dim() == 2 && problem_sizes.size(1) == 3 && problem_sizes.scalar_type() == at::kInt,
              "problem_sizes must be int32 [E, 3]");
  TORCH_CHECK(expert_offsets.scalar_type() == at::kInt, "expert_offsets must be int32");
  const int64_t E = b.size(0), K = b.size(1), N = b.size(2);
  TORCH_CHECK(a.size(1) == K && output.size(1) == N && output.size(0) == a.size(0), "shapes do not match");
  const c10::cuda::CUDAGuard guard(a.device());
  check_rc(sglb200_fp8_blockwise_scaled_grouped_mm(
               a.data_ptr(), b.data_ptr(), scales_a.data_ptr<float>(), scales_b.data_ptr<float>(), output.data_ptr(),
               expert_offsets.data_ptr<int32_t>(), problem_sizes.data_ptr<int32_t>(), a.size(0), E, N, K, a.stride(0),
               b.stride(2), b.stride(0), output.stride(0), scales_a.stride(0), scales_a.stride(1), scales_b.stride(0),
               scales_b.stride(2), scales_b.stride(1), dtype_code(output.scalar_type()), stream_of(a)),
           "fp8_blockwise_scaled_grouped_mm");
}

// common_extension.cc:281-285
void prepare_moe_input(const torch::Tensor& topk_ids, torch::Tensor& expert_offsets,
                       const c10::optional<torch::Tensor>& blockscale_offsets, torch::Tensor& problem_sizes1,
                       torch::Tensor& problem_sizes2, torch::Tensor& input_permutation, torch::Tensor& output_permutation,
                       int64_t num_experts, int64_t n, int64_t k) {
  TORCH_CHECK(!blockscale_offsets.has_value(), "blockscale_offsets (FP4) is outside the block-FP8 path");
  TORCH_CHECK(topk_ids.is_cuda() && topk_ids.scalar_type() == at::kInt && topk_ids.is_contiguous() && topk_ids.dim() == 2,
              "topk_ids must be a contiguous int32 CUDA tensor [M, topk]");
  const c10::cuda::CUDAGuard guard(topk_ids.device());
  check_rc(sglb200_prepare_moe_input(topk_ids.data_ptr<int32_t>(), expert_offsets.data_ptr<int32_t>(),
                                     problem_sizes1.data_ptr<int32_t>(), problem_sizes2.data_ptr<int32_t>(),
                                     input_permutation.data_ptr<int32_t>(), output_permutation.data_ptr<int32_t>(),
                                     topk_ids.size(0), topk_ids.size(1), num_experts, n, k, stream_of(topk_ids)),
           "prepare_moe_input");
}

// common_extension.cc:287-288
void shuffle_rows(const torch::Tensor& input, const torch::Tensor& dst2src_map, torch::Tensor& output) {
  TORCH_CHECK(input.is_cuda() && input.is_contiguous() && output.is_contiguous(), "input / output must be contiguous CUDA tensors");
  TORCH_CHECK(dst2src_map.scalar_type() == at::kInt, "dst2src_map must be int32");
  TORCH_CHECK(input.scalar_type() == output.scalar_type() && input.size(-1) == output.size(-1), "row types must match");
  const c10::cuda::CUDAGuard guard(input.device());
  check_rc(sglb200_shuffle_rows(input.data_ptr(), dst2src_map.data_ptr<int32_t>(), output.data_ptr(), output.size(0),
                                input.size(-1) * (int64_t)input.element_size(), stream_of(input)),
           "shuffle_rows");
}

// common_extension.cc:289-290; fp32 products as the reference kernel (prepare_moe_input.cu:258-392)
void apply_shuffle_mul_sum(const torch::Tensor& input, torch::Tensor& output, const torch::Tensor& permutation,
                           const c10::optional<torch::Tensor>& factors) {
  TORCH_CHECK(input.is_cuda() && input.is_contiguous() && output.is_contiguous(), "input / output must be contiguous CUDA tensors");
  TORCH_CHECK(permutation.scalar_type() == at::kInt, "permutation must be int32");
  const int64_t m = output.size(0), hidden = output.size(1);
  TORCH_CHECK(m > 0 && permutation.numel() % m == 0, "permutation must hold topk entries per output row");
  const int64_t topk = permutation.numel() / m;
  const void* f = nullptr;
  if (factors.has_value()) {
    TORCH_CHECK(factors->scalar_type() == input.scalar_type() && factors->numel() == m * topk, "factors must be [m * topk] in the row type");
    f = factors->data_ptr();
  }
  const c10::cuda::CUDAGuard guard(input.device());
  check_rc(sglb200_apply_shuffle_mul_sum(input.data_ptr(), output.data_ptr(), permutation.data_ptr<int32_t>(), f, m, topk,
                                         hidden, dtype_code(input.scalar_type()), /*round_products=*/0, stream_of(input)),
           "apply_shuffle_mul_sum");
}

// common_extension.cc:82-83
void silu_and_mul(torch::Tensor& out, const torch::Tensor& input) {
  TORCH_CHECK(input.is_cuda() && input.is_contiguous() && out.is_contiguous(), "tensors must be contiguous CUDA tensors");
  const int64_t d = input.size(-1) / 2;
  const int64_t rows = d ? input.numel() / (2 * d) : 0;
  const c10::cuda::CUDAGuard guard(input.device());
  check_rc(sglb200_silu_and_mul(input.data_ptr(), out.data_ptr(), rows, d, dtype_code(input.scalar_type()), stream_of(input)),
           "silu_and_mul");
}

// common_extension.cc:262-263
void moe_sum_reduce(const torch::Tensor& input, torch::Tensor& output, double routed_scaling_factor) {
  TORCH_CHECK(input.is_cuda() && input.dim() == 3 && input.is_contiguous() && output.is_contiguous(),
              "input must be a contiguous [M, topk, H] CUDA tensor");
  const c10::cuda::CUDAGuard guard(input.device());
  check_rc(sglb200_moe_sum_reduce(input.data_ptr(), output.data_ptr(), input.size(0), input.size(1), input.size(2),
                                  dtype_code(input.scalar_type()), (float)routed_scaling_factor, stream_of(input)),
           "moe_sum_reduce");
}

}  // namespace

TORCH_LIBRARY_FRAGMENT(sgl_kernel, m) {
  m.def("fp8_blockwise_scaled_mm(Tensor mat_a, Tensor mat_b, Tensor scales_a, Tensor scales_b, ScalarType out_dtype) -> Tensor");
  m.impl("fp8_blockwise_scaled_mm", torch::kCUDA, &fp8_blockwise_scaled_mm);
  m.def("sgl_per_token_group_quant_8bit(Tensor input, Tensor output_q, Tensor output_s, int group_size,"
        " float eps, float fp8_min, float fp8_max, bool scale_ue8m0) -> ()");
  m.impl("sgl_per_token_group_quant_8bit", torch::kCUDA, &sgl_per_token_group_quant_8bit);
  m.def("sgl_per_token_group_quant_8bit_v2(Tensor input, Tensor output_q, Tensor output_s, int group_size,"
        " float eps, float fp8_min, float fp8_max, bool scale_ue8m0, bool fuse_silu_and_mul, Tensor? masked_m) -> ()");
  m.impl("sgl_per_token_group_quant_8bit_v2", torch::kCUDA, &sgl_per_token_group_quant_8bit_v2);
  m.def("fp8_blockwise_scaled_grouped_mm(Tensor output, Tensor a_ptrs, Tensor b_ptrs, Tensor out_ptrs, Tensor "
        "a_scales_ptrs, Tensor b_scales_ptrs, Tensor a, Tensor b, Tensor scales_a, Tensor scales_b, Tensor "
        "stride_a, Tensor stride_b, Tensor stride_c, Tensor layout_sfa, Tensor layout_sfb, Tensor problem_sizes, Tensor "
        "expert_offsets, Tensor workspace) -> ()");
  m.impl("fp8_blockwise_scaled_grouped_mm", torch::kCUDA, &fp8_blockwise_scaled_grouped_mm);
  m.def("prepare_moe_input(Tensor topk_ids, Tensor expert_offsets, Tensor? blockscale_offsets, Tensor problem_sizes1,"
        " Tensor problem_sizes2, Tensor input_permutation, Tensor output_permutation, int num_experts, int n, int k) -> ()");
  m.impl("prepare_moe_input", torch::kCUDA, &prepare_moe_input);
  m.def("shuffle_rows(Tensor input, Tensor dst2src_map, Tensor output) -> ()");
  m.impl("shuffle_rows", torch::kCUDA, &shuffle_rows);
  m.def("apply_shuffle_mul_sum(Tensor input, Tensor output, Tensor permutation, Tensor? factors) -> ()");
  m.impl("apply_shuffle_mul_sum", torch::kCUDA, &apply_shuffle_mul_sum);
  m.def("silu_and_mul(Tensor! out, Tensor input) -> ()");
  m.impl("silu_and_mul", torch::kCUDA, &silu_and_mul);
  m.def("moe_sum_reduce(Tensor input, Tensor output, float routed_scaling_factor) -> ()");
  m.impl("moe_sum_reduce", torch::kCUDA, &moe_sum_reduce);
}
