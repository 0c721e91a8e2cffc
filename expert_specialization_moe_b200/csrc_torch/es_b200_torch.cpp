// Torch operator registration of the es_b200 library: the three operators of the reference extension
// (expert_specialization/csrc/expert_specialization.cpp:56-73) under the namespace `es_b200`, with the reference's
// schemas word for word — argument order (a, b, sfa, sfb, d, ...) of the MXFP8 GEMM included — CUDA dispatch key only.
// Each implementation does the reference's TORCH_CHECKs (es_sm100_mxfp8_blockscaled.cu:15-25,
// es_sm100_mxfp8_blockscaled_group_quant.cu:13-24, es_fp8_blockwise.cu:47-56) plus the ones the reference leaves
// implicit, takes the current CUDA stream and forwards raw pointers to the C ABI (include/es_b200.h).  The namespace
// differs from the reference's so that both libraries can be loaded into one process side by side.
#include <ATen/core/Tensor.h>
#include <ATen/ops/zeros.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <mutex>
#include <unordered_map>

#include "es_b200.h"

namespace {

int dtype_code(const at::Tensor& t, const char* what) {
  if (t.scalar_type() == at::kBFloat16) return ES_B200_BF16;
  if (t.scalar_type() == at::kHalf) return ES_B200_FP16;
  TORCH_CHECK(false, what, ": dtype must be kFloat16 or kBFloat16");
  return -1;
}

void check_rc(int rc) {
  if (rc == ES_B200_OK) return;
  const char* msg = es_b200_last_error();
  TORCH_CHECK(false, (msg && msg[0]) ? msg : es_b200_strerror(rc));
}

// Work-counter scratch of the grouped GEMM, one per (device, stream): zeroed when created, left zeroed by every call,
// and zeroed again (on the stream, before the call) when a device-side error has been reported since.
struct Scratch {
  at::Tensor buf;
  uint64_t epoch;
};
at::Tensor& mm_scratch(const at::Tensor& like, cudaStream_t stream) {
  static std::mutex mu;
  static std::unordered_map<uint64_t, Scratch> cache;
  const uint64_t key = (reinterpret_cast<uint64_t>(stream) << 8) ^ static_cast<uint64_t>(like.get_device() + 1);
  const uint64_t epoch = es_b200_error_epoch();
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it == cache.end()) {
    const int64_t n = static_cast<int64_t>(es_b200_grouped_mm_scratch_bytes(0, 0, 0, 0));
    it = cache.emplace(key, Scratch{at::zeros({n}, like.options().dtype(at::kByte)), epoch}).first;   // on the current stream
  } else if (it->second.epoch != epoch) {
    it->second.buf.zero_();
    it->second.epoch = epoch;
  }
  return it->second.buf;
}

void check_problem_tensors(const at::Tensor& problem_sizes, const at::Tensor& expert_offsets) {
  TORCH_CHECK(problem_sizes.dim() == 2, "problem_sizes must be 2D tensor");
  TORCH_CHECK(problem_sizes.size(1) == 3, "problem_sizes must have shape (num_experts, 3)");
  TORCH_CHECK(problem_sizes.size(0) == expert_offsets.size(0),
              "Number of experts in problem_sizes must match expert_offsets");
  TORCH_CHECK(problem_sizes.scalar_type() == at::kInt, "problem_sizes must be int32");
  TORCH_CHECK(expert_offsets.scalar_type() == at::kInt && expert_offsets.dim() == 1, "expert_offsets must be 1D int32");
  TORCH_CHECK(problem_sizes.is_contiguous() && expert_offsets.is_contiguous(),
              "problem_sizes / expert_offsets must be contiguous");
}

void grouped_quant_common(const at::Tensor& input, const at::Tensor& problem_sizes, const at::Tensor& expert_offsets,
                          const at::Tensor& blockscale_offsets, at::Tensor& quant_output, at::Tensor& scale_factor,
                          bool silu_mul) {
  TORCH_CHECK(input.dim() == 2, "input must be 2D tensor");
  const int64_t k = silu_mul ? input.size(1) / 2 : input.size(1);
  TORCH_CHECK(k % 128 == 0 && (!silu_mul || input.size(1) % 256 == 0), "k must align to 128");
  TORCH_CHECK(input.stride(1) == 1, "input must be row major");
  TORCH_CHECK(problem_sizes.dim() == 2, "problem_sizes must be 2D tensor");
  const int64_t groups = problem_sizes.size(0);
  TORCH_CHECK(expert_offsets.dim() == 1 && expert_offsets.size(0) == groups,
              "expert_offsets must be 1D and have size equal to the number of groups");
  TORCH_CHECK(blockscale_offsets.dim() == 1 && blockscale_offsets.size(0) == groups,
              "blockscale_offsets must be 1D and have size equal to the number of groups");
  // implicit in the reference (it reinterprets the raw pointers)
  TORCH_CHECK(problem_sizes.size(1) == 3 && problem_sizes.scalar_type() == at::kInt && problem_sizes.is_contiguous(),
              "problem_sizes must be a contiguous int32 tensor of shape (num_experts, 3)");
  TORCH_CHECK(expert_offsets.scalar_type() == at::kInt && blockscale_offsets.scalar_type() == at::kInt,
              "expert_offsets and blockscale_offsets must be int32");
  TORCH_CHECK(expert_offsets.is_contiguous() && blockscale_offsets.is_contiguous(), "offsets must be contiguous");
  TORCH_CHECK(input.stride(0) == input.size(1), "input rows must be densely packed");
  TORCH_CHECK(quant_output.is_contiguous() && quant_output.numel() == input.size(0) * k &&
                  quant_output.element_size() == 1,
              "quant_output must be a contiguous 1-byte tensor of shape (rows, k)");
  TORCH_CHECK(scale_factor.is_contiguous() && scale_factor.element_size() == 1,
              "scale_factor must be a contiguous 1-byte tensor");
  const int dt = dtype_code(input, "input");
  c10::cuda::CUDAGuard guard(input.device());
  void* stream = c10::cuda::getCurrentCUDAStream(input.get_device()).stream();
  auto fn = silu_mul ? es_b200_mxfp8_silu_mul_grouped_quant : es_b200_mxfp8_grouped_quant;
  check_rc(fn(input.data_ptr(), dt, problem_sizes.data_ptr<int32_t>(), expert_offsets.data_ptr<int32_t>(),
              blockscale_offsets.data_ptr<int32_t>(), quant_output.data_ptr(),
              static_cast<uint8_t*>(scale_factor.data_ptr()), static_cast<int>(groups), input.size(0),
              static_cast<int>(k), stream));
}

// reference: es_sm100_mxfp8_blockscaled_group_quant.cu:5-39
void es_sm100_mxfp8_blockscaled_grouped_quant(const at::Tensor& input, const at::Tensor& problem_sizes,
                                              const at::Tensor& expert_offsets, const at::Tensor& blockscale_offsets,
                                              at::Tensor& quant_output, at::Tensor& scale_factor) {
  grouped_quant_common(input, problem_sizes, expert_offsets, blockscale_offsets, quant_output, scale_factor, false);
}

// no counterpart in the reference: silu(gate) * up fused in front of the quantisation, gate_up = [rows, 2k]
void es_sm100_mxfp8_silu_mul_grouped_quant(const at::Tensor& gate_up, const at::Tensor& problem_sizes,
                                           const at::Tensor& expert_offsets, const at::Tensor& blockscale_offsets,
                                           at::Tensor& quant_output, at::Tensor& scale_factor) {
  grouped_quant_common(gate_up, problem_sizes, expert_offsets, blockscale_offsets, quant_output, scale_factor, true);
}

// reference: es_sm100_mxfp8_blockscaled.cu:5-40 (argument order of the op schema: a, b, sfa, sfb, d, ...)
void es_sm100_mxfp8_blockscaled_grouped_mm(const at::Tensor& a, const at::Tensor& b, const at::Tensor& sfa,
                                           const at::Tensor& sfb, at::Tensor& d, const at::Tensor& problem_sizes,
                                           const at::Tensor& expert_offsets, const at::Tensor& blockscale_offsets) {
  check_problem_tensors(problem_sizes, expert_offsets);
  TORCH_CHECK(a.dim() == 2, "a must be a 2D tensor of shape (num_tokens, k)");
  TORCH_CHECK(b.dim() == 3, "b must be a 3D tensor of shape (num_experts, k, n)");
  TORCH_CHECK(a.size(1) == b.size(1) && a.size(1) % 128 == 0, "k should align 128");
  TORCH_CHECK(b.size(2) % 128 == 0, "n should align 128");
  TORCH_CHECK(a.stride(1) == 1, "a must be row major");
  TORCH_CHECK(b.stride(1) == 1, "a must be column major");
  // implicit in the reference
  const int64_t E = b.size(0), K = b.size(1), N = b.size(2);
  TORCH_CHECK(E == problem_sizes.size(0), "b must hold one matrix per expert");
  TORCH_CHECK(b.stride(2) == K && b.stride(0) == N * K, "b must be a transposed view of contiguous [E, N, K] memory");
  TORCH_CHECK(a.stride(0) == K, "a rows must be densely packed");
  TORCH_CHECK(a.element_size() == 1 && b.element_size() == 1, "a and b must be float8_e4m3fn");
  TORCH_CHECK(d.dim() == 2 && d.size(0) == a.size(0) && d.size(1) == N && d.is_contiguous(),
              "output must be a contiguous (num_tokens, n) tensor");
  TORCH_CHECK(blockscale_offsets.scalar_type() == at::kInt && blockscale_offsets.dim() == 1 &&
                  blockscale_offsets.size(0) == E && blockscale_offsets.is_contiguous(),
              "offsets must be int32 of length num_experts");
  TORCH_CHECK(sfa.element_size() == 1 && sfb.element_size() == 1, "sfa and sfb must be 1-byte UE8M0 tensors");
  const int dt = dtype_code(d, "output");
  c10::cuda::CUDAGuard guard(a.device());
  cudaStream_t stream = c10::cuda::getCurrentCUDAStream(a.get_device()).stream();
  at::Tensor& scratch = mm_scratch(a, stream);
  check_rc(es_b200_mxfp8_grouped_mm(a.data_ptr(), b.data_ptr(), static_cast<const uint8_t*>(sfa.data_ptr()),
                                    static_cast<const uint8_t*>(sfb.data_ptr()), d.data_ptr(), dt,
                                    problem_sizes.data_ptr<int32_t>(), expert_offsets.data_ptr<int32_t>(),
                                    blockscale_offsets.data_ptr<int32_t>(), static_cast<int>(E), a.size(0),
                                    static_cast<int>(N), static_cast<int>(K), sfa.numel() / (K / 32),
                                    scratch.data_ptr(), static_cast<size_t>(scratch.numel()), stream));
}

// reference: es_fp8_blockwise.cu:34-193.  stride_a / stride_b / stride_d and workspace are accepted for signature
// compatibility; rows must be densely packed (K, K, N), as every caller of the reference passes them.
void es_fp8_blockwise_scaled_grouped_mm(at::Tensor& output, const at::Tensor& a, const at::Tensor& b,
                                        const at::Tensor& scales_a, const at::Tensor& scales_b,
                                        const at::Tensor& /*stride_a*/, const at::Tensor& /*stride_b*/,
                                        const at::Tensor& /*stride_d*/, const at::Tensor& problem_sizes,
                                        const at::Tensor& expert_offsets, const at::Tensor& /*workspace*/) {
  check_problem_tensors(problem_sizes, expert_offsets);
  TORCH_CHECK(a.scalar_type() == at::kFloat8_e4m3fn, "a must be kFloat8_e4m3fn");
  TORCH_CHECK(b.scalar_type() == at::kFloat8_e4m3fn, "b must be kFloat8_e4m3fn");
  TORCH_CHECK(output.scalar_type() == at::kBFloat16 || output.scalar_type() == at::kHalf,
              "output must be bfloat16 or half");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 3, "a must be (num_tokens, k) and b (num_experts, k, n)");
  const int64_t E = b.size(0), K = b.size(1), N = b.size(2);
  TORCH_CHECK(a.size(1) == K && K % 128 == 0, "k should align 128");
  TORCH_CHECK(N % 128 == 0, "n should align 128");
  TORCH_CHECK(b.stride(1) == 1 && b.stride(2) == K && b.stride(0) == N * K,
              "b must be a transposed view of contiguous [E, N, K] memory");
  TORCH_CHECK(a.stride(1) == 1 && a.stride(0) == K, "a must be row major with densely packed rows");
  TORCH_CHECK(E == problem_sizes.size(0), "b must hold one matrix per expert");
  TORCH_CHECK(scales_a.scalar_type() == at::kFloat && scales_a.dim() == 2 && scales_a.size(0) == a.size(0) &&
                  scales_a.size(1) == K / 128 && scales_a.is_contiguous(),
              "scales_a must be contiguous f32 (num_tokens, k/128)");
  TORCH_CHECK(scales_b.scalar_type() == at::kFloat && scales_b.dim() == 3 && scales_b.size(0) == E &&
                  scales_b.size(1) == K / 128 && scales_b.size(2) == N / 128 && scales_b.stride(1) == 1 &&
                  scales_b.stride(2) == K / 128,
              "scales_b must be the (E, k/128, n/128) transposed view of contiguous f32 [E, n/128, k/128] memory");
  TORCH_CHECK(output.dim() == 2 && output.size(0) == a.size(0) && output.size(1) == N && output.is_contiguous(),
              "output must be a contiguous (num_tokens, n) tensor");
  const int dt = dtype_code(output, "output");
  c10::cuda::CUDAGuard guard(a.device());
  void* stream = c10::cuda::getCurrentCUDAStream(a.get_device()).stream();
  check_rc(es_b200_fp8_blockwise_grouped_mm(a.data_ptr(), b.data_ptr(), scales_a.data_ptr<float>(),
                                            scales_b.data_ptr<float>(), output.data_ptr(), dt,
                                            problem_sizes.data_ptr<int32_t>(), expert_offsets.data_ptr<int32_t>(),
                                            static_cast<int>(E), a.size(0), static_cast<int>(N), static_cast<int>(K),
                                            nullptr, 0, stream));
}

}  // namespace

TORCH_LIBRARY(es_b200, m) {
  m.def(
      "es_fp8_blockwise_scaled_grouped_mm(Tensor output, Tensor a, Tensor b, Tensor scales_a, Tensor scales_b, Tensor "
      "stride_a, Tensor stride_b, Tensor stride_d, Tensor problem_sizes, Tensor expert_offsets, Tensor workspace) -> "
      "()");
  m.def(
      "es_sm100_mxfp8_blockscaled_grouped_mm(Tensor a, Tensor b, Tensor sfa, Tensor sfb, Tensor d, Tensor "
      "problem_sizes, Tensor expert_offsets, Tensor blockscale_offsets) -> ()");
  m.def(
      "es_sm100_mxfp8_blockscaled_grouped_quant(Tensor input, Tensor problem_sizes, Tensor expert_offsets, Tensor "
      "blockscale_offsets, Tensor quant_output, Tensor scale_factor) -> () ");
  m.def(
      "es_sm100_mxfp8_silu_mul_grouped_quant(Tensor gate_up, Tensor problem_sizes, Tensor expert_offsets, Tensor "
      "blockscale_offsets, Tensor quant_output, Tensor scale_factor) -> ()");
}

TORCH_LIBRARY_IMPL(es_b200, CUDA, m) {
  m.impl("es_fp8_blockwise_scaled_grouped_mm", &es_fp8_blockwise_scaled_grouped_mm);
  m.impl("es_sm100_mxfp8_blockscaled_grouped_mm", &es_sm100_mxfp8_blockscaled_grouped_mm);
  m.impl("es_sm100_mxfp8_blockscaled_grouped_quant", &es_sm100_mxfp8_blockscaled_grouped_quant);
  m.impl("es_sm100_mxfp8_silu_mul_grouped_quant", &es_sm100_mxfp8_silu_mul_grouped_quant);
}
