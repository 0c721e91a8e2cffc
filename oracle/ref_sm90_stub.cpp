// TEST INFRASTRUCTURE ONLY (checker side, never shipped or measured as the product).
//
// The reference registers three torch ops in one TORCH_LIBRARY block
// (expert_specialization/csrc/expert_specialization.cpp:56-73).  Its FP8-blockwise op
// (expert_specialization/csrc/cuda/es_fp8_blockwise.cu) is Hopper-only device code and cannot
// be built for sm_100a, so the reference build used as an on-GPU checker links this
// throwing stand-in for that one symbol.  Nothing here restates reference arithmetic.
#include <torch/all.h>

void es_fp8_blockwise_scaled_grouped_mm(
    torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&,
    const torch::Tensor&, const torch::Tensor&, const torch::Tensor&, const torch::Tensor&,
    const torch::Tensor&, const torch::Tensor&, const torch::Tensor&) {
  TORCH_CHECK(false, "reference es_fp8_blockwise_scaled_grouped_mm is sm_90a-only; not built for sm_100a");
}
