"""Drop-in operator surface: same names, argument order and in-place semantics as the reference's
expert_specialization/ops.py:4-50, and the same mechanics: each function is a thin wrapper over a torch operator
(`torch.ops.es_b200.*`, registered by csrc_torch/es_b200_torch.cpp with the reference's schemas and the CUDA dispatch
key only).  The registered implementation validates its tensors the way the reference's host entry points do
(TORCH_CHECK -> RuntimeError before anything is launched), then hands raw device pointers and the current CUDA stream
to the C ABI (include/es_b200.h).  Nothing here computes: without the CUDA library the calls fail, and CPU tensors are
refused by the dispatcher (no CPU kernel is registered), as with the reference.
"""
from __future__ import annotations

from . import _cabi

__all__ = [
    "es_fp8_blockwise_scaled_grouped_mm",
    "es_sm100_mxfp8_blockscaled_grouped_mm",
    "es_sm100_mxfp8_blockscaled_grouped_quant",
    "es_sm100_mxfp8_silu_mul_grouped_quant",
]

_quant = _silu_quant = _mm = _blockwise_mm = None


def _bind():
    global _quant, _silu_quant, _mm, _blockwise_mm
    ops = _cabi.torch_ops()
    _quant = ops.es_sm100_mxfp8_blockscaled_grouped_quant.default
    _silu_quant = ops.es_sm100_mxfp8_silu_mul_grouped_quant.default
    _mm = ops.es_sm100_mxfp8_blockscaled_grouped_mm.default
    _blockwise_mm = ops.es_fp8_blockwise_scaled_grouped_mm.default


def es_sm100_mxfp8_blockscaled_grouped_quant(
    input, problem_sizes, expert_offsets, blockscale_offsets, quant_output, scale_factor
):
    """bf16/fp16 [T,K] -> e4m3 codes [T,K] + swizzled UE8M0 scales (reference: ops.py:40-50,
    es_sm100_mxfp8_blockscaled_group_quant.cu:5-39).  Writes quant_output and scale_factor in place."""
    if _quant is None:
        _bind()
    _quant(input, problem_sizes, expert_offsets, blockscale_offsets, quant_output, scale_factor)


def es_sm100_mxfp8_silu_mul_grouped_quant(
    gate_up, problem_sizes, expert_offsets, blockscale_offsets, quant_output, scale_factor
):
    """Fused silu(gate) * up -> MXFP8 grouped quantisation; gate_up is [T, 2K] (gate | up), outputs as for
    es_sm100_mxfp8_blockscaled_grouped_quant with K columns.  An addition of this library (the reference has no fused
    ops): same bits as the unfused sequence, one pass over memory."""
    if _silu_quant is None:
        _bind()
    _silu_quant(gate_up, problem_sizes, expert_offsets, blockscale_offsets, quant_output, scale_factor)


def es_sm100_mxfp8_blockscaled_grouped_mm(
    output, a, b, sfa, sfb, problem_sizes, expert_offsets, blockscale_offsets
):
    """MXFP8 (e4m3 + UE8M0 per 32) grouped GEMM, bf16/fp16 out (reference: ops.py:32-37,
    es_sm100_mxfp8_blockscaled.cu:5-40).  `b` is the reference's [E, K, N] view of [E, N, K] memory.  As in the
    reference, the registered operator takes the output in fifth place."""
    if _mm is None:
        _bind()
    _mm(a, b, sfa, sfb, output, problem_sizes, expert_offsets, blockscale_offsets)


def es_fp8_blockwise_scaled_grouped_mm(
    output,
    a,
    b,
    scales_a,
    scales_b,
    stride_a,
    stride_b,
    stride_d,
    problem_sizes,
    expert_offsets,
    workspace,
):
    """e4m3 x e4m3 grouped GEMM with fp32 scales (1x128 on a, 128x128 on b), bf16/fp16 out (reference: ops.py:4-29,
    es_fp8_blockwise.cu:34-193).  stride_a / stride_b / stride_d and workspace are accepted for signature
    compatibility; the strides must describe densely packed rows (K, K, N), as the reference's callers pass them, and
    the workspace is not used."""
    if _blockwise_mm is None:
        _bind()
    _blockwise_mm(output, a, b, scales_a, scales_b, stride_a, stride_b, stride_d, problem_sizes, expert_offsets,
                  workspace)
