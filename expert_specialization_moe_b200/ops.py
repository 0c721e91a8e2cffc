"""Drop-in operator surface: same names, argument order and in-place semantics as the reference's
expert_specialization/ops.py:4-50.  Each function validates its tensors the way the reference's host entry points
do (TORCH_CHECK -> RuntimeError before anything is launched), then hands raw device pointers and the current CUDA
stream to the C ABI (include/es_b200.h).  Nothing here computes: without the CUDA library the calls fail.
"""
from __future__ import annotations

import torch

from . import _cabi

__all__ = [
    "es_fp8_blockwise_scaled_grouped_mm",
    "es_sm100_mxfp8_blockscaled_grouped_mm",
    "es_sm100_mxfp8_blockscaled_grouped_quant",
    "es_sm100_mxfp8_silu_mul_grouped_quant",
]


def _check(cond: bool, msg: str):
    if not cond:
        raise RuntimeError(msg)


def _dtype_code(dt: torch.dtype, what: str) -> int:
    if dt == torch.bfloat16:
        return _cabi.BF16
    if dt == torch.float16:
        return _cabi.FP16
    raise RuntimeError(f"{what}: dtype must be kFloat16 or kBFloat16")


def _stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(*tensors):
    for t in tensors:
        _check(t.is_cuda, "expert_specialization ops are CUDA-only (no CPU implementation exists)")


def _scratch(lib, num_experts: int, num_rows: int, n: int, k: int, device) -> torch.Tensor:
    nbytes = int(lib.es_b200_grouped_mm_scratch_bytes(num_experts, num_rows, n, k))
    return torch.empty(nbytes, dtype=torch.uint8, device=device) if nbytes else None


def es_sm100_mxfp8_blockscaled_grouped_quant(
    input, problem_sizes, expert_offsets, blockscale_offsets, quant_output, scale_factor
):
    """bf16/fp16 [T,K] -> e4m3 codes [T,K] + swizzled UE8M0 scales (reference: ops.py:40-50,
    es_sm100_mxfp8_blockscaled_group_quant.cu:5-39).  Writes quant_output and scale_factor in place."""
    _require_cuda(input, problem_sizes, expert_offsets, blockscale_offsets, quant_output, scale_factor)
    _check(input.dim() == 2, "input must be 2D tensor")
    _check(input.size(1) % 128 == 0, "k must align to 128")
    _check(input.stride(1) == 1, "input must be row major")
    _check(problem_sizes.dim() == 2, "problem_sizes must be 2D tensor")
    groups = problem_sizes.size(0)
    _check(expert_offsets.dim() == 1 and expert_offsets.size(0) == groups,
           "expert_offsets must be 1D and have size equal to the number of groups")
    _check(blockscale_offsets.dim() == 1 and blockscale_offsets.size(0) == groups,
           "blockscale_offsets must be 1D and have size equal to the number of groups")
    # checks the reference leaves implicit (it reinterprets the raw pointers)
    _check(problem_sizes.size(1) == 3 and problem_sizes.dtype == torch.int32 and problem_sizes.is_contiguous(),
           "problem_sizes must be a contiguous int32 tensor of shape (num_experts, 3)")
    _check(expert_offsets.dtype == torch.int32 and blockscale_offsets.dtype == torch.int32,
           "expert_offsets and blockscale_offsets must be int32")
    _check(expert_offsets.is_contiguous() and blockscale_offsets.is_contiguous(), "offsets must be contiguous")
    _check(input.stride(0) == input.size(1), "input rows must be densely packed")
    _check(quant_output.is_contiguous() and quant_output.numel() == input.numel()
           and quant_output.element_size() == 1, "quant_output must be a contiguous 1-byte tensor shaped like input")
    _check(scale_factor.is_contiguous() and scale_factor.element_size() == 1,
           "scale_factor must be a contiguous 1-byte tensor")
    dt = _dtype_code(input.dtype, "input")
    lib = _cabi.load()
    _cabi.check(lib.es_b200_mxfp8_grouped_quant(
        input.data_ptr(), dt, problem_sizes.data_ptr(), expert_offsets.data_ptr(), blockscale_offsets.data_ptr(),
        quant_output.data_ptr(), scale_factor.data_ptr(), groups, input.size(0), input.size(1),
        _stream_ptr(input)))


def es_sm100_mxfp8_silu_mul_grouped_quant(
    gate_up, problem_sizes, expert_offsets, blockscale_offsets, quant_output, scale_factor
):
    """Fused silu(gate) * up -> MXFP8 grouped quantisation; gate_up is [T, 2K] (gate | up), outputs as for
    es_sm100_mxfp8_blockscaled_grouped_quant with K columns.  An addition of this library (the reference has no fused
    ops): same bits as the unfused sequence, one pass over memory."""
    _require_cuda(gate_up, problem_sizes, expert_offsets, blockscale_offsets, quant_output, scale_factor)
    _check(gate_up.dim() == 2 and gate_up.size(1) % 256 == 0, "gate_up must be (rows, 2k) with k aligned to 128")
    _check(gate_up.stride(1) == 1 and gate_up.stride(0) == gate_up.size(1), "gate_up must be densely packed row major")
    k = gate_up.size(1) // 2
    groups = problem_sizes.size(0)
    _check(problem_sizes.dim() == 2 and problem_sizes.size(1) == 3 and problem_sizes.dtype == torch.int32
           and problem_sizes.is_contiguous(), "problem_sizes must be a contiguous int32 tensor of shape (num_experts, 3)")
    _check(expert_offsets.dim() == 1 and expert_offsets.size(0) == groups and expert_offsets.dtype == torch.int32
           and expert_offsets.is_contiguous(), "expert_offsets must be contiguous int32 of length num_experts")
    _check(blockscale_offsets.dim() == 1 and blockscale_offsets.size(0) == groups
           and blockscale_offsets.dtype == torch.int32 and blockscale_offsets.is_contiguous(),
           "blockscale_offsets must be contiguous int32 of length num_experts")
    _check(quant_output.is_contiguous() and quant_output.numel() == gate_up.size(0) * k
           and quant_output.element_size() == 1, "quant_output must be a contiguous 1-byte (rows, k) tensor")
    _check(scale_factor.is_contiguous() and scale_factor.element_size() == 1,
           "scale_factor must be a contiguous 1-byte tensor")
    dt = _dtype_code(gate_up.dtype, "gate_up")
    lib = _cabi.load()
    _cabi.check(lib.es_b200_mxfp8_silu_mul_grouped_quant(
        gate_up.data_ptr(), dt, problem_sizes.data_ptr(), expert_offsets.data_ptr(), blockscale_offsets.data_ptr(),
        quant_output.data_ptr(), scale_factor.data_ptr(), groups, gate_up.size(0), k, _stream_ptr(gate_up)))


def es_sm100_mxfp8_blockscaled_grouped_mm(
    output, a, b, sfa, sfb, problem_sizes, expert_offsets, blockscale_offsets
):
    """MXFP8 (e4m3 + UE8M0 per 32) grouped GEMM, bf16/fp16 out (reference: ops.py:32-37,
    es_sm100_mxfp8_blockscaled.cu:5-40).  `b` is the reference's [E, K, N] view of [E, N, K] memory."""
    _require_cuda(output, a, b, sfa, sfb, problem_sizes, expert_offsets, blockscale_offsets)
    _check(problem_sizes.dim() == 2, "problem_sizes must be 2D tensor")
    _check(problem_sizes.size(1) == 3, "problem_sizes must have shape (num_experts, 3)")
    _check(problem_sizes.size(0) == expert_offsets.size(0),
           "Number of experts in problem_sizes must match expert_offsets")
    _check(problem_sizes.dtype == torch.int32, "problem_sizes must be int32")
    _check(a.dim() == 2, "a must be a 2D tensor of shape (num_tokens, k)")
    _check(b.dim() == 3, "b must be a 3D tensor of shape (num_experts, k, n)")
    _check(a.size(1) == b.size(1) and a.size(1) % 128 == 0, "k should align 128")
    _check(b.size(2) % 128 == 0, "n should align 128")
    _check(a.stride(1) == 1, "a must be row major")
    _check(b.stride(1) == 1, "a must be column major")
    # implicit in the reference
    E, K, N = b.size(0), b.size(1), b.size(2)
    _check(E == problem_sizes.size(0), "b must hold one matrix per expert")
    _check(b.stride(2) == K and b.stride(0) == N * K, "b must be a transposed view of contiguous [E, N, K] memory")
    _check(a.stride(0) == K, "a rows must be densely packed")
    _check(a.element_size() == 1 and b.element_size() == 1, "a and b must be float8_e4m3fn")
    _check(output.dim() == 2 and output.size(0) == a.size(0) and output.size(1) == N and output.is_contiguous(),
           "output must be a contiguous (num_tokens, n) tensor")
    _check(expert_offsets.dtype == torch.int32 and blockscale_offsets.dtype == torch.int32
           and blockscale_offsets.size(0) == E, "offsets must be int32 of length num_experts")
    _check(problem_sizes.is_contiguous() and expert_offsets.is_contiguous() and blockscale_offsets.is_contiguous(),
           "problem_sizes / offsets must be contiguous")
    _check(sfa.element_size() == 1 and sfb.element_size() == 1, "sfa and sfb must be 1-byte UE8M0 tensors")
    dt = _dtype_code(output.dtype, "output")
    lib = _cabi.load()
    T = a.size(0)
    sfa_rows = sfa.numel() // (K // 32)
    scratch = _scratch(lib, E, T, N, K, a.device)
    _cabi.check(lib.es_b200_mxfp8_grouped_mm(
        a.data_ptr(), b.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), output.data_ptr(), dt,
        problem_sizes.data_ptr(), expert_offsets.data_ptr(), blockscale_offsets.data_ptr(), E, T, N, K, sfa_rows,
        scratch.data_ptr() if scratch is not None else None, scratch.numel() if scratch is not None else 0,
        _stream_ptr(a)))


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
    _require_cuda(output, a, b, scales_a, scales_b, problem_sizes, expert_offsets)
    _check(problem_sizes.dim() == 2, "problem_sizes must be 2D tensor")
    _check(problem_sizes.size(1) == 3, "problem_sizes must have shape (num_experts, 3)")
    _check(problem_sizes.size(0) == expert_offsets.size(0),
           "Number of experts in problem_sizes must match expert_offsets")
    _check(problem_sizes.dtype == torch.int32, "problem_sizes must be int32")
    _check(a.dtype == torch.float8_e4m3fn, "a must be kFloat8_e4m3fn")
    _check(b.dtype == torch.float8_e4m3fn, "b must be kFloat8_e4m3fn")
    _check(output.dtype in (torch.bfloat16, torch.float16), "output must be bfloat16 or half")
    _check(a.dim() == 2 and b.dim() == 3, "a must be (num_tokens, k) and b (num_experts, k, n)")
    E, K, N = b.size(0), b.size(1), b.size(2)
    _check(a.size(1) == K and K % 128 == 0, "k should align 128")
    _check(N % 128 == 0, "n should align 128")
    _check(b.stride(1) == 1 and b.stride(2) == K and b.stride(0) == N * K,
           "b must be a transposed view of contiguous [E, N, K] memory")
    _check(a.stride(1) == 1 and a.stride(0) == K, "a must be row major with densely packed rows")
    _check(E == problem_sizes.size(0), "b must hold one matrix per expert")
    _check(scales_a.dtype == torch.float32 and scales_a.dim() == 2 and scales_a.size(0) == a.size(0)
           and scales_a.size(1) == K // 128 and scales_a.is_contiguous(), "scales_a must be contiguous f32 (num_tokens, k/128)")
    _check(scales_b.dtype == torch.float32 and scales_b.dim() == 3 and scales_b.size(0) == E
           and scales_b.size(1) == K // 128 and scales_b.size(2) == N // 128
           and scales_b.stride(1) == 1 and scales_b.stride(2) == K // 128,
           "scales_b must be the (E, k/128, n/128) transposed view of contiguous f32 [E, n/128, k/128] memory")
    _check(output.dim() == 2 and output.size(0) == a.size(0) and output.size(1) == N and output.is_contiguous(),
           "output must be a contiguous (num_tokens, n) tensor")
    _check(expert_offsets.dtype == torch.int32 and expert_offsets.is_contiguous() and problem_sizes.is_contiguous(),
           "problem_sizes / expert_offsets must be contiguous int32")
    dt = _dtype_code(output.dtype, "output")
    lib = _cabi.load()
    T = a.size(0)
    scratch = _scratch(lib, E, T, N, K, a.device)
    _cabi.check(lib.es_b200_fp8_blockwise_grouped_mm(
        a.data_ptr(), b.data_ptr(), scales_a.data_ptr(), scales_b.data_ptr(), output.data_ptr(), dt,
        problem_sizes.data_ptr(), expert_offsets.data_ptr(), E, T, N, K,
        scratch.data_ptr() if scratch is not None else None, scratch.numel() if scratch is not None else 0,
        _stream_ptr(a)))
