"""CPU oracle for the two grouped GEMMs.  TEST INFRASTRUCTURE ONLY.

* MXFP8 block-scaled grouped GEMM: semantics of the reference's CUTLASS instantiation
    expert_specialization/csrc/cuda/es_sm100_mxfp8_blockscaled_traits.cuh:44-72  (e4m3 operands, UE8M0 scale per
        32 K elements, fp32 accumulation, round-to-nearest to bf16/fp16, no C operand)
    expert_specialization/csrc/cuda/es_sm100_mxfp8_blockscaled_functor.cuh:61-75 (per-expert addressing:
        A + off_e*K, B + e*N*K, SFA + bsoff_e*K/32, SFB + e*N*K/32, D + off_e*N)
  restated as dequantise -> per-expert fp32 matmul, modelled on the reference's torch path
    test/test_es_grouped_gemm.py:62-86 (baseline_scaled_mm).
* FP8-blockwise grouped GEMM (fp32 scales: 1x128 on A, 128x128 on B):
    test/test_es_grouped_gemm.py:36-86 (per_token_cast_to_fp8, per_block_cast_to_fp8, baseline_scaled_mm)
    expert_specialization/csrc/cuda/es_fp8_blockwise_functor.cuh:57-74 (addressing).

Floating-point results are compared with tolerances (relative error <= 1e-2, cosine >= 0.9999, and the reference's
own criterion calc_diff < 1e-3), never bit-wise.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
"""
from __future__ import annotations

import numpy as np
import torch

from . import mxfp8_quant_oracle as Q


def calc_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2<x,y>/(|x|^2+|y|^2): the acceptance metric of the reference's tests (test_es_grouped_gemm.py:25-29)."""
    x, y = x.double(), y.double()
    den = (x * x + y * y).sum()
    if den == 0:
        return 0.0
    return float(1 - 2 * (x * y).sum() / den)


def rel_err_and_cosine(x: torch.Tensor, y: torch.Tensor):
    x, y = x.double().flatten(), y.double().flatten()
    ny = y.norm()
    rel = float((x - y).norm() / ny) if ny > 0 else float((x - y).norm())
    den = x.norm() * ny
    cos = float((x * y).sum() / den) if den > 0 else 1.0
    return rel, cos


def dequant_mxfp8(codes_u8: torch.Tensor, sf_rowmajor_u8: torch.Tensor) -> torch.Tensor:
    """codes [R,K] u8 (e4m3 bits), sf [R,K/32] u8 (UE8M0) -> fp32 [R,K] = code * 2^(sf-127)."""
    vals = codes_u8.view(torch.float8_e4m3fn).to(torch.float32)
    scale = torch.exp2(sf_rowmajor_u8.to(torch.float32) - 127.0)
    R, K = vals.shape
    return (vals.view(R, K // 32, 32) * scale.unsqueeze(-1)).view(R, K)


def unswizzle_sf_torch(sf_flat_u8: torch.Tensor, base: int, m: int, K: int) -> torch.Tensor:
    if m == 0:
        return torch.zeros((0, K // 32), dtype=torch.uint8)
    idx = torch.from_numpy(Q.sf_swizzled_offsets(m, K)) + base
    return sf_flat_u8.reshape(-1)[idx]


def mxfp8_grouped_mm(a_u8, b_u8, sfa_u8, sfb_u8, problem_sizes, expert_offsets, blockscale_offsets,
                     out_dtype=torch.bfloat16, out=None, experts=None):
    """a [T,K] u8; b memory layout [E,N,K] u8; sfa / sfb flat swizzled u8.  Returns d [T,N] (rows outside every
    expert are zero unless `out` is given).  `experts` restricts the computation to a subset (bounded CPU timing)."""
    T, K = a_u8.shape
    E, N, _ = b_u8.shape
    d = out if out is not None else torch.zeros((T, N), dtype=out_dtype)
    for e in (range(E) if experts is None else experts):
        m = int(problem_sizes[e][0])
        if m == 0:
            continue
        off = int(expert_offsets[e])
        sa = unswizzle_sf_torch(sfa_u8, int(blockscale_offsets[e]) * (K // 32), m, K)
        sb = unswizzle_sf_torch(sfb_u8, e * N * (K // 32), N, K)
        af = dequant_mxfp8(a_u8[off:off + m], sa)
        bf = dequant_mxfp8(b_u8[e], sb)
        d[off:off + m] = torch.mm(af, bf.t()).to(d.dtype)
    return d


# ---- FP8-blockwise (fp32 scales) -------------------------------------------------------------
def per_token_cast_to_fp8(x: torch.Tensor):
    """Restates test_es_grouped_gemm.py:36-44 for K % 128 == 0: 1x128 groups, scale = amax/448, amax clamped 1e-4."""
    m, k = x.shape
    assert k % 128 == 0
    xv = x.view(m, -1, 128)
    amax = xv.abs().float().amax(dim=2).view(m, -1).clamp(1e-4)
    q = (xv * (448.0 / amax.unsqueeze(2))).to(torch.float8_e4m3fn)
    return q.view(m, k), (amax / 448.0).view(m, -1)


def per_block_cast_to_fp8(x: torch.Tensor):
    """Restates test_es_grouped_gemm.py:47-59 for dims % 128 == 0: 128x128 blocks."""
    m, n = x.shape
    assert m % 128 == 0 and n % 128 == 0
    xv = x.view(-1, 128, n // 128, 128)
    amax = xv.abs().float().amax(dim=(1, 3), keepdim=True).clamp(1e-4)
    q = (xv * (448.0 / amax)).to(torch.float8_e4m3fn)
    return q.view(m, n).contiguous(), (amax / 448.0).view(xv.size(0), xv.size(2))


def fp8_blockwise_grouped_mm(a_u8, b_u8, scales_a, scales_b, problem_sizes, expert_offsets,
                             out_dtype=torch.bfloat16, out=None, experts=None):
    """a [T,K] u8 (e4m3); b memory [E,N,K] u8; scales_a [T,K/128] f32; scales_b memory [E,N/128,K/128] f32.
    d[off_e:off_e+m] = (sa (x) a) @ (sb (x) b)^T in fp32, cast to out_dtype (test_es_grouped_gemm.py:62-86)."""
    T, K = a_u8.shape
    E, N, _ = b_u8.shape
    d = out if out is not None else torch.zeros((T, N), dtype=out_dtype)
    for e in (range(E) if experts is None else experts):
        m = int(problem_sizes[e][0])
        if m == 0:
            continue
        off = int(expert_offsets[e])
        af = a_u8[off:off + m].view(torch.float8_e4m3fn).float() * scales_a[off:off + m].repeat_interleave(128, dim=1)
        bf = b_u8[e].view(torch.float8_e4m3fn).float() * \
            scales_b[e].repeat_interleave(128, dim=0).repeat_interleave(128, dim=1)
        d[off:off + m] = torch.mm(af, bf.t()).to(d.dtype)
    return d
