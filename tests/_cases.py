"""Seeded input builders shared by the CPU and GPU tests."""
from __future__ import annotations

import numpy as np
import torch

from oracle import mxfp8_quant_oracle as Q


def f32_to_bf16_bits(a):
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def activations_bits(T, K, seed, is_bf16=True, outliers=True):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((T, K), dtype=np.float32)
    if outliers:
        x *= np.where(rng.random((T, K), dtype=np.float32) < 0.01, np.float32(50.0), np.float32(1.0))
    if is_bf16:
        return f32_to_bf16_bits(x)
    return x.astype(np.float16).view(np.uint16)


def bits_to_tensor(x_bits, is_bf16, device):
    dt = torch.bfloat16 if is_bf16 else torch.float16
    return torch.from_numpy(x_bits.view(np.int16)).to(device).view(dt)


def run_quant_op(x_bits, is_bf16, counts, device="cuda", sf_fill=0xCD, ps_n=0):
    """Calls the product op through ops.py -> C ABI.  Returns (codes u8 [T,K], sf flat u8, ps, eo, bo)."""
    from expert_specialization_moe_b200 import es_sm100_mxfp8_blockscaled_grouped_quant
    T, K = x_bits.shape
    ps, eo, bo, sf_rows = Q.offsets_from_counts(counts, ps_n, K)
    x = bits_to_tensor(x_bits, is_bf16, device)
    codes = torch.zeros((T, K), dtype=torch.uint8, device=device).view(torch.float8_e4m3fn)
    sf = torch.full((max(sf_rows, 1), K // 32), sf_fill, dtype=torch.uint8, device=device)
    es_sm100_mxfp8_blockscaled_grouped_quant(
        x, torch.from_numpy(ps).to(device), torch.from_numpy(eo).to(device), torch.from_numpy(bo).to(device), codes, sf)
    torch.cuda.synchronize()
    return codes.view(torch.uint8).cpu().numpy(), sf.cpu().numpy().reshape(-1)[: sf_rows * (K // 32)], ps, eo, bo


def oracle_quant(x_bits, is_bf16, counts, rcp448_bits=Q.RCP_448_BITS_DEFAULT, sf_fill=0xCD):
    T, K = x_bits.shape
    ps, eo, bo, sf_rows = Q.offsets_from_counts(counts, 0, K)
    codes = np.zeros((T, K), dtype=np.uint8)
    sf = np.full(sf_rows * (K // 32), sf_fill, dtype=np.uint8)
    Q.grouped_quant(x_bits, is_bf16, ps, eo, bo, codes, sf, rcp448_bits)
    return codes, sf


def valid_sf_index(counts, bo, K):
    idx = [int(bo[e]) * (K // 32) + Q.sf_swizzled_offsets(int(counts[e]), K).ravel()
           for e in range(len(counts)) if counts[e] > 0]
    return np.concatenate(idx) if idx else np.zeros(0, dtype=np.int64)


# ---- grouped GEMM cases ------------------------------------------------------------------------
def mxfp8_gemm_inputs(counts, N, K, seed, w_std=0.02):
    """Seeded MXFP8 operands built on the CPU with the oracle quantiser (bit-identical to the CUDA quantiser):
    returns dict of numpy arrays: a_codes [T,K], sfa flat, w_codes [E,N,K], sfb flat, ps, eo, bo."""
    rng = np.random.default_rng(seed)
    E = len(counts)
    T = int(sum(counts))
    ps, eo, bo, sfa_rows = Q.offsets_from_counts(counts, N, K)
    a_bits = f32_to_bf16_bits(rng.standard_normal((max(T, 1), K), dtype=np.float32))[:T]
    w_bits = f32_to_bf16_bits(rng.standard_normal((E * N, K), dtype=np.float32) * np.float32(w_std))
    a_codes = np.zeros((T, K), dtype=np.uint8)
    sfa = np.zeros(max(sfa_rows, 1) * (K // 32), dtype=np.uint8)
    Q.grouped_quant(a_bits, True, ps, eo, bo, a_codes, sfa)
    wps, weo, wbo, sfb_rows = Q.offsets_from_counts([N] * E, 0, K)
    w_codes = np.zeros((E * N, K), dtype=np.uint8)
    sfb = np.zeros(sfb_rows * (K // 32), dtype=np.uint8)
    Q.grouped_quant(w_bits, True, wps, weo, wbo, w_codes, sfb)
    return dict(a_codes=a_codes, sfa=sfa, w_codes=w_codes.reshape(E, N, K), sfb=sfb, ps=ps, eo=eo, bo=bo)


def run_mxfp8_mm_op(inp, out_dtype=torch.bfloat16, device="cuda", fill=None):
    """Calls the product GEMM through ops.py -> C ABI.  Returns d [T,N] on the CPU."""
    from expert_specialization_moe_b200 import es_sm100_mxfp8_blockscaled_grouped_mm
    E, N, K = inp["w_codes"].shape
    T = inp["a_codes"].shape[0]
    a = torch.from_numpy(inp["a_codes"]).to(device).view(torch.float8_e4m3fn)
    b = torch.from_numpy(inp["w_codes"]).to(device).view(torch.float8_e4m3fn).transpose(1, 2)   # [E,K,N] view
    sfa = torch.from_numpy(inp["sfa"]).to(device)
    sfb = torch.from_numpy(inp["sfb"]).to(device)
    d = torch.zeros((T, N), dtype=out_dtype, device=device)
    if fill is not None:
        d.fill_(fill)
    es_sm100_mxfp8_blockscaled_grouped_mm(
        d, a, b, sfa, sfb, torch.from_numpy(inp["ps"]).to(device), torch.from_numpy(inp["eo"]).to(device),
        torch.from_numpy(inp["bo"]).to(device))
    torch.cuda.synchronize()
    return d.cpu()


def device_status():
    from expert_specialization_moe_b200 import _cabi
    import ctypes
    lib = _cabi.load()
    raw = ctypes.c_uint32(0)
    rc = lib.es_b200_check_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(raw))
    return rc, raw.value


def fp8_blockwise_inputs(counts, N, K, seed, dtype=torch.bfloat16):
    """Operands of the FP8-blockwise op built with the (restated) reference quantisers on the CPU."""
    from oracle import grouped_gemm_oracle as G
    g = torch.Generator().manual_seed(seed)
    E, T = len(counts), int(sum(counts))
    ps, eo, _, _ = Q.offsets_from_counts(counts, N, K)
    a = torch.randn((max(T, 1), K), generator=g, dtype=torch.float32).to(dtype)[:T]
    w = torch.randn((E, N, K), generator=g, dtype=torch.float32).to(dtype)
    if T:
        a_q, sa = G.per_token_cast_to_fp8(a)
    else:
        a_q, sa = torch.zeros((0, K), dtype=torch.float8_e4m3fn), torch.zeros((0, K // 128))
    w_q = torch.empty((E, N, K), dtype=torch.float8_e4m3fn)
    sb = torch.empty((E, N // 128, K // 128), dtype=torch.float32)
    for e in range(E):
        w_q[e], sb[e] = G.per_block_cast_to_fp8(w[e])
    return dict(a=a, w=w, a_q=a_q.contiguous(), sa=sa.float().contiguous(), w_q=w_q, sb=sb, ps=ps, eo=eo)


def run_fp8_blockwise_op(inp, out_dtype=torch.bfloat16, device="cuda", fill=None):
    from expert_specialization_moe_b200 import es_fp8_blockwise_scaled_grouped_mm
    E, N, K = inp["w_q"].shape
    T = inp["a_q"].shape[0]
    a = inp["a_q"].to(device)
    b = inp["w_q"].to(device).transpose(1, 2)                 # [E, K, N] view, stride(1) == 1
    sa = inp["sa"].to(device)
    sb = inp["sb"].to(device).transpose(1, 2)                 # [E, K/128, N/128] view
    d = torch.zeros((T, N), dtype=out_dtype, device=device)
    if fill is not None:
        d.fill_(fill)
    strides = torch.full((E,), K, dtype=torch.int64, device=device)
    d_strides = torch.full((E,), N, dtype=torch.int64, device=device)
    workspace = torch.empty(1024, dtype=torch.uint8, device=device)
    es_fp8_blockwise_scaled_grouped_mm(d, a, b, sa, sb, strides, strides, d_strides,
                                       torch.from_numpy(inp["ps"]).to(device), torch.from_numpy(inp["eo"]).to(device),
                                       workspace)
    torch.cuda.synchronize()
    return d.cpu()
