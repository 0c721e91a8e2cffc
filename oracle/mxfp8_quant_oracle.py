"""CPU oracle for the SM100 MXFP8 grouped quantisation.  TEST INFRASTRUCTURE ONLY.

numpy restatement of the reference kernel
  expert_specialization/csrc/cuda/es_sm100_mxfp8_blockscaled_group_quant.cuh
      :36-134   cvt_warp_fp16_to_mxfp8     (amax -> UE8M0 scale -> e4m3 codes)
      :17-25, :294-310                     (512-byte swizzled scale-factor atoms, per-expert base)
      :261-355  mxfp8_group_quant          (which rows of which expert are touched)
and of the CUDA conversion intrinsics it calls (cuda_fp8.hpp: __nv_cvt_float_to_e8m0 with
__NV_SATFINITE / cudaRoundPosInf, the e8m0 -> float cast, __nv_fp8x2_e4m3(float2)).

Parity status: the reference ships no golden vectors for this op.  The oracle is pinned by fixtures
produced by running the reference's own kernel on a B200 (tests/golden/, made by
tests/golden/make_reference_fixtures.py); see the test-suite for which fixtures exist.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.
"""
from __future__ import annotations

import numpy as np

# Bit pattern returned by `rcp.approx.ftz.f32 448.0f` on B200 (the single hardware-dependent constant of the
# algorithm, group_quant.cuh:81).  RN(1/448) = 0x3B124925; tests/golden holds the value measured on the GPU.
RCP_448_BITS_DEFAULT = 0x3B124925

SF_BLOCK = 32        # elements per scale factor (MX block)
ATOM_ROWS = 128      # rows per swizzled scale-factor atom
ATOM_KBLOCKS = 4     # K blocks per atom  -> 512 bytes


# ----------------------------------------------------------------------------------------------
# scalar-format helpers (all vectorised over numpy arrays)
# ----------------------------------------------------------------------------------------------
def bf16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f16_bits_to_f32(u16: np.ndarray) -> np.ndarray:
    return u16.view(np.float16).astype(np.float32)


def f32_to_ue8m0_rp_satfinite(x: np.ndarray) -> np.ndarray:
    """`cvt.rp.satfinite.ue8m0x2.f32` on |x| (cuda_fp8.hpp __nv_cvt_float_to_e8m0, used at group_quant.cuh:86).

    Round toward +inf to a power of two 2^(sf-127); |x| <= 2^-127 -> 0; non-NaN overflow -> 0xFE; NaN -> 0xFF.
    """
    bits = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32) & np.uint32(0x7FFFFFFF)
    exp = (bits >> np.uint32(23)).astype(np.int32)
    man = bits & np.uint32(0x7FFFFF)
    res = exp + (man != 0)
    # f32 subnormals: only values strictly above 2^-127 (mantissa 0x400000) round up to 2^-126
    res = np.where(exp == 0, (man > np.uint32(0x400000)).astype(np.int32), res)
    res = np.minimum(res, 254)
    res = np.where((exp == 255) & (man != 0), 255, res)   # NaN
    return res.astype(np.uint8)


def ue8m0_to_f32(sf: np.ndarray) -> np.ndarray:
    """`static_cast<float>(__nv_fp8_e8m0)` (group_quant.cuh:87): 2^(sf-127); 0 -> 2^-127 (f32 subnormal); 0xFF -> NaN."""
    sf = sf.astype(np.uint32)
    bits = sf << np.uint32(23)
    bits = np.where(sf == 0, np.uint32(0x00400000), bits)
    bits = np.where(sf == 255, np.uint32(0x7FFFFFFF), bits)
    return bits.astype(np.uint32).view(np.float32)


def rcp_approx_ftz_of_scale(sf: np.ndarray) -> np.ndarray:
    """`rcp.approx.ftz.f32` of ue8m0_to_f32(sf) (group_quant.cuh:90,28-32).

    The argument is always a power of two, where the approximation is exact: 2^(127-sf).  Flush-to-zero edge
    cases: sf == 0 (argument 2^-127 is subnormal, flushed to 0 -> +inf); sf == 254 (result 2^-127 is subnormal,
    flushed to +0); sf == 255 -> NaN.
    """
    sf = sf.astype(np.int32)
    e = 127 - sf + 127                       # biased exponent of 2^(127-sf)
    bits = (np.clip(e, 0, 254).astype(np.uint32)) << np.uint32(23)
    bits = np.where(sf == 0, np.uint32(0x7F800000), bits)
    bits = np.where(sf >= 254, np.uint32(0), bits)
    bits = np.where(sf == 255, np.uint32(0x7FFFFFFF), bits)
    return bits.astype(np.uint32).view(np.float32)


def f32_to_e4m3_rn_satfinite(v: np.ndarray) -> np.ndarray:
    """`cvt.rn.satfinite.e4m3x2.f32` (via __nv_fp8x2_e4m3(float2), group_quant.cuh:109-116).

    Round to nearest even on the e4m3fn grid, |v| > 448 (incl. inf) -> +-448 (0x7E / 0xFE), NaN -> 0x7F,
    the sign of zero is kept.
    """
    v = np.ascontiguousarray(v, dtype=np.float32)
    bits = v.view(np.uint32)
    sign = ((bits >> np.uint32(24)) & np.uint32(0x80)).astype(np.uint8)
    abits = bits & np.uint32(0x7FFFFFFF)
    a = abits.view(np.float32)
    isnan = abits > np.uint32(0x7F800000)
    # normal range of e4m3 (>= 2^-6): round the f32 mantissa to 3 bits, ties to even
    lsb = (abits >> np.uint32(20)) & np.uint32(1)
    rb = (abits + np.uint32(0x7FFFF) + lsb) & np.uint32(0xFFF00000)
    e = (rb >> np.uint32(23)).astype(np.int32) - 127
    m3 = ((rb >> np.uint32(20)) & np.uint32(7)).astype(np.int32)
    code_norm = ((e + 7) << 3) | m3
    # subnormal range (< 2^-6): multiples of 2^-9, ties to even (np.rint)
    with np.errstate(invalid="ignore", over="ignore"):
        q = np.rint(a.astype(np.float64) * 512.0)
    q = np.where(np.isfinite(q), q, 0.0)
    code_sub = np.minimum(q, 8.0).astype(np.int32)
    small = a < np.float32(2.0 ** -6)
    code = np.where(small, code_sub, code_norm)
    code = np.where(a > np.float32(448.0), 0x7E, code)           # satfinite (also catches rounding to 512 / inf)
    code = np.where(code > 0x7E, 0x7E, code)
    out = code.astype(np.uint8) | sign
    out = np.where(isnan, np.uint8(0x7F), out)
    return out.astype(np.uint8)


_E4M3_LUT = None


def e4m3_to_f32(codes: np.ndarray) -> np.ndarray:
    """Decode e4m3fn bytes (bias 7, no inf, 0x7F/0xFF = NaN)."""
    global _E4M3_LUT
    if _E4M3_LUT is None:
        c = np.arange(256, dtype=np.int32)
        e = (c >> 3) & 0xF
        m = c & 7
        val = np.where(e == 0, m * 2.0 ** -9, (1.0 + m / 8.0) * np.exp2((e - 7).astype(np.float64)))
        val = np.where((c & 0x7F) == 0x7F, np.nan, val)
        val = np.where(c >= 128, -val, val)
        _E4M3_LUT = val.astype(np.float32)
    return _E4M3_LUT[codes]


# ----------------------------------------------------------------------------------------------
# per-row quantisation (group_quant.cuh:36-134)
# ----------------------------------------------------------------------------------------------
def quantize_rows(x_bits: np.ndarray, is_bf16: bool, rcp448_bits: int = RCP_448_BITS_DEFAULT):
    """x_bits: uint16 [R, K] raw bf16/fp16 bits, K % 32 == 0.  Returns (codes u8 [R,K], sf u8 [R,K/32])."""
    assert x_bits.dtype == np.uint16 and x_bits.ndim == 2 and x_bits.shape[1] % SF_BLOCK == 0
    R, K = x_bits.shape
    x = bf16_bits_to_f32(x_bits) if is_bf16 else f16_bits_to_f32(x_bits)
    xb = x.reshape(R, K // SF_BLOCK, SF_BLOCK)
    # __habs2/__hmax2/__hmax drop NaN operands (cuh:67-79): NaN only if the whole block is NaN
    with np.errstate(invalid="ignore"):
        amax = np.fmax.reduce(np.abs(xb), axis=2)
    rcp448 = np.array([rcp448_bits], dtype=np.uint32).view(np.float32)[0]
    with np.errstate(invalid="ignore", over="ignore", under="ignore"):
        s = (amax * rcp448).astype(np.float32)                      # cuh:81, IEEE fp32 multiply
    sf = f32_to_ue8m0_rp_satfinite(s)                               # cuh:85-88
    inv = rcp_approx_ftz_of_scale(sf)                               # cuh:90
    inv = np.where(amax != 0, inv, np.float32(0.0)).astype(np.float32)
    with np.errstate(invalid="ignore", over="ignore", under="ignore"):
        scaled = (xb * inv[:, :, None]).astype(np.float32)          # cuh:102-103
    codes = f32_to_e4m3_rn_satfinite(scaled).reshape(R, K)
    return codes, sf


def silu_mul_bits(gate_up_bits: np.ndarray, is_bf16: bool) -> np.ndarray:
    """[R, 2K] raw bits (gate | up) -> [R, K] raw bits of round_to_input_type(silu(gate) * up), fp32 arithmetic
    x / (1 + exp(-x)).  (No reference counterpart: restates the unfused torch sequence silu(g.float()) * u.float().)
    numpy's float32 exp can differ from the GPU's expf in the last bit, which rarely survives the rounding to 16 bits;
    tests compare with a stated mismatch allowance and, exactly, with the unfused GPU sequence."""
    R, K2 = gate_up_bits.shape
    K = K2 // 2
    conv = bf16_bits_to_f32 if is_bf16 else f16_bits_to_f32
    g, u = conv(gate_up_bits[:, :K]), conv(gate_up_bits[:, K:])
    with np.errstate(over="ignore", invalid="ignore"):
        act = (g / (np.float32(1.0) + np.exp(-g, dtype=np.float32))).astype(np.float32) * u
    if is_bf16:
        b = np.ascontiguousarray(act, dtype=np.float32).view(np.uint32)
        nan = (b & np.uint32(0x7FFFFFFF)) > np.uint32(0x7F800000)
        r = ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)
        return np.where(nan, np.uint16(0x7FFF), r).astype(np.uint16)
    return act.astype(np.float16).view(np.uint16)


# ----------------------------------------------------------------------------------------------
# swizzled scale-factor layout (group_quant.cuh:25,294-310)
# ----------------------------------------------------------------------------------------------
def align128(m):
    return (m + 127) // 128 * 128


def sf_swizzled_offsets(rows: int, K: int) -> np.ndarray:
    """Byte offsets [rows, K/32] (relative to the expert's base) of the scale factor of (row r, K block kb).

    off = (r/128)*(K/128)*512 + (kb/4)*512 + (r%32)*16 + ((r%128)/32)*4 + kb%4
    """
    r = np.arange(rows, dtype=np.int64)[:, None]
    kb = np.arange(K // SF_BLOCK, dtype=np.int64)[None, :]
    kt = K // 128
    return (r // 128) * kt * 512 + (kb // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + (kb % 4)


def swizzle_sf(sf_rowmajor: np.ndarray, K: int, fill: int = 0) -> np.ndarray:
    """[m, K/32] row-major scale bytes -> flat swizzled bytes of length align128(m) * K/32 (padding = fill)."""
    m = sf_rowmajor.shape[0]
    out = np.full(align128(m) * (K // SF_BLOCK), fill, dtype=np.uint8)
    if m:
        out[sf_swizzled_offsets(m, K).ravel()] = sf_rowmajor.ravel()
    return out


def unswizzle_sf(sf_flat: np.ndarray, m: int, K: int) -> np.ndarray:
    """Inverse of swizzle_sf on the valid rows: flat swizzled bytes -> [m, K/32] row-major."""
    if m == 0:
        return np.zeros((0, K // SF_BLOCK), dtype=np.uint8)
    return sf_flat[sf_swizzled_offsets(m, K)]


# ----------------------------------------------------------------------------------------------
# the grouped op (group_quant.cuh:261-355; host checks in ..._group_quant.cu:13-24)
# ----------------------------------------------------------------------------------------------
def grouped_quant(x_bits, is_bf16, problem_sizes, expert_offsets, blockscale_offsets, codes_out, sf_out,
                  rcp448_bits: int = RCP_448_BITS_DEFAULT, zero_padding_rows: bool = True):
    """In-place grouped quantisation with the reference's addressing.

    x_bits [T,K] u16; problem_sizes [E,3] (m,n,k) int; expert_offsets [E]; blockscale_offsets [E];
    codes_out [T,K] u8 (rows outside every expert's range are left untouched); sf_out flat u8 of
    sum(align128(m)) * K/32 bytes.  The reference leaves the scale bytes of padding rows (m <= r < align128(m))
    unspecified; with zero_padding_rows they are set to 0, which is what the CUDA path of this repo writes.
    """
    T, K = x_bits.shape
    assert K % 128 == 0
    kb = K // SF_BLOCK
    sf_flat = sf_out.reshape(-1)
    for e in range(len(problem_sizes)):
        m = int(problem_sizes[e][0])
        if m == 0:
            continue
        off = int(expert_offsets[e])
        base = int(blockscale_offsets[e]) * kb
        c, s = quantize_rows(x_bits[off:off + m], is_bf16, rcp448_bits)
        codes_out[off:off + m] = c
        mp = align128(m)
        if zero_padding_rows:
            sf_flat[base: base + mp * kb] = swizzle_sf(s, K, 0)
        else:
            sf_flat[base + sf_swizzled_offsets(m, K).ravel()] = s.ravel()
    return codes_out, sf_out


# ----------------------------------------------------------------------------------------------
# synthetic workloads (token counts: Zipf(alpha) over experts; values: N(0,1) with sparse outliers)
# ----------------------------------------------------------------------------------------------
def zipf_counts(T: int, E: int, alpha: float = 1.2, seed: int = 0) -> np.ndarray:
    rng = np.random.default_rng(seed)
    p = np.arange(1, E + 1, dtype=np.float64) ** -alpha
    p /= p.sum()
    counts = rng.multinomial(T, p)
    rng.shuffle(counts)
    return counts.astype(np.int64)


def offsets_from_counts(counts, N: int, K: int):
    counts = np.asarray(counts, dtype=np.int64)
    E = len(counts)
    eo = np.zeros(E, dtype=np.int32)
    bo = np.zeros(E, dtype=np.int32)
    eo[1:] = np.cumsum(counts)[:-1]
    bo[1:] = np.cumsum(align128(counts))[:-1]
    ps = np.stack([counts, np.full(E, N), np.full(E, K)], axis=1).astype(np.int32)
    return ps, eo, bo, int(align128(counts).sum())


def edge_case_rows_bf16(K: int, seed: int = 0) -> np.ndarray:
    """bf16 bit patterns [R,K] whose 32-blocks hit every special branch of the scale derivation:
    all-zero / signed-zero blocks, amax = 1.75*2^n (the ulp-sensitive significand of amax/448), exact powers of
    two, NaN / inf members, all-NaN blocks, bf16 subnormals, values at the e4m3 saturation and tie points."""
    rng = np.random.default_rng(seed)
    nb = K // SF_BLOCK
    rows = []

    def f32_to_bf16_bits(a):
        b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
        return ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)

    base = f32_to_bf16_bits(rng.standard_normal((16, K)))
    # row 0: zeros / negative zeros
    r = np.zeros(K, dtype=np.uint16); r[1::2] = 0x8000; rows.append(r)
    # rows with amax = 1.75 * 2^n for a sweep of n, one block each
    for n0 in range(-20, 20, nb if nb < 40 else 40):
        r = base[1].copy().reshape(nb, 32)
        for b in range(nb):
            n = n0 + b
            r[b] = f32_to_bf16_bits(rng.uniform(-1, 1, 32) * 2.0 ** n)
            r[b, rng.integers(32)] = f32_to_bf16_bits(np.array([1.75 * 2.0 ** n]))[0]
        rows.append(r.reshape(-1))
    # exact powers of two and 448 * 2^n as amax
    r = base[2].copy().reshape(nb, 32)
    for b in range(nb):
        n = (b % 30) - 15
        r[b] = f32_to_bf16_bits(rng.uniform(-0.5, 0.5, 32) * 2.0 ** n)
        r[b, 0] = f32_to_bf16_bits(np.array([(448.0 if b % 2 else 1.0) * 2.0 ** n]))[0]
    rows.append(r.reshape(-1))
    # NaN / inf members, all-NaN block, all-inf block
    r = base[3].copy().reshape(nb, 32)
    r[0, 3] = 0x7FC0; r[0, 4] = 0xFFC0
    if nb > 1: r[1, 5] = 0x7F80
    if nb > 2: r[2, 6] = 0xFF80; r[2, 7] = 0x7FC0
    if nb > 3: r[3, :] = 0x7FC0
    if nb > 4: r[4, :] = 0x7F80
    rows.append(r.reshape(-1))
    # bf16 subnormals and tiny normals (scale exponent clamps at 0), huge values
    r = base[4].copy().reshape(nb, 32)
    r[0, :] = rng.integers(0, 0x80, 32).astype(np.uint16)
    if nb > 1: r[1, :] = rng.integers(0x80, 0x400, 32).astype(np.uint16)
    if nb > 2: r[2, :] = rng.integers(0x7F00, 0x7F80, 32).astype(np.uint16)
    if nb > 3: r[3, :] = 0; r[3, 9] = 0x0001
    rows.append(r.reshape(-1))
    # e4m3 tie points: values k/16 * amax with amax = 448 exactly -> scaled values on half-ulp boundaries
    r = base[5].copy().reshape(nb, 32)
    ties = np.array([448, 464, 480, 432, 416, 15.5, 14.5, 13.5, 1.0625, 1.1875, 0.001953125 * 3, 0.0009765625,
                     0.0029296875, 2 ** -10, 2 ** -9, 2 ** -8, 17, 18, 19, 20, 21, 22, 23, 25, 27, 29, 31, 33, 35, 37,
                     39, 41], dtype=np.float32)
    r[0, :] = f32_to_bf16_bits(ties * np.where(np.arange(32) % 2, -1, 1))
    rows.append(r.reshape(-1))
    rows.extend(list(base[6:]))
    return np.stack(rows).astype(np.uint16)
