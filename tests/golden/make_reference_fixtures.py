"""Generate the golden fixtures in this directory by running the REFERENCE's own SM100 kernels on a B200.

    oracle/build_ref.sh <reference checkout>        # builds oracle/_ref/libes_reference.so (CPU box, no GPU needed)
    python tests/golden/make_reference_fixtures.py [--out DIR]   # on a machine with a B200; default DIR = here

The reference holds no golden vectors for these ops, so its compiled kernels are the only ground truth for the
bit-level contract (e4m3 codes, UE8M0 scale bytes, swizzled placement) and for the bf16 GEMM results.  Inputs are
seeded numpy data; outputs of the reference's `es_sm100_mxfp8_blockscaled_grouped_quant` and
`es_sm100_mxfp8_blockscaled_grouped_mm` are stored next to them as compressed .npz files (a few hundred KB).
Nothing from this repository's own kernels is involved in producing the fixtures.
"""
from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
OUT = Path(sys.argv[sys.argv.index("--out") + 1]) if "--out" in sys.argv else HERE
sys.path.insert(0, str(ROOT))
from oracle import mxfp8_quant_oracle as Q  # noqa: E402  (input generators only)

SF_FILL = 0xCD   # scale buffer is pre-filled with this so that bytes the reference never writes are recognisable


def load_reference():
    lib = ROOT / "oracle" / "_ref" / "libes_reference.so"
    torch.ops.load_library(str(lib))
    return torch.ops.expert_specialization


def f32_to_bf16_bits(a):
    b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


def run_ref_quant(ref, x_bits, is_bf16, ps, eo, bo, sf_rows):
    dev = "cuda"
    dt = torch.bfloat16 if is_bf16 else torch.float16
    x = torch.from_numpy(x_bits.view(np.int16)).to(dev).view(dt)
    T, K = x.shape
    codes = torch.zeros((T, K), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    sf = torch.full((sf_rows, K // 32), SF_FILL, dtype=torch.uint8, device=dev)
    ref.es_sm100_mxfp8_blockscaled_grouped_quant(
        x, torch.from_numpy(ps).to(dev), torch.from_numpy(eo).to(dev), torch.from_numpy(bo).to(dev), codes, sf)
    torch.cuda.synchronize()
    return codes.view(torch.uint8).cpu().numpy(), sf.cpu().numpy().reshape(-1)


def quant_case(ref, name, x_bits, is_bf16, counts):
    K = x_bits.shape[1]
    ps, eo, bo, sf_rows = Q.offsets_from_counts(counts, 0, K)
    assert sum(counts) == x_bits.shape[0]
    codes, sf = run_ref_quant(ref, x_bits, is_bf16, ps, eo, bo, sf_rows)
    np.savez_compressed(OUT / f"ref_quant_{name}.npz", x_bits=x_bits, is_bf16=np.array(is_bf16), ps=ps, eo=eo, bo=bo,
                        sf_rows=np.array(sf_rows), codes=codes, sf=sf, sf_fill=np.array(SF_FILL))
    print(f"wrote ref_quant_{name}.npz  T={x_bits.shape[0]} K={K} E={len(counts)}")


def gemm_case(ref, name, counts, N, K, out_dtype, seed):
    """Inputs quantised by the reference quant op (A rows and, with the transposed problem list, the weights —
    exactly as test/test_es_sm100_mxfp8_blockscaled_grouped_quant.py:53,87-96 does), then the reference GEMM."""
    dev = "cuda"
    rng = np.random.default_rng(seed)
    E = len(counts)
    T = int(sum(counts))
    a_bits = f32_to_bf16_bits(rng.standard_normal((T, K)))
    w_bits = f32_to_bf16_bits(rng.standard_normal((E * N, K)) * 0.05)
    ps, eo, bo, sfa_rows = Q.offsets_from_counts(counts, N, K)
    a_codes, sfa = run_ref_quant(ref, a_bits, True, ps, eo, bo, sfa_rows)
    wps, weo, wbo, sfb_rows = Q.offsets_from_counts([N] * E, 0, K)
    w_codes, sfb = run_ref_quant(ref, w_bits, True, wps, weo, wbo, sfb_rows)
    # (padding rows of sfa hold whatever the reference left there; they only feed output rows that are never stored)
    a_t = torch.from_numpy(a_codes).to(dev).view(torch.float8_e4m3fn)
    b_t = torch.from_numpy(w_codes).to(dev).view(torch.float8_e4m3fn).view(E, N, K).transpose(1, 2)
    d = torch.zeros((T, N), dtype=out_dtype, device=dev)
    ref.es_sm100_mxfp8_blockscaled_grouped_mm(
        a_t, b_t, torch.from_numpy(sfa).to(dev), torch.from_numpy(sfb).to(dev), d,
        torch.from_numpy(ps).to(dev), torch.from_numpy(eo).to(dev), torch.from_numpy(bo).to(dev))
    torch.cuda.synchronize()
    np.savez_compressed(OUT / f"ref_gemm_{name}.npz", a_codes=a_codes, sfa=sfa, w_codes=w_codes.reshape(E, N, K),
                        sfb=sfb, ps=ps, eo=eo, bo=bo, d_bits=d.view(torch.int16).cpu().numpy().view(np.uint16),
                        out_is_bf16=np.array(out_dtype == torch.bfloat16))
    print(f"wrote ref_gemm_{name}.npz  counts={list(counts)} N={N} K={K}")


def big_quant_digest(ref, T, K, E, seed):
    """Full-size run (the grouped-quant benchmark shape): store only SHA-256 digests of the reference's outputs."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((T, K), dtype=np.float32)
    x *= np.where(rng.random((T, K), dtype=np.float32) < 0.01, np.float32(50.0), np.float32(1.0))
    x_bits = f32_to_bf16_bits(x)
    counts = Q.zipf_counts(T, E, 1.2, seed)
    ps, eo, bo, sf_rows = Q.offsets_from_counts(counts, 0, K)
    codes, sf = run_ref_quant(ref, x_bits, True, ps, eo, bo, sf_rows)
    h_codes = hashlib.sha256(codes.tobytes()).hexdigest()
    valid = np.concatenate([int(bo[e]) * (K // 32) + Q.sf_swizzled_offsets(int(counts[e]), K).ravel()
                            for e in range(E) if counts[e] > 0])
    h_sf = hashlib.sha256(sf[valid].tobytes()).hexdigest()
    return {"T": T, "K": K, "E": E, "seed": seed, "codes_sha256": h_codes, "sf_valid_sha256": h_sf,
            "input_sha256": hashlib.sha256(x_bits.tobytes()).hexdigest()}


def main():
    assert torch.cuda.is_available(), "needs a B200"
    ref = load_reference()
    OUT.mkdir(parents=True, exist_ok=True)
    rng = np.random.default_rng(1234)

    # 1. edge cases, one expert (bf16): every special branch of the scale derivation
    edge = Q.edge_case_rows_bf16(512, seed=0)
    quant_case(ref, "edge_bf16", edge, True, [edge.shape[0]])

    # 2. ragged experts incl. empty ones (bf16), N(0,1) with 1% x50 outliers
    counts = [1, 127, 128, 129, 0, 300, 0, 17]
    T = sum(counts)
    x = rng.standard_normal((T, 256)).astype(np.float32)
    x *= np.where(rng.random((T, 256)) < 0.01, 50.0, 1.0).astype(np.float32)
    quant_case(ref, "ragged_bf16", f32_to_bf16_bits(x), True, counts)

    # 3. fp16 input, incl. fp16 subnormals / max values
    counts = [33, 0, 200, 5]
    T = sum(counts)
    xh = (rng.standard_normal((T, 384)) * 3).astype(np.float16)
    xh[0, :32] = np.float16(6e-8)
    xh[1, :32] = np.float16(65504.0)
    xh[2, :64] = 0
    xh[3, 5] = np.float16(np.nan)
    xh[4, 40:48] = np.float16(np.inf)
    quant_case(ref, "ragged_fp16", xh.view(np.uint16), False, counts)

    # 4. grouped GEMM outputs of the reference on small problems
    gemm_case(ref, "small_bf16", [5, 0, 130, 64, 1, 257], 256, 384, torch.bfloat16, 7)
    gemm_case(ref, "small_fp16", [16, 3, 0, 129], 128, 128, torch.float16, 8)

    # 5. digests at the full benchmark shape
    digests = [big_quant_digest(ref, 32768, 7168, 256, 0)]
    (OUT / "ref_quant_digests.json").write_text(json.dumps(digests, indent=1))
    print("wrote ref_quant_digests.json", digests)


if __name__ == "__main__":
    main()
