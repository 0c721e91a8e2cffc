"""CPU tests of the oracle: it must reproduce the golden fixtures that pin it.

* tests/golden/ref_quant_*.npz, ref_gemm_*.npz, ref_quant_digests.json: outputs of the reference's own SM100 kernels
  (run on a B200 by tests/golden/make_reference_fixtures.py);
* tests/golden/ref_blockwise_*.npz: outputs of the reference's own torch quantisers / dequant-matmul path
  (run on the CPU by tests/golden/make_blockwise_fixtures.py);
* tests/golden/b200_probe.json: the bit pattern of rcp.approx.ftz.f32(448) measured on a B200.
"""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import grouped_gemm_oracle as G
from oracle import mxfp8_quant_oracle as Q
from tests import _cases as C

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_rcp_constant_matches_hardware_probe():
    probe = json.loads((GOLDEN / "b200_probe.json").read_text())
    assert int(probe["rcp448_bits"], 16) == Q.RCP_448_BITS_DEFAULT
    assert probe["pow2_mismatches"] == 0            # rcp.approx.ftz is exact on powers of two
    assert int(probe["rcp_2m127"], 16) == 0x7F800000 and int(probe["rcp_2p127"], 16) == 0


@pytest.mark.parametrize("name", ["edge_bf16", "ragged_bf16", "ragged_fp16"])
def test_quant_oracle_reproduces_reference_kernel(name):
    z = np.load(GOLDEN / f"ref_quant_{name}.npz")
    x_bits, is_bf16 = z["x_bits"], bool(z["is_bf16"])
    counts = z["ps"][:, 0]
    codes, sf = C.oracle_quant(x_bits, is_bf16, counts)
    assert np.array_equal(codes, z["codes"]), "e4m3 codes differ from the reference kernel"
    idx = C.valid_sf_index(counts, z["bo"], x_bits.shape[1])
    assert np.array_equal(sf[idx], z["sf"][idx]), "UE8M0 scale bytes differ from the reference kernel"


def test_quant_oracle_special_values():
    K = 128
    x = np.zeros((6, K), dtype=np.uint16)
    x[1, :] = 0x8000                    # -0
    x[2, :32] = 0x7FC0                  # all-NaN block
    x[3, 0] = 0x7F80                    # +inf member
    x[4, 0] = 0x43E0                    # 448.0 -> scale exponent 127, code 0x7E
    x[5, 0] = 0x0001                    # smallest bf16 subnormal
    codes, sf = Q.quantize_rows(x, True)
    assert (codes[0] == 0).all() and (sf[0] == 0).all()
    assert (codes[1] == 0x80).all() and (sf[1] == 0).all()            # sign of zero is kept
    assert sf[2, 0] == 0xFF and (codes[2, :32] == 0x7F).all()
    assert sf[3, 0] == 0xFE and codes[3, 0] == 0x7F and (codes[3, 1:32] == 0).all()   # inf * 0 = NaN, finite * 0 = 0
    assert sf[4, 0] == 127 and codes[4, 0] == 0x7E
    assert sf[5, 0] == 0 and codes[5, 0] == 0x7E                      # scale underflows: inverse is +inf, saturates


def test_swizzle_roundtrip_and_formula():
    rng = np.random.default_rng(0)
    for m, K in [(1, 128), (127, 256), (128, 384), (300, 7168)]:
        sf = rng.integers(0, 255, size=(m, K // 32), dtype=np.uint8)
        flat = Q.swizzle_sf(sf, K, fill=0)
        assert flat.size == Q.align128(m) * (K // 32)
        assert np.array_equal(Q.unswizzle_sf(flat, m, K), sf)
    # one hand-computed offset: row 200, K block 9, K = 512 (4 K tiles): atom (1, 2) -> (1*4+2)*512; row 200%32=8,
    # (200%128)/32=2; kb%4=1
    off = Q.sf_swizzled_offsets(256, 512)[200, 9]
    assert off == (1 * 4 + 2) * 512 + 8 * 16 + 2 * 4 + 1


def test_zipf_workload_statistics():
    c = Q.zipf_counts(32768, 256, 1.2, 0)
    assert c.sum() == 32768 and c.max() == 8409 and int(Q.align128(c).sum()) == 56960
    assert sorted(c)[-5:] == [1185, 1552, 2222, 3608, 8409]
    c4 = Q.zipf_counts(512, 256, 1.2, 0)
    assert c4.sum() == 512 and (c4 == 0).sum() == 147 and c4.max() == 117


@pytest.mark.parametrize("name", ["small_bf16", "small_fp16"])
def test_gemm_oracle_reproduces_reference_kernel(name):
    z = np.load(GOLDEN / f"ref_gemm_{name}.npz")
    out_dtype = torch.bfloat16 if bool(z["out_is_bf16"]) else torch.float16
    d = G.mxfp8_grouped_mm(torch.from_numpy(z["a_codes"]), torch.from_numpy(z["w_codes"]), torch.from_numpy(z["sfa"]),
                           torch.from_numpy(z["sfb"]), z["ps"], z["eo"], z["bo"], out_dtype=out_dtype)
    ref = torch.from_numpy(z["d_bits"].view(np.int16)).view(out_dtype)
    for e in range(len(z["ps"])):
        m, off = int(z["ps"][e][0]), int(z["eo"][e])
        if m == 0:
            continue
        rel, cos = G.rel_err_and_cosine(d[off:off + m].float(), ref[off:off + m].float())
        assert rel <= 1e-2 and cos >= 0.9999, (e, rel, cos)
        assert G.calc_diff(d[off:off + m], ref[off:off + m]) < 1e-3


@pytest.mark.parametrize("name", ["c1_bf16", "small_fp16"])
def test_blockwise_oracle_reproduces_reference_torch_path(name):
    z = np.load(GOLDEN / f"ref_blockwise_{name}.npz")
    dtype = torch.bfloat16 if bool(z["is_bf16"]) else torch.float16
    N, K = int(z["N"]), int(z["K"])
    for e, m in enumerate(z["counts"]):
        if m == 0:
            continue
        a = torch.from_numpy(z[f"a_{e}"].view(np.int16)).view(dtype)
        w = torch.from_numpy(z[f"w_{e}"].view(np.int16)).view(dtype)
        a_q, sa = G.per_token_cast_to_fp8(a)
        w_q, sb = G.per_block_cast_to_fp8(w)
        assert np.array_equal(a_q.view(torch.uint8).numpy(), z[f"aq_{e}"])
        assert np.array_equal(w_q.view(torch.uint8).numpy(), z[f"wq_{e}"])
        assert np.array_equal(sa.float().numpy(), z[f"sa_{e}"]) and np.array_equal(sb.float().numpy(), z[f"sb_{e}"])
        ps = np.array([[m, N, K]], dtype=np.int32)
        d = G.fp8_blockwise_grouped_mm(a_q.view(torch.uint8), w_q.view(torch.uint8).view(1, N, K), sa.float(),
                                       sb.float().view(1, N // 128, K // 128), ps, [0], out_dtype=dtype)
        ref = torch.from_numpy(z[f"d_{e}"].view(np.int16)).view(dtype)
        rel, cos = G.rel_err_and_cosine(d.float(), ref.float())
        assert rel <= 1e-3 and cos >= 0.99999, (e, rel, cos)    # same math, fp32 summation order may differ
