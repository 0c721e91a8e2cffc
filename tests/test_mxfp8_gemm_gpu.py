"""GPU parity of the MXFP8 block-scaled grouped GEMM (ops.py -> C ABI -> tcgen05 kernel).

Oracle: dequantise (code * 2^(sf-127)) and multiply in fp32 on the CPU.  Tolerances (floating point, stated by the
build target): relative error <= 1e-2 and cosine >= 0.9999 per expert, plus the reference tests' own criterion
calc_diff < 1e-3.  Also compared with outputs of the reference's CUTLASS kernel stored in tests/golden."""
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import grouped_gemm_oracle as G
from tests import _cases as C

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"
REL_TOL, COS_TOL, DIFF_TOL = 1e-2, 0.9999, 1e-3


def _check_against_oracle(inp, d, out_dtype):
    ref = G.mxfp8_grouped_mm(torch.from_numpy(inp["a_codes"]), torch.from_numpy(inp["w_codes"]),
                             torch.from_numpy(inp["sfa"]), torch.from_numpy(inp["sfb"]), inp["ps"], inp["eo"],
                             inp["bo"], out_dtype=out_dtype)
    for e in range(len(inp["ps"])):
        m, off = int(inp["ps"][e][0]), int(inp["eo"][e])
        if m == 0:
            continue
        x, y = d[off:off + m].float(), ref[off:off + m].float()
        rel, cos = G.rel_err_and_cosine(x, y)
        assert rel <= REL_TOL and cos >= COS_TOL, f"expert {e} (m={m}): rel={rel:.3e} cos={cos:.6f}"
        assert G.calc_diff(x, y) < DIFF_TOL
    rc, raw = C.device_status()
    assert rc == 0, f"device status {raw:#x}"


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("counts,N,K", [
    ([1], 128, 128),
    ([16], 128, 256),
    ([128], 256, 128),
    ([5, 0, 130, 64, 1, 257], 256, 384),
    ([0, 1, 3, 7, 16, 64, 128, 293], 1024, 512),
    ([0, 0, 0], 128, 128),
    ([17, 33, 65, 129], 384, 1152),
    ([193, 385, 577, 64], 256, 256),      # token tiles that start mid scale-atom
    ([1000], 128, 128),                   # odd number of 128-wide weight tiles: one CTA of the pair idles
    ([200, 9], 384, 256),
])
def test_mm_matches_oracle(counts, N, K, out_dtype):
    inp = C.mxfp8_gemm_inputs(counts, N, K, seed=N + K + len(counts))
    if sum(counts) == 0:
        inp["a_codes"] = np.zeros((4, K), dtype=np.uint8)    # buffer rows that belong to no expert
        d = C.run_mxfp8_mm_op(inp, out_dtype, fill=7.0)
        assert (d == 7.0).all()
        return
    d = C.run_mxfp8_mm_op(inp, out_dtype)
    _check_against_oracle(inp, d, out_dtype)


def test_mm_many_small_experts():
    from oracle import mxfp8_quant_oracle as Q
    counts = list(Q.zipf_counts(512, 256, 1.2, 0))
    inp = C.mxfp8_gemm_inputs(counts, 256, 512, seed=3)
    d = C.run_mxfp8_mm_op(inp)
    _check_against_oracle(inp, d, torch.bfloat16)


def test_mm_does_not_write_outside_experts():
    counts = [3, 20]
    inp = C.mxfp8_gemm_inputs(counts, 128, 128, seed=9)
    # leave a gap of 5 rows between the two experts and 4 rows at the end
    T = 3 + 5 + 20 + 4
    a = np.zeros((T, 128), dtype=np.uint8)
    a[0:3] = inp["a_codes"][0:3]
    a[8:28] = inp["a_codes"][3:23]
    inp2 = dict(inp, a_codes=a, eo=np.array([0, 8], dtype=np.int32))
    d = C.run_mxfp8_mm_op(inp2, fill=3.0)
    assert (d[3:8] == 3.0).all() and (d[28:] == 3.0).all()
    ref = C.run_mxfp8_mm_op(inp)
    assert torch.equal(d[0:3], ref[0:3]) and torch.equal(d[8:28], ref[3:23])


@pytest.mark.parametrize("name", ["small_bf16", "small_fp16"])
def test_mm_matches_reference_kernel_fixture(name):
    f = GOLDEN / f"ref_gemm_{name}.npz"
    z = np.load(f)
    out_dtype = torch.bfloat16 if bool(z["out_is_bf16"]) else torch.float16
    inp = {k: z[k] for k in ("a_codes", "sfa", "w_codes", "sfb", "ps", "eo", "bo")}
    d = C.run_mxfp8_mm_op(inp, out_dtype)
    ref = torch.from_numpy(z["d_bits"].view(np.int16)).view(out_dtype)
    for e in range(len(inp["ps"])):
        m, off = int(inp["ps"][e][0]), int(inp["eo"][e])
        if m == 0:
            continue
        rel, cos = G.rel_err_and_cosine(d[off:off + m].float(), ref[off:off + m].float())
        assert rel <= REL_TOL and cos >= COS_TOL, f"expert {e}: rel={rel:.3e} cos={cos:.6f}"
    # both kernels accumulate the same fp32 products; in practice the outputs agree to the last bf16/fp16 bit
    # almost everywhere -- report how many do not
    frac = float((d.view(torch.int16) != ref.view(torch.int16)).float().mean())
    assert frac < 0.05, f"{frac:.4f} of outputs differ from the reference kernel in the last bit"
    _check_against_oracle(inp, d, out_dtype)
