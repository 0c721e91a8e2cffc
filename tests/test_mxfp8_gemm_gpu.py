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


def test_mm_more_experts_than_the_shared_memory_tables_hold():
    """Beyond 256 experts only part of the per-expert tables fits behind the item prefix in shared memory (300 experts:
    the first 241); the others are read from global memory.  All three buckets have experts on both sides."""
    counts = [(7 * e) % 41 for e in range(300)]
    counts[3], counts[250], counts[280], counts[299] = 200, 150, 70, 33
    inp = C.mxfp8_gemm_inputs(counts, 256, 256, seed=21)
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


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("counts,N,K", [
    ([5, 0, 130, 64, 1, 257], 256, 384),      # all three buckets; the CTA-pair kernel holds its chunks before storing
    ([193, 385, 577, 64], 256, 256),          # two K blocks: the CTA-pair kernel stores each chunk as it is read
    ([1000, 20], 128, 128),                   # one K block, odd number of weight tiles
    ([400, 33, 7], 512, 768),
])
def test_scatter_epilogue_equals_dense_output(counts, N, K, out_dtype):
    """es_b200_mxfp8_grouped_mm_scatter with a random permutation of the rows into one local buffer: row r of the dense
    result must arrive, bit for bit, in row perm[r] (same kernels, same arithmetic, only the epilogue's destination
    differs); rows of the buffer that no output row maps to stay untouched."""
    import ctypes
    from expert_specialization_moe_b200 import _cabi
    inp = C.mxfp8_gemm_inputs(counts, N, K, seed=3)
    dense = C.run_mxfp8_mm_op(inp, out_dtype)
    dev = torch.device("cuda")
    E = len(counts)
    T = inp["a_codes"].shape[0]
    slots = T + 5
    a = torch.from_numpy(inp["a_codes"]).to(dev)
    w = torch.from_numpy(inp["w_codes"]).to(dev)
    sfa = torch.from_numpy(inp["sfa"]).to(dev)
    sfb = torch.from_numpy(inp["sfb"]).to(dev)
    ps, eo, bo = (torch.from_numpy(inp[k]).to(dev) for k in ("ps", "eo", "bo"))
    g = torch.Generator(device="cpu")
    g.manual_seed(7)
    perm = torch.randperm(slots, generator=g)[:T].to(torch.int32)
    meta = torch.stack([torch.zeros_like(perm), perm], dim=1).contiguous().to(dev)
    out = torch.full((slots, N), 7.0, dtype=out_dtype, device=dev)
    table = (ctypes.c_void_p * 1)(out.data_ptr())
    stream = torch.cuda.current_stream(dev).cuda_stream
    scratch = _cabi.grouped_mm_scratch(dev, stream)
    dt = _cabi.BF16 if out_dtype == torch.bfloat16 else _cabi.FP16
    _cabi.check(_cabi.load().es_b200_mxfp8_grouped_mm_scatter(
        a.data_ptr(), w.data_ptr(), sfa.data_ptr(), sfb.data_ptr(), dt, ps.data_ptr(), eo.data_ptr(), bo.data_ptr(),
        E, T, N, K, sfa.numel() // (K // 32), meta.data_ptr(), table, 1, slots, scratch.data_ptr(), scratch.numel(),
        stream))
    torch.cuda.synchronize()
    rc, raw = C.device_status()
    assert rc == 0, f"device status {raw:#x}"
    out = out.cpu()
    valid = torch.zeros(T, dtype=torch.bool)
    for e, m in enumerate(counts):
        valid[int(inp["eo"][e]):int(inp["eo"][e]) + m] = True
    rows = perm.long()[valid]
    assert torch.equal(out[rows].view(torch.int16), dense[valid].view(torch.int16))
    untouched = torch.ones(slots, dtype=torch.bool)
    untouched[rows] = False
    assert bool((out[untouched] == 7.0).all())
