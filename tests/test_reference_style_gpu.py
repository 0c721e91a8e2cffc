"""The reference's own three test programs, re-stated for this library (same parametrisation, same acceptance
criterion calc_diff < 1e-3 against the UNQUANTISED matmul):

* test/test_es_grouped_gemm.py:101-202            -> test_fp8_blockwise_scaled_grouped_mm
* test/test_es_sm100_mxfp8_blockscaled_grouped_quant.py:22-114 -> test_mxfp8_quant_then_grouped_mm (A and, with the
  transposed problem list, the weights are quantised by the grouped quant op, then multiplied by the grouped GEMM)
* test/test_es_sm100_mxfp8_blockscaled_grouped_gemm.py:23-84 uses TensorRT-LLM's quantiser for its inputs; here the
  inputs come from this library's quant op, whose output is bit-identical to the reference's quant kernel.
Shapes are drawn from seeded generators (the reference draws n, k in 128*[1,64] and m in [1,256] / [1,4096])."""
import random

import pytest
import torch

from oracle.grouped_gemm_oracle import calc_diff
from tests import _cases as C

pytestmark = pytest.mark.gpu


def _align(v, a=128):
    return (v + a - 1) // a * a


@pytest.mark.parametrize("num_experts", [8, 16, 32, 64, 128])
@pytest.mark.parametrize("out_dtype", [torch.half, torch.bfloat16])
def test_fp8_blockwise_scaled_grouped_mm(num_experts, out_dtype):
    rnd = random.Random(num_experts * 7 + (1 if out_dtype == torch.half else 0))
    n_g, k_g = rnd.randint(1, 24) * 128, rnd.randint(1, 24) * 128       # the reference draws up to 64*128
    counts = [rnd.randint(1, 256) for _ in range(num_experts)]
    inp = C.fp8_blockwise_inputs(counts, n_g, k_g, seed=num_experts, dtype=out_dtype)
    d = C.run_fp8_blockwise_op(inp, out_dtype)
    dev = "cuda"
    for g in range(num_experts):
        off, m = int(inp["eo"][g]), counts[g]
        baseline = (inp["a"][off:off + m].to(dev).float() @ inp["w"][g].to(dev).float().t()).cpu()
        diff = calc_diff(d[off:off + m], baseline)
        assert diff < 0.001, f"expert {g}: m={m} n={n_g} k={k_g} diff={diff:.5f}"


@pytest.mark.parametrize("num_experts,out_dtype", [(8, torch.bfloat16), (8, torch.float16), (16, torch.bfloat16),
                                                   (16, torch.float16)])
def test_mxfp8_quant_then_grouped_mm(num_experts, out_dtype):
    from expert_specialization_moe_b200 import (es_sm100_mxfp8_blockscaled_grouped_mm as grouped_mm,
                                                es_sm100_mxfp8_blockscaled_grouped_quant as grouped_quant)
    rnd = random.Random(42 + num_experts)
    torch.manual_seed(42)
    dev = "cuda"
    n_g, k_g = rnd.randint(1, 24) * 128, rnd.randint(1, 24) * 128
    eo, aux_eo, a_bo, b_bo, ps, aux_ps, a_list, b_list, ref = [], [], [], [], [], [], [], [], []
    off = aoff = abo = bbo = 0
    for g in range(num_experts):
        m_g = rnd.randint(1, 1024)                                      # the reference draws up to 4096
        eo.append(off); off += m_g
        aux_eo.append(aoff); aoff += n_g
        a_bo.append(abo); abo += _align(m_g)
        b_bo.append(bbo); bbo += n_g
        ps.append([m_g, n_g, k_g]); aux_ps.append([n_g, m_g, k_g])
        a = torch.normal(0.0, 1.0, size=(m_g, k_g), device=dev, dtype=out_dtype)
        b = torch.normal(0.0, 1.0, size=(n_g, k_g), device=dev, dtype=out_dtype)
        a_list.append(a); b_list.append(b); ref.append(a.float() @ b.float().T)
    a, b = torch.concat(a_list, 0), torch.concat(b_list, 0)
    t32 = lambda v: torch.tensor(v, device=dev, dtype=torch.int32)
    _ps, _aux_ps, _eo, _aux_eo, _a_bo, _b_bo = t32(ps), t32(aux_ps), t32(eo), t32(aux_eo), t32(a_bo), t32(b_bo)
    a_quant = torch.zeros(a.shape, device=dev, dtype=torch.uint8).view(torch.float8_e4m3fn)
    a_sf = torch.zeros((abo, k_g // 32), dtype=torch.uint8, device=dev)
    b_quant = torch.zeros(b.shape, device=dev, dtype=torch.uint8).view(torch.float8_e4m3fn)
    b_sf = torch.zeros((num_experts, n_g, k_g // 32), dtype=torch.uint8, device=dev)
    grouped_quant(a, _ps, _eo, _a_bo, a_quant, a_sf)
    grouped_quant(b, _aux_ps, _aux_eo, _b_bo, b_quant, b_sf)
    b_q = b_quant.view(num_experts, n_g, k_g).transpose(1, 2)
    b_s = b_sf.view(num_experts, n_g, k_g // 32).transpose(1, 2)
    d = torch.empty((off, n_g), device=dev, dtype=out_dtype)
    grouped_mm(d, a_quant, b_q, a_sf, b_s, _ps, _eo, _a_bo)
    torch.cuda.synchronize()
    for g in range(num_experts):
        actual = d[eo[g]: eo[g] + ps[g][0]]
        diff = calc_diff(actual.float().cpu(), ref[g].cpu())
        assert diff < 0.001, f"expert {g}: m={ps[g][0]} n={n_g} k={k_g} diff={diff:.5f}"
    rc, raw = C.device_status()
    assert rc == 0, raw
