"""GPU parity of the MXFP8 grouped quantisation (through ops.py -> C ABI) against the CPU oracle and against the
golden fixtures produced by the reference's own kernel.  Bit-exact: codes everywhere, scale bytes on valid rows,
zeros on the padding rows."""
import hashlib
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import mxfp8_quant_oracle as Q
from tests import _cases as C

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def _compare(x_bits, is_bf16, counts):
    codes, sf, ps, eo, bo = C.run_quant_op(x_bits, is_bf16, counts)
    ocodes, osf = C.oracle_quant(x_bits, is_bf16, counts)
    assert np.array_equal(codes, ocodes), f"codes differ at {np.argwhere(codes != ocodes)[:5]}"
    assert np.array_equal(sf, osf), f"scale bytes differ at {np.argwhere(sf != osf)[:5]}"


@pytest.mark.parametrize("is_bf16", [True, False])
@pytest.mark.parametrize("counts,K", [
    ([1], 128), ([0, 0, 5], 128), ([127, 128, 129], 256), ([8, 0, 300, 17, 1, 1, 64], 384),
    ([513], 1152), ([3] * 40, 7168), ([0], 128),
])
def test_quant_matches_oracle(counts, K, is_bf16):
    x = C.activations_bits(sum(counts), K, seed=sum(counts) + K, is_bf16=is_bf16)
    if sum(counts) == 0:
        x = np.full((1, K), 0x3F80, dtype=np.uint16)   # an all-empty problem list must leave the outputs untouched
        codes, sf, *_ = C.run_quant_op(x, is_bf16, [0])
        assert not codes.any()
        return
    _compare(x, is_bf16, counts)


def test_quant_edge_values():
    x = Q.edge_case_rows_bf16(512, seed=0)
    _compare(x, True, [x.shape[0]])
    _compare(x, True, [7, 0, x.shape[0] - 7])


def test_quant_many_experts():
    counts = list(Q.zipf_counts(4096, 1024, 1.2, 3))
    _compare(C.activations_bits(4096, 256, 5), True, counts)


def test_quant_rows_outside_experts_untouched():
    """expert ranges need not cover the buffer: rows that belong to no expert keep their previous contents."""
    import torch
    from expert_specialization_moe_b200 import es_sm100_mxfp8_blockscaled_grouped_quant as quant
    K = 256
    x_bits = C.activations_bits(64, K, 11)
    x = C.bits_to_tensor(x_bits, True, "cuda")
    ps = torch.tensor([[10, 0, K], [5, 0, K]], dtype=torch.int32, device="cuda")
    eo = torch.tensor([4, 40], dtype=torch.int32, device="cuda")
    bo = torch.tensor([0, 128], dtype=torch.int32, device="cuda")
    codes = torch.full((64, K), 0x55, dtype=torch.uint8, device="cuda")
    sf = torch.full((256, K // 32), 0xCD, dtype=torch.uint8, device="cuda")
    quant(x, ps, eo, bo, codes, sf)
    torch.cuda.synchronize()
    c = codes.cpu().numpy()
    oc, osf = Q.quantize_rows(x_bits, True)
    touched = np.zeros(64, dtype=bool); touched[4:14] = True; touched[40:45] = True
    assert np.array_equal(c[touched], oc[touched])
    assert (c[~touched] == 0x55).all()
    s = sf.cpu().numpy().reshape(-1)
    assert np.array_equal(Q.unswizzle_sf(s[: 128 * (K // 32)], 10, K), osf[4:14])
    assert np.array_equal(Q.unswizzle_sf(s[128 * (K // 32):], 5, K), osf[40:45])


@pytest.mark.parametrize("name", ["edge_bf16", "ragged_bf16", "ragged_fp16"])
def test_quant_matches_reference_fixture(name):
    f = GOLDEN / f"ref_quant_{name}.npz"
    if not f.exists():
        pytest.skip("fixture not generated yet")
    z = np.load(f)
    counts = z["ps"][:, 0]
    codes, sf, ps, eo, bo = C.run_quant_op(z["x_bits"], bool(z["is_bf16"]), counts)
    assert np.array_equal(codes, z["codes"])
    idx = C.valid_sf_index(counts, bo, z["x_bits"].shape[1])
    assert np.array_equal(sf[idx], z["sf"][idx])


def test_quant_full_size_digest_matches_reference():
    """The benchmark shape (T=32768, K=7168, E=256, Zipf counts): SHA-256 of all codes and of the valid scale bytes
    equals the digest of the reference kernel's output on the same seeded input."""
    f = GOLDEN / "ref_quant_digests.json"
    if not f.exists():
        pytest.skip("fixture not generated yet")
    for d in json.loads(f.read_text()):
        T, K, E, seed = d["T"], d["K"], d["E"], d["seed"]
        x_bits = C.activations_bits(T, K, seed)
        assert hashlib.sha256(x_bits.tobytes()).hexdigest() == d["input_sha256"]
        counts = Q.zipf_counts(T, E, 1.2, seed)
        codes, sf, ps, eo, bo = C.run_quant_op(x_bits, True, counts)
        assert hashlib.sha256(codes.tobytes()).hexdigest() == d["codes_sha256"]
        idx = C.valid_sf_index(counts, bo, K)
        assert hashlib.sha256(sf[idx].tobytes()).hexdigest() == d["sf_valid_sha256"]


# ---- fused SiLU * mul + quant -----------------------------------------------------------------------------------
def _run_silu_mul_quant(gu_bits, is_bf16, counts):
    import torch
    from expert_specialization_moe_b200 import es_sm100_mxfp8_silu_mul_grouped_quant as fused
    T, K2 = gu_bits.shape
    K = K2 // 2
    ps, eo, bo, sf_rows = Q.offsets_from_counts(counts, 0, K)
    dev = "cuda"
    gu = C.bits_to_tensor(gu_bits, is_bf16, dev)
    codes = torch.zeros((T, K), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
    sf = torch.full((max(sf_rows, 1), K // 32), 0xCD, dtype=torch.uint8, device=dev)
    fused(gu, torch.from_numpy(ps).to(dev), torch.from_numpy(eo).to(dev), torch.from_numpy(bo).to(dev), codes, sf)
    torch.cuda.synchronize()
    return codes.view(torch.uint8).cpu().numpy(), sf.cpu().numpy().reshape(-1)[: sf_rows * (K // 32)], gu


@pytest.mark.parametrize("is_bf16", [True, False])
@pytest.mark.parametrize("counts,K", [([5, 0, 130, 64], 128), ([300], 768), ([1] * 7 + [90], 2048)])
def test_fused_silu_mul_quant_equals_unfused_sequence(counts, K, is_bf16):
    """Bit-exact against the unfused GPU sequence (torch silu*mul in fp32 -> input type -> grouped quant op)."""
    import torch
    gu_bits = C.activations_bits(sum(counts), 2 * K, seed=K + len(counts), is_bf16=is_bf16, outliers=False)
    codes, sf, gu = _run_silu_mul_quant(gu_bits, is_bf16, counts)
    act = (torch.nn.functional.silu(gu[:, :K].float()) * gu[:, K:].float()).to(gu.dtype)
    act_bits = act.view(torch.int16).cpu().numpy().view(np.uint16)
    ucodes, usf, *_ = C.run_quant_op(act_bits, is_bf16, counts)
    assert np.array_equal(codes, ucodes)
    assert np.array_equal(sf, usf)


def test_fused_silu_mul_quant_matches_cpu_oracle():
    """Against the numpy oracle; its float32 exp may differ from the GPU's in the last bit, so a small fraction of
    16-bit activations (and with them codes) may differ: allowance 1e-3 of the codes, scales 1e-3 of the bytes."""
    counts, K = [40, 3, 200], 512
    gu_bits = C.activations_bits(sum(counts), 2 * K, seed=5, outliers=False)
    codes, sf, _ = _run_silu_mul_quant(gu_bits, True, counts)
    act_bits = Q.silu_mul_bits(gu_bits, True)
    ocodes, osf = C.oracle_quant(act_bits, True, counts)
    assert (codes != ocodes).mean() < 1e-3
    assert (sf != osf).mean() < 1e-3
