"""Generate tests/golden/ref_blockwise_*.npz by running the REFERENCE's own torch code on the CPU.

    python tests/golden/make_blockwise_fixtures.py /path/to/reference

The reference's test module (test/test_es_grouped_gemm.py) defines the quantisers per_token_cast_to_fp8 /
per_block_cast_to_fp8 and the dequantise-and-matmul path baseline_scaled_mm.  The module imports the compiled
extension and probes the GPU at import time, so it is imported here with a stand-in `expert_specialization.ops` module
and a stubbed torch.cuda.get_device_capability; only its pure-torch functions are then called, on CPU tensors.
The fixtures pin oracle/grouped_gemm_oracle.py (the restatement of these functions) bit for bit.
"""
from __future__ import annotations

import importlib.util
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REF = Path(sys.argv[1]) if len(sys.argv) > 1 else HERE.parent.parent.parent / "reference"   # a sibling checkout


def load_reference_test_module():
    pkg = types.ModuleType("expert_specialization")
    ops = types.ModuleType("expert_specialization.ops")
    ops.es_fp8_blockwise_scaled_grouped_mm = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("not available"))
    pkg.ops = ops
    sys.modules["expert_specialization"] = pkg
    sys.modules["expert_specialization.ops"] = ops
    torch.cuda.get_device_capability = lambda device=None: (0, 0)
    spec = importlib.util.spec_from_file_location("ref_test_es_grouped_gemm", REF / "test" / "test_es_grouped_gemm.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def make_case(ref, name, counts, N, K, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    out = {"counts": np.array(counts, dtype=np.int64), "N": np.array(N), "K": np.array(K),
           "is_bf16": np.array(dtype == torch.bfloat16)}
    for e, m in enumerate(counts):
        if m == 0:
            continue
        a = torch.randn((m, K), generator=g, dtype=torch.float32).to(dtype)
        w = (torch.randn((N, K), generator=g, dtype=torch.float32) * 0.02).to(dtype)
        a_q, sa = ref.per_token_cast_to_fp8(a)
        w_q, sb = ref.per_block_cast_to_fp8(w)                       # weights as [N, K]: scale blocks [N/128, K/128]
        # reference GEMM path: (M,K) x (K,N), scales broadcast to element shape
        d = ref.baseline_scaled_mm(a_q, w_q.t(), sa, sb.t(), dtype)
        out[f"a_{e}"] = bits(a); out[f"w_{e}"] = bits(w)
        out[f"aq_{e}"] = a_q.contiguous().view(torch.uint8).numpy(); out[f"sa_{e}"] = sa.float().numpy()
        out[f"wq_{e}"] = w_q.contiguous().view(torch.uint8).numpy(); out[f"sb_{e}"] = sb.float().numpy()
        out[f"d_{e}"] = bits(d)
    np.savez_compressed(HERE / f"ref_blockwise_{name}.npz", **out)
    print(f"wrote ref_blockwise_{name}.npz", counts, N, K)


def main():
    ref = load_reference_test_module()
    # the CPU-runnable configuration at reduced N (fixture size), same K and token counts
    make_case(ref, "c1_bf16", [0, 1, 3, 7, 16, 64, 128, 293], 128, 512, torch.bfloat16, 0)
    make_case(ref, "small_fp16", [5, 130], 128, 256, torch.float16, 1)


if __name__ == "__main__":
    main()
