"""TEST INFRASTRUCTURE ONLY.  Single-GPU A/B of this library's kernels against the reference's own SM100 kernels
(oracle/_ref/libes_reference.so, built by oracle/build_ref.sh) on identical device inputs.

    python oracle/compare_with_reference_gpu.py [--workload gate_up|down] [--steps 20] [--quant]

Prints one JSON line per measurement: device time per call (CUDA events, after warm-up) of both implementations and
the output agreement.  Never run on more than one GPU: the reference kernel issues cluster-multicast TMA loads.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def timeit(fn, steps, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="gate_up")
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--quant", action="store_true", help="also compare the grouped quant at T=32768,K=7168,E=256")
    args = ap.parse_args()
    torch.ops.load_library(str(ROOT / "oracle" / "_ref" / "libes_reference.so"))
    ref = torch.ops.expert_specialization
    from expert_specialization_moe_b200 import (es_sm100_mxfp8_blockscaled_grouped_mm as our_mm,
                                                es_sm100_mxfp8_blockscaled_grouped_quant as our_quant)
    dev = torch.device("cuda", 0)
    E, T, N, K, desc = bench.WORKLOADS[args.workload]
    counts = bench.zipf_counts(T, E, 1.2, 0)
    wl = bench.build_device_workload(counts, N, K, dev, seed=1000)
    flops = 2.0 * T * N * K
    abytes = bench.algorithmic_bytes(counts, N, K)

    d_ref = torch.zeros_like(wl["d"])
    t_ours = timeit(lambda: our_mm(wl["d"], wl["a"], wl["b"], wl["sfa"], wl["sfb"], wl["ps"], wl["eo"], wl["bo"]), args.steps)
    t_ref = timeit(lambda: ref.es_sm100_mxfp8_blockscaled_grouped_mm(wl["a"], wl["b"], wl["sfa"], wl["sfb"], d_ref, wl["ps"], wl["eo"], wl["bo"]), args.steps)
    x, y = wl["d"].float(), d_ref.float()
    rel = float((x - y).norm() / y.norm())
    same = float((wl["d"].view(torch.int16) == d_ref.view(torch.int16)).float().mean())
    print(json.dumps({"op": "mxfp8_grouped_mm", "workload": desc, "ours_ms": t_ours, "reference_ms": t_ref,
                      "speedup": t_ref / t_ours, "ours_tflops": flops / t_ours / 1e9, "reference_tflops": flops / t_ref / 1e9,
                      "ours_gbs": abytes / t_ours / 1e6, "reference_gbs": abytes / t_ref / 1e6,
                      "rel_diff_vs_reference": rel, "bit_identical_fraction": same}))

    if args.quant:
        Tq, Kq, Eq = 32768, 7168, 256
        cq = bench.zipf_counts(Tq, Eq, 1.2, 0)
        ps, eo, bo, sf_rows = bench.offsets(cq, 0, Kq)
        t = lambda a: torch.from_numpy(a).to(dev)
        ps, eo, bo = t(ps), t(eo), t(bo)
        xq = torch.randn((Tq, Kq), device=dev, dtype=torch.float32)
        xq = (xq * torch.where(torch.rand_like(xq) < 0.01, 50.0, 1.0)).to(torch.bfloat16)
        c1 = torch.zeros((Tq, Kq), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        c2 = torch.zeros_like(c1)
        s1 = torch.zeros((sf_rows, Kq // 32), dtype=torch.uint8, device=dev)
        s2 = torch.zeros_like(s1)
        tq_ours = timeit(lambda: our_quant(xq, ps, eo, bo, c1, s1), args.steps)
        tq_ref = timeit(lambda: ref.es_sm100_mxfp8_blockscaled_grouped_quant(xq, ps, eo, bo, c2, s2), args.steps)
        qbytes = 2 * Tq * Kq + Tq * Kq + Tq * Kq // 32
        print(json.dumps({"op": "mxfp8_grouped_quant", "T": Tq, "K": Kq, "E": Eq, "ours_ms": tq_ours, "reference_ms": tq_ref,
                          "speedup": tq_ref / tq_ours, "ours_gbs": qbytes / tq_ours / 1e6, "reference_gbs": qbytes / tq_ref / 1e6,
                          "codes_identical": bool(torch.equal(c1.view(torch.uint8), c2.view(torch.uint8)))}))


if __name__ == "__main__":
    main()
