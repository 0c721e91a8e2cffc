"""TEST INFRASTRUCTURE ONLY.  Single-GPU A/B of this library's kernels against the reference's own SM100 kernels
(oracle/_ref/libes_reference.so, built by oracle/build_ref.sh) on identical device inputs, in one process.

    python oracle/compare_with_reference_gpu.py [--workloads gate_up,down,heavy,ref_dist,ref_dist_ep8] [--steps 20,200]
                                                [--repeats 5] [--quant]

For every workload and step count the two implementations run INTERLEAVED (ours, reference, ours, reference, ...),
`repeats` timed groups of `steps` calls each (CUDA events on the launching stream, after warm-up; groups of fewer than
100 calls start after 1.5 s of idle GPU: the burst regime, as `bench.py --steps 20` in a fresh process); the SM clock is
sampled with nvidia-smi while each arm runs (groups of 100 calls or more).  One JSON line per measurement: medians of
ms per call for both arms, their ratio, ms x median SM MHz (what the call costs in SM cycles, comparable across
power-cap states) and the output agreement.  Never run on more than one GPU: the reference kernel issues
cluster-multicast TMA loads.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def timed_group(fn, steps, dev):
    # the clock is only sampled on long groups: nvidia-smi needs a few hundred ms to start delivering samples
    sample = steps >= 100
    sampler = bench.ClockSampler(dev.index or 0)
    if sample:
        sampler.start()
        time.sleep(0.3)
        fn()
    else:
        # short groups measure the burst regime: a few calls of this arm (so that nothing of the other arm is in
        # flight or in the caches), then 1.5 s of idle GPU.  Back to back with the other arm's group they would run
        # inside the clock governor's settling time after the other kernel's different power draw.
        for _ in range(3):
            fn()
        torch.cuda.synchronize(dev)
        time.sleep(1.5)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize(dev)
    clocks = sampler.stop() if sample else {}
    return e0.elapsed_time(e1) / steps, clocks.get("sm_mhz")


def interleaved(ours, ref, steps, repeats, dev):
    for _ in range(3):
        ours(); ref()
    torch.cuda.synchronize(dev)
    t_o, t_r, c_o, c_r = [], [], [], []
    for _ in range(repeats):
        t, c = timed_group(ours, steps, dev); t_o.append(t); c_o.append(c)
        t, c = timed_group(ref, steps, dev); t_r.append(t); c_r.append(c)
    med = lambda v: float(np.median([x for x in v if x is not None])) if any(x is not None for x in v) else None
    mo, mr, co, cr = med(t_o), med(t_r), med(c_o), med(c_r)
    out = {"steps": steps, "repeats": repeats, "ours_ms": mo, "reference_ms": mr, "speedup": mr / mo,
           "ours_ms_all": [round(x, 4) for x in t_o], "reference_ms_all": [round(x, 4) for x in t_r],
           "ours_sm_mhz": co, "reference_sm_mhz": cr}
    if co and cr:
        out["ours_ms_x_mhz"], out["reference_ms_x_mhz"] = mo * co, mr * cr
        out["speedup_in_sm_cycles"] = (mr * cr) / (mo * co)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workloads", default="gate_up,down,heavy,ref_dist,ref_dist_ep8")
    ap.add_argument("--steps", default="20,200")
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--quant", action="store_true", help="also compare the grouped quant at T=32768,K=7168,E=256")
    args = ap.parse_args()
    assert torch.cuda.device_count() >= 1
    ref = bench.reference_ops()
    assert ref is not None, "oracle/_ref/libes_reference.so is missing: run oracle/build_ref.sh"
    from expert_specialization_moe_b200 import (es_sm100_mxfp8_blockscaled_grouped_mm as our_mm,
                                                es_sm100_mxfp8_blockscaled_grouped_quant as our_quant)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    step_counts = [int(x) for x in args.steps.split(",")]

    for name in [w for w in args.workloads.split(",") if w]:
        E, T, N, K, desc = bench.WORKLOADS[name]
        counts = bench.workload_counts(name)
        T = int(counts.sum())
        wl = bench.build_device_workload(counts, N, K, dev, seed=1000)
        d_ref = torch.zeros_like(wl["d"])
        ours = lambda: our_mm(wl["d"], wl["a"], wl["b"], wl["sfa"], wl["sfb"], wl["ps"], wl["eo"], wl["bo"])
        theirs = lambda: ref.es_sm100_mxfp8_blockscaled_grouped_mm(wl["a"], wl["b"], wl["sfa"], wl["sfb"], d_ref,
                                                                   wl["ps"], wl["eo"], wl["bo"])
        flops = 2.0 * T * N * K
        abytes = bench.algorithmic_bytes(counts, N, K)
        for steps in step_counts:
            r = interleaved(ours, theirs, steps, args.repeats, dev)
            same = float((wl["d"].view(torch.int16) == d_ref.view(torch.int16)).float().mean())
            r.update({"op": "mxfp8_grouped_mm", "workload": name, "ours_tflops": flops / r["ours_ms"] / 1e9,
                      "reference_tflops": flops / r["reference_ms"] / 1e9, "ours_gbs": abytes / r["ours_ms"] / 1e6,
                      "reference_gbs": abytes / r["reference_ms"] / 1e6, "bit_identical_fraction": same})
            print(json.dumps(r), flush=True)
        del wl, d_ref
        torch.cuda.empty_cache()

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
        qbytes = 2 * Tq * Kq + Tq * Kq + Tq * Kq // 32
        for steps in step_counts:
            r = interleaved(lambda: our_quant(xq, ps, eo, bo, c1, s1),
                            lambda: ref.es_sm100_mxfp8_blockscaled_grouped_quant(xq, ps, eo, bo, c2, s2), steps,
                            args.repeats, dev)
            r.update({"op": "mxfp8_grouped_quant", "workload": "quant", "ours_gbs": qbytes / r["ours_ms"] / 1e6,
                      "reference_gbs": qbytes / r["reference_ms"] / 1e6,
                      "codes_identical": bool(torch.equal(c1.view(torch.uint8), c2.view(torch.uint8)))})
            print(json.dumps(r), flush=True)


if __name__ == "__main__":
    main()
