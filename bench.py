#!/usr/bin/env python
"""Benchmark of the MoE grouped-GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload gate_up|down|quant]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W

Default workload ("gate_up"): DeepSeek-V3-shaped gate_up MXFP8 grouped GEMM, prefill — E=256 experts, 32768 routed rows
split by Zipf(1.2) counts, N=4096, K=7168, e4m3 operands with UE8M0 scales per 32, bf16 output.  One step = one call of
es_sm100_mxfp8_blockscaled_grouped_mm over the whole batch.  With N GPUs the experts are sharded contiguously
(E/N per GPU, expert-parallel, no data-path collective); the step time is the slowest rank's.

Prints ONE JSON line (rank 0).  `value` is the device-timed throughput with operands resident in HBM; `e2e` is the same
metric through the public op with the activations, their scales and the problem list copied from pinned host memory and
the output copied back inside the timed region (weights are model state and stay resident).
`--impl reference` on one GPU runs the reference's own SM100 kernels (the unmodified reference sources built by
oracle/build_ref.sh into oracle/_ref/, called through the reference's torch ops) on the same workload and prints the
same line; where that library is absent (it never travels to a multi-GPU call: its kernel issues cluster-multicast
loads) the arm falls back to the CPU dequant+matmul path (the reference's torch path restated in oracle/) on a
bounded sample of the workload and says so in `reference_kind`.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (E, T, N, K, description)
    "gate_up": (256, 32768, 4096, 7168, "DeepSeek-V3 gate_up MXFP8 grouped GEMM, prefill: E=256, 32768 routed rows "
                                        "(4096 tokens x top-8), Zipf(1.2) counts, N=4096, K=7168"),
    "down": (256, 512, 7168, 2048, "DeepSeek-V3 down-proj MXFP8 grouped GEMM, decode: E=256, 512 routed rows "
                                   "(64 tokens x top-8), Zipf(1.2) counts, N=7168, K=2048"),
    # small cases for profiler captures (a few GB at most on the device; weights still larger than L2)
    "gate_up_small": (32, 4096, 4096, 7168, "gate_up shape at 1/8 scale for profiler captures: E=32, 4096 routed rows, "
                                            "Zipf(1.2) counts, N=4096, K=7168"),
    "down_small": (64, 128, 7168, 2048, "down-proj shape at 1/4 scale for profiler captures: E=64, 128 routed rows, "
                                        "Zipf(1.2) counts, N=7168, K=2048"),
    "heavy": (8, 32768, 4096, 7168, "compute-bound probe: E=8 experts x 4096 rows each, N=4096, K=7168"),
    # grouped MXFP8 quantisation alone (N is unused): bf16 N(0,1) with 1% outliers x50
    "quant": (256, 32768, 0, 7168, "grouped MXFP8 quantisation: bf16 [32768, 7168], E=256, Zipf(1.2) counts, "
                                   "e4m3 codes + swizzled UE8M0 scales"),
    "qwen3_ep": (128, 0, 0, 0, "Qwen3-30B-A3B-shaped MoE layer with expert parallelism (N >= 2), dispatch / combine "
                               "over peer memory (FusedExchange)"),
    "qwen3_ep_pipelined": (128, 0, 0, 0, "the qwen3_ep layer as two half-batches on two streams (PipelinedExchange)"),
    "qwen3_ep_nccl": (128, 0, 0, 0, "Qwen3-30B-A3B-shaped MoE layer with expert parallelism (N >= 2), NCCL all-to-all "
                                    "dispatch / combine"),
    # the reference's own published benchmark (benchmark/benchmark_es_fp8_blockwise_moe.py: uniform-random top-8
    # routing, bf16 output), FP8-blockwise op; T = batch x top-8.  H200 numbers of the reference for these two points:
    # 264.8 us = 113.6 TFLOP/s and 187.2 us = 80.3 TFLOP/s (media/performance_data/H200_bench.log:14-16, 62-64)
    "blockwise_gate_up": (256, 4096, 512, 7168, "FP8-blockwise grouped GEMM, DeepSeek-R1 gate_up TP8 of the reference's "
                                                "benchmark: E=256, batch 512 x top-8 uniform-random routing, n=512, k=7168"),
    "blockwise_down": (256, 4096, 7168, 256, "FP8-blockwise grouped GEMM, DeepSeek-R1 down TP8 of the reference's "
                                             "benchmark: E=256, batch 512 x top-8 uniform-random routing, n=7168, k=256"),
    # the reference's own SM100 benchmark (benchmark/benchmark_sm100_mxfp8_blockscaled_moe.py:17-33,153-166): per-expert
    # row counts drawn 70 % from [1, 32], 15 % from [32, 64], 10 % from [64, 128], 5 % from [128, 1024]
    "ref_dist": (256, None, 512, 7168, "MXFP8 grouped GEMM on the reference's SM100 benchmark: DeepSeek-R1 gate_up TP8 "
                                       "(n=512, k=7168, E=256), row counts 70/15/10/5 % from 1-32/32-64/64-128/128-1024"),
    "ref_dist_ep8": (32, None, 4096, 7168, "MXFP8 grouped GEMM on the reference's SM100 benchmark: DeepSeek-R1 gate_up "
                                           "EP8 decode (n=4096, k=7168, E=32), row counts 70/15/10/5 % from "
                                           "1-32/32-64/64-128/128-1024"),
    # the other four shapes of that benchmark (same row distribution)
    "ref_dist_down": (256, None, 7168, 256, "MXFP8 grouped GEMM on the reference's SM100 benchmark: DeepSeek-R1 down TP8 "
                                            "(n=7168, k=256, E=256), the benchmark's row distribution"),
    "ref_dist_qwen_gate_up": (128, None, 768, 4096, "MXFP8 grouped GEMM on the reference's SM100 benchmark: Qwen3 gate_up "
                                                    "TP4 (n=768, k=4096, E=128), the benchmark's row distribution"),
    "ref_dist_qwen_down": (128, None, 4096, 384, "MXFP8 grouped GEMM on the reference's SM100 benchmark: Qwen3 down TP4 "
                                                 "(n=4096, k=384, E=128), the benchmark's row distribution"),
    "ref_dist_ep16": (16, None, 4096, 7168, "MXFP8 grouped GEMM on the reference's SM100 benchmark: DeepSeek-R1 gate_up "
                                            "EP16 decode (n=4096, k=7168, E=16), the benchmark's row distribution"),
    # weight-streaming probe: 128 experts of 1..32 rows, every tile streams a [128 x 7168] slab once; with
    # --tunable mm_stream_max_ctas=<n> it gives the per-SM ingest rate of the streaming kernel at n CTAs
    "stream_probe": (128, None, 4096, 7168, "weight-streaming probe: E=128 experts of 1..32 rows (uniform), N=4096, K=7168"),
    "quant_small": (64, 8192, 0, 7168, "grouped MXFP8 quantisation at 1/4 scale for profiler captures: bf16 "
                                       "[8192, 7168], E=64"),
}
FALLBACK_HBM_GBS = 6650.0


def zipf_counts(T, E, alpha=1.2, seed=0):
    rng = np.random.default_rng(seed)
    p = np.arange(1, E + 1, dtype=np.float64) ** -alpha
    p /= p.sum()
    counts = rng.multinomial(T, p)
    rng.shuffle(counts)
    return counts.astype(np.int64)


def ref_dist_counts(E, seed=1):
    """Row counts with the distribution of the reference's SM100 benchmark (its generator draws a class per expert:
    70 % 1-32 rows, 15 % 32-64, 10 % 64-128, 5 % 128-1024)."""
    rng = np.random.default_rng(seed)
    u = rng.random(E)
    lo = np.where(u <= 0.7, 1, np.where(u <= 0.85, 32, np.where(u <= 0.95, 64, 128)))
    hi = np.where(u <= 0.7, 32, np.where(u <= 0.85, 64, np.where(u <= 0.95, 128, 1024)))
    return rng.integers(lo, hi + 1).astype(np.int64)


def workload_counts(name):
    E, T, N, K, _ = WORKLOADS[name]
    if name == "heavy":
        return np.full(E, T // E, dtype=np.int64)
    if name.startswith("ref_dist"):
        return ref_dist_counts(E)
    if name == "stream_probe":
        return np.random.default_rng(0).integers(1, 33, size=E).astype(np.int64)
    return zipf_counts(T, E, 1.2, 0)


REF_LIB = ROOT / "oracle" / "_ref" / "libes_reference.so"


def reference_ops():
    """torch ops of the reference's own SM100 build (oracle/_ref), or None where that library is absent."""
    if not REF_LIB.exists():
        return None
    torch.ops.load_library(str(REF_LIB))
    return torch.ops.expert_specialization


def align128(x):
    return (x + 127) // 128 * 128


def offsets(counts, N, K):
    counts = np.asarray(counts, dtype=np.int64)
    E = len(counts)
    eo = np.zeros(E, dtype=np.int32)
    bo = np.zeros(E, dtype=np.int32)
    eo[1:] = np.cumsum(counts)[:-1]
    bo[1:] = np.cumsum(align128(counts))[:-1]
    ps = np.stack([counts, np.full(E, N), np.full(E, K)], axis=1).astype(np.int32)
    return ps, eo, bo, int(align128(counts).sum())


def algorithmic_bytes(counts, N, K):
    """A + SFA + B + SFB of the experts that have rows + bf16 D (padding rows and empty experts not counted)."""
    counts = np.asarray(counts, dtype=np.int64)
    T = int(counts.sum())
    active = int((counts > 0).sum())
    return T * K + T * K // 32 + active * N * K + active * N * K // 32 + 2 * T * N


def shard_counts(counts_all, world, placement):
    """Row counts of the experts each rank owns.  contiguous: experts [r*E/G, (r+1)*E/G).  balanced: experts sorted by
    rows, each assigned to the least-loaded rank that still has room (E/G experts per rank) — the static placement an
    expert-parallel deployment would derive from load statistics."""
    E = len(counts_all)
    per = E // world
    if placement == "contiguous" or world == 1:
        return [counts_all[r * per:(r + 1) * per] for r in range(world)]
    order = np.argsort(-counts_all, kind="stable")
    load = [0] * world
    owned = [[] for _ in range(world)]
    for e in order:
        r = min((i for i in range(world) if len(owned[i]) < per), key=lambda i: load[i])
        owned[r].append(int(e)); load[r] += int(counts_all[e])
    return [counts_all[np.array(sorted(o))] for o in owned]


def peak_hbm():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


def read_traffic(key):
    """DRAM bytes per launch from the committed ncu capture summary (profiles/traffic.txt), or None."""
    f = ROOT / "profiles" / "traffic.txt"
    if not f.exists():
        return None
    for line in f.read_text().splitlines():
        p = line.split()
        if len(p) == 2 and p[0] == key:
            return float(p[1])
    return None


class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.idx), f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [s for s in sm if s > 0.5 * max(sm)] or sm
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------------
def build_device_workload(counts, N, K, device, seed, quant=None):
    """Quantised operands resident on `device`, produced with the grouped quant op (this library's, bit-identical to
    the reference's, unless `quant` is given): activations N(0,1), weights N(0,0.02), both bf16 -> e4m3 + UE8M0."""
    if quant is None:
        from expert_specialization_moe_b200 import es_sm100_mxfp8_blockscaled_grouped_quant as quant
    E = len(counts)
    T = int(counts.sum())
    ps, eo, bo, sfa_rows = offsets(counts, N, K)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    t = lambda a: torch.from_numpy(a).to(device)
    ps_d, eo_d, bo_d = t(ps), t(eo), t(bo)
    x = torch.randn((max(T, 1), K), generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)[:T]
    a = torch.zeros((T, K), dtype=torch.uint8, device=device).view(torch.float8_e4m3fn)
    sfa = torch.zeros((max(sfa_rows, 1), K // 32), dtype=torch.uint8, device=device)
    quant(x, ps_d, eo_d, bo_d, a, sfa)
    del x
    w = torch.empty((E, N, K), dtype=torch.uint8, device=device).view(torch.float8_e4m3fn)
    sfb = torch.empty((E, N, K // 32), dtype=torch.uint8, device=device)
    chunk = 8
    for e0 in range(0, E, chunk):
        ne = min(chunk, E - e0)
        wb = (torch.randn((ne * N, K), generator=g, device=device, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        wps, weo, wbo, _ = offsets([N] * ne, 0, K)
        quant(wb, t(wps), t(weo), t(wbo), w[e0:e0 + ne].view(ne * N, K), sfb[e0:e0 + ne].view(ne * N, K // 32))
        del wb
    torch.cuda.synchronize(device)
    d = torch.empty((T, N), dtype=torch.bfloat16, device=device)
    return dict(a=a, sfa=sfa, b=w.transpose(1, 2), w=w, sfb=sfb, d=d, ps=ps_d, eo=eo_d, bo=bo_d,
                ps_h=ps, eo_h=eo, bo_h=bo)


class CpuReferenceSample:
    """Bounded sample of the workload for the CPU path (dequantise + per-expert fp32 torch.mm,
    oracle/grouped_gemm_oracle.py — the restatement of the reference's torch dequant-matmul path).  Operands are built
    once; run() times one pass over the sample on all host threads."""

    def __init__(self, counts, N, K, seed, max_flops):
        from oracle import mxfp8_quant_oracle as Q
        rng = np.random.default_rng(seed)
        self.N, self.K = N, K

        def random_mxfp8(rows):
            # operand bytes drawn directly (finite e4m3 codes of either sign, scale exponents around 2^-7): the CPU
            # time of dequantise + matmul does not depend on the values, and quantising 29 M weights per expert with
            # the numpy oracle would dominate the wall clock of this leg
            codes = rng.integers(0, 0x7F, size=(rows, K), dtype=np.uint8) | (rng.integers(0, 2, size=(rows, K), dtype=np.uint8) << 7)
            sf = rng.integers(118, 123, size=(rows, K // 32), dtype=np.uint8)
            return torch.from_numpy(codes), torch.from_numpy(Q.swizzle_sf(sf, K))

        self.w, self.sfb = random_mxfp8(N)
        self.w = self.w.view(1, N, K)
        self.items, self.flops, self.rows, self.experts = [], 0.0, 0, []
        for e in range(len(counts)):
            m = int(counts[e])
            if m == 0:
                continue
            a, sfa = random_mxfp8(m)
            self.items.append((a, sfa, np.array([[m, N, K]], dtype=np.int32)))
            self.flops += 2.0 * m * N * K
            self.rows += m
            self.experts.append(e)
            if self.flops >= max_flops:
                break

    def run(self, threads=None):
        from oracle import grouped_gemm_oracle as G
        threads = threads or os.cpu_count() or 1
        torch.set_num_threads(threads)
        t0 = time.perf_counter()
        for a, sfa, ps in self.items:
            G.mxfp8_grouped_mm(a, self.w, sfa, self.sfb, ps, [0], [0])
        secs = time.perf_counter() - t0
        return self.flops / secs / 1e12, threads, secs

    def describe(self, secs):
        return (f"experts {self.experts[0]}..{self.experts[-1]} of the workload ({len(self.experts)} non-empty experts, "
                f"{self.rows} rows, {self.flops / 1e9:.1f} GFLOP) in {secs:.1f} s: unswizzle + dequantise + fp32 "
                f"torch.mm per expert")


def oracle_spot_check(wl, counts, N, K):
    """Part of the cpu_baseline leg: the CPU path (oracle dequantise + fp32 matmul) on the DEVICE's own operands for
    one small expert and one 128-column tile, against what the GPU wrote there — so the two arms of this benchmark
    are seen to compute the same thing, not only to be timed on the same shapes."""
    from oracle import grouped_gemm_oracle as G
    from oracle import mxfp8_quant_oracle as Q
    nz = [e for e in range(len(counts)) if counts[e] > 0]
    e = min(nz, key=lambda i: (abs(int(counts[i]) - 24), i))          # an expert of about two dozen rows
    m, off, bo, kb = int(counts[e]), int(wl["eo_h"][e]), int(wl["bo_h"][e]), K // 32
    a = wl["a"].view(torch.uint8)[off:off + m].cpu()
    sa = wl["sfa"].reshape(-1)[(torch.from_numpy(Q.sf_swizzled_offsets(m, K)) + bo * kb).to(wl["sfa"].device)].cpu()
    w = wl["w"].view(torch.uint8)[e, :128].cpu()
    sb = wl["sfb"].reshape(-1)[(torch.from_numpy(Q.sf_swizzled_offsets(N, K))[:128] + e * N * kb).to(wl["sfb"].device)].cpu()
    ref = torch.mm(G.dequant_mxfp8(a, sa), G.dequant_mxfp8(w, sb).t())
    got = wl["d"][off:off + m, :128].float().cpu()
    rel, cos = G.rel_err_and_cosine(got, ref)
    return {"expert": int(e), "rows": m, "columns": "0..127", "rel_err": rel, "cosine": cos,
            "ok": bool(rel <= 1e-2 and cos >= 0.9999)}


def cpu_reference_rate(counts, N, K, seed, budget_s=20.0, threads=None):
    """One timed pass over a sample sized for about `budget_s` seconds (assuming ~0.2 TFLOP/s of host throughput)."""
    sample = CpuReferenceSample(counts, N, K, seed, max_flops=budget_s * 0.2e12)
    rate, threads, secs = sample.run(threads)
    return rate, threads, sample.describe(secs)


def bench_ep_layer(args, device, rank, world, dist):
    """Qwen3-30B-A3B-shaped MoE layer, expert parallel: E=128, top-8, hidden 2048, moe_intermediate 768, 16384 tokens
    per GPU, router logits N(0,1) -> softmax -> top-8.  One step = count exchange + NCCL all-to-all dispatch + grouped
    quant + gate_up grouped GEMM + fused SiLU*mul/requant + down grouped GEMM + all-to-all combine with top-k weights
    (expert_parallel.moe_forward), or the same layer over peer memory (expert_parallel.FusedExchange).  value =
    expert-GEMM FLOPs of all ranks / step time."""
    from expert_specialization_moe_b200 import expert_parallel as ep
    E, topk, H, I, tokens = 128, 8, 2048, 768, 16384
    assert dist is not None and E % world == 0, "the expert-parallel layer benchmark runs on 1, 2, 4 or 8 ranks"
    e_local = E // world
    g = torch.Generator(device=device); g.manual_seed(1234)           # same weights everywhere; each rank keeps a shard
    w1 = (torch.randn((E, 2 * I, H), generator=g, device=device) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn((E, H, I), generator=g, device=device) * 0.02).to(torch.bfloat16)
    shard = ep.ExpertShard(w1[rank * e_local:(rank + 1) * e_local].contiguous(),
                           w2[rank * e_local:(rank + 1) * e_local].contiguous())
    del w1, w2
    g.manual_seed(99 + rank)
    x = torch.randn((tokens, H), generator=g, device=device).to(torch.bfloat16)
    p = torch.softmax(torch.randn((tokens, E), generator=g, device=device), -1)
    wts, ids = torch.topk(p, topk, dim=-1)
    wts = (wts / wts.sum(-1, keepdim=True)).to(torch.float32)
    fused = args.workload in ("qwen3_ep", "qwen3_ep_pipelined")
    if fused:
        # capacity: 2x the balanced share is ample for softmax-of-N(0,1) routing; overflow would be reported as an
        # out-of-range destination by es_b200_check_status below
        if args.workload == "qwen3_ep_pipelined":
            fx = ep.PipelinedExchange(E, topk, tokens, H, device, capacity_rows=2 * tokens * topk)
        else:
            fx = ep.FusedExchange(E, topk, tokens, H, device, capacity_rows=2 * tokens * topk)
        out_buf = None if args.workload == "qwen3_ep_pipelined" else torch.empty_like(x)
        step = (lambda: fx.forward(x, ids, wts, shard)) if out_buf is None else \
               (lambda: fx.forward(x, ids, wts, shard, out=out_buf))
    else:
        step = lambda: ep.moe_forward(x, ids, wts, E, shard.forward)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(device.index or 0)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=device)
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    import ctypes
    from expert_specialization_moe_b200 import _cabi
    raw = ctypes.c_uint32(0)
    _cabi.load().es_b200_check_status(torch.cuda.current_stream(device).cuda_stream, ctypes.byref(raw))
    st = torch.tensor([int(raw.value)], dtype=torch.int64, device=device)
    dist.all_reduce(st, op=dist.ReduceOp.MAX)
    status = int(st[0])
    line = None
    if rank == 0:
        flops = 2.0 * tokens * topk * world * (2 * I * H + H * I)
        line = {"metric": "MoE layer (expert parallel) grouped-GEMM TFLOPS incl. dispatch/combine",
                "value": flops / (float(ms[0]) * 1e-3) / 1e12, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": float(ms[0]), "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "mxfp8_e4m3", "data": "synthetic",
                "config": {"workload": "Qwen3-30B-A3B-shaped MoE layer: E=128, top-8, hidden 2048, intermediate 768, "
                                       "16384 tokens per GPU, " + ("dispatch/combine as peer-memory stores fused with "
                                       "the quantisation (FusedExchange)" + (", two half-batches on two streams"
                                       if args.workload == "qwen3_ep_pipelined" else "") if fused
                                       else "NCCL all-to-all dispatch/combine"),
                           "experts_per_gpu": e_local},
                "clocks": clocks, "device_status": status,
                # ours per step: route count + tables, dispatch-quant-push, unpack, 2 barriers, 3 + 3 GEMM launches,
                # silu-quant, weighted sum (fused) / 2 quant kernels + GEMMs (all-to-all path)
                "gpu_launches": args.steps * ((28 if args.workload == "qwen3_ep_pipelined" else 14) if fused else 9)}
    del shard, x
    torch.cuda.empty_cache()
    return line


def bench_quant(args, E, T, K, desc, device, rank, world, dist, quant=None):
    """Grouped quant alone; with N GPUs each rank quantises its own E/N experts' rows (no collective).  `quant`: the
    reference's op for the reference arm."""
    is_reference = quant is not None
    if quant is None:
        from expert_specialization_moe_b200 import es_sm100_mxfp8_blockscaled_grouped_quant as quant
    counts_all = zipf_counts(T, E, 1.2, 0)
    counts = counts_all[rank * (E // world):(rank + 1) * (E // world)]
    Tl = int(counts.sum())
    ps, eo, bo, sf_rows = offsets(counts, 0, K)
    t = lambda a: torch.from_numpy(a).to(device)
    ps, eo, bo = t(ps), t(eo), t(bo)
    g = torch.Generator(device=device); g.manual_seed(7 + rank)
    # Three input / output sets (2.1 GB in all) taken in turn: every step streams 0.7 GB that the two steps before it
    # have pushed out of the 126 MB L2 many times over, and no flush kernel leaves dirty lines behind for the timed
    # kernel to write back (a 256 MB memset before each step did: ~0.1 GB of extra HBM writes inside the timed region).
    NSETS = 3
    xs, codes, sfs = [], [], []
    for i in range(NSETS):
        x = torch.randn((Tl, K), generator=g, device=device, dtype=torch.float32)
        xs.append((x * torch.where(torch.rand((Tl, K), generator=g, device=device) < 0.01, 50.0, 1.0)).to(torch.bfloat16))
        del x
        codes.append(torch.empty((Tl, K), dtype=torch.uint8, device=device).view(torch.float8_e4m3fn))
        sfs.append(torch.empty((max(sf_rows, 128), K // 32), dtype=torch.uint8, device=device))
    step = lambda i: quant(xs[i % NSETS], ps, eo, bo, codes[i % NSETS], sfs[i % NSETS])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(device.index or 0)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1) / args.steps
    abytes_local = 3 * Tl * K + Tl * K // 32
    stats = torch.tensor([ms], dtype=torch.float64, device=device)
    sums = torch.tensor([float(abytes_local)], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    if rank == 0:
        peak, peak_kind = peak_hbm()
        achieved = abytes_local / (ms * 1e-3) / 1e9
        line = {"metric": "MXFP8 grouped quantisation GB/s (algorithmic bytes)", "value": float(sums[0]) / (float(stats[0]) * 1e-3) / 1e9,
                "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(stats[0]),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16->e4m3+ue8m0",
                "data": "synthetic", "config": {"workload": desc, "l2": "three input/output sets (2.1 GB) in rotation: inputs larger than L2, no flush"},
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "traffic": read_traffic(f"{args.workload}_n{world}"), "peak_kind": peak_kind, "algorithmic_bytes": abytes_local,
                             "kernel": "mxfp8_group_quant_kernel", "kernel_ms": ms},
                "clocks": clocks, "gpu_launches": args.steps}
        if is_reference:
            line["impl"] = "reference"
            line["reference_kind"] = "gpu_kernel: the reference's own mxfp8_group_quant kernel (oracle/_ref)"
            line["roofline"]["kernel"] = "reference mxfp8_group_quant"
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def reference_blockwise(args, E, T, N, K, desc):
    """CPU arm of the blockwise workloads: the reference test's torch dequant + matmul (restated in oracle/) on the
    first experts of the same routing, as many as fit about a second per step, all host threads."""
    from oracle import grouped_gemm_oracle as G
    rng = np.random.default_rng(3)
    counts = np.bincount(rng.integers(0, E, size=T), minlength=E).astype(np.int64)
    n_exp = int(max(1, min(E, 0.05e12 / max(1.0, 2.0 * counts.mean() * N * K + 4.0 * N * K))))
    counts = counts[:n_exp]
    rows = int(counts.sum())
    g = torch.Generator(); g.manual_seed(5)
    a = torch.randint(0, 0x78, (rows, K), dtype=torch.uint8, generator=g)
    w = torch.randint(0, 0x78, (n_exp, N, K), dtype=torch.uint8, generator=g)
    sa = torch.rand((rows, K // 128), generator=g) * 0.01 + 0.001
    sb = torch.rand((n_exp, N // 128, K // 128), generator=g) * 0.01 + 0.001
    eo = np.zeros(n_exp, dtype=np.int64); eo[1:] = np.cumsum(counts)[:-1]
    ps = np.stack([counts, np.full(n_exp, N), np.full(n_exp, K)], axis=1)
    rates, secs = [], 0.0
    for i in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        G.fp8_blockwise_grouped_mm(a, w, sa, sb, ps, eo)
        secs = time.perf_counter() - t0
        if i >= args.warmup:
            rates.append(2.0 * rows * N * K / secs / 1e12)
    v = float(np.mean(rates)) if rates else 0.0
    cores = torch.get_num_threads()
    line = {"impl": "reference", "metric": "FP8-blockwise grouped GEMM TFLOPS", "value": v, "unit": "TFLOP/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 2.0 * T * N * K / (v * 1e12) * 1e3 if v else None, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3 x fp32 block scales", "data": "synthetic",
            "config": {"workload": desc},
            "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                             "sample": f"first {n_exp} of {E} experts ({rows} rows), {secs:.2f} s per step"},
            "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


PUBLISHED_H200_TFLOPS = {"blockwise_gate_up": 113.6, "blockwise_down": 80.3}


def bench_blockwise(args, E, T, N, K, desc, device, rank, world, dist):
    """es_fp8_blockwise_scaled_grouped_mm on a shape of the reference's benchmark script; experts sharded E/N per GPU."""
    from expert_specialization_moe_b200 import es_fp8_blockwise_scaled_grouped_mm as op
    rng = np.random.default_rng(3)
    ids = rng.integers(0, E, size=T)                        # uniform-random top-k routing, as the reference benchmark
    counts_all = np.bincount(ids, minlength=E).astype(np.int64)
    el = E // world
    counts = counts_all[rank * el:(rank + 1) * el]
    rows = int(counts.sum())
    g = torch.Generator(device=device); g.manual_seed(11 + rank)
    # random finite e4m3 codes and positive scales: timing does not depend on the values
    w = torch.randint(0, 0x78, (el, N, K), dtype=torch.uint8, device=device, generator=g).view(torch.float8_e4m3fn)
    a = torch.randint(0, 0x78, (max(rows, 1), K), dtype=torch.uint8, device=device, generator=g).view(torch.float8_e4m3fn)[:rows]
    sb = torch.rand((el, N // 128, K // 128), device=device, generator=g) * 0.01 + 0.001
    sa = torch.rand((rows, K // 128), device=device, generator=g) * 0.01 + 0.001
    d = torch.empty((rows, N), dtype=torch.bfloat16, device=device)
    eo = np.zeros(el, dtype=np.int32); eo[1:] = np.cumsum(counts)[:-1]
    ps = np.stack([counts, np.full(el, N), np.full(el, K)], axis=1).astype(np.int32)
    ps, eo = torch.from_numpy(ps).to(device), torch.from_numpy(eo).to(device)
    st = torch.full((el,), K, dtype=torch.int64, device=device)
    ws = torch.empty(16, dtype=torch.uint8, device=device)
    step = lambda: op(d, a, w.transpose(1, 2), sa, sb.transpose(1, 2), st, st, st, ps, eo, ws)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(device.index or 0)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = e0.elapsed_time(e1) / args.steps
    abytes_local = el * N * K + rows * K + rows * N * 2 + 4 * (el * (N // 128) * (K // 128) + rows * (K // 128))
    stats = torch.tensor([ms], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    if rank == 0:
        peak, peak_kind = peak_hbm()
        achieved = abytes_local / (ms * 1e-3) / 1e9
        value = 2.0 * T * N * K / (float(stats[0]) * 1e-3) / 1e12
        buckets = 1 + (rows > 32)        # launches: the <= 32-row shape, then the two larger shapes in one launch
        line = {"metric": "FP8-blockwise grouped GEMM TFLOPS", "value": value, "unit": "TFLOP/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(stats[0]), "higher_is_better": True,
                "scaling": "strong", "vs_baseline": value / PUBLISHED_H200_TFLOPS[args.workload],
                "vs_baseline_note": "published number is the reference's Hopper kernel on H200",
                "dtype": "fp8_e4m3 x fp32 block scales", "data": "synthetic",
                "config": {"workload": desc, "experts_per_gpu": el, "out_dtype": "bf16",
                           "l2": "inputs larger than L2 (weights %.2f GB per GPU), no flush" % (el * N * K / 1e9)},
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                             "traffic": read_traffic(f"{args.workload}_n{world}"), "peak_kind": peak_kind,
                             "algorithmic_bytes": abytes_local, "kernel": "fp8_blockwise_grouped_mm_kernel (<= 32 rows) + fp8_blockwise_two_shapes_kernel",
                             "kernel_ms": ms},
                "clocks": clocks, "gpu_launches": int(args.steps * buckets)}
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------------
def place_experts(counts_all, world, placement, N, K):
    """Experts (and their row counts) of every rank.  Returns (list of count arrays, note).
    contiguous: experts [r*E/G, (r+1)*E/G).  balanced: E/G experts per rank, largest first to the least-loaded rank.
    load_balanced: what an expert-parallel deployment derives from load statistics — an expert with more rows than
    one rank's fair share is REPLICATED (weights on several ranks, its rows split evenly between the replicas), then
    every (replica of an) expert goes, most expensive first, to the rank with the least estimated time, where an
    expert costs max(its weight bytes at HBM speed, its FLOPs at tensor speed)."""
    E = len(counts_all)
    per = E // world
    if placement == "contiguous" or world == 1:
        return [counts_all[r * per:(r + 1) * per] for r in range(world)], "contiguous blocks of E/N experts"
    if placement == "balanced":
        return shard_counts(counts_all, world, "balanced"), "E/N experts per rank, greedy by rows"
    fair = max(1, int(counts_all.sum()) // world)
    virtual, replicated = [], 0
    for m in counts_all:
        m = int(m)
        parts = max(1, -(-m // fair)) if m > fair else 1
        replicated += parts > 1
        base, extra = divmod(m, parts)
        virtual += [base + (1 if i < extra else 0) for i in range(parts)]
    cost = lambda m: max(N * K * (1 + 1 / 32) / 6.2e12, 2.0 * m * N * K / 2.4e15) if m > 0 else 0.0
    load = [0.0] * world
    owned = [[] for _ in range(world)]
    for m in sorted(virtual, key=lambda m: -cost(m)):
        r = min(range(world), key=lambda i: (load[i], len(owned[i])))
        owned[r].append(m); load[r] += cost(m)
    width = max(len(o) for o in owned)
    shards = [np.array(sorted(o, reverse=True) + [0] * (width - len(o)), dtype=np.int64) for o in owned]
    return shards, (f"load-balanced: {replicated} expert(s) with more rows than a rank's fair share replicated "
                    f"(rows split between the replicas), experts placed by estimated time; {width} expert slots per rank")


def run_gemm_arm(args, wl, grouped_mm, counts, N, K, device, rank, world, dist, local_rank):
    """Times args.steps calls of `grouped_mm` on the resident workload, then the same call end to end with host
    buffers.  Returns (elapsed_ms, my_ms, e2e tuple or None, clocks, host_us_per_call)."""
    def step():
        grouped_mm(wl["d"], wl["a"], wl["b"], wl["sfa"], wl["sfb"], wl["ps"], wl["eo"], wl["bo"])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    elapsed_ms = ev0.elapsed_time(ev1)
    clocks = sampler.stop() if rank == 0 else None

    # host time of one call (argument checks, tensor maps, launches): 50 calls enqueued back to back, no sync inside
    torch.cuda.synchronize(device)
    t0 = time.perf_counter()
    for _ in range(50):
        step()
    host_us = (time.perf_counter() - t0) / 50 * 1e6
    torch.cuda.synchronize(device)

    e2e = None
    if not args.no_e2e:
        # Pinned host buffers; per step: H2D of the activations (e4m3 codes + scales) and the problem list, the op, D2H of
        # the bf16 result.  The three legs run on three streams over double-buffered device tensors, so step i+1's
        # upload and step i-1's download overlap step i's kernel (PCIe is full duplex); every step's copies are inside
        # the timed region.
        a_h = wl["a"].view(torch.uint8).cpu().pin_memory()
        sfa_h = wl["sfa"].cpu().pin_memory()
        ps_h = torch.from_numpy(wl["ps_h"]).pin_memory()
        eo_h = torch.from_numpy(wl["eo_h"]).pin_memory()
        bo_h = torch.from_numpy(wl["bo_h"]).pin_memory()
        NB = 2
        d_h = [torch.empty(wl["d"].shape, dtype=wl["d"].dtype).pin_memory() for _ in range(NB)]
        a_d = [torch.empty_like(wl["a"]) for _ in range(NB)]
        sfa_d = [torch.empty_like(wl["sfa"]) for _ in range(NB)]
        ps_d = [torch.empty_like(wl["ps"]) for _ in range(NB)]
        eo_d = [torch.empty_like(wl["eo"]) for _ in range(NB)]
        bo_d = [torch.empty_like(wl["bo"]) for _ in range(NB)]
        d_d = [torch.empty_like(wl["d"]) for _ in range(NB)]
        s_in, s_mm, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device), torch.cuda.Stream(device)
        ev_in = [torch.cuda.Event() for _ in range(NB)]
        ev_mm = [torch.cuda.Event() for _ in range(NB)]
        ev_out = [torch.cuda.Event() for _ in range(NB)]

        def e2e_step(i):
            b = i % NB
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_mm[b])            # the kernel that last read these input buffers is done
                a_d[b].view(torch.uint8).copy_(a_h, non_blocking=True)
                sfa_d[b].copy_(sfa_h, non_blocking=True)
                ps_d[b].copy_(ps_h, non_blocking=True); eo_d[b].copy_(eo_h, non_blocking=True)
                bo_d[b].copy_(bo_h, non_blocking=True)
                ev_in[b].record(s_in)
            with torch.cuda.stream(s_mm):
                s_mm.wait_event(ev_in[b])
                s_mm.wait_event(ev_out[b])           # the download that last read this output buffer is done
                grouped_mm(d_d[b], a_d[b], wl["b"], sfa_d[b], wl["sfb"], ps_d[b], eo_d[b], bo_d[b])
                ev_mm[b].record(s_mm)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_mm[b])
                d_h[b].copy_(d_d[b], non_blocking=True)
                ev_out[b].record(s_out)

        def e2e_join():
            cur = torch.cuda.current_stream(device)
            for st in (s_in, s_mm, s_out):
                cur.wait_stream(st)

        for i in range(2):
            e2e_step(i)
        e2e_join()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for st in (s_in, s_mm, s_out):
            st.wait_event(f0)
        for i in range(args.steps):
            e2e_step(i)
        e2e_join()
        f1.record()
        barrier()
        e2e_ms = f0.elapsed_time(f1)
        if not torch.equal(d_h[(args.steps - 1) % NB], wl["d"].cpu()):
            raise SystemExit("e2e result differs from the device-resident result")
        h2d = a_h.numel() + sfa_h.numel() + 4 * (ps_h.numel() + eo_h.numel() + bo_h.numel())
        d2h = d_h[0].numel() * d_h[0].element_size()
        e2e = (e2e_ms, h2d, d2h)
    return elapsed_ms, float(ev0.elapsed_time(ev1)) / args.steps, e2e, clocks, host_us


def compare_with_reference_kernel(wl, ours, ref_mm, device, repeats=3, steps=100, settle=20):
    """Outside every timed region, one GPU only: this library's call and the reference's own SM100 kernel on the same
    resident operands, interleaved (ours, reference, ours, ...), `repeats` groups of `steps` calls each; medians.
    Each group starts with `settle` untimed calls of its own kernel: on a GPU at its power cap the clock governor needs
    tens of milliseconds to settle after the other kernel's different draw, and with 20-call groups back to back both
    arms were timed inside that transient (this library's call 1.92 ms in such groups, 1.79 ms in groups of 200)."""
    d_ref = torch.zeros_like(wl["d"])
    ref = lambda: ref_mm(wl["a"], wl["b"], wl["sfa"], wl["sfb"], d_ref, wl["ps"], wl["eo"], wl["bo"])
    mine = lambda: ours(wl["d"], wl["a"], wl["b"], wl["sfa"], wl["sfb"], wl["ps"], wl["eo"], wl["bo"])

    def timed(fn):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        # a short idle gap first, as oracle/compare_with_reference_gpu.py does for its long groups: straight after the
        # other arm's group this library's call measured 5 % slower than in any run of its own (decode workload: 0.268
        # vs 0.254 ms), the reference's kernel did not
        torch.cuda.synchronize(device)
        time.sleep(0.3)
        for _ in range(settle):
            fn()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / steps

    for _ in range(3):
        ref(); mine()
    torch.cuda.synchronize(device)
    t_ours, t_ref = [], []
    for _ in range(repeats):
        t_ours.append(timed(mine))
        t_ref.append(timed(ref))
    same = float((wl["d"].view(torch.int16) == d_ref.view(torch.int16)).float().mean())
    mo, mr = float(np.median(t_ours)), float(np.median(t_ref))
    return {"ms_per_step": mr, "ours_ms_per_step": mo, "ratio": mr / mo, "bit_identical_fraction": same,
            "how": f"interleaved, {repeats} x {steps} calls each after 0.3 s idle and {settle} untimed ones, medians; reference = "
                   f"its own SM100 CUTLASS kernel built from its sources (oracle/_ref)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="gate_up", choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-budget", type=float, default=20.0, help="seconds of CPU work for the cpu_baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip the side-by-side run of the reference kernel")
    ap.add_argument("--reference-cpu", action="store_true", help="--impl reference: time the CPU port even on one GPU")
    ap.add_argument("--placement", default=None, choices=["contiguous", "balanced", "load_balanced"],
                    help="expert-to-GPU placement for N > 1 (default load_balanced): contiguous blocks of E/N experts; "
                         "E/N experts per GPU chosen greedily by rows; or load-aware with the hottest expert "
                         "replicated (see place_experts)")
    ap.add_argument("--tunable", action="append", default=[], metavar="NAME=VALUE",
                    help="set a dispatcher tunable of the library before the run (es_b200_set_tunable), e.g. "
                         "mm_pair_first_clusters=0, mm_stream_max_ctas=64, mm_stream_lsu=0; repeatable")
    ap.add_argument("--ep-layer-steps", type=int, default=10,
                    help="N > 1, default workload: steps of the expert-parallel layer run after the headline (0 = skip)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    E, T, N, K, desc = WORKLOADS[args.workload]
    counts_all = workload_counts(args.workload)
    if T is None:
        T = int(counts_all.sum())
    placement = args.placement or ("load_balanced" if world > 1 else "contiguous")
    metric = "MoE-layer grouped-GEMM TFLOPS"
    config = {"workload": desc, "experts_per_gpu": E // max(world, 1), "placement": placement,
              "l2": "inputs larger than L2 (weights %.2f GB per GPU), no flush" % ((E // max(world, 1)) * N * K / 1e9),
              "out_dtype": "bf16"}
    gemm_workload = not (args.workload.startswith("quant") or args.workload.startswith("qwen3_ep")
                         or args.workload.startswith("blockwise"))

    ref = None
    if args.impl == "reference":
        # One GPU and the reference's own build present: its SM100 kernels, through its torch ops.  Otherwise the CPU
        # restatement of its torch dequant-matmul path on a bounded sample (rank 0 only).
        if (world == 1 and not args.reference_cpu and torch.cuda.is_available()
                and (gemm_workload or args.workload.startswith("quant"))):
            ref = reference_ops()
        if ref is None:
            if rank != 0:
                return
            if args.workload.startswith("blockwise"):
                return reference_blockwise(args, E, T, N, K, desc)
            rates = []
            cores = os.cpu_count() or 1
            # the whole run (warm-up + steps) is kept to about two minutes: each step times one pass over a sample sized
            # for total / (steps + warm-up) seconds at ~0.2 TFLOP/s
            per_step_budget = min(args.cpu_budget, max(0.25, 100.0 / max(1, args.steps + args.warmup)))
            sample = CpuReferenceSample(counts_all, N, K, seed=100, max_flops=per_step_budget * 0.2e12)
            sdesc = ""
            for i in range(args.warmup + args.steps):
                r, cores, secs = sample.run()
                if i >= args.warmup:
                    rates.append(r)
                    sdesc = sample.describe(secs)
            v = float(np.mean(rates)) if rates else 0.0
            flops_total = 2.0 * T * N * K
            line = {
                "impl": "reference", "reference_kind": "cpu_port: the reference's torch dequant + per-expert matmul "
                "path restated (oracle/), host cores; the reference's own SM100 build is not on this box",
                "metric": metric, "value": v, "unit": "TFLOP/s", "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": flops_total / (v * 1e12) * 1e3 if v else None,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "mxfp8_e4m3",
                "data": "synthetic", "config": config,
                "cpu_baseline": {"value": v, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sdesc},
                "e2e": {"value": v, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0,
            }
            print(json.dumps(line))
            return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU fallback")
    if args.tunable:
        from expert_specialization_moe_b200 import _cabi as _tun
        for item in args.tunable:
            name, _, value = item.partition("=")
            _tun.set_tunable(name.strip(), int(value))
        config["tunables"] = list(args.tunable)
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)

    if args.workload.startswith("quant"):
        return bench_quant(args, E, T, K, desc, device, rank, world, dist,
                           quant=ref.es_sm100_mxfp8_blockscaled_grouped_quant if ref is not None else None)
    if args.workload.startswith("qwen3_ep"):
        if dist is None:                         # one GPU: a process group of one, all experts local
            import socket
            import torch.distributed as dist
            with socket.socket() as sock:
                sock.bind(("127.0.0.1", 0))
                port = sock.getsockname()[1]
            dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1,
                                    device_id=device)
        line = bench_ep_layer(args, device, rank, world, dist)
        if rank == 0:
            print(json.dumps(line))
        dist.barrier()
        dist.destroy_process_group()
        return
    if args.workload.startswith("blockwise"):
        return bench_blockwise(args, E, T, N, K, desc, device, rank, world, dist)

    # expert-parallel shard
    assert E % world == 0
    shards, placement_note = place_experts(counts_all, world, placement, N, K)
    counts = shards[rank]
    config["placement_note"] = placement_note
    config["experts_per_gpu"] = int(len(counts))
    config["l2"] = "inputs larger than L2 (weights %.2f GB per GPU), no flush" % (int((counts > 0).sum()) * N * K / 1e9)
    from expert_specialization_moe_b200 import es_sm100_mxfp8_blockscaled_grouped_mm as our_mm
    from expert_specialization_moe_b200 import _cabi
    if ref is not None:
        wl = build_device_workload(counts, N, K, device, seed=1000 + rank,
                                   quant=ref.es_sm100_mxfp8_blockscaled_grouped_quant)
        grouped_mm = lambda d, a, b, sfa, sfb, ps, eo, bo: ref.es_sm100_mxfp8_blockscaled_grouped_mm(
            a, b, sfa, sfb, d, ps, eo, bo)
    else:
        wl = build_device_workload(counts, N, K, device, seed=1000 + rank)
        grouped_mm = our_mm

    elapsed_ms, my_ms, e2e, clocks, host_us = run_gemm_arm(args, wl, grouped_mm, counts, N, K, device, rank, world,
                                                           dist, local_rank)
    if ref is None:
        import ctypes
        raw = ctypes.c_uint32(0)
        rc = _cabi.load().es_b200_check_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(raw))
        if rc != 0:
            raise SystemExit(f"device-side status {raw.value:#x}: a bounded wait gave up; the timing is invalid")

    # ---- reduce over ranks: slowest rank's time, summed work
    flops_local = 2.0 * float(counts.sum()) * N * K
    stats = torch.tensor([elapsed_ms, e2e[0] if e2e else 0.0], dtype=torch.float64, device=device)
    sums = torch.tensor([flops_local, float(e2e[1]) if e2e else 0.0, float(e2e[2]) if e2e else 0.0],
                        dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    elapsed_ms, e2e_ms = float(stats[0]), float(stats[1])
    flops_total, h2d_total, d2h_total = float(sums[0]), float(sums[1]), float(sums[2])

    # one call launches the streaming kernel (both shapes in one launch), the CTA-pair kernel when the host-known row
    # count can reach its bucket (>= 113 rows at most shapes), and a leading capped CTA-pair launch when the call is split
    # (256 rows or more)
    rows_local = int(counts.sum())
    launches_per_step = 1 + (rows_local >= 113) + (rows_local >= 256)
    line = None
    if rank == 0:
        ms_per_step = elapsed_ms / args.steps
        value = flops_total / (ms_per_step * 1e-3) / 1e12
        peak, peak_kind = peak_hbm()
        # roofline of the call's kernel chain, rank 0's launch: algorithmic bytes of rank 0's shard / its own time
        abytes = algorithmic_bytes(counts, N, K)
        achieved = abytes / (my_ms * 1e-3) / 1e9
        traffic = read_traffic(f"{args.workload}_n{world}")
        line = {
            "metric": metric, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "mxfp8_e4m3", "data": "synthetic",
            "config": config,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_kind": peak_kind, "algorithmic_bytes": abytes,
                         "kernel": ("mxfp8_grouped_mm_pair_kernel (capped) | mxfp8_grouped_mm_kernel (32- and 112-token "
                                    "shapes in one launch) | mxfp8_grouped_mm_pair_kernel: one PDL chain per call, "
                                    "buckets side by side"
                                    if launches_per_step == 3 else "mxfp8_grouped_mm_kernel chain"),
                         "kernel_ms": my_ms},
            "clocks": clocks, "gpu_launches": args.steps * launches_per_step, "host_us_per_call": host_us,
        }
        if ref is not None:
            line["impl"] = "reference"
            line["reference_kind"] = ("gpu_kernel: the reference's own SM100 CUTLASS grouped GEMM, unmodified sources "
                                      "built by oracle/build_ref.sh, called through its torch op")
            line["roofline"]["kernel"] = "reference CUTLASS kernel (pre-compute + grouped GEMM)"
            line["gpu_launches"] = args.steps * 2
        if e2e:
            e2e_step_ms = e2e_ms / args.steps
            line["e2e"] = {"value": flops_total / (e2e_step_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                           "h2d_bytes_per_step": int(h2d_total), "d2h_bytes_per_step": int(d2h_total),
                           "ms_per_step": e2e_step_ms}
        if world == 1 and ref is None and not args.no_reference_gpu:
            ref_side = reference_ops()
            if ref_side is not None:
                line["reference_gpu"] = compare_with_reference_kernel(
                    wl, our_mm, ref_side.es_sm100_mxfp8_blockscaled_grouped_mm, device)
        if world == 1 and not args.no_cpu_baseline:
            r, cores, sdesc = cpu_reference_rate(counts_all, N, K, seed=100, budget_s=args.cpu_budget)
            line["cpu_baseline"] = {"value": r, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sdesc}
            if ref is None:
                line["cpu_baseline"]["gpu_result_check"] = oracle_spot_check(wl, counts, N, K)
    del wl
    torch.cuda.empty_cache()
    # N > 1, default workload: the expert-parallel layer (dispatch / combine over peer memory) rides along, outside the
    # headline's timed region, so that a multi-GPU record also carries the exchange
    if world > 1 and args.workload == "gate_up" and ref is None and args.ep_layer_steps > 0:
        ep_args = argparse.Namespace(**vars(args))
        ep_args.workload, ep_args.steps, ep_args.warmup = "qwen3_ep", args.ep_layer_steps, 3
        ep_line = bench_ep_layer(ep_args, device, rank, world, dist)
        if rank == 0:
            line["ep_layer"] = {k: ep_line[k] for k in ("ms_per_step", "value", "unit", "device_status")}
            line["ep_layer"]["workload"] = ep_line["config"]["workload"]
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
