"""CPU tests of the benchmark's host logic: expert sharding for N > 1, algorithmic byte counts, and the reference arm
(`--impl reference`), which runs the CPU path on a bounded sample and prints the contract's JSON line."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_shard_counts_partition_all_experts():
    counts = bench.zipf_counts(32768, 256, 1.2, 0)
    for world in (1, 2, 4, 8):
        for placement in ("contiguous", "balanced"):
            shards = bench.shard_counts(counts, world, placement)
            assert len(shards) == world and all(len(s) == 256 // world for s in shards)
            assert sum(int(s.sum()) for s in shards) == 32768
            assert sorted(np.concatenate(shards).tolist()) == sorted(counts.tolist())
    cont = [int(s.sum()) for s in bench.shard_counts(counts, 8, "contiguous")]
    bal = [int(s.sum()) for s in bench.shard_counts(counts, 8, "balanced")]
    assert cont == [4893, 1987, 2040, 5036, 11822, 1130, 957, 4903]
    assert max(bal) < max(cont) and max(bal) >= counts.max()


def test_algorithmic_bytes():
    counts = np.array([0, 3, 130])
    N, K = 256, 512
    T, act = 133, 2
    assert bench.algorithmic_bytes(counts, N, K) == T * K + T * K // 32 + act * N * K + act * N * K // 32 + 2 * T * N
    # the headline workload: 8.26 GB
    c = bench.zipf_counts(32768, 256, 1.2, 0)
    assert bench.algorithmic_bytes(c, 4096, 7168) == 8261730304


def test_offsets_layout():
    ps, eo, bo, rows = bench.offsets([5, 0, 130], 64, 128)
    assert eo.tolist() == [0, 5, 5] and bo.tolist() == [0, 128, 128] and rows == 128 + 256
    assert ps.tolist() == [[5, 64, 128], [0, 64, 128], [130, 64, 128]]


def test_reference_arm_prints_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                          "--cpu-budget", "0.25", "--workload", "down"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    for key in ("metric", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "dtype", "data",
                "config"):
        assert key in line


def test_load_balanced_placement_replicates_the_hottest_expert_and_keeps_every_row():
    counts = bench.zipf_counts(32768, 256, 1.2, 0)
    for world in (2, 4, 8):
        shards, note = bench.place_experts(counts, world, "load_balanced", 4096, 7168)
        assert len(shards) == world and len({len(s) for s in shards}) == 1          # same number of expert slots
        assert sum(int(s.sum()) for s in shards) == 32768                            # replicas split rows, none lost
        rows = [int(s.sum()) for s in shards]
        contiguous = [int(s.sum()) for s in bench.place_experts(counts, world, "contiguous", 4096, 7168)[0]]
        assert max(rows) <= max(contiguous)
        fair = 32768 // world
        assert max(int(s.max()) for s in shards) <= max(fair, int(counts.max()) // 2 + 1)
    shards8, note8 = bench.place_experts(counts, 8, "load_balanced", 4096, 7168)
    assert "1 expert(s)" in note8 and max(int(s.sum()) for s in shards8) < 5000       # 11822 rows under contiguous


def test_reference_benchmark_row_distribution():
    c = bench.ref_dist_counts(4096, seed=3)
    assert c.min() >= 1 and c.max() <= 1024
    share = [(c <= 32).mean(), ((c >= 32) & (c <= 64)).mean(), ((c >= 64) & (c <= 128)).mean(), (c >= 128).mean()]
    assert abs(share[0] - 0.70) < 0.03 and abs(share[3] - 0.05) < 0.015
