"""GPU parity of the MXFP8 grouped GEMM at the sizes of the two benchmark configurations:

    gate_up  E=256, 32768 routed rows split by Zipf(1.2), N=4096, K=7168   (one expert of 8409 rows: 22 CTA-pair items
             of 384 rows, 56 K steps through the 5-stage ring, two sub-tiles and three scale atoms per item)
    down     E=256, 512 routed rows (147 empty experts, most others 1-3 rows), N=7168, K=2048

Operands are built on the device with the grouped quant op (bit-exact against the oracle in test_quant_gpu.py).  The
whole output is too large to evaluate on the CPU in test time, so the oracle (dequantise + fp32 matmul,
oracle/grouped_gemm_oracle.py) is evaluated on a SAMPLE: the largest expert (its first rows, the rows around the
sub-tile boundary 380..390, its last partial item), one expert of 33..128 rows, three of at most 32 rows including the
smallest, each at the first and the last 128-column tile of N.  Tolerances (floating point, the build target's):
relative error <= 1e-2, cosine >= 0.9999.  Buffer rows that belong to no expert must stay untouched, the device status
word must be clean, and every call must leave the work counters in the scratch zeroed.  Where the reference's own
kernel was built (oracle/_ref, single-GPU boxes only) the whole output is also compared with the reference kernel's:
bit for bit where the accumulation order is the reference's, to two ulps elsewhere.
"""
from pathlib import Path

import numpy as np
import pytest
import torch

import bench
from oracle import grouped_gemm_oracle as G
from oracle import mxfp8_quant_oracle as Q
from tests import _cases as C

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
REL_TOL, COS_TOL = 1e-2, 0.9999
CANARY_ROWS = 8


def _workload(name):
    E, T, N, K, _ = bench.WORKLOADS[name]
    counts = bench.zipf_counts(T, E, 1.2, 0)
    dev = torch.device("cuda", 0)
    wl = bench.build_device_workload(counts, N, K, dev, seed=4242)
    # rows past the last expert: inputs are zero, outputs must not be written
    a = torch.zeros((T + CANARY_ROWS, K), dtype=torch.uint8, device=dev)
    a[:T] = wl["a"].view(torch.uint8)
    wl["a"] = a.view(torch.float8_e4m3fn)
    wl["counts"], wl["dims"] = counts, (E, T, N, K)
    return wl


@pytest.fixture(scope="module")
def gate_up():
    wl = _workload("gate_up")
    yield wl
    wl.clear()
    torch.cuda.empty_cache()


@pytest.fixture(scope="module")
def down():
    wl = _workload("down")
    yield wl
    wl.clear()
    torch.cuda.empty_cache()


def _run(wl, out_dtype):
    from expert_specialization_moe_b200 import es_sm100_mxfp8_blockscaled_grouped_mm as mm
    E, T, N, K = wl["dims"]
    d = torch.full((T + CANARY_ROWS, N), 3.0, dtype=out_dtype, device=wl["a"].device)
    mm(d, wl["a"], wl["b"], wl["sfa"], wl["sfb"], wl["ps"], wl["eo"], wl["bo"])
    torch.cuda.synchronize()
    return d


def _oracle_block(wl, e, rows, n_lo, n_hi, out_dtype):
    """Oracle value of d[expert e, rows, n_lo:n_hi] (rows = indices inside the expert)."""
    E, T, N, K = wl["dims"]
    m = int(wl["counts"][e])
    off, bo = int(wl["eo_h"][e]), int(wl["bo_h"][e])
    kb = K // 32
    rows_t = torch.as_tensor(rows, dtype=torch.int64)
    a = wl["a"].view(torch.uint8)[off + rows_t.to(wl["a"].device)].cpu()
    sf_idx = torch.from_numpy(Q.sf_swizzled_offsets(m, K))[rows_t] + bo * kb
    sa = wl["sfa"].reshape(-1)[sf_idx.to(wl["sfa"].device)].cpu()
    w = wl["w"].view(torch.uint8)[e, n_lo:n_hi].cpu()
    sfb_idx = torch.from_numpy(Q.sf_swizzled_offsets(N, K))[n_lo:n_hi] + e * N * kb
    sb = wl["sfb"].reshape(-1)[sfb_idx.to(wl["sfb"].device)].cpu()
    return torch.mm(G.dequant_mxfp8(a, sa), G.dequant_mxfp8(w, sb).t()).to(out_dtype)


def _sample(counts):
    """(expert, row indices inside the expert) pairs: see the module docstring."""
    counts = np.asarray(counts)
    picks = []
    big = int(np.argmax(counts))
    m = int(counts[big])
    if m > 32:
        rows = list(range(0, min(m, 8)))
        if m > 390:
            rows += list(range(380, 390))
        last_item = (m - 1) // 384 * 384
        rows += list(range(max(last_item - 2, 0), min(last_item + 6, m))) + list(range(max(m - 4, 0), m))
        picks.append((big, sorted(set(rows))))
    mid = [int(e) for e in np.argsort(-counts) if 33 <= counts[e] <= 128]
    if mid:
        e = mid[0]
        picks.append((e, list(range(int(counts[e])))))
    small = [int(e) for e in np.argsort(counts) if 1 <= counts[e] <= 32]
    for e in (small[:1] + small[len(small) // 2:len(small) // 2 + 1] + small[-1:]):
        picks.append((e, list(range(int(counts[e])))))
    return picks


def _check(wl, d, out_dtype):
    E, T, N, K = wl["dims"]
    picks = _sample(wl["counts"])
    assert len(picks) >= 3
    for e, rows in picks:
        off = int(wl["eo_h"][e])
        idx = torch.as_tensor(rows, dtype=torch.int64, device=d.device) + off
        for n_lo in (0, N - 128):
            ref = _oracle_block(wl, e, rows, n_lo, n_lo + 128, out_dtype)
            got = d[idx, n_lo:n_lo + 128].cpu()
            rel, cos = G.rel_err_and_cosine(got.float(), ref.float())
            assert rel <= REL_TOL and cos >= COS_TOL, \
                f"expert {e} (m={int(wl['counts'][e])}), columns {n_lo}..: rel={rel:.3e} cos={cos:.6f}"
    assert bool((d[T:] == 3.0).all()), "rows that belong to no expert were written"
    assert bool(torch.isfinite(d[:T].float()).all())
    rc, raw = C.device_status()
    assert rc == 0, f"device status {raw:#x}"


def _reference_ops():
    lib = ROOT / "oracle" / "_ref" / "libes_reference.so"
    if not lib.exists() or torch.cuda.device_count() != 1:
        return None
    torch.ops.load_library(str(lib))
    return torch.ops.expert_specialization


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_gate_up_config_matches_the_oracle_on_a_sample(gate_up, out_dtype):
    d = _run(gate_up, out_dtype)
    _check(gate_up, d, out_dtype)
    d2 = _run(gate_up, out_dtype)                       # same call again: counters were reset, result is deterministic
    assert torch.equal(d, d2)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float16])
def test_down_config_matches_the_oracle_on_a_sample(down, out_dtype):
    d = _run(down, out_dtype)
    _check(down, d, out_dtype)
    # every non-empty expert of the decode configuration is small enough to check in full at one column tile
    E, T, N, K = down["dims"]
    for e in np.nonzero(down["counts"])[0][::7]:
        rows = list(range(int(down["counts"][e])))
        ref = _oracle_block(down, int(e), rows, 3584, 3712, out_dtype)
        off = int(down["eo_h"][e])
        rel, cos = G.rel_err_and_cosine(d[off:off + len(rows), 3584:3712].cpu().float(), ref.float())
        assert rel <= REL_TOL and cos >= COS_TOL, f"expert {e}: rel={rel:.3e} cos={cos:.6f}"


@pytest.mark.parametrize("name", ["gate_up", "down"])
def test_output_against_the_reference_kernels_whole_output(name, request):
    """Whole output against the reference's own CUTLASS kernel on the same operands.  Experts on the CTA-pair kernel
    (113 rows and more) accumulate every product in the reference's order: bit-identical.  Experts on the streaming
    shapes add two or four partial accumulators at the end, so a few outputs round differently: at least 99.9 %
    bit-identical, the rest within two bf16 ulps (2^-7 relative) or 1e-5 absolute."""
    ref = _reference_ops()
    if ref is None:
        pytest.skip("the reference's own kernel is only built and run on single-GPU boxes")
    wl = request.getfixturevalue(name)
    E, T, N, K = wl["dims"]
    d = _run(wl, torch.bfloat16)
    d_ref = torch.full_like(d, 3.0)
    ref.es_sm100_mxfp8_blockscaled_grouped_mm(wl["a"], wl["b"], wl["sfa"], wl["sfb"], d_ref, wl["ps"], wl["eo"],
                                              wl["bo"])
    torch.cuda.synchronize()
    counts = torch.from_numpy(np.asarray(wl["counts"])).to(d.device)
    heavy_row = torch.repeat_interleave(counts >= 113, counts)
    same = d[:T].view(torch.int16) == d_ref[:T].view(torch.int16)
    if bool(heavy_row.any()):
        assert bool(same[heavy_row].all()), "CTA-pair experts differ from the reference kernel"
    light = ~heavy_row
    if bool(light.any()):
        frac = float(same[light].float().mean())
        assert frac >= 0.999, f"only {frac:.5f} of the streaming experts' outputs equal the reference kernel's"
        x, y = d[:T][light].float(), d_ref[:T][light].float()
        # (outputs are O(1); near a zero of the sum the fp32 rounding of the partial sums, ~1e-7, can move a tiny result
        # by several of ITS ulps, hence the absolute term)
        assert bool(((x - y).abs() <= y.abs() * 2.0 ** -7 + 1e-5).all())


def test_split_and_unsplit_calls_agree(gate_up):
    """The same call with the buckets side by side (work counters) and one after the other (no scratch semantics):
    per-tile arithmetic does not depend on which CTA ran the tile."""
    from expert_specialization_moe_b200 import _cabi
    d_split = _run(gate_up, torch.bfloat16)
    _cabi.set_tunable("mm_dynamic", 0)
    try:
        d_serial = _run(gate_up, torch.bfloat16)
    finally:
        _cabi.set_tunable("mm_dynamic", 1)
    assert torch.equal(d_split, d_serial)
    rc, raw = C.device_status()
    assert rc == 0, f"device status {raw:#x}"


def test_order_of_the_streaming_shapes_does_not_change_the_output(gate_up):
    """The two single-CTA shapes share one launch; how many CTAs of the 112-token shape get the lowest CTA indices (and
    so start first) is a tunable and must not change a bit of the result."""
    from expert_specialization_moe_b200 import _cabi
    lib = _cabi.load()
    outs = []
    try:
        for lead in (0, 20, 100000):              # none, a few, all of them
            _cabi.set_tunable("mm_stream_mid_lead_ctas", lead)
            outs.append(_run(gate_up, torch.bfloat16))
    finally:
        lib.es_b200_set_tunable(b"mm_stream_mid_lead_ctas", -1)      # back to the built-in default (see below)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    rc, raw = C.device_status()
    assert rc == 0, f"device status {raw:#x}"


def test_c_abi_call_with_caller_scratch_leaves_the_work_counters_zeroed(gate_up):
    """Straight through the C ABI with the caller's own scratch: same output as the torch operator, and the scratch
    is all zero again after every call (which is what lets one buffer serve every call on a stream)."""
    from expert_specialization_moe_b200 import _cabi
    lib = _cabi.load()
    wl = gate_up
    E, T, N, K = wl["dims"]
    want = _run(wl, torch.bfloat16)
    nbytes = int(lib.es_b200_grouped_mm_scratch_bytes(E, T, N, K))
    scratch = torch.zeros(nbytes, dtype=torch.uint8, device=want.device)
    stream = torch.cuda.current_stream(want.device).cuda_stream
    for _ in range(2):
        d = torch.full_like(want, 3.0)
        rc = lib.es_b200_mxfp8_grouped_mm(wl["a"].data_ptr(), wl["w"].data_ptr(), wl["sfa"].data_ptr(),
                                          wl["sfb"].data_ptr(), d.data_ptr(), _cabi.BF16, wl["ps"].data_ptr(),
                                          wl["eo"].data_ptr(), wl["bo"].data_ptr(), E, T + CANARY_ROWS, N, K,
                                          wl["sfa"].numel() // (K // 32), scratch.data_ptr(), nbytes, stream)
        assert rc == 0, lib.es_b200_last_error().decode()
        torch.cuda.synchronize()
        assert int(scratch.view(torch.int32).abs().sum()) == 0, "work counters were not left zeroed"
        assert torch.equal(d, want)
    # too small a scratch is refused before anything is launched
    rc = lib.es_b200_mxfp8_grouped_mm(wl["a"].data_ptr(), wl["w"].data_ptr(), wl["sfa"].data_ptr(), wl["sfb"].data_ptr(),
                                      want.data_ptr(), _cabi.BF16, wl["ps"].data_ptr(), wl["eo"].data_ptr(),
                                      wl["bo"].data_ptr(), E, T + CANARY_ROWS, N, K, wl["sfa"].numel() // (K // 32),
                                      scratch.data_ptr(), 8, stream)
    assert rc == 4 and b"scratch" in lib.es_b200_last_error()
    rc, raw = C.device_status()
    assert rc == 0, f"device status {raw:#x}"


def test_misaligned_blockscale_offset_is_reported_and_skipped():
    """blockscale_offsets must be multiples of 128 rows (they are cumulative round-ups).  An expert whose offset is not
    cannot be addressed by the scale loads: its rows are left unwritten, the status word says so, nothing faults."""
    inp = C.mxfp8_gemm_inputs([40, 200, 20], 256, 256, seed=5)
    good = C.run_mxfp8_mm_op(inp, fill=5.0)
    rc, raw = C.device_status()
    assert rc == 0
    assert list(inp["bo"]) == [0, 128, 384]
    from expert_specialization_moe_b200 import _cabi
    epoch = int(_cabi.load().es_b200_error_epoch())
    bad = dict(inp, bo=np.array([0, 192, 384], dtype=np.int32))       # expert 1: 64 rows off an atom
    d = C.run_mxfp8_mm_op(bad, fill=5.0)
    rc, raw = C.device_status()
    assert rc != 0 and (raw & 0x80)
    assert int(_cabi.load().es_b200_error_epoch()) == epoch + 1       # owners of scratch buffers re-zero them on this
    assert torch.equal(d[:40], good[:40]) and torch.equal(d[240:], good[240:])
    assert bool((d[40:240] == 5.0).all())
    rc, raw = C.device_status()
    assert rc == 0
    assert torch.equal(C.run_mxfp8_mm_op(inp, fill=5.0), good)         # the next call is unaffected
