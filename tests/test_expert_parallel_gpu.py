"""Two-GPU test of the expert-parallel layer: NCCL all-to-all dispatch -> grouped quant -> gate_up grouped GEMM ->
SiLU*mul -> grouped quant -> down grouped GEMM -> all-to-all combine, against an unquantised fp32 evaluation of the
same layer.  Floating point: calc_diff < 5e-3 (two chained MXFP8 GEMMs; the reference's single-GEMM tests use 1e-3)."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        from expert_specialization_moe_b200 import expert_parallel as ep
        from oracle.grouped_gemm_oracle import calc_diff

        E, topk, H, I, tokens = 8, 2, 256, 128, 300
        dev = torch.device("cuda", rank)
        gw = torch.Generator(device=dev).manual_seed(1)            # same weights on every rank
        w1 = (torch.randn((E, 2 * I, H), generator=gw, device=dev) * 0.05).to(torch.bfloat16)
        w2 = (torch.randn((E, H, I), generator=gw, device=dev) * 0.05).to(torch.bfloat16)
        g = torch.Generator(device=dev).manual_seed(10 + rank)
        x = torch.randn((tokens, H), generator=g, device=dev).to(torch.bfloat16)
        p = torch.softmax(torch.randn((tokens, E), generator=g, device=dev), -1)
        wts, ids = torch.topk(p, topk, dim=-1)
        wts = wts / wts.sum(-1, keepdim=True)
        e_local = E // world
        shard = ep.ExpertShard(w1[rank * e_local:(rank + 1) * e_local].contiguous(),
                               w2[rank * e_local:(rank + 1) * e_local].contiguous())
        out = ep.moe_forward(x, ids, wts, E, shard.forward)
        torch.cuda.synchronize()
        # unquantised evaluation of my tokens
        ref = torch.zeros((tokens, H), dtype=torch.float32, device=dev)
        for kk in range(topk):
            for e in range(E):
                sel = ids[:, kk] == e
                if sel.any():
                    h = x[sel].float() @ w1[e].float().t()
                    a = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
                    ref[sel] += wts[sel, kk:kk + 1] * (a @ w2[e].float().t())
        q.put((rank, float(calc_diff(out.float().cpu(), ref.cpu())), None))
        dist.destroy_process_group()
    except Exception:
        import traceback
        q.put((rank, None, traceback.format_exc()))


def _worker_fused(rank, world, port, q):
    """Fused exchange (peer-memory dispatch / combine) against the all-to-all path on the same inputs."""
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        from expert_specialization_moe_b200 import expert_parallel as ep
        from expert_specialization_moe_b200 import es_sm100_mxfp8_blockscaled_grouped_quant as quant
        from expert_specialization_moe_b200 import _cabi
        import ctypes

        E, topk, H, I, tokens = 8, 2, 256, 128, 300
        dev = torch.device("cuda", rank)
        gw = torch.Generator(device=dev).manual_seed(1)
        w1 = (torch.randn((E, 2 * I, H), generator=gw, device=dev) * 0.05).to(torch.bfloat16)
        w2 = (torch.randn((E, H, I), generator=gw, device=dev) * 0.05).to(torch.bfloat16)
        e_local = E // world
        shard = ep.ExpertShard(w1[rank * e_local:(rank + 1) * e_local].contiguous(),
                               w2[rank * e_local:(rank + 1) * e_local].contiguous())
        fx = ep.FusedExchange(E, topk, tokens, H, dev)
        worst = 0.0
        for it in range(3):                       # several rounds: the receive buffers and flags are reused
            g = torch.Generator(device=dev).manual_seed(10 + rank + 100 * it)
            x = torch.randn((tokens, H), generator=g, device=dev).to(torch.bfloat16)
            p = torch.softmax(torch.randn((tokens, E), generator=g, device=dev), -1)
            wts, ids = torch.topk(p, topk, dim=-1)
            wts = wts / wts.sum(-1, keepdim=True)
            # all-to-all path
            plan = ep.make_plan(ids, E)
            rows = ep.dispatch(x, plan)
            ps, eo, bo, sf_rows = plan.problem_tensors(2 * I, H)
            a_ref = torch.empty((rows.shape[0], H), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
            sf_ref = torch.zeros((max(sf_rows, 128), H // 32), dtype=torch.uint8, device=dev)
            quant(rows, ps, eo, bo, a_ref, sf_ref)
            out_ref = ep.combine(shard.forward(rows, plan), plan, wts)
            # fused path
            fplan = fx.plan(ids)
            # the device-side routing kernels against the same arithmetic in torch
            cnt = torch.bincount(ids.reshape(-1), minlength=E)
            cnt_all = torch.empty((world, E), dtype=cnt.dtype, device=dev)
            dist.all_gather_into_tensor(cnt_all, cnt)
            want = ep.routing_tables(ids, cnt_all, rank, H)
            for key, val in want.items():
                assert torch.equal(fplan[key].to(val.dtype), val), f"routing table {key} differs"
            a, sfa = fx.dispatch(x, fplan)
            torch.cuda.synchronize()
            n = rows.shape[0]
            assert int(fplan["total_rows"]) == n
            assert torch.equal(fplan["expert_offsets"], eo) and torch.equal(fplan["blockscale_offsets"], bo)
            assert torch.equal(a[:n].view(torch.uint8), a_ref.view(torch.uint8)), "dispatched codes differ"
            # scale bytes of valid rows: compare through the row -> offset map of the swizzled layout
            kt = H // 128
            counts = fplan["rows"].tolist()
            for le, m in enumerate(counts):
                r = torch.arange(m, device=dev)
                base = int(bo[le]) * (H // 32) + (r // 128) * kt * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4
                idx = (base.unsqueeze(1) + torch.arange(kt, device=dev).unsqueeze(0) * 512).unsqueeze(2) \
                    + torch.arange(4, device=dev).view(1, 1, 4)
                assert torch.equal(sfa.reshape(-1)[idx], sf_ref.reshape(-1)[idx]), f"scales of local expert {le} differ"
            for fuse in (False, True):            # combine as its own kernel / fused into the down GEMM's epilogue
                out = fx.forward(x, ids, wts, shard, fuse_combine=fuse)
                torch.cuda.synchronize()
                worst = max(worst, float((out.float() - out_ref.float()).abs().max()
                                         / out_ref.float().abs().max().clamp_min(1e-6)))
                if fuse:
                    assert torch.equal(out, out_unfused), "fused and unfused combine differ"
                out_unfused = out
        # the same layer as two half-batches on two streams: the same values up to fp32 summation order (an expert's
        # rows split in two may fall into another row-count bucket, which adds its partial accumulators differently)
        px = ep.PipelinedExchange(E, topk, tokens, H, dev)
        out_p = px.forward(x, ids, wts, shard)
        torch.cuda.synchronize()
        d_p = float((out_p.float() - out.float()).abs().max() / out.float().abs().max().clamp_min(1e-6))
        assert d_p < 1e-2, f"pipelined and single-stream exchange differ by {d_p}"
        raw = ctypes.c_uint32(0)
        rc = _cabi.load().es_b200_check_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(raw))
        q.put((rank, worst if rc == 0 else float("inf"), None))
        dist.destroy_process_group()
    except Exception:
        import traceback
        q.put((rank, None, traceback.format_exc()))


def test_two_gpu_fused_exchange():
    """Peer-memory dispatch (quantise once, push codes + scales + return address) and combine against the all-to-all
    path: dispatched codes and scales bit-identical, layer output equal up to the summation order of the top-k rows."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_fused, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, err, tb in res:
        assert tb is None, f"rank {rank}:\n{tb}"
        assert err < 1e-2, f"rank {rank}: relative max difference {err}"


def test_two_gpu_moe_layer():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, diff, tb in res:
        assert tb is None, f"rank {rank}:\n{tb}"
        assert diff < 5e-3, f"rank {rank}: calc_diff {diff}"


def test_route_tables_cut_rows_at_the_capacity():
    """More rows routed to a GPU than its receive buffers hold (one GPU, through the C ABI): the problem description
    handed to the GEMMs stops at the capacity, the surplus pairs keep destinations past it (which the dispatch kernel
    skips), and es_b200_check_status reports the overflow once."""
    import ctypes
    from expert_specialization_moe_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    E, tokens, topk, H, capacity = 8, 64, 2, 256, 100
    g = torch.Generator(device=dev).manual_seed(3)
    ids = torch.randint(0, E, (tokens, topk), generator=g, device=dev, dtype=torch.int64)
    pairs = tokens * topk
    i32 = lambda *s: torch.zeros(s, dtype=torch.int32, device=dev)
    seg_counts, seg_base, counts_all = i32(256, E), i32(256, E), i32(1, E)
    dst_rank, dst_row, rows, eo, bo, total = i32(pairs), i32(pairs), i32(E), i32(E), i32(E), i32(1)
    sf_off = torch.zeros(pairs, dtype=torch.int64, device=dev)
    table = (ctypes.c_void_p * 1)(counts_all.data_ptr())
    stream = torch.cuda.current_stream(dev).cuda_stream
    raw = ctypes.c_uint32(0)
    lib.es_b200_check_status(stream, ctypes.byref(raw))          # start from a clean status word
    assert lib.es_b200_ep_route_count(ids.data_ptr(), 1, pairs, E, seg_counts.data_ptr(), seg_base.data_ptr(), table,
                                      0, 1, stream) == 0
    assert lib.es_b200_ep_route_tables(ids.data_ptr(), 1, pairs, E, seg_base.data_ptr(), counts_all.data_ptr(), 0, 1, H,
                                       dst_rank.data_ptr(), dst_row.data_ptr(), sf_off.data_ptr(), rows.data_ptr(),
                                       eo.data_ptr(), bo.data_ptr(), total.data_ptr(), capacity, stream) == 0
    assert lib.es_b200_check_status(stream, ctypes.byref(raw)) != 0 and raw.value != 0
    assert lib.es_b200_check_status(stream, ctypes.byref(raw)) == 0
    assert int(total) == capacity and int(rows.sum()) == capacity
    counts = torch.bincount(ids.reshape(-1), minlength=E)
    assert torch.equal(eo.to(torch.int64), torch.cumsum(counts, 0) - counts)       # offsets are those of the full problem
    assert bool(((rows == 0) | ((eo + rows) <= capacity)).all())
    assert int((dst_row >= capacity).sum()) == pairs - capacity
    assert sorted(dst_row.tolist()) == list(range(pairs))
