"""Expert-parallel exchange on ONE GPU (the two-GPU tests of test_expert_parallel_gpu.py are skipped on a one-GPU box).

* FusedExchange / PipelinedExchange with a process group of one, at the dimensions of the Qwen3-30B-A3B layer (E=128,
  top-8, hidden 2048, intermediate 768, 2048 tokens): routing kernels against the same arithmetic in torch
  (expert_parallel.routing_tables), the layer against an unquantised fp32 evaluation (floating point: calc_diff < 5e-3,
  two chained MXFP8 GEMMs; the reference's single-GEMM tests use 1e-3), both combine modes.  This runs ep_route,
  dispatch_quant_push, unpack_side, the scatter epilogue of the grouped GEMM and its K=768 CTA-pair path.
* Two ranks EMULATED on one GPU through the C ABI: two sets of buffers, every step issued for rank 0 then rank 1 on
  one stream (stream order stands in for the barrier kernel, which must never wait for a launch of the same GPU).
  Routing tables against routing_tables() with world = 2, then the whole layer against the fp32 evaluation.
* The barrier's bounded wait made to run out: rank 0 of a world of two whose partner never arrives, with a 20 ms limit.
  The kernel returns, the status word reports the barrier bit once, nothing faults and the next check is clean.
* A pair dropped at dispatch (receive buffer full) contributes 0 to the weighted sum, not a stale row.
"""
import ctypes
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

ERR_BAD_DESTINATION, ERR_BARRIER_TIMEOUT = 0x10000, 0x20000


def _layer_reference(x, ids, wts, w1, w2):
    """Unquantised fp32 evaluation of the MoE layer on the tokens' device."""
    tokens, H = x.shape
    I = w2.shape[2]
    ref = torch.zeros((tokens, H), dtype=torch.float32, device=x.device)
    for e in range(w1.shape[0]):
        tok, j = torch.nonzero(ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        h = x[tok].float() @ w1[e].float().t()
        a = torch.nn.functional.silu(h[:, :I]) * h[:, I:]
        ref.index_add_(0, tok, wts[tok, j].unsqueeze(1).float() * (a @ w2[e].float().t()))
    return ref


def _status(lib, dev):
    raw = ctypes.c_uint32(0)
    rc = lib.es_b200_check_status(torch.cuda.current_stream(dev).cuda_stream, ctypes.byref(raw))
    return rc, raw.value


@pytest.fixture(scope="module")
def group_of_one():
    import torch.distributed as dist
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1, device_id=dev)
    yield dev
    dist.destroy_process_group()


def test_fused_exchange_layer_on_one_gpu(group_of_one):
    from expert_specialization_moe_b200 import _cabi
    from expert_specialization_moe_b200 import expert_parallel as ep
    from oracle.grouped_gemm_oracle import calc_diff
    dev = group_of_one
    lib = _cabi.load()
    E, topk, H, I, tokens = 128, 8, 2048, 768, 2048
    g = torch.Generator(device=dev).manual_seed(21)
    w1 = (torch.randn((E, 2 * I, H), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    w2 = (torch.randn((E, H, I), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    shard = ep.ExpertShard(w1, w2)
    fx = ep.FusedExchange(E, topk, tokens, H, dev)
    px = ep.PipelinedExchange(E, topk, tokens, H, dev)
    _status(lib, dev)
    for it in range(2):                                   # twice: receive buffers, flags and counters are reused
        g.manual_seed(100 + it)
        x = torch.randn((tokens, H), generator=g, device=dev).to(torch.bfloat16)
        logits = torch.randn((tokens, E), generator=g, device=dev)
        logits[:, 5] += 3.0                               # one expert with several hundred rows: CTA-pair tiles
        wts, ids = torch.topk(torch.softmax(logits, -1), topk, dim=-1)
        wts = (wts / wts.sum(-1, keepdim=True)).float()
        plan = fx.plan(ids)
        counts = torch.bincount(ids.reshape(-1), minlength=E).view(1, E)
        want = ep.routing_tables(ids, counts, 0, H)
        for key, val in want.items():
            assert torch.equal(plan[key].to(val.dtype), val), f"routing table {key} differs"
        assert int(plan["rows"].max()) > 384
        ref = _layer_reference(x, ids, wts, w1, w2)
        outs = []
        for fuse in (False, True):
            out = fx.forward(x, ids, wts, shard, fuse_combine=fuse)
            torch.cuda.synchronize()
            diff = calc_diff(out.float().cpu(), ref.cpu())
            assert diff < 5e-3, f"fuse_combine={fuse}: calc_diff {diff}"
            outs.append(out)
        assert torch.equal(outs[0], outs[1]), "combine kernel and scatter epilogue disagree"
        # two half-batches: an expert's rows split in two may fall into another row-count bucket, whose kernel adds its
        # partial accumulators in another order — same values up to fp32 summation order
        out_p = px.forward(x, ids, wts, shard)
        torch.cuda.synchronize()
        assert calc_diff(out_p.float().cpu(), outs[1].float().cpu()) < 1e-5, "two half-batches disagree with one batch"
    rc, raw = _status(lib, dev)
    assert rc == 0, f"device status {raw:#x}"


class _EmulatedRank:
    """Buffers of one rank of an emulated world (all on one GPU)."""

    def __init__(self, lib, rank, world, E, topk, tokens, H, dev):
        self.lib, self.rank, self.world, self.E, self.topk, self.tokens, self.H, self.dev = \
            lib, rank, world, E, topk, tokens, H, dev
        self.e_local = E // world
        self.capacity = world * tokens * topk
        self.side_bytes = int(lib.es_b200_ep_side_record_bytes(H))
        u8 = lambda *s: torch.zeros(s, dtype=torch.uint8, device=dev)
        i32 = lambda *s: torch.zeros(s, dtype=torch.int32, device=dev)
        self.codes, self.side = u8(self.capacity, H), u8(self.capacity, self.side_bytes)
        self.scale_rows = (self.capacity + 128 * self.e_local + 127) // 128 * 128
        self.scales = u8(self.scale_rows, H // 32)
        self.meta = i32(self.capacity, 2)
        self.pairs = torch.zeros((tokens * topk, H), dtype=torch.bfloat16, device=dev)
        self.counts_all = i32(world, E)
        self.seg_counts, self.seg_base = i32(256, E), i32(256, E)
        p = tokens * topk
        self.t = {"dst_rank": i32(p), "dst_row": i32(p), "dst_scale_offset": torch.zeros(p, dtype=torch.int64, device=dev),
                  "rows": i32(self.e_local), "expert_offsets": i32(self.e_local),
                  "blockscale_offsets": i32(self.e_local), "total_rows": i32(1)}
        self.work = {}


def test_two_emulated_ranks_on_one_gpu():
    from expert_specialization_moe_b200 import _cabi
    from expert_specialization_moe_b200 import expert_parallel as ep
    from oracle.grouped_gemm_oracle import calc_diff
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    world, E, topk, H, I, tokens = 2, 16, 4, 512, 256, 700
    g = torch.Generator(device=dev).manual_seed(33)
    w1 = (torch.randn((E, 2 * I, H), generator=g, device=dev) * 0.03).to(torch.bfloat16)
    w2 = (torch.randn((E, H, I), generator=g, device=dev) * 0.03).to(torch.bfloat16)
    el = E // world
    shards = [ep.ExpertShard(w1[r * el:(r + 1) * el].contiguous(), w2[r * el:(r + 1) * el].contiguous())
              for r in range(world)]
    ranks = [_EmulatedRank(lib, r, world, E, topk, tokens, H, dev) for r in range(world)]
    table = lambda attr: (ctypes.c_void_p * world)(*[getattr(r, attr).data_ptr() for r in ranks])
    peer_counts, peer_codes, peer_side, peer_pairs = (table(a) for a in ("counts_all", "codes", "side", "pairs"))
    stream = torch.cuda.current_stream(dev).cuda_stream
    ok = lambda rc: _cabi.check(rc)
    _status(lib, dev)
    for it in range(2):
        xs, idss, wtss = [], [], []
        for r in range(world):
            g.manual_seed(1000 * it + r)
            xs.append(torch.randn((tokens, H), generator=g, device=dev).to(torch.bfloat16))
            wts, ids = torch.topk(torch.softmax(torch.randn((tokens, E), generator=g, device=dev), -1), topk, dim=-1)
            idss.append(ids.contiguous())
            wtss.append((wts / wts.sum(-1, keepdim=True)).float().contiguous())
        pairs = tokens * topk
        # step 1: every rank's histogram lands in every rank's count matrix
        for r in ranks:
            ok(lib.es_b200_ep_route_count(idss[r.rank].data_ptr(), 1, pairs, E, r.seg_counts.data_ptr(),
                                          r.seg_base.data_ptr(), peer_counts, r.rank, world, stream))
        # step 2: tables
        for r in ranks:
            t = r.t
            ok(lib.es_b200_ep_route_tables(idss[r.rank].data_ptr(), 1, pairs, E, r.seg_base.data_ptr(),
                                           r.counts_all.data_ptr(), r.rank, world, H, t["dst_rank"].data_ptr(),
                                           t["dst_row"].data_ptr(), t["dst_scale_offset"].data_ptr(),
                                           t["rows"].data_ptr(), t["expert_offsets"].data_ptr(),
                                           t["blockscale_offsets"].data_ptr(), t["total_rows"].data_ptr(), r.capacity,
                                           stream))
        torch.cuda.synchronize()
        cnt_all = torch.stack([torch.bincount(ids.reshape(-1), minlength=E) for ids in idss])
        assert torch.equal(ranks[0].counts_all.long(), cnt_all) and torch.equal(ranks[1].counts_all.long(), cnt_all)
        for r in ranks:
            want = ep.routing_tables(idss[r.rank], cnt_all, r.rank, H)
            for key, val in want.items():
                assert torch.equal(r.t[key].to(val.dtype), val), f"rank {r.rank}: routing table {key} differs"
        # step 3: dispatch (quantise once, push codes + side records to the owners), then unpack on the owners
        for r in ranks:
            t = r.t
            ok(lib.es_b200_ep_dispatch_quant_push(xs[r.rank].data_ptr(), _cabi.BF16, t["dst_rank"].data_ptr(),
                                                  t["dst_row"].data_ptr(), t["dst_scale_offset"].data_ptr(), peer_codes,
                                                  peer_side, r.rank, world, tokens, topk, H, r.capacity,
                                                  r.pairs.data_ptr(), H * 2, stream))
        for r in ranks:
            ok(lib.es_b200_ep_unpack_side(r.side.data_ptr(), r.t["total_rows"].data_ptr(), r.scales.data_ptr(),
                                          r.meta.data_ptr(), H, r.capacity, r.scales.numel(), stream))
        # step 4: expert GEMMs on each owner; the down GEMM's epilogue stores into the senders' (token, j) slots
        for r in ranks:
            shards[r.rank].forward_codes(r.codes.view(torch.float8_e4m3fn), r.scales, r.t["rows"],
                                         r.t["expert_offsets"], r.t["blockscale_offsets"], r.work,
                                         (r.meta, peer_pairs, world, pairs))
        # step 5: weighted sum on each sender
        for r in ranks:
            out = torch.empty((tokens, H), dtype=torch.bfloat16, device=dev)
            ok(lib.es_b200_ep_topk_weighted_sum(r.pairs.data_ptr(), _cabi.BF16, wtss[r.rank].data_ptr(),
                                                out.data_ptr(), tokens, topk, H, stream))
            torch.cuda.synchronize()
            ref = _layer_reference(xs[r.rank], idss[r.rank], wtss[r.rank], w1, w2)
            diff = calc_diff(out.float().cpu(), ref.cpu())
            assert diff < 5e-3, f"round {it}, rank {r.rank}: calc_diff {diff}"
        # every row a rank received came from the rank its return address names
        for r in ranks:
            n = int(r.t["total_rows"])
            assert n == int(cnt_all[:, r.rank * el:(r.rank + 1) * el].sum())
            src = r.meta[:n, 0]
            assert int(src.min()) >= 0 and int(src.max()) < world
    rc, raw = _status(lib, dev)
    assert rc == 0, f"device status {raw:#x}"


def test_barrier_wait_runs_out_and_reports():
    from expert_specialization_moe_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    _status(lib, dev)
    mine = torch.zeros(17, dtype=torch.int32, device=dev)
    absent = torch.zeros(17, dtype=torch.int32, device=dev)      # the flags of a partner that never calls the barrier
    flags = (ctypes.c_void_p * 2)(mine.data_ptr(), absent.data_ptr())
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    assert lib.es_b200_ep_barrier_limit(flags, 0, 2, 20_000_000, stream) == 0
    ev1.record()
    rc, raw = _status(lib, dev)
    assert rc != 0 and raw == ERR_BARRIER_TIMEOUT, f"status {raw:#x}"
    assert 15.0 < ev0.elapsed_time(ev1) < 2000.0               # gave up after about the 20 ms it was given
    assert b"bounded device-side wait" in lib.es_b200_last_error()
    # rank 0 did announce itself to the partner and to itself before it gave up
    assert int(absent[0]) == 1 and int(mine[0]) == 1 and int(mine[1]) == 0
    rc, raw = _status(lib, dev)
    assert rc == 0 and raw == 0
    # a world of one never waits: the same flags, complete
    solo = (ctypes.c_void_p * 1)(mine.data_ptr())
    assert lib.es_b200_ep_barrier(solo, 0, 1, stream) == 0
    rc, raw = _status(lib, dev)
    assert rc == 0
    assert lib.es_b200_ep_barrier_limit(flags, 0, 2, 0, stream) != 0      # a limit must be positive


def test_dropped_pairs_add_zero_to_the_weighted_sum():
    """Receive buffer too small for the rows routed to it: the surplus pairs are dropped at dispatch, reported, and
    their (token, j) slots cleared, so the weighted sum does not pick up rows left there by an earlier step."""
    from expert_specialization_moe_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    E, tokens, topk, H, capacity = 8, 64, 2, 256, 100
    g = torch.Generator(device=dev).manual_seed(3)
    ids = torch.randint(0, E, (tokens, topk), generator=g, device=dev, dtype=torch.int64)
    x = torch.randn((tokens, H), generator=g, device=dev).to(torch.bfloat16)
    pairs = tokens * topk
    i32 = lambda *s: torch.zeros(s, dtype=torch.int32, device=dev)
    seg_counts, seg_base, counts_all = i32(256, E), i32(256, E), i32(1, E)
    dst_rank, dst_row, rows, eo, bo, total = i32(pairs), i32(pairs), i32(E), i32(E), i32(E), i32(1)
    sf_off = torch.zeros(pairs, dtype=torch.int64, device=dev)
    side_bytes = int(lib.es_b200_ep_side_record_bytes(H))
    codes = torch.zeros((capacity, H), dtype=torch.uint8, device=dev)
    side = torch.zeros((capacity, side_bytes), dtype=torch.uint8, device=dev)
    slots = torch.full((pairs, H), 7.0, dtype=torch.bfloat16, device=dev)          # "rows of an earlier step"
    t1 = lambda t: (ctypes.c_void_p * 1)(t.data_ptr())
    stream = torch.cuda.current_stream(dev).cuda_stream
    _status(lib, dev)
    assert lib.es_b200_ep_route_count(ids.data_ptr(), 1, pairs, E, seg_counts.data_ptr(), seg_base.data_ptr(),
                                      t1(counts_all), 0, 1, stream) == 0
    assert lib.es_b200_ep_route_tables(ids.data_ptr(), 1, pairs, E, seg_base.data_ptr(), counts_all.data_ptr(), 0, 1, H,
                                       dst_rank.data_ptr(), dst_row.data_ptr(), sf_off.data_ptr(), rows.data_ptr(),
                                       eo.data_ptr(), bo.data_ptr(), total.data_ptr(), capacity, stream) == 0
    assert lib.es_b200_ep_dispatch_quant_push(x.data_ptr(), _cabi.BF16, dst_rank.data_ptr(), dst_row.data_ptr(),
                                              sf_off.data_ptr(), t1(codes), t1(side), 0, 1, tokens, topk, H, capacity,
                                              slots.data_ptr(), H * 2, stream) == 0
    rc, raw = _status(lib, dev)
    assert rc != 0 and (raw & ERR_BAD_DESTINATION)
    dropped = dst_row >= capacity
    assert int(dropped.sum()) == pairs - capacity
    assert bool((slots[dropped] == 0).all()), "slots of dropped pairs were not cleared"
    assert bool((slots[~dropped] == 7.0).all()), "slots of delivered pairs must be left to the combine"
