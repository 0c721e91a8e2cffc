"""World-size-2 and -4 tests of the expert-parallel plumbing on CPU ranks (gloo): routing counts, dispatch
permutation, regrouping by local expert, combine with top-k weights.  The expert computation is a stand-in closed
form (row * (global expert id + 1)), so the expected result is computable without any GEMM."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, num_experts, tokens, topk, hidden, q):
    try:
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world)
        from expert_specialization_moe_b200 import expert_parallel as ep

        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn((tokens, hidden), generator=g)
        logits = torch.randn((tokens, num_experts), generator=g)
        w, ids = torch.topk(torch.softmax(logits, -1), topk, dim=-1)
        w = w / w.sum(-1, keepdim=True)
        if rank == 0:
            ids[:, 0] = 0                      # skew: every token of rank 0 also goes to expert 0
        e_local = num_experts // world

        seen = {}

        def expert_fn(rows, plan):
            ps, eo, bo, sf_rows = plan.problem_tensors(64, hidden)
            assert ps.shape == (e_local, 3) and ps.dtype == torch.int32
            assert int(ps[:, 0].sum()) == rows.shape[0] == plan.rows_in
            assert torch.equal(eo[1:].long(), torch.cumsum(ps[:, 0].long(), 0)[:-1])
            assert sf_rows == int(((ps[:, 0].long() + 127) // 128 * 128).sum())
            assert all(int(b) % 128 == 0 for b in bo)
            gid = torch.repeat_interleave(torch.arange(e_local) + rank * e_local, plan.local_counts)
            seen["rows"] = rows.shape[0]
            return rows * (gid + 1).unsqueeze(1).to(rows.dtype)

        out = ep.moe_forward(x, ids, w, num_experts, expert_fn)
        expect = (x.unsqueeze(1) * (ids + 1).unsqueeze(-1).float() * w.unsqueeze(-1)).sum(1)
        err = float((out - expect).abs().max())
        # global conservation: rows received over all ranks == tokens * topk * world
        total = torch.tensor([seen["rows"]])
        dist.all_reduce(total)
        q.put((rank, err, int(total), None))
        dist.destroy_process_group()
    except Exception as exc:  # surface the failure in the parent
        import traceback
        q.put((rank, None, None, traceback.format_exc()))


@pytest.mark.parametrize("world,num_experts,topk", [(2, 8, 2), (4, 16, 4), (2, 6, 3)])
def test_dispatch_combine_roundtrip(world, num_experts, topk):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    tokens, hidden = 37, 16
    procs = [ctx.Process(target=_worker, args=(r, world, port, num_experts, tokens, topk, hidden, q))
             for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, err, total, tb in results:
        assert tb is None, f"rank {rank} failed:\n{tb}"
        assert err < 1e-5, f"rank {rank}: max error {err}"
        assert total == tokens * topk * world


def test_silu_mul():
    from expert_specialization_moe_b200.expert_parallel import silu_mul
    g = torch.randn(5, 8)
    out = silu_mul(g)
    assert torch.allclose(out, torch.nn.functional.silu(g[:, :4]) * g[:, 4:], atol=1e-6)


@pytest.mark.parametrize("world,num_experts,topk,tokens", [(2, 8, 2, 37), (4, 16, 4, 21), (8, 128, 8, 64)])
def test_routing_tables_of_the_fused_exchange(world, num_experts, topk, tokens):
    """routing_tables (the address arithmetic of the peer-memory dispatch) for every rank of a simulated job: the
    destinations of all ranks tile each owner's receive buffer exactly, rows of one expert are contiguous and ordered
    by (source rank, token, j) — the order the all-to-all path delivers — and the scale offsets are the swizzled
    positions of those rows."""
    from expert_specialization_moe_b200.expert_parallel import routing_tables
    hidden = 256
    g = torch.Generator().manual_seed(world * 100 + topk)
    ids = [torch.stack([torch.randperm(num_experts, generator=g)[:topk] for _ in range(tokens)]) for _ in range(world)]
    counts_all = torch.stack([torch.bincount(i.reshape(-1), minlength=num_experts) for i in ids])
    tabs = [routing_tables(ids[r], counts_all, r, hidden) for r in range(world)]
    e_local = num_experts // world
    kt = hidden // 128
    for d in range(world):
        total = int(tabs[d]["total_rows"])
        # expected arrival order on owner d: expert-major, then source rank, then the source's (token, j) order
        expected = []
        for e in range(d * e_local, (d + 1) * e_local):
            for s in range(world):
                flat = ids[s].reshape(-1)
                expected += [(s, int(p)) for p in torch.nonzero(flat == e).reshape(-1)]
        assert len(expected) == total
        got = [None] * total
        for s in range(world):
            t = tabs[s]
            for p in torch.nonzero(t["dst_rank"] == d).reshape(-1).tolist():
                row = int(t["dst_row"][p])
                assert 0 <= row < total and got[row] is None
                got[row] = (s, p)
                # scale offset of the row: expert's blockscale offset + swizzled position inside the expert
                e = int(ids[s].reshape(-1)[p])
                le = e - d * e_local
                r_local = row - int(tabs[d]["expert_offsets"][le])
                want = (int(tabs[d]["blockscale_offsets"][le]) * (hidden // 32) + (r_local // 128) * kt * 512
                        + (r_local % 32) * 16 + ((r_local % 128) // 32) * 4)
                assert int(t["dst_scale_offset"][p]) == want
        assert got == expected
        rows = tabs[d]["rows"].to(torch.int64)
        assert int(rows.sum()) == total
        assert torch.equal(tabs[d]["expert_offsets"].to(torch.int64), torch.cumsum(rows, 0) - rows)
        mp128 = (rows + 127) // 128 * 128
        assert torch.equal(tabs[d]["blockscale_offsets"].to(torch.int64), torch.cumsum(mp128, 0) - mp128)
