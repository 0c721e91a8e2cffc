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
