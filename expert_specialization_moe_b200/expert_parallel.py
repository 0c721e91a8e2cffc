"""Expert-parallel execution of an MoE layer's expert GEMMs: E/G experts per GPU, tokens move.

The reference has no distributed code; this module is the expert-parallel mode that the grouped GEMM operators are
deployed in: one process per GPU, `torch.distributed` all-to-all (NCCL over NVLink / NVSwitch on GPUs, gloo in the CPU
tests) for token dispatch and combine, and the grouped quant / grouped GEMM operators of this package for the
compute on each rank's expert shard.  Nothing here computes a GEMM itself.

    plan   = make_plan(topk_ids, num_experts, group)        # counts exchange + permutations (host-visible sizes)
    x_e    = dispatch(x, plan)                              # rows of my experts, grouped by expert
    y_e    = expert_fn(x_e, plan.problem_sizes(...), ...)   # gate_up -> SiLU*mul -> down on the local shard
    y      = combine(y_e, plan, topk_weights)               # rows return and are summed per token with their weights

Expert e lives on rank e // (E / G) (contiguous shards), local index e % (E / G).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.distributed as dist


def _align128(x: torch.Tensor) -> torch.Tensor:
    return (x + 127) // 128 * 128


@dataclass
class DispatchPlan:
    """Everything both directions of the exchange need; all index tensors live on the tokens' device."""
    num_experts: int
    world_size: int
    rank: int
    topk: int
    num_tokens: int
    send_order: torch.Tensor        # [tokens*topk] permutation of the (token, k) pairs into expert order
    send_counts: torch.Tensor       # [E] rows I send to each (global) expert
    send_splits: list               # [G] rows I send to each rank
    recv_counts: torch.Tensor       # [G, E_local] rows each source rank sends to each of my experts
    recv_splits: list               # [G] rows I receive from each rank
    recv_order: torch.Tensor        # [rows_in] permutation of the received rows into local-expert order
    local_counts: torch.Tensor      # [E_local] rows per local expert after regrouping

    @property
    def experts_per_rank(self) -> int:
        return self.num_experts // self.world_size

    @property
    def rows_in(self) -> int:
        return int(sum(self.recv_splits))

    def problem_tensors(self, n: int, k: int):
        """(problem_sizes [E_local,3], expert_offsets [E_local], blockscale_offsets [E_local], scale_rows) in the
        layout the grouped operators take (int32, on the plan's device)."""
        c = self.local_counts.to(torch.int64)
        dev = c.device
        eo = torch.zeros_like(c)
        bo = torch.zeros_like(c)
        if c.numel() > 1:
            eo[1:] = torch.cumsum(c, 0)[:-1]
            bo[1:] = torch.cumsum(_align128(c), 0)[:-1]
        ps = torch.stack([c, torch.full_like(c, n), torch.full_like(c, k)], dim=1)
        return (ps.to(torch.int32).contiguous(), eo.to(torch.int32), bo.to(torch.int32),
                int(_align128(c).sum().item()) if c.numel() else 0)


def make_plan(topk_ids: torch.Tensor, num_experts: int, group: Optional[dist.ProcessGroup] = None) -> DispatchPlan:
    """topk_ids [tokens, topk] (int64, values in [0, E)).  One all-to-all of per-expert counts, then host-visible split
    sizes (torch.distributed needs them on the host; this is the only synchronisation point of the layer)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    assert num_experts % world == 0, "experts must divide evenly over the ranks"
    e_local = num_experts // world
    tokens, topk = topk_ids.shape
    flat = topk_ids.reshape(-1)
    # stable sort by expert: rows for one destination rank are contiguous and already ordered by expert
    send_order = torch.sort(flat, stable=True).indices
    send_counts = torch.bincount(flat, minlength=num_experts)
    recv_counts = torch.empty((world, e_local), dtype=send_counts.dtype, device=send_counts.device)
    dist.all_to_all_single(recv_counts.view(-1), send_counts.contiguous(), group=group)
    send_splits = send_counts.view(world, e_local).sum(1).tolist()
    recv_splits = recv_counts.sum(1).tolist()
    # received rows arrive grouped by source rank, inside each source by expert; regroup by expert (stable)
    src_expert = torch.repeat_interleave(
        torch.arange(e_local, device=flat.device).repeat(world), recv_counts.reshape(-1))
    recv_order = torch.sort(src_expert, stable=True).indices
    local_counts = recv_counts.sum(0)
    return DispatchPlan(num_experts, world, rank, topk, tokens, send_order, send_counts, send_splits, recv_counts,
                        recv_splits, recv_order, local_counts)


def dispatch(x: torch.Tensor, plan: DispatchPlan, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """x [tokens, H] -> rows routed to my experts, grouped by local expert: [rows_in, H]."""
    token_of_pair = plan.send_order // plan.topk
    send = x.index_select(0, token_of_pair).contiguous()
    recv = torch.empty((plan.rows_in, x.shape[1]), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(recv, send, output_split_sizes=plan.recv_splits, input_split_sizes=plan.send_splits,
                           group=group)
    return recv.index_select(0, plan.recv_order)


def combine(y: torch.Tensor, plan: DispatchPlan, topk_weights: torch.Tensor,
            group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """y [rows_in, H] (local-expert order) -> [tokens, H] = sum_k w[token,k] * y(token,k), accumulated in fp32."""
    back = torch.empty_like(y)
    back[plan.recv_order] = y                      # undo the regrouping: source-rank order again
    out_rows = torch.empty((plan.num_tokens * plan.topk, y.shape[1]), dtype=y.dtype, device=y.device)
    dist.all_to_all_single(out_rows, back.contiguous(), output_split_sizes=plan.send_splits,
                           input_split_sizes=plan.recv_splits, group=group)
    pairs = torch.empty_like(out_rows)
    pairs[plan.send_order] = out_rows              # (token, k) order
    w = topk_weights.reshape(-1, 1).to(torch.float32)
    acc = (pairs.to(torch.float32) * w).view(plan.num_tokens, plan.topk, -1).sum(1)
    return acc.to(y.dtype)


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[rows, 2I] -> [rows, I]: silu(gate) * up with gate = first half of the columns."""
    i = gate_up.shape[1] // 2
    return torch.nn.functional.silu(gate_up[:, :i].float()).mul_(gate_up[:, i:].float()).to(gate_up.dtype)


class ExpertShard:
    """MXFP8 weights of this rank's experts: gate_up [E_local, 2I, H] and down [E_local, H, I], e4m3 + swizzled UE8M0,
    quantised once with the grouped quant operator (as the reference's own test quantises weights:
    test/test_es_sm100_mxfp8_blockscaled_grouped_quant.py:53,87-96)."""

    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor):
        self.e_local, self.n1, self.h = w_gate_up.shape
        _, self.h2, self.i = w_down.shape
        assert self.h2 == self.h and self.n1 == 2 * self.i
        self.w1, self.sf1 = self._quantise(w_gate_up)
        self.w2, self.sf2 = self._quantise(w_down)

    @staticmethod
    def _quantise(w: torch.Tensor):
        from .ops import es_sm100_mxfp8_blockscaled_grouped_quant as quant
        e, n, k = w.shape
        dev = w.device
        ps = torch.tensor([[n, 0, k]] * e, dtype=torch.int32, device=dev)
        off = torch.arange(e, dtype=torch.int32, device=dev) * n
        codes = torch.empty((e * n, k), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        sf = torch.zeros((e * n, k // 32), dtype=torch.uint8, device=dev)
        quant(w.reshape(e * n, k).contiguous(), ps, off, off, codes, sf)
        return codes.view(e, n, k), sf

    def forward(self, x: torch.Tensor, plan: DispatchPlan) -> torch.Tensor:
        """x [rows_in, H] bf16 grouped by local expert -> [rows_in, H] bf16."""
        from .ops import es_sm100_mxfp8_blockscaled_grouped_mm as mm
        from .ops import es_sm100_mxfp8_blockscaled_grouped_quant as quant
        from .ops import es_sm100_mxfp8_silu_mul_grouped_quant as silu_mul_quant
        rows = x.shape[0]
        dev = x.device
        ps1, eo, bo, sf_rows = plan.problem_tensors(self.n1, self.h)
        a = torch.empty((rows, self.h), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        sfa = torch.empty((max(sf_rows, 128), self.h // 32), dtype=torch.uint8, device=dev)
        quant(x, ps1, eo, bo, a, sfa)
        h1 = torch.empty((rows, self.n1), dtype=x.dtype, device=dev)
        mm(h1, a, self.w1.transpose(1, 2), sfa, self.sf1, ps1, eo, bo)
        ps2, _, _, _ = plan.problem_tensors(self.h, self.i)
        a2 = torch.empty((rows, self.i), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn)
        sfa2 = torch.empty((max(sf_rows, 128), self.i // 32), dtype=torch.uint8, device=dev)
        silu_mul_quant(h1, ps2, eo, bo, a2, sfa2)      # fused SiLU * mul + requantisation, one pass over h1
        out = torch.empty((rows, self.h), dtype=x.dtype, device=dev)
        mm(out, a2, self.w2.transpose(1, 2), sfa2, self.sf2, ps2, eo, bo)
        return out


def moe_forward(x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, num_experts: int,
                expert_fn: Callable[[torch.Tensor, DispatchPlan], torch.Tensor],
                group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """dispatch -> expert_fn on the local shard -> combine.  `expert_fn` is ExpertShard.forward on GPUs."""
    plan = make_plan(topk_ids, num_experts, group)
    rows = dispatch(x, plan, group)
    y = expert_fn(rows, plan)
    return combine(y, plan, topk_weights, group)
