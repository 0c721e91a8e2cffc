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

`FusedExchange` is the same layer without the all-to-alls: every rank quantises its tokens once and stores codes,
scales and return addresses straight into the owners' receive buffers over NVLink (peer-mapped symmetric memory),
the expert outputs are stored straight back into the senders' (token, j) slots, and the per-expert counts travel the
same way.  Nothing in it needs a size on the host, so a layer is a fixed sequence of launches.
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


def routing_tables(topk_ids: torch.Tensor, counts_all: torch.Tensor, rank: int, hidden: int):
    """Where every (token, j) pair of THIS rank goes, and what this rank's experts receive — tensor arithmetic only
    (no host synchronisation; runs on CPU tensors too).

    topk_ids [tokens, topk] expert ids; counts_all [G, E]: counts_all[s, e] = pairs rank s routes to expert e.
    On the owner, the rows of one expert are ordered by source rank, inside a source by (token, j) order.
    Returns a dict of tensors: dst_rank, dst_row (int32 [tokens*topk]), dst_scale_offset (int64: byte offset of the
    row's scale word for K tile 0 in the owner's swizzled scale buffer), rows (int32 [E_local], m_e of my experts),
    expert_offsets, blockscale_offsets (int32 [E_local]), total_rows (int32 [1])."""
    world, num_experts = counts_all.shape
    e_local = num_experts // world
    kt = hidden // 128
    counts_all = counts_all.to(torch.int64)
    m = counts_all.sum(0)                                                    # rows per expert on its owner
    m_owner = m.view(world, e_local)
    eo_all = (torch.cumsum(m_owner, 1) - m_owner).reshape(-1)               # row offset of expert e on its owner
    mp = _align128(m_owner)
    bo_all = (torch.cumsum(mp, 1) - mp).reshape(-1)                         # scale-row offset of expert e on its owner
    src_off = torch.cumsum(counts_all, 0) - counts_all                      # [G, E]: rows of lower ranks in expert e
    flat = topk_ids.reshape(-1).to(torch.int64)
    pairs = flat.numel()
    order = torch.sort(flat, stable=True).indices
    mine = counts_all[rank]
    start = torch.cumsum(mine, 0) - mine
    pos_sorted = torch.arange(pairs, device=flat.device) - start[flat[order]]
    pos = torch.empty_like(pos_sorted)
    pos[order] = pos_sorted                                                  # rank of the pair among my pairs to its expert
    r_local = src_off[rank][flat] + pos                                      # row inside the expert, on the owner
    dst_rank = torch.div(flat, e_local, rounding_mode="floor")
    dst_row = eo_all[flat] + r_local
    sf_off = (bo_all[flat] * (hidden // 32) + (r_local >> 7) * (kt * 512) + (r_local & 31) * 16
              + ((r_local & 127) >> 5) * 4)
    lo, hi = rank * e_local, (rank + 1) * e_local
    return {
        "dst_rank": dst_rank.to(torch.int32), "dst_row": dst_row.to(torch.int32), "dst_scale_offset": sf_off,
        "rows": m[lo:hi].to(torch.int32), "expert_offsets": eo_all[lo:hi].to(torch.int32),
        "blockscale_offsets": bo_all[lo:hi].to(torch.int32), "total_rows": m[lo:hi].sum().to(torch.int32).reshape(1),
    }


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

    def forward_codes(self, a: torch.Tensor, sfa: torch.Tensor, rows: torch.Tensor, eo: torch.Tensor,
                      bo: torch.Tensor, work: dict, scatter=None) -> Optional[torch.Tensor]:
        """a [capacity, H] e4m3 + sfa (swizzled) as delivered by FusedExchange.dispatch, grouped by local expert with
        `rows[e]` valid rows at expert_offsets eo / blockscale_offsets bo (all on the device).  `work` caches the
        capacity-sized intermediates.  Returns [capacity, H] (rows past the valid ones are undefined) — or, with
        `scatter` = (row_meta, peer table, world, slots), nothing: the down GEMM then stores every output row
        straight into its (GPU, slot) destination (es_b200_mxfp8_grouped_mm_scatter)."""
        from .ops import es_sm100_mxfp8_blockscaled_grouped_mm as mm
        from .ops import es_sm100_mxfp8_silu_mul_grouped_quant as silu_mul_quant
        cap, dev = a.shape[0], a.device
        if work.get("cap") != cap:
            work.clear()
            ps = lambda n, k: torch.tensor([[0, n, k]] * self.e_local, dtype=torch.int32, device=dev)
            work.update(cap=cap,
                        h1=torch.empty((cap, self.n1), dtype=torch.bfloat16, device=dev),
                        a2=torch.empty((cap, self.i), dtype=torch.uint8, device=dev).view(torch.float8_e4m3fn),
                        sfa2=torch.zeros((sfa.shape[0], self.i // 32), dtype=torch.uint8, device=dev),
                        ps1=ps(self.n1, self.h), ps2=ps(self.h, self.i))
        # problem lists live in the work set: only the row counts change from step to step (no allocation per step)
        ps1, ps2 = work["ps1"], work["ps2"]
        ps1[:, 0].copy_(rows)
        ps2[:, 0].copy_(rows)
        mm(work["h1"], a, self.w1.transpose(1, 2), sfa, self.sf1, ps1, eo, bo)
        silu_mul_quant(work["h1"], ps2, eo, bo, work["a2"], work["sfa2"])
        if scatter is None:
            if "out" not in work:
                work["out"] = torch.empty((cap, self.h), dtype=torch.bfloat16, device=dev)
            mm(work["out"], work["a2"], self.w2.transpose(1, 2), work["sfa2"], self.sf2, ps2, eo, bo)
            return work["out"]
        from . import _cabi
        meta, table, world, slots = scatter
        stream = torch.cuda.current_stream(dev).cuda_stream
        scratch = _cabi.grouped_mm_scratch(dev, stream)
        _cabi.check(_cabi.load().es_b200_mxfp8_grouped_mm_scatter(
            work["a2"].data_ptr(), self.w2.data_ptr(), work["sfa2"].data_ptr(), self.sf2.data_ptr(), _cabi.BF16,
            ps2.data_ptr(), eo.data_ptr(), bo.data_ptr(), self.e_local, cap, self.h, self.i,
            work["sfa2"].numel() // (self.i // 32), meta.data_ptr(), table, world, slots,
            scratch.data_ptr(), scratch.numel(), stream))
        return None

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


class FusedExchange:
    """Dispatch and combine of one MoE layer over peer memory (see the module docstring).  One instance per rank holds
    one symmetric allocation: receive buffers for codes [capacity, H] and side records (return address, scale position,
    scale bytes of each row), the (token, j) slots [tokens * topk, H] the expert outputs come back to, the count
    matrix and the barrier flags.  `capacity` defaults to the worst case (every pair of every rank routed here)."""

    def __init__(self, num_experts: int, topk: int, tokens: int, hidden: int, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None, capacity_rows: Optional[int] = None,
                 dtype: torch.dtype = torch.bfloat16):
        import ctypes
        import torch.distributed._symmetric_memory as symm
        from . import _cabi
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        assert num_experts % self.world == 0 and hidden % 128 == 0
        self.num_experts, self.topk, self.tokens, self.hidden, self.dtype = num_experts, topk, tokens, hidden, dtype
        self.e_local = num_experts // self.world
        self.capacity = int(capacity_rows or self.world * tokens * topk)
        self.scale_rows = (self.capacity + 128 * self.e_local + 127) // 128 * 128
        self.scale_bytes = self.scale_rows * (hidden // 32)
        self._lib = _cabi.load()
        self.side_bytes = int(self._lib.es_b200_ep_side_record_bytes(hidden))
        sizes = [self.capacity * hidden, self.capacity * self.side_bytes, 0, tokens * topk * hidden * 2, 17 * 4,
                 self.world * num_experts * 4]
        offs, total = [], 0
        for sz in sizes:
            offs.append(total)
            total += (sz + 255) // 256 * 256
        self.buf = symm.empty((total,), dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.hdl = symm.rendezvous(self.buf, self.group)
        self.codes = self.buf[offs[0]:offs[0] + sizes[0]].view(torch.float8_e4m3fn).view(self.capacity, hidden)
        self.side = self.buf[offs[1]:offs[1] + sizes[1]].view(self.capacity, self.side_bytes)
        self.scales = torch.zeros((self.scale_rows, hidden // 32), dtype=torch.uint8, device=device)   # local
        self.meta = torch.zeros((self.capacity, 2), dtype=torch.int32, device=device)                  # local
        self.pairs = self.buf[offs[3]:offs[3] + sizes[3]].view(dtype).view(tokens * topk, hidden)
        table = lambda k: (ctypes.c_void_p * self.world)(*[int(p) + offs[k] for p in self.hdl.buffer_ptrs])
        (self._peer_codes, self._peer_side, _, self._peer_pairs, self._peer_flags,
         self._peer_counts) = (table(k) for k in range(6))
        self.counts_all = self.buf[offs[5]:offs[5] + sizes[5]].view(torch.int32).view(self.world, num_experts)
        pairs = tokens * topk
        i32 = lambda *shape: torch.empty(shape, dtype=torch.int32, device=device)
        self._seg_counts, self._seg_base = i32(256, num_experts), i32(256, num_experts)
        self._tables = {"dst_rank": i32(pairs), "dst_row": i32(pairs),
                        "dst_scale_offset": torch.empty(pairs, dtype=torch.int64, device=device),
                        "rows": i32(self.e_local), "expert_offsets": i32(self.e_local),
                        "blockscale_offsets": i32(self.e_local), "total_rows": i32(1)}
        self._check = _cabi.check
        self._dtype_code = _cabi.BF16 if dtype == torch.bfloat16 else _cabi.FP16
        self.work = {}
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)          # every rank's buffers (and flags) are zeroed before anyone stores

    def barrier(self, device):
        """Stream-ordered barrier of the ranks (bounded wait on the device; see es_b200_ep_barrier)."""
        self._check(self._lib.es_b200_ep_barrier(self._peer_flags, self.rank, self.world,
                                                 torch.cuda.current_stream(device).cuda_stream))

    def plan(self, topk_ids: torch.Tensor) -> dict:
        """Routing tables of this step (three small launches and a barrier; the returned tensors are reused by the
        next call).  `routing_tables` is the same arithmetic in torch."""
        assert topk_ids.shape == (self.tokens, self.topk) and topk_ids.is_contiguous()
        assert topk_ids.dtype in (torch.int32, torch.int64)
        dev = topk_ids.device
        s = torch.cuda.current_stream(dev).cuda_stream
        is64 = 1 if topk_ids.dtype == torch.int64 else 0
        pairs = self.tokens * self.topk
        t = self._tables
        self._check(self._lib.es_b200_ep_route_count(topk_ids.data_ptr(), is64, pairs, self.num_experts,
                                                     self._seg_counts.data_ptr(), self._seg_base.data_ptr(),
                                                     self._peer_counts, self.rank, self.world, s))
        self.barrier(dev)                       # every rank's counts have arrived in my count matrix
        self._check(self._lib.es_b200_ep_route_tables(
            topk_ids.data_ptr(), is64, pairs, self.num_experts, self._seg_base.data_ptr(), self.counts_all.data_ptr(),
            self.rank, self.world, self.hidden, t["dst_rank"].data_ptr(), t["dst_row"].data_ptr(),
            t["dst_scale_offset"].data_ptr(), t["rows"].data_ptr(), t["expert_offsets"].data_ptr(),
            t["blockscale_offsets"].data_ptr(), t["total_rows"].data_ptr(), self.capacity, s))
        return t

    def dispatch(self, x: torch.Tensor, plan: dict):
        """x [tokens, H] -> (codes [capacity, H] e4m3, swizzled scales) of the rows routed to my experts."""
        assert x.shape == (self.tokens, self.hidden) and x.dtype == self.dtype and x.is_contiguous()
        s = torch.cuda.current_stream(x.device).cuda_stream
        self._check(self._lib.es_b200_ep_dispatch_quant_push(
            x.data_ptr(), self._dtype_code, plan["dst_rank"].data_ptr(), plan["dst_row"].data_ptr(),
            plan["dst_scale_offset"].data_ptr(), self._peer_codes, self._peer_side, self.rank, self.world, self.tokens,
            self.topk, self.hidden, self.capacity, self.pairs.data_ptr(), self.hidden * 2, s))
        self.barrier(x.device)                  # all ranks' stores into my buffers are complete and visible
        self._check(self._lib.es_b200_ep_unpack_side(self.side.data_ptr(), plan["total_rows"].data_ptr(),
                                                     self.scales.data_ptr(), self.meta.data_ptr(), self.hidden,
                                                     self.capacity, self.scale_bytes, s))
        return self.codes, self.scales

    def combine(self, y: torch.Tensor, plan: dict, topk_weights: torch.Tensor,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """y [capacity, H] expert outputs in receive order -> [tokens, H] = sum_j w[token, j] * y(token, j)."""
        assert y.shape == (self.capacity, self.hidden) and y.dtype == self.dtype and y.is_contiguous()
        s = torch.cuda.current_stream(y.device).cuda_stream
        self._check(self._lib.es_b200_ep_combine_push(
            y.data_ptr(), self.meta.data_ptr(), plan["total_rows"].data_ptr(), self._peer_pairs, self.world,
            self.capacity, self.tokens * self.topk, self.hidden, 2, s))
        return self.reduce(topk_weights, out)

    def reduce(self, topk_weights: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """After every rank's expert outputs have arrived in my (token, j) slots: out[t] = sum_j w[t, j] * slot(t, j).
        `out`: caller's [tokens, H] result buffer (a serving loop passes the same one every step: no allocation)."""
        dev = self.pairs.device
        self.barrier(dev)
        if out is None:
            out = torch.empty((self.tokens, self.hidden), dtype=self.dtype, device=dev)
        w = topk_weights if (topk_weights.dtype == torch.float32 and topk_weights.is_contiguous()) \
            else topk_weights.to(torch.float32).contiguous()
        self._check(self._lib.es_b200_ep_topk_weighted_sum(self.pairs.data_ptr(), self._dtype_code, w.data_ptr(),
                                                           out.data_ptr(), self.tokens, self.topk, self.hidden,
                                                           torch.cuda.current_stream(dev).cuda_stream))
        return out

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, shard: ExpertShard,
                fuse_combine: bool = True, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One MoE layer.  With fuse_combine the down GEMM's epilogue stores each output row straight into the
        sender's slot; otherwise the rows go through a dense output and es_b200_ep_combine_push."""
        assert self.dtype == torch.bfloat16 or not fuse_combine
        plan = self.plan(topk_ids)
        a, sfa = self.dispatch(x, plan)
        scatter = (self.meta, self._peer_pairs, self.world, self.tokens * self.topk) if fuse_combine else None
        y = shard.forward_codes(a, sfa, plan["rows"], plan["expert_offsets"], plan["blockscale_offsets"], self.work,
                                scatter)
        if fuse_combine:
            return self.reduce(topk_weights, out)
        return self.combine(y, plan, topk_weights, out)


class PipelinedExchange:
    """The same layer on two halves of the token batch, each with its own FusedExchange and CUDA stream, so that one
    half's NVLink-bound steps (dispatch, the down GEMM's scatter epilogue) can run while the other half computes."""

    def __init__(self, num_experts: int, topk: int, tokens: int, hidden: int, device: torch.device,
                 group: Optional[dist.ProcessGroup] = None, capacity_rows: Optional[int] = None):
        assert tokens % 2 == 0
        self.half = tokens // 2
        cap = None if capacity_rows is None else capacity_rows // 2
        self.parts = [FusedExchange(num_experts, topk, self.half, hidden, device, group, cap) for _ in range(2)]
        self.streams = [torch.cuda.Stream(device=device) for _ in range(2)]

    def forward(self, x, topk_ids, topk_weights, shard: ExpertShard):
        cur = torch.cuda.current_stream(x.device)
        outs = []
        for i, (fx, st) in enumerate(zip(self.parts, self.streams)):
            lo, hi = i * self.half, (i + 1) * self.half
            st.wait_stream(cur)
            with torch.cuda.stream(st):
                outs.append(fx.forward(x[lo:hi], topk_ids[lo:hi].contiguous(), topk_weights[lo:hi], shard))
        for st in self.streams:
            cur.wait_stream(st)
        return torch.cat(outs, 0)
