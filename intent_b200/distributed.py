"""Multi-GPU forms of the programs: one process per GPU, ``torch.distributed``.

The reference is single-device (each artifact binds one CUDA device,
python/intent/runtime/artifact.py:216-237); what is here is the sharding the
benchmark configurations ask for.

  * Dense W4A16 prefill and W8A8 shard over output columns: rank r owns a
    contiguous block of columns of the weight (and of its scales), activations are
    replicated, every rank writes its own block of Y.  No collective on the path.
  * MoE is expert-parallel: rank r owns experts [r*E/g, (r+1)*E/g).  Tokens are
    routed where they live, token rows travel to the owners of their experts with
    one all-to-all, the expert FFN runs on the received rows, the f32 result rows
    travel back with the reverse all-to-all and are combined per token.  The rows a
    kernel reads are always in local memory.
"""
from __future__ import annotations

from dataclasses import dataclass


def column_shard(columns: int, world: int, rank: int, multiple: int = 256) -> slice:
    """Contiguous block of output columns owned by ``rank``; block edges are multiples of
    ``multiple`` (one kernel tile) except the last edge."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    tiles = -(-columns // multiple)
    first = (tiles * rank) // world * multiple
    last = min(columns, (tiles * (rank + 1)) // world * multiple)
    return slice(first, max(first, last))


@dataclass
class ExchangePlan:
    """Row counts of one all-to-all: what this rank sends to / receives from every rank."""

    send: list
    receive: list

    @property
    def received_rows(self) -> int:
        return int(sum(self.receive))


def exchange_counts(send_counts, group=None) -> ExchangePlan:
    """All ranks tell each other how many rows they will send (one small all-to-all);
    the counts come back to the host because the collective needs them as split sizes."""
    import torch
    import torch.distributed as dist

    send = send_counts.to(torch.int64)
    received = torch.empty_like(send)
    dist.all_to_all_single(received, send, group=group)
    return ExchangePlan([int(v) for v in send.cpu()], [int(v) for v in received.cpu()])


def dispatch_rows(rows, plan: ExchangePlan, group=None):
    """rows sorted by destination rank [sum(send), ...] -> rows received, grouped by source rank."""
    import torch
    import torch.distributed as dist

    out = torch.empty((plan.received_rows, *rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=plan.receive, input_split_sizes=plan.send,
                           group=group)
    return out


def return_rows(rows, plan: ExchangePlan, group=None):
    """Inverse of :func:`dispatch_rows`: results for received rows go back to their senders and
    arrive in the order the rows were sent."""
    import torch
    import torch.distributed as dist

    out = torch.empty((int(sum(plan.send)), *rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=plan.send, input_split_sizes=plan.receive,
                           group=group)
    return out


class ExpertParallelMoE:
    """Expert-parallel SiLU-gated int4 MoE FFN.  ``experts`` is the global expert count,
    ``tokens`` the number of tokens routed by THIS rank per call; every rank holds the weights of
    its own ``experts // world`` experts."""

    def __init__(self, *, tokens, hidden, intermediate, experts, top_k=2, group_size=128, zero_point=8,
                 act_dtype="bf16", capacity_rows=None, target=None, group=None):
        import torch.distributed as dist

        from . import programs
        from .compiler import compile as _compile
        from .moe import MoEAlignment, MoEW4A16FFN

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if experts % self.world:
            raise ValueError("the expert count must be a multiple of the number of ranks")
        self.local_experts = experts // self.world
        self.tokens, self.hidden, self.top_k = tokens, hidden, top_k
        self.routes = tokens * top_k
        # rows this rank may receive; the worst case is every route of every rank
        self.capacity = capacity_rows or self.routes * self.world
        self.router = _compile(programs.moe_route_top2, target=target)
        # sorting routes by destination rank is the same stable partition as the expert alignment
        self.by_rank = MoEAlignment.build(tokens=tokens, top_k=top_k, experts=self.world, block_size=1,
                                          target=target)
        rank_constexprs = {"TOKENS": tokens, "TOP_K": top_k, "EXPERTS": self.world, "BLOCK_SIZE": 1}
        self.send_positions = _compile(programs.moe_route_positions, target=target, constexprs=rank_constexprs)
        self.gather = _compile(programs.moe_gather_rows, target=target,
                               constexprs={"ACT_DTYPE": act_dtype, "TOP_K": top_k})
        self.local = MoEW4A16FFN(tokens=self.capacity, hidden=hidden, intermediate=intermediate,
                                 experts=self.local_experts, top_k=1, group_size=group_size,
                                 zero_point=zero_point, act_dtype=act_dtype, target=target)
        self.combine = _compile(programs.moe_combine, target=target)

    def forward(self, logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales):
        """logits [T, E] f32 and x [T, H] of this rank's tokens; weights of this rank's experts.
        Returns y [T, H] f32."""
        import torch

        ids, weights = self.router.run(logits)
        destination = torch.div(ids, self.local_experts, rounding_mode="floor").to(torch.int32)
        sorted_routes, _, total = self.by_rank.run(destination)            # routes grouped by destination rank
        counts = torch.bincount(destination.flatten(), minlength=self.world)
        plan = exchange_counts(counts, self.group)
        send_rows = self.gather.run(x, sorted_routes, total)[: self.routes]
        send_experts = (ids.flatten()[sorted_routes[: self.routes].long()] % self.local_experts).to(torch.int32)
        received = dispatch_rows(send_rows, plan, self.group)
        received_experts = dispatch_rows(send_experts.unsqueeze(1), plan, self.group)
        n = plan.received_rows
        if n > self.capacity:
            raise RuntimeError(f"received {n} rows, capacity is {self.capacity}")
        results = torch.zeros((n, self.hidden), dtype=torch.float32, device=x.device)
        if n:
            rows, positions = self.local.experts_forward(received, received_experts.contiguous(), up_gate_packed,
                                                         up_gate_scales, down_packed, down_scales)
            ones = torch.ones((n, 1), dtype=torch.float32, device=x.device)
            self.combine.run(rows, positions[:n], ones, results)            # back to arrival order
        returned = return_rows(results, plan, self.group)                   # [routes, H] in send order
        send_position = self.send_positions.run(sorted_routes, total)       # route -> slot in send order
        y = torch.zeros((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
        self.combine.run(returned, send_position, weights, y)
        return y

    __call__ = forward
