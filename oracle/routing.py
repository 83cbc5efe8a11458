"""Oracle restatements of the MoE router and the route alignment
(test infrastructure).

Reference sources followed:
  * softmax            examples/kernels/normalization/softmax.py:23-37,
                       experiments/cpu/baselines/pytorch/cpu_runtime.py:300-303
  * insertion top-k    examples/kernels/sampling/top_k.py:10-33,
                       cpu_runtime.py:759-773  (strict ``>``: lower index wins ties)
  * count / prefix / scatter / mark
                       examples/kernels/routing/moe_align.py:14-86,
                       examples/programs/composition.py:98-174,
                       cpu_runtime.py:1076-1097
  * canonical compare  experiments/cpu/providers/mojo/routing.py:27-43
"""
from __future__ import annotations

import torch


def softmax_f32(x: torch.Tensor) -> torch.Tensor:
    """exp(x - max) / sum in f32 (cpu_runtime.py:300-303)."""
    values = x.float()
    numerator = torch.exp(values - values.amax(dim=-1, keepdim=True))
    return numerator / numerator.sum(dim=-1, keepdim=True)


def insertion_top_k(logits: torch.Tensor, k: int):
    """Insertion top-k with a strict ``>`` compare, vectorised over rows exactly
    as cpu_runtime.py:759-773 does it (k is 8 there; a parameter here)."""
    rows = logits.shape[0]
    values = torch.full((rows, k), -torch.inf, dtype=logits.dtype)
    indices = torch.full((rows, k), -1, dtype=torch.int32)
    for candidate in range(logits.shape[1]):
        carry_value = logits[:, candidate]
        carry_index = torch.full((rows,), candidate, dtype=torch.int32)
        for slot in range(k):
            current_value = values[:, slot].clone()
            current_index = indices[:, slot].clone()
            swap = carry_value > current_value
            values[:, slot] = torch.where(swap, carry_value, current_value)
            indices[:, slot] = torch.where(swap, carry_index, current_index)
            carry_value = torch.where(swap, current_value, carry_value)
            carry_index = torch.where(swap, current_index, carry_index)
    return values, indices


def moe_route_top2(logits: torch.Tensor):
    """Router of the MoE benchmark configuration: top-2 experts per token with
    ties broken by the lower expert id, plus the two softmax probabilities.

    Selection runs on the raw f32 logits: softmax is strictly monotone in exact
    arithmetic, and selecting on logits keeps the index result independent of
    how exp() is rounded.  The route weights are the (not renormalised) f32
    softmax probabilities of the two chosen experts.  Returns (ids i32 [T,2],
    weights f32 [T,2]).
    """
    _, ids = insertion_top_k(logits.float(), 2)
    probabilities = softmax_f32(logits)
    weights = torch.gather(probabilities, 1, ids.long())
    return ids, weights


def moe_count_routes(topk_ids: torch.Tensor, num_experts: int) -> torch.Tensor:
    """counts[e] = number of routes to e (moe_align.py:14-29, cpu_runtime.py:1076-1078)."""
    return torch.bincount(topk_ids.flatten().long(), minlength=num_experts).int()


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int):
    """Restates cpu_runtime.py:1081-1097: per-expert spans padded to
    ``block_size``; inside a span the route ids appear in ascending order (stable
    argsort), the padding holds the sentinel ``routes``; ``expert_ids[b]`` is the
    expert owning block b.  Returns (sorted_ids, expert_ids, total_padded[1],
    offsets[E+1]) - the fourth value is what moe_prefix_routes writes
    (moe_align.py:32-49).  Blocks past ``total_padded`` are left at -1 here (the
    reference leaves them uninitialised).
    """
    flat = topk_ids.flatten()
    routes = flat.numel()
    counts = torch.bincount(flat.long(), minlength=num_experts)
    padded = (counts + block_size - 1) // block_size * block_size
    offsets = torch.cat((torch.zeros(1, dtype=torch.int64), padded.cumsum(0)))
    order = torch.argsort(flat, stable=True).to(torch.int32)
    capacity = routes + num_experts * (block_size - 1)
    sorted_ids = torch.full((capacity,), routes, dtype=torch.int32)
    expert_ids = torch.full(((capacity + block_size - 1) // block_size,), -1, dtype=torch.int32)
    source = 0
    for expert in range(num_experts):
        begin, end = int(offsets[expert]), int(offsets[expert + 1])
        count = int(counts[expert])
        sorted_ids[begin:begin + count] = order[source:source + count]
        expert_ids[begin // block_size:end // block_size] = expert
        source += count
    return sorted_ids, expert_ids, offsets[-1:].to(torch.int32), offsets.to(torch.int32)


def canonical_alignment(sorted_ids, expert_ids, total, *, block_size: int, num_experts: int):
    """Order-free view used by the reference to compare an atomically scattered
    alignment (mojo/routing.py:27-43): sort the ids inside each expert span."""
    total_value = int(total.reshape(-1)[0].item())
    blocks = total_value // block_size
    canonical = sorted_ids[:total_value].clone()
    active = expert_ids[:blocks]
    for expert in range(num_experts):
        owned = torch.nonzero(active == expert).flatten()
        if owned.numel() == 0:
            continue
        begin = int(owned[0]) * block_size
        end = (int(owned[-1]) + 1) * block_size
        canonical[begin:end] = torch.sort(canonical[begin:end]).values
    return canonical, active, total
