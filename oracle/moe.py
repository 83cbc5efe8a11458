"""Oracle restatements of the ragged / MoE programs (test infrastructure).

Reference sources followed:
  * ragged grouped GEMM        examples/kernels/ragged/grouped_gemm.py:11-70,
                               experiments/cpu/baselines/pytorch/cpu_runtime.py:859-864
  * routed expert projection   grouped_gemm.py:101-138, cpu_runtime.py:874-881
  * MoE expert FFN             examples/kernels/ragged/moe.py:12-53, cpu_runtime.py:1279-1286
  * SiLU gate                  examples/kernels/activation/swiglu.py:27-46,
                               cpu_runtime.py:274-278, 76-78
"""
from __future__ import annotations

import torch

from .contraction import dequantize_int4


def ragged_grouped_gemm(x, offsets, weight):
    """rows offsets[g]:offsets[g+1] of X times W[g] (cpu_runtime.py:859-864)."""
    output = torch.zeros((x.shape[0], weight.shape[2]), dtype=x.dtype)
    for group in range(weight.shape[0]):
        begin, end = int(offsets[group]), int(offsets[group + 1])
        output[begin:end] = (x[begin:end].float() @ weight[group].float()).to(x.dtype)
    return output


def routed_expert_projection(x, offsets, member_routes, weight):
    """out[token, slot, :] = x[token] @ W[e].T for every route of expert e, with
    token = route // top_k and slot = route % top_k (cpu_runtime.py:874-881);
    weight is [E, N, K]."""
    top_k = member_routes.numel() // x.shape[0]
    output = torch.zeros((x.shape[0] * top_k, weight.shape[1]), dtype=x.dtype)
    for expert in range(weight.shape[0]):
        routes = member_routes[int(offsets[expert]):int(offsets[expert + 1])].long()
        values = x[routes // top_k].float() @ weight[expert].float().T
        output[routes] = values.to(x.dtype)
    return output.reshape(x.shape[0], top_k, weight.shape[1])


def moe_expert_ffn(x, route_offsets, member_routes, route_token, route_weights, w1, w2, y, *, round_hidden=False):
    """The reference's dense-weight MoE FFN (cpu_runtime.py:1279-1286): ReLU
    between the two products, weighted add into the f32 InOut ``y``.  The kernel
    body rounds the hidden activation to the input dtype between the products
    (moe.py:42); the torch reference does not - both are inside the reference's
    own tolerance.  The default follows the torch reference; ``round_hidden``
    follows the kernel body."""
    for expert in range(w1.shape[0]):
        routes = member_routes[int(route_offsets[expert]):int(route_offsets[expert + 1])].long()
        tokens = route_token[routes].long()
        hidden = torch.relu(x[tokens].float() @ w1[expert].float())
        if round_hidden:
            hidden = hidden.to(x.dtype).float()
        values = hidden @ w2[expert].float()
        y.index_add_(0, tokens, route_weights[routes, None] * values)
    return y


def silu_and_mul(gate_up: torch.Tensor, out_dtype=None):
    """Packed SiLU gate: first half of the columns is the gate, second half the
    up projection; ``silu(gate) * up`` evaluated in f32 with one final rounding
    (swiglu.py:35-46 'silu_and_mul_packed'; sigmoid as 1/(1+exp(-g)),
    cpu_runtime.py:274-278)."""
    half = gate_up.shape[1] // 2
    gate = gate_up[:, :half].float()
    up = gate_up[:, half:].float()
    sigmoid = 1.0 / (1.0 + torch.exp(-gate))
    result = gate * sigmoid * up
    return result if out_dtype is None else result.to(out_dtype)


def grouped_w4a16_gemm(x_sorted, expert_of_row, packed, scales, *, group_size, zero_point):
    """Rows already sorted by expert: out[r] = x_sorted[r] @ dequant(W[expert_of_row[r]])
    in f32.  packed is [E, K/8, N] i32, scales [E, K/G, N]."""
    out = torch.zeros((x_sorted.shape[0], packed.shape[2]), dtype=torch.float32)
    for expert in range(packed.shape[0]):
        rows = torch.nonzero(expert_of_row == expert).flatten()
        if rows.numel() == 0:
            continue
        weight = dequantize_int4(packed[expert], scales[expert], group_size=group_size,
                                 zero_point=zero_point)
        out[rows] = x_sorted[rows].float() @ weight
    return out


def moe_w4a16_swiglu_ffn(x, topk_ids, topk_weights, up_gate_packed, up_gate_scales,
                         down_packed, down_scales, *, group_size=128, zero_point=8,
                         round_hidden: bool = True):
    """MoE FFN of the benchmark configuration, per-expert loop in route order
    (restated from cpu_runtime.py:1279-1286 with int4 dequantisation and a SiLU
    gate in place of ReLU):

        for every route (token t, choice c) with expert e = topk_ids[t, c]:
            gu = x[t] @ dequant(W_upgate[e])      # [2*I], gate = first I columns
            h  = silu(gate) * up                  # f32; rounded to x.dtype when
                                                  # round_hidden (moe.py:42 rounds
                                                  # the hidden activation likewise)
            o  = h @ dequant(W_down[e])           # [H] f32
            y[t] += topk_weights[t, c] * o        # f32

    Returns y f32 [T, H].
    """
    tokens, hidden = x.shape
    experts = up_gate_packed.shape[0]
    top_k = topk_ids.shape[1]
    y = torch.zeros((tokens, hidden), dtype=torch.float32)
    flat = topk_ids.flatten().long()
    member_routes = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=experts)
    offsets = torch.cat((torch.zeros(1, dtype=torch.int64), counts.cumsum(0)))
    weights = topk_weights.flatten().float()
    for expert in range(experts):
        routes = member_routes[int(offsets[expert]):int(offsets[expert + 1])]
        if routes.numel() == 0:
            continue
        token = routes // top_k
        w_up = dequantize_int4(up_gate_packed[expert], up_gate_scales[expert],
                               group_size=group_size, zero_point=zero_point)
        w_down = dequantize_int4(down_packed[expert], down_scales[expert],
                                 group_size=group_size, zero_point=zero_point)
        gate_up = x[token].float() @ w_up
        h = silu_and_mul(gate_up)
        if round_hidden:
            h = h.to(x.dtype).float()
        out = h @ w_down
        y.index_add_(0, token, weights[routes, None] * out)
    return y
