"""Seeded synthetic inputs for the benchmark configurations.

All tensors are drawn on the CPU from one ``torch.Generator`` seeded with
``seed`` in a fixed draw order (documented per function), so the same values
are produced on every machine.  The distributions are the ones the benchmark
configurations state; the packing follows the reference's recipe
(experiments/cpu/providers/mojo/contraction.py:193-195: low nibble = lowest k).
"""
from __future__ import annotations

import torch

PACK_FACTOR = 8


def pack_int4(logical: torch.Tensor) -> torch.Tensor:
    """[K, N] integers (low 4 bits kept) -> [K/8, N] int32, low nibble = lowest k."""
    K, N = logical.shape
    if K % PACK_FACTOR:
        raise ValueError("K must be a multiple of 8")
    logical = logical.to(torch.int32)
    packed = torch.zeros((K // PACK_FACTOR, N), dtype=torch.int32)
    for lane in range(PACK_FACTOR):
        packed |= (logical[lane::PACK_FACTOR] & 15) << (4 * lane)
    return packed


def _generator(seed: int) -> torch.Generator:
    return torch.Generator(device="cpu").manual_seed(int(seed))


def w4a16_inputs(M: int, K: int, N: int, *, dtype=torch.float16, group_size: int = 128,
                 seed: int = 0, activation_scale: float = 1.0):
    """Draw order: X ~ N(0,1) [M,K]; q ~ U{0..15} [K,N]; S = 0.002 + 0.01|N(0,1)| [K/G,N].

    Returns (X dtype, packed i32 [K/8,N], scales dtype [K/G,N]).  The zero-point
    of these unsigned nibbles is 8.
    """
    g = _generator(seed)
    x = (torch.randn((M, K), generator=g, dtype=torch.float32) * activation_scale).to(dtype)
    q = torch.randint(0, 16, (K, N), generator=g, dtype=torch.int32)
    scales = (0.002 + 0.01 * torch.randn((K // group_size, N), generator=g,
                                         dtype=torch.float32).abs()).to(dtype)
    return x, pack_int4(q), scales


def w8a8_inputs(M: int, K: int, N: int, *, seed: int = 0):
    """Draw order: A ~ U{-127..127} [M,K]; sa = 0.01|N(0,1)|+1e-3 [M]; B ~ U{-127..127} [K,N];
    sb same distribution [N].  Returns (A i8, B i8, sa f32, sb f32)."""
    g = _generator(seed)
    a = torch.randint(-127, 128, (M, K), generator=g, dtype=torch.int8)
    sa = 0.01 * torch.randn((M,), generator=g, dtype=torch.float32).abs() + 1e-3
    b = torch.randint(-127, 128, (K, N), generator=g, dtype=torch.int8)
    sb = 0.01 * torch.randn((N,), generator=g, dtype=torch.float32).abs() + 1e-3
    return a, b, sa, sb


def moe_inputs(tokens: int, hidden: int, experts: int, intermediate: int, *,
               dtype=torch.bfloat16, group_size: int = 128, seed: int = 0):
    """Draw order: logits ~ N(0,1) f32 [T,E]; x ~ N(0,1)/sqrt(H) [T,H]; then per
    tensor (up_gate, down): q ~ U{0..15}, S = 0.002 + 0.01|N(0,1)|.

    Returns dict with logits, x, up_gate_packed [E,H/8,2I], up_gate_scales
    [E,H/G,2I], down_packed [E,I/8,H], down_scales [E,I/G,H].  The 1/sqrt(H)
    activation scale follows the reference's MoE case
    (experiments/cpu/providers/mojo/ragged.py:197-206).
    """
    g = _generator(seed)
    logits = torch.randn((tokens, experts), generator=g, dtype=torch.float32)
    x = (torch.randn((tokens, hidden), generator=g, dtype=torch.float32) / hidden ** 0.5).to(dtype)

    def quantised(K, N):
        q = torch.randint(0, 16, (experts * K, N), generator=g, dtype=torch.int32)
        packed = pack_int4(q).reshape(experts, K // PACK_FACTOR, N)
        scales = (0.002 + 0.01 * torch.randn((experts, K // group_size, N), generator=g,
                                             dtype=torch.float32).abs()).to(dtype)
        return packed, scales

    up_gate_packed, up_gate_scales = quantised(hidden, 2 * intermediate)
    down_packed, down_scales = quantised(intermediate, hidden)
    return dict(logits=logits, x=x, up_gate_packed=up_gate_packed, up_gate_scales=up_gate_scales,
                down_packed=down_packed, down_scales=down_scales)


def moe_activations(tokens: int, hidden: int, experts: int, *, dtype=torch.bfloat16, seed: int = 0):
    """Router logits ~ N(0,1) f32 [T,E] and x ~ N(0,1)/sqrt(H) [T,H]: the first two draws of
    :func:`moe_inputs`, so both functions give the same activations for one seed."""
    g = _generator(seed)
    logits = torch.randn((tokens, experts), generator=g, dtype=torch.float32)
    x = (torch.randn((tokens, hidden), generator=g, dtype=torch.float32) / hidden ** 0.5).to(dtype)
    return logits, x


def moe_expert_weights(first: int, count: int, hidden: int, intermediate: int, *, dtype=torch.bfloat16,
                       group_size: int = 128, seed: int = 0):
    """Int4 weights of experts ``first .. first+count-1``, each expert from its own generator (seeded with
    ``seed`` and the expert's global id), so any rank can draw exactly its own experts.

    The packed words are drawn directly as uniform 32-bit integers: eight independent nibbles uniform on
    0..15, i.e. the same distribution as packing ``q ~ U{0..15}``, at an eighth of the draws (64 experts
    of the benchmark shape take about a second instead of half a minute).  Scales are
    0.002 + 0.01|N(0,1)|.  Returns (up_gate_packed [n,H/8,2I], up_gate_scales [n,H/G,2I],
    down_packed [n,I/8,H], down_scales [n,I/G,H]).
    """
    out = [[], [], [], []]
    for expert in range(first, first + count):
        g = _generator(seed * 1000003 + 7919 * (expert + 1))
        for slot, (K, N) in ((0, (hidden, 2 * intermediate)), (2, (intermediate, hidden))):
            out[slot].append(torch.randint(-2 ** 31, 2 ** 31, (K // PACK_FACTOR, N), generator=g,
                                           dtype=torch.int64).to(torch.int32))
            out[slot + 1].append((0.002 + 0.01 * torch.randn((K // group_size, N), generator=g,
                                                             dtype=torch.float32).abs()).to(dtype))
    return tuple(torch.stack(parts) for parts in out)
