"""Oracle restatements of the packed-weight contractions next to the W4A16 path
(test infrastructure; the product never imports this module).

Reference sources followed:
  * w4a8_packed_matmul        examples/kernels/contraction/weight_only_int4.py:54-91,
                              experiments/cpu/baselines/pytorch/cpu_runtime.py:105-108
  * bitnet_int2_matmul        weight_only_int4.py:94-123, cpu_runtime.py:111-114
  * dequant_bf16_fp4_matmul   weight_only_int4.py:126-175, cpu_runtime.py:117-124

Pinned by tests/golden/{w4a8_small,bitnet_int2_*,dequant_bf16_fp4_*}.npz, which hold the
outputs of the reference's own torch functions.  The integer products are evaluated in
int64 and wrapped to int32, which is the kernel bodies' stated arithmetic (the reference's
torch functions go through f32, exact only while every sum stays below 2**24).
"""
from __future__ import annotations

import torch


def _wrap_i32(value: torch.Tensor) -> torch.Tensor:
    return ((value + 2 ** 31) % 2 ** 32 - 2 ** 31).to(torch.int32)


def unpack_w4a8(packed: torch.Tensor) -> torch.Tensor:
    """u8 [N, K/2] -> signed int4 values [N, K] as int8; the low nibble is the even k
    (weight_only_int4.py:66-85)."""
    nibbles = torch.stack((packed & 15, packed >> 4), dim=-1).flatten(1).to(torch.int16)
    return (nibbles - ((nibbles & 8) << 1)).to(torch.int8)


def w4a8_packed_matmul(activation: torch.Tensor, packed: torch.Tensor) -> torch.Tensor:
    """output[N, M] = i32(signed(W)[N, K] . activation[M, K]^T)."""
    return _wrap_i32(unpack_w4a8(packed).to(torch.int64) @ activation.to(torch.int64).T)


def unpack_bitnet_int2(packed: torch.Tensor) -> torch.Tensor:
    """u8 [N, K/4] -> values 0..3 [N, K] as int8.  Sixteen values share a 4-byte word:
    value k of the word sits in byte k % 4 at bit 2 * (k // 4) (weight_only_int4.py:105-117)."""
    groups = packed.reshape(packed.shape[0], -1, 4)
    lanes = torch.stack(tuple((groups >> (lane * 2)) & 3 for lane in range(4)), dim=2)
    return lanes.flatten(1).to(torch.int8)


def bitnet_int2_matmul(activation: torch.Tensor, packed: torch.Tensor) -> torch.Tensor:
    """output[M, N] = i32(activation[M, K] . decoded[N, K]^T)."""
    return _wrap_i32(activation.to(torch.int64) @ unpack_bitnet_int2(packed).to(torch.int64).T)


def decode_fp4_bf16(packed: torch.Tensor) -> torch.Tensor:
    """u8 [N, K/2] -> bf16 [N, K]: two bytes form a big-endian 16-bit word of four e2m1 codes whose
    sign / exponent / mantissa bits are moved to bf16 positions and rescaled by 2**126
    (weight_only_int4.py:141-167)."""
    word = (packed[:, 0::2].to(torch.int32) << 8) | packed[:, 1::2].to(torch.int32)
    bits = torch.stack((word & 0x81C0, (word << 3) & 0x81C0, (word << 6) & 0x81C0,
                        ((word << 1) & 0x8000) | ((word >> 3) & 0x0180) | ((word >> 7) & 0x0040)),
                       dim=-1).flatten(1).to(torch.int16)
    return (bits.view(torch.bfloat16).float() * (2.0 ** 126)).bfloat16()


def dequant_bf16_fp4_matmul(activation: torch.Tensor, packed: torch.Tensor) -> torch.Tensor:
    """output[M, N] = bf16(activation[M, K] . decoded[N, K]^T), f32 accumulation."""
    return (activation.float() @ decode_fp4_bf16(packed).float().T).bfloat16()
