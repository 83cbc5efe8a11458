"""Oracle restatements of the dense quantized contractions (test infrastructure).

Reference sources followed:
  * W4A16 kernel body   examples/kernels/contraction/weight_only_int4.py:18-51
  * W4A16 torch-CPU ref experiments/cpu/baselines/pytorch/cpu_runtime.py:97-102
  * packing recipe      experiments/cpu/providers/mojo/contraction.py:190-198
  * gemm_i8 kernel body examples/kernels/contraction/gemm.py:29-39
  * exact-int recipe    experiments/cpu/providers/weft/matrix.py:82-83
"""
from __future__ import annotations

import torch

PACK_FACTOR = 8  # weight_only_int4.py:8


def pack_int4(logical: torch.Tensor) -> torch.Tensor:
    """Pack a [K, N] integer tensor (only the low 4 bits of each entry are kept)
    into [K/8, N] int32, low nibble = lowest k.

    Follows the loop at experiments/cpu/providers/mojo/contraction.py:193-195
    (``packed |= (logical[lane::8] & 15) << (4 * lane)``).
    """
    K, N = logical.shape
    if K % PACK_FACTOR:
        raise ValueError("K must be a multiple of 8")
    logical = logical.to(torch.int32)
    packed = torch.zeros((K // PACK_FACTOR, N), dtype=torch.int32)
    for lane in range(PACK_FACTOR):
        packed |= (logical[lane::PACK_FACTOR] & 15) << (4 * lane)
    return packed


def unpack_int4(packed: torch.Tensor) -> torch.Tensor:
    """[K/8, N] int32 -> [K, N] int32 nibbles in 0..15 (cpu_runtime.py:98-99)."""
    K = packed.shape[0] * PACK_FACTOR
    positions = torch.arange(K)
    return (packed[positions // 8] >> ((positions % 8) * 4)[:, None]) & 15


def dequantize_int4(packed, scales, *, group_size: int, zero_point: int | None):
    """f32 dequantised weight [K, N].

    zero_point None  -> the reference's two's-complement nibble
                        (``nibble - ((nibble & 8) << 1)``, cpu_runtime.py:100);
    zero_point z     -> unsigned nibble minus z (z = 8 for the benchmark
                        configurations).  The two agree when the packed words
                        differ by ``^ 0x88888888``.
    """
    nibble = unpack_int4(packed)
    if zero_point is None:
        signed = nibble - ((nibble & 8) << 1)
    else:
        signed = nibble - int(zero_point)
    return signed.float() * scales.float().repeat_interleave(group_size, dim=0)


def weight_only_int4_matmul(activation, packed, scales, *, group_size: int = 64,
                            zero_point: int | None = None, out_dtype=None):
    """``(X.float() @ dequant_f32).to(out_dtype)``.

    With the defaults this is exactly cpu_runtime.py:97-102 (group 64, signed
    nibble, f16 result).  ``group_size``/``zero_point``/``out_dtype`` carry the
    benchmark configurations (group 128, zero-point 8, bf16).
    """
    out_dtype = activation.dtype if out_dtype is None else out_dtype
    dequantized = dequantize_int4(packed, scales, group_size=group_size, zero_point=zero_point)
    return (activation.float() @ dequantized).to(out_dtype)


def weight_only_int4_matmul_rounded(activation, packed, scales, *, group_size: int = 64,
                                    zero_point: int | None = None, out_dtype=None):
    """Same contraction with the dequantised weight rounded to the activation
    dtype before the f32-accumulated product, i.e. the kernel body's own order
    of operations (weight_only_int4.py:42: ``cast(unpacked, f16) * group_scales``
    is an f16 multiply; :43-47 accumulate in f32).  Used to bound the
    difference between the two legal contracts.
    """
    out_dtype = activation.dtype if out_dtype is None else out_dtype
    nibble = unpack_int4(packed)
    signed = nibble - ((nibble & 8) << 1) if zero_point is None else nibble - int(zero_point)
    expanded = scales.repeat_interleave(group_size, dim=0)
    dequantized = (signed.to(activation.dtype) * expanded.to(activation.dtype))
    return (activation.float() @ dequantized.float()).to(out_dtype)


def gemm_i8_exact_f64(a, b, bias=None):
    """i8 x i8 -> i32 through an f64 matmul (weft/matrix.py:82-83); exact because
    |sum| <= K * 127^2 < 2^53."""
    acc = (a.double() @ b.double()).to(torch.int64)
    if bias is not None:
        acc = acc + bias.to(torch.int64)[None, :]
    # two's-complement wrap to i32 (numerics spec: integers wrap)
    return ((acc + 2**31) % 2**32 - 2**31).to(torch.int32)


def gemm_i8(a, b, bias=None):
    """``C = i32(sum_k A[m,k] * B[k,n]) + bias[n]`` (gemm.py:29-39).

    Uses torch's CPU integer matmul; :func:`gemm_i8_exact_f64` is the
    reference's own recipe and the two are compared in the CPU tests.
    """
    M, K = a.shape
    if hasattr(torch, "_int_mm") and M > 0 and K > 0 and b.shape[1] > 0:
        try:
            acc = torch._int_mm(a.contiguous(), b.contiguous())
        except RuntimeError:
            return gemm_i8_exact_f64(a, b, bias)
    else:
        return gemm_i8_exact_f64(a, b, bias)
    if bias is not None:
        acc = acc + bias[None, :].to(torch.int32)
    return acc


def w8a8_scaled_gemm(a, b, a_scales, b_scales, *, out_dtype=torch.bfloat16):
    """``out = out_dtype(f32(acc) * sa[m] * sb[n])`` with the exact i32
    accumulator of :func:`gemm_i8`.  The per-token x per-channel epilogue is the
    benchmark's extension of gemm_i8; the nearest reference precedent is the
    per-channel scale of quantized_gemm (gemm.py:83-106).  Multiplication order
    is (acc * sa) * sb, all in f32, one rounding to the output type.
    """
    acc = gemm_i8(a, b)
    return ((acc.float() * a_scales.float()[:, None]) * b_scales.float()[None, :]).to(out_dtype), acc


def gemm(a, b, *, relu: bool = False):
    """Dense 16-bit GEMM with f32 accumulation and one rounding to the input type
    (examples/kernels/contraction/gemm.py:40-80)."""
    accumulator = a.float() @ b.float()
    if relu:
        accumulator = torch.relu(accumulator)
    return accumulator.to(a.dtype)


def quantized_gemm(a, b, bias, residual, scale):
    """GEMM + bias + ReLU + residual + per-channel scale + clamp + truncating int8 cast
    (examples/kernels/contraction/gemm.py:83-106, cpu_runtime.py:91-94)."""
    accumulator = a.float() @ b.float()
    fused = torch.relu(accumulator + bias) + residual.float()
    return (fused / scale).clamp(-128.0, 127.0).to(torch.int8)
