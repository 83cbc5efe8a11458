"""Packed-weight contractions (int4 x int8, interleaved int2 x int8, fp4 -> bf16) against the
reference's golden outputs and the oracle.  The integer programs must be bit-exact
(the reference compares them with atol 0: experiments/cpu/providers/mojo/contraction.py:201-217);
the fp4 program uses the reference's atol 1.0 / rtol 2e-2 (contraction.py:220-224) and the
benchmark's max|y - ref| <= 2e-2 * max|ref|."""
import pytest
import torch

import intent_b200 as ib
import oracle
from intent_b200.runtime import native
from conftest import load_golden, max_abs_rel

pytestmark = pytest.mark.gpu


def _clean():
    lib = native.library()
    return lib.intent_b200_i8_gemm_device_status() == 0 and lib.intent_b200_grouped_gemm16_device_status() == 0


def _pad_rows(t, multiple):
    rows = -(-t.shape[0] // multiple) * multiple
    out = torch.zeros((rows,) + tuple(t.shape[1:]), dtype=t.dtype)
    out[:t.shape[0]] = t
    return out


def test_w4a8_golden(cuda_device):
    g = load_golden("w4a8_small")                       # M = 24: padded to the kernel's multiple of 16
    activation = _pad_rows(g["activation"], 16)
    artifact = ib.compile(ib.programs.w4a8_packed_matmul, target=ib.B200Target(0))
    out = artifact.run(activation.to(cuda_device), g["packed"].to(cuda_device))
    torch.cuda.synchronize()
    assert _clean() and out.dtype == torch.int32
    assert torch.equal(out.cpu()[:, :24], g["output"])
    assert torch.all(out.cpu()[:, 24:] == 0)


@pytest.mark.parametrize("M,K,N", [(16, 32, 8), (128, 256, 200), (272, 4096, 1000), (4096, 1024, 512)])
def test_w4a8_exact(cuda_device, M, K, N):
    gen = torch.Generator().manual_seed(M + K + N)
    activation = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=gen)
    packed = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=gen)
    artifact = ib.compile(ib.programs.w4a8_packed_matmul, target=ib.B200Target(0))
    out = artifact.run(activation.to(cuda_device), packed.to(cuda_device))
    torch.cuda.synchronize()
    assert _clean() and out.shape == (N, M)
    assert torch.equal(out.cpu(), oracle.w4a8_packed_matmul(activation, packed))


@pytest.mark.parametrize("tag", ["small", "full_range"])
def test_bitnet_golden(cuda_device, tag):
    g = load_golden(f"bitnet_int2_{tag}")
    packed = _pad_rows(g["packed"], 16)                 # N = 40 / 72: padded to the kernel's multiple of 16
    artifact = ib.compile(ib.programs.bitnet_int2_matmul, target=ib.B200Target(0))
    out = artifact.run(g["activation"].to(cuda_device), packed.to(cuda_device))
    torch.cuda.synchronize()
    n = g["output"].shape[1]
    assert _clean() and torch.equal(out.cpu()[:, :n], g["output"])


@pytest.mark.parametrize("M,K,N", [(1, 4096, 4096), (5, 64, 16), (300, 1024, 272)])
def test_bitnet_exact(cuda_device, M, K, N):
    gen = torch.Generator().manual_seed(M + K + N)
    activation = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=gen)
    packed = torch.randint(0, 256, (N, K // 4), dtype=torch.uint8, generator=gen)
    artifact = ib.compile(ib.programs.bitnet_int2_matmul, target=ib.B200Target(0))
    out = artifact.run(activation.to(cuda_device), packed.to(cuda_device))
    torch.cuda.synchronize()
    assert _clean() and out.shape == (M, N)
    assert torch.equal(out.cpu(), oracle.bitnet_int2_matmul(activation, packed))


@pytest.mark.parametrize("tag", ["small", "all_codes"])
def test_fp4_golden(cuda_device, tag):
    g = load_golden(f"dequant_bf16_fp4_{tag}")
    artifact = ib.compile(ib.programs.dequant_bf16_fp4_matmul, target=ib.B200Target(0))
    out = artifact.run(g["activation"].to(cuda_device), g["packed"].to(cuda_device))
    torch.cuda.synchronize()
    assert _clean()
    assert torch.allclose(out.cpu().float(), g["output"].float(), atol=1.0, rtol=2e-2)
    assert max_abs_rel(out.cpu(), g["output"]) <= 2e-2


@pytest.mark.parametrize("M,K,N", [(8, 64, 8), (130, 520, 264), (1024, 4096, 1024)])
def test_fp4_matches_oracle(cuda_device, M, K, N):
    gen = torch.Generator().manual_seed(M + K + N)
    activation = (torch.randn((M, K), generator=gen) * 0.125).bfloat16()
    packed = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=gen)
    artifact = ib.compile(ib.programs.dequant_bf16_fp4_matmul, target=ib.B200Target(0))
    out = artifact.run(activation.to(cuda_device), packed.to(cuda_device))
    torch.cuda.synchronize()
    assert _clean() and out.shape == (M, N)
    reference = oracle.dequant_bf16_fp4_matmul(activation, packed)
    assert max_abs_rel(out.cpu(), reference) <= 2e-2
    assert torch.allclose(out.cpu().float(), reference.float(), rtol=2.0 ** -6, atol=2e-2)


def test_packed_shape_rules(cuda_device):
    artifact = ib.compile(ib.programs.w4a8_packed_matmul, target=ib.B200Target(0))
    a = torch.zeros((16, 64), dtype=torch.int8, device=cuda_device)
    with pytest.raises(ValueError):
        artifact.run(a, torch.zeros((8, 30), dtype=torch.uint8, device=cuda_device))      # P * 2 != K
    with pytest.raises(TypeError):
        artifact.run(a, torch.zeros((8, 32), dtype=torch.int8, device=cuda_device))       # dtype is not coerced
