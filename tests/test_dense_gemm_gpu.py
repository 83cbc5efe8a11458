"""Dense 16-bit GEMM programs of the reference's gemm.py on the ragged tcgen05 kernel:
gemm (f16, optional ReLU), bf16_gemm and quantized_gemm (int8 epilogue, the reference's
IntegerTolerance(max_abs=2): experiments/cpu/providers/mojo/contraction.py:177-186)."""
import pytest
import torch

import intent_b200 as ib
import oracle
from intent_b200.runtime import native
from conftest import load_golden, max_abs_rel

pytestmark = pytest.mark.gpu


def _status():
    return native.library().intent_b200_grouped_gemm16_device_status()


@pytest.mark.parametrize("activation", ["none", "relu"])
@pytest.mark.parametrize("M,K,N", [(128, 64, 256), (37, 200, 72), (1000, 1032, 520)])
def test_gemm_f16(cuda_device, activation, M, K, N):
    gen = torch.Generator().manual_seed(M + K + N)
    a = (torch.randn((M, K), generator=gen) / K ** 0.5).half()
    b = torch.randn((K, N), generator=gen).half()
    artifact = ib.compile(ib.programs.gemm, target=ib.B200Target(0), constexprs={"ACTIVATION": activation})
    c = artifact.run(a.to(cuda_device), b.to(cuda_device))
    torch.cuda.synchronize()
    assert _status() == 0
    reference = oracle.gemm(a, b, relu=activation == "relu")
    assert max_abs_rel(c.cpu(), reference) <= 2e-2
    assert torch.allclose(c.cpu().float(), reference.float(), rtol=2.0 ** -9, atol=1e-3)
    if activation == "relu":
        assert torch.all(c >= 0)


@pytest.mark.parametrize("M,K,N", [(256, 512, 256), (77, 136, 1000)])
def test_bf16_gemm(cuda_device, M, K, N):
    gen = torch.Generator().manual_seed(M + K + N)
    a = (torch.randn((M, K), generator=gen) / K ** 0.5).bfloat16()
    b = torch.randn((K, N), generator=gen).bfloat16()
    artifact = ib.compile(ib.programs.bf16_gemm, target=ib.B200Target(0))
    c = artifact.run(a.to(cuda_device), b.to(cuda_device))
    torch.cuda.synchronize()
    assert _status() == 0
    reference = oracle.gemm(a, b)
    assert max_abs_rel(c.cpu(), reference) <= 2e-2
    assert torch.allclose(c.cpu().float(), reference.float(), rtol=2.0 ** -6, atol=1e-3)


def test_quantized_gemm_golden(cuda_device):
    g = load_golden("quantized_gemm_small")
    artifact = ib.compile(ib.programs.quantized_gemm, target=ib.B200Target(0))
    out = artifact.run(*(g[k].to(cuda_device) for k in ("a", "b", "bias", "residual", "scale")))
    torch.cuda.synchronize()
    assert _status() == 0 and out.dtype == torch.int8
    difference = (out.cpu().int() - g["output"].int()).abs()
    assert difference.max().item() <= 2
    assert (difference > 0).float().mean().item() < 0.02      # a truncation boundary is crossed rarely


@pytest.mark.parametrize("M,K,N", [(130, 520, 264), (1024, 1024, 2048)])
def test_quantized_gemm_matches_oracle(cuda_device, M, K, N):
    gen = torch.Generator().manual_seed(M + K + N)
    a = (torch.randn((M, K), generator=gen) / K ** 0.5).half()
    b = torch.randn((K, N), generator=gen).half()
    bias = torch.randn((N,), generator=gen) * 0.25
    residual = (torch.randn((M, N), generator=gen) * 0.25).half()
    scale = torch.linspace(1.0 / 48.0, 1.0 / 24.0, N, dtype=torch.float32)
    artifact = ib.compile(ib.programs.quantized_gemm, target=ib.B200Target(0))
    out = artifact.run(a.to(cuda_device), b.to(cuda_device), bias.to(cuda_device), residual.to(cuda_device),
                       scale.to(cuda_device))
    torch.cuda.synchronize()
    assert _status() == 0
    reference = oracle.quantized_gemm(a, b, bias, residual, scale)
    difference = (out.cpu().int() - reference.int()).abs()
    assert difference.max().item() <= 2
    assert (difference > 0).float().mean().item() < 0.02
    assert out.min().item() >= -128 and out.max().item() <= 127 and (out == 127).any()   # saturation is reached
