"""int8 tensor-core GEMM: the int32 accumulator must be bit-exact, the scaled bf16
epilogue within 2e-2 * max|ref| (in practice one bf16 rounding)."""
import pytest
import torch

import intent_b200 as ib
import oracle
from intent_b200.runtime import native
from conftest import load_golden, max_abs_rel

pytestmark = pytest.mark.gpu


def _status():
    return native.library().intent_b200_i8_gemm_device_status()


@pytest.mark.parametrize("tag", ["small"])
def test_gemm_i8_golden(cuda_device, tag):
    g = load_golden(f"gemm_i8_{tag}")
    artifact = ib.compile(ib.programs.gemm_i8, target=ib.B200Target(0))
    out = artifact.run(g["a"].to(cuda_device), g["b"].to(cuda_device), g["bias"].to(cuda_device))
    torch.cuda.synchronize()
    assert _status() == 0
    assert out.dtype == torch.int32
    assert torch.equal(out.cpu(), g["output"])


@pytest.mark.parametrize("M,K,N", [(128, 128, 256), (37, 384, 144), (300, 1040, 528), (1024, 4096, 1024),
                                   (129, 16, 16)])
def test_gemm_i8_exact(cuda_device, M, K, N):
    gen = torch.Generator().manual_seed(M + K + N)
    a = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=gen)
    b = torch.randint(-128, 128, (K, N), dtype=torch.int8, generator=gen)
    bias = torch.randint(-2**31, 2**31 - 1, (N,), dtype=torch.int64, generator=gen).to(torch.int32)  # exercises wraparound
    artifact = ib.compile(ib.programs.gemm_i8, target=ib.B200Target(0))
    out = artifact.run(a.to(cuda_device), b.to(cuda_device), bias.to(cuda_device))
    torch.cuda.synchronize()
    assert _status() == 0
    assert torch.equal(out.cpu(), oracle.gemm_i8_exact_f64(a, b, bias))


def test_gemm_i8_extremes(cuda_device):
    a = torch.full((128, 8192), -128, dtype=torch.int8)
    b = torch.full((8192, 256), -128, dtype=torch.int8)
    artifact = ib.compile(ib.programs.gemm_i8, target=ib.B200Target(0))
    out = artifact.run(a.to(cuda_device), b.to(cuda_device), torch.zeros(256, dtype=torch.int32, device=cuda_device))
    assert torch.equal(out.cpu(), torch.full((128, 256), 8192 * 128 * 128, dtype=torch.int32))


@pytest.mark.parametrize("M,K,N", [(256, 512, 256), (100, 1024, 272)])
def test_w8a8_scaled_epilogue(cuda_device, M, K, N):
    a, b, sa, sb = ib.workloads.w8a8_inputs(M, K, N, seed=3)
    artifact = ib.compile(ib.programs.w8a8_gemm, target=ib.B200Target(0))
    out = artifact.run(a.to(cuda_device), b.to(cuda_device), sa.to(cuda_device), sb.to(cuda_device))
    torch.cuda.synchronize()
    assert _status() == 0
    ref, _ = oracle.w8a8_scaled_gemm(a, b, sa, sb)
    assert out.dtype == torch.bfloat16
    assert max_abs_rel(out.cpu(), ref) <= 2e-2
    assert torch.equal(out.cpu(), ref)          # same f32 operation order, one rounding: identical bits


def test_w8a8_full_size_accumulator_bit_exact(cuda_device):
    """Benchmark configuration 3 (4096 x 8192 x 8192): the raw accumulator through gemm_i8 with a zero
    bias must equal the CPU integer matmul on sampled rows; the bf16 output must equal the epilogue
    formula applied to that accumulator everywhere (checked on the GPU)."""
    M, K, N = 4096, 8192, 8192
    a, b, sa, sb = ib.workloads.w8a8_inputs(M, K, N, seed=0)
    ad, bd, sad, sbd = (t.to(cuda_device) for t in (a, b, sa, sb))
    acc = ib.compile(ib.programs.gemm_i8, target=ib.B200Target(0)).run(
        ad, bd, torch.zeros(N, dtype=torch.int32, device=cuda_device))
    out = ib.compile(ib.programs.w8a8_gemm, target=ib.B200Target(0)).run(ad, bd, sad, sbd)
    torch.cuda.synchronize()
    assert _status() == 0
    rows = torch.tensor([0, 127, 128, 2047, 4095])
    assert torch.equal(acc[rows.to(cuda_device)].cpu(), oracle.gemm_i8(a[rows], b))
    expected = ((acc.float() * sad[:, None]) * sbd[None, :]).to(torch.bfloat16)
    assert torch.equal(out, expected)
    # a checksum that does not depend on the tiling: column sums of the accumulator
    assert torch.equal(acc.sum(dim=0, dtype=torch.int64).cpu(),
                       (a.to(torch.int64).sum(dim=0)[None, :].double() @ b.double()).to(torch.int64).flatten())
