"""W4A16 tensor-core (tcgen05) GEMM parity through the artifact surface.

Tolerance: the benchmark criterion max|y - ref| <= 2e-2 * max|ref| against the
f32-accumulate dequant oracle; the kernel rounds the dequantised weight to the
activation type first (the reference kernel body's order), which the second
oracle form reproduces to accumulation-order noise.
"""
import pytest
import torch

import intent_b200 as ib
import oracle
from intent_b200.runtime import native
from conftest import load_golden, max_abs_rel

pytestmark = pytest.mark.gpu


def _compile(dtype, group, zero_point, kernel="gemm"):
    return ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(0),
                      constexprs={"GROUP_SIZE": group, "ZERO_POINT": zero_point, "ACT_DTYPE": dtype,
                                  "KERNEL": kernel})


def _device_status():
    lib = native.library()
    return lib.intent_b200_w4a16_gemm_device_status()


@pytest.mark.parametrize("dtype,M,K,N,group", [
    (torch.bfloat16, 128, 256, 256, 128),
    (torch.float16, 128, 256, 256, 128),
    (torch.bfloat16, 200, 512, 264, 128),      # ragged M and N tiles
    (torch.float16, 77, 1024, 512, 64),
    (torch.bfloat16, 300, 384, 256, 32),       # two scale rows per k block, K not a multiple of 128
    (torch.bfloat16, 1024, 4096, 1024, 128),
    (torch.float16, 16, 4096, 4096, 128),      # the CPU-runnable benchmark configuration forced onto tensor cores
])
def test_gemm_matches_oracle(cuda_device, dtype, M, K, N, group):
    x, p, s = ib.workloads.w4a16_inputs(M, K, N, dtype=dtype, group_size=group, seed=5)
    artifact = _compile("f16" if dtype == torch.float16 else "bf16", group, 8)
    out = artifact.run(x.to(cuda_device), p.to(cuda_device), s.to(cuda_device))
    torch.cuda.synchronize()
    assert _device_status() == 0
    ref = oracle.weight_only_int4_matmul(x, p, s, group_size=group, zero_point=8)
    rounded = oracle.weight_only_int4_matmul_rounded(x, p, s, group_size=group, zero_point=8)
    assert out.dtype == dtype and out.shape == (M, N)
    assert max_abs_rel(out.cpu(), ref) <= 2e-2
    assert max_abs_rel(out.cpu(), rounded) <= (2e-3 if dtype == torch.float16 else 1.6e-2)


def test_gemm_golden_reference_layout(cuda_device):
    """Reference constants (group 64, two's-complement nibbles, f16), M = 33 golden vector."""
    g = load_golden("w4a16_wide")
    for kernel in ("gemm", "auto"):
        artifact = _compile("f16", 64, "twos_complement", kernel)
        out = artifact.run(g["activation"].to(cuda_device), g["packed"].to(cuda_device), g["scales"].to(cuda_device))
        torch.cuda.synchronize()
        assert (out.cpu().float() - g["output"].float()).abs().max() <= 4e-2      # the reference's own tolerance
        assert max_abs_rel(out.cpu(), g["output"]) <= 2e-2
    assert _device_status() == 0


def test_gemm_full_size_prefill_rows(cuda_device):
    """Benchmark configuration 2 (8192^3, bf16): rows sampled across M tiles against the oracle,
    plus linearity in X (a size-independent property): f(2x) == 2 f(x) exactly."""
    M = K = N = 8192
    x, p, s = ib.workloads.w4a16_inputs(M, K, N, dtype=torch.bfloat16, group_size=128, seed=0)
    artifact = _compile("bf16", 128, 8)
    xd, pd, sd = x.to(cuda_device), p.to(cuda_device), s.to(cuda_device)
    out = artifact.run(xd, pd, sd)
    doubled = artifact.run(xd * 2, pd, sd)
    torch.cuda.synchronize()
    assert _device_status() == 0
    assert torch.equal(doubled, out * 2)
    seen = artifact.observation            # the plan this shape selects: CTA pairs, one pair per two SMs
    assert seen.kernel.startswith("w4a16_gemm_pair_kernel") and seen.cluster == 2 and seen.grid % 2 == 0
    assert seen.registers > 0 and seen.shared_dynamic > 100 * 1024
    # 80 rows: five in each of the 16 pair tiles of 512 rows - first and last row of the tile, and rows of
    # both CTAs of the pair (each owns 256 rows) and of both of their 128-row blocks
    rows = torch.cat([torch.tensor([0, 130, 255, 300, 511]) + 512 * tile for tile in range(16)])
    ref = oracle.weight_only_int4_matmul(x[rows], p, s, group_size=128, zero_point=8)
    assert max_abs_rel(out[rows.to(cuda_device)].cpu(), ref) <= 2e-2
    # a column checksum over ALL rows: sum_m y[m, :] = (sum_m x[m, :]) @ W', W' being the dequantised weight
    # rounded to bf16 as the kernel rounds it.  What remains is the rounding of the 8192 outputs of a column
    # (each about 4 in magnitude, 2^-9 relative: 0.4 rms in the sum); a 512-row tile that was skipped or
    # doubled would move its columns' sums by about 100.
    column_sum = out.float().sum(dim=0).cpu()
    signed = (oracle.unpack_int4(p) - 8).to(torch.bfloat16)
    weight = (signed * s.repeat_interleave(128, dim=0)).float()
    expected_sum = x.float().sum(dim=0) @ weight
    assert (column_sum - expected_sum).abs().max() <= 5.0
    # every tile was written: no element is left at the fill value
    assert torch.isfinite(out).all()


def test_reference_case_on_cta_pairs(cuda_device):
    """The reference's own W4A16 case at its own size (M512 K2048 N4096, group 64, signed nibbles, f16;
    experiments/cpu/providers/mojo/contraction.py:190-198): this is the CTA-pair kernel in two's-complement
    mode.  Checked against stored rows of the reference module's output at the reference's atol = 4e-2,
    against the oracle on every row, and at the benchmark's 2e-2 * max|ref|."""
    import importlib.util
    from pathlib import Path

    spec = importlib.util.spec_from_file_location("golden_generate", Path(__file__).parent / "golden" / "generate.py")
    generate = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(generate)
    g = load_golden("w4a16_reference_case_rows")
    activation, packed, scales = generate.reference_case_inputs()
    assert torch.equal(generate.digest(packed), g["packed_digest"])
    for kernel in ("auto", "gemm"):
        artifact = _compile("f16", 64, "twos_complement", kernel)
        out = artifact.run(activation.to(cuda_device), packed.to(cuda_device), scales.to(cuda_device))
        torch.cuda.synchronize()
        assert _device_status() == 0
        out = out.cpu()
        rows = g["rows"].long()
        assert (out[rows].float() - g["output_rows"].float()).abs().max() <= 4e-2
        ref = oracle.weight_only_int4_matmul(activation, packed, scales)          # reference defaults
        assert (out.float() - ref.float()).abs().max() <= 4e-2
        assert max_abs_rel(out, ref) <= 2e-2
        assert max_abs_rel(out, ref) <= 2e-3          # what the kernel really achieves on f16


@pytest.mark.parametrize("M,K,N", [(512, 512, 256), (1100, 1024, 776), (2048, 2048, 2048)])
def test_cta_pair_kernel_equals_single_cta_kernel(cuda_device, M, K, N):
    """M >= 512 runs on CTA pairs (cta_group::2); the k loop and the rounding are the same as in the
    single-CTA kernel, so the two must agree bit for bit, and with the oracle within tolerance."""
    lib = native.library()
    x, p, s = ib.workloads.w4a16_inputs(M, K, N, dtype=torch.bfloat16, group_size=128, seed=9)
    artifact = _compile("bf16", 128, 8)
    xd, pd, sd = x.to(cuda_device), p.to(cuda_device), s.to(cuda_device)
    try:
        lib.intent_b200_w4a16_gemm_pairs(1)
        paired = artifact.run(xd, pd, sd)
        lib.intent_b200_w4a16_gemm_pairs(0)
        single = artifact.run(xd, pd, sd)
        torch.cuda.synchronize()
    finally:
        lib.intent_b200_w4a16_gemm_pairs(1)
    assert _device_status() == 0
    assert torch.equal(paired, single)
    ref = oracle.weight_only_int4_matmul(x, p, s, group_size=128, zero_point=8)
    assert max_abs_rel(paired.cpu(), ref) <= 2e-2


def test_host_pipeline_of_row_pieces_gives_the_whole_product(cuda_device):
    """ColumnShardedRows on one GPU: rows uploaded, multiplied and downloaded in (tapered) pieces give the bits
    of one launch over all rows (a row's sums do not depend on which rows share its tile)."""
    from intent_b200.distributed import ColumnShardedRows
    M, K, N = 2048, 1024, 512
    x, p, s = ib.workloads.w4a16_inputs(M, K, N, dtype=torch.bfloat16, group_size=128, seed=4)
    artifact = ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(0),
                          constexprs={"GROUP_SIZE": 128, "ZERO_POINT": 8, "ACT_DTYPE": "bf16"})
    pd, sd = p.to(cuda_device), s.to(cuda_device)
    expected = artifact.run(x.to(cuda_device), pd, sd).cpu()
    px = x.pin_memory()
    py = torch.empty((M, N), dtype=torch.bfloat16).pin_memory()
    for taper in (True, False):
        pipeline = ColumnShardedRows(artifact, (pd, sd), rows=M, width=K, n_local=N, in_dtype=torch.bfloat16,
                                     out_dtype=torch.bfloat16, device=cuda_device, chunks=8, taper=taper)
        assert sum(pipeline.sizes) == M and (len(pipeline.sizes) == 10) == taper
        for _ in range(2):                   # buffers are reused from run to run
            py.zero_()
            pipeline.run(px, py)
            torch.cuda.synchronize()
            assert torch.equal(py, expected)
