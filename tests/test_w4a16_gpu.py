"""W4A16 parity on the GPU, through the artifact surface (which calls the C ABI).

Tolerances: the benchmark's criterion  max|y - ref| <= 2e-2 * max|ref|  against
the f32-accumulate dequant oracle, and the reference's own Tolerance(atol=4e-2)
on its own case recipe (experiments/cpu/providers/mojo/contraction.py:190-198).
"""
import pytest
import torch

import intent_b200 as ib
import oracle
from conftest import load_golden, max_abs_rel

pytestmark = pytest.mark.gpu

BENCH_TOL = 2e-2


def _compile(dtype="f16", group=128, zero_point=8, kernel="auto"):
    return ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(0),
                      constexprs={"GROUP_SIZE": group, "ZERO_POINT": zero_point, "ACT_DTYPE": dtype,
                                  "KERNEL": kernel})


@pytest.mark.parametrize("tag", ["small", "ragged_m"])
def test_golden_reference_layout(cuda_device, tag):
    """The reference's own constants (group 64, two's-complement nibbles, f16) on golden vectors."""
    g = load_golden(f"w4a16_{tag}")
    artifact = _compile("f16", 64, "twos_complement")
    out = artifact.run(g["activation"].to(cuda_device), g["packed"].to(cuda_device), g["scales"].to(cuda_device))
    torch.cuda.synchronize()
    assert out.dtype == torch.float16 and out.shape == g["output"].shape
    assert (out.cpu().float() - g["output"].float()).abs().max() <= 4e-2      # reference tolerance
    assert max_abs_rel(out.cpu(), g["output"]) <= BENCH_TOL
    assert max_abs_rel(out.cpu(), g["output"]) <= 2e-3                         # what the kernel really achieves


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("M,K,N", [(1, 4096, 14336), (1, 14336, 4096), (4, 4096, 14336), (8, 14336, 4096),
                                   (16, 4096, 4096), (3, 256, 72), (8, 128, 8), (16, 512, 200), (9, 1024, 64), (2, 128, 8)])
def test_skinny_matches_oracle(cuda_device, dtype, M, K, N):
    x, p, s = ib.workloads.w4a16_inputs(M, K, N, dtype=dtype, group_size=128, seed=0)
    artifact = _compile("f16" if dtype == torch.float16 else "bf16", 128, 8, "gemv")
    out = artifact.run(x.to(cuda_device), p.to(cuda_device), s.to(cuda_device))
    torch.cuda.synchronize()
    ref = oracle.weight_only_int4_matmul(x, p, s, group_size=128, zero_point=8)
    assert out.dtype == dtype
    assert max_abs_rel(out.cpu(), ref) <= BENCH_TOL
    # rounding of the result to 16 bits dominates: a few ulp of the output type
    assert max_abs_rel(out.cpu(), ref) <= (2e-3 if dtype == torch.float16 else 1.6e-2)


@pytest.mark.parametrize("group", [32, 64, 128])
def test_group_sizes_and_auto_dispatch(cuda_device, group):
    x, p, s = ib.workloads.w4a16_inputs(5, 512, 96, dtype=torch.float16, group_size=group, seed=4)
    artifact = _compile("f16", group, 8, "auto")
    out = artifact.run(x.to(cuda_device), p.to(cuda_device), s.to(cuda_device))
    ref = oracle.weight_only_int4_matmul(x, p, s, group_size=group, zero_point=8)
    assert max_abs_rel(out.cpu(), ref) <= 2e-3


def test_work_splits_are_reproducible_and_agree(cuda_device):
    """Any split of the weight stream over CTAs sums in a fixed order: one split is
    bit-reproducible, different splits agree to rounding, and splits that make column
    tiles straddle CTAs exercise the scratch/ticket path."""
    from intent_b200.runtime import native

    lib = native.library()
    artifact = _compile("f16", 128, 8, "gemv")
    try:
        for M, K, N in [(4, 4096, 1024), (1, 14336, 512), (8, 1024, 2048)]:
            x, p, s = ib.workloads.w4a16_inputs(M, K, N, dtype=torch.float16, seed=7)
            xd, pd, sd = x.to(cuda_device), p.to(cuda_device), s.to(cuda_device)
            ref = oracle.weight_only_int4_matmul(x, p, s, group_size=128, zero_point=8)
            for ctas in (0, 148, 37, 7, 1, 100000):
                assert lib.intent_b200_w4a16_gemv_grid(ctas) == 0
                first = artifact.run(xd, pd, sd)
                second = artifact.run(xd, pd, sd)
                torch.cuda.synchronize()
                assert torch.equal(first, second), (M, K, N, ctas)
                assert max_abs_rel(first.cpu(), ref) <= 2e-3, (M, K, N, ctas)
        # launch overlap on: same bits as with it off (back-to-back launches on one stream)
        lib.intent_b200_w4a16_gemv_grid(0)
        plain = artifact.run(xd, pd, sd)
        assert lib.intent_b200_w4a16_gemv_overlap(1) == 0
        outs = [artifact.run(xd, pd, sd) for _ in range(4)]
        torch.cuda.synchronize()
        assert all(torch.equal(o, plain) for o in outs)
    finally:
        lib.intent_b200_w4a16_gemv_grid(0)
        lib.intent_b200_w4a16_gemv_overlap(0)


def test_workspace_stays_clean_and_status_word_is_zero(cuda_device):
    x, p, s = ib.workloads.w4a16_inputs(2, 14336, 256, dtype=torch.float16, seed=1)
    artifact = _compile("f16", 128, 8, "gemv")
    call = artifact.prepare(x.to(cuda_device), p.to(cuda_device), s.to(cuda_device))
    for _ in range(3):
        call.launch()
    torch.cuda.synchronize()
    (workspace,) = call._workspace
    assert workspace.numel() > 0
    header = workspace[:256 + 4 * (256 // 32)].cpu()               # status word + one ticket counter per 32 columns
    assert int(header[:4].view(torch.int32)[0]) == 0                # status word
    assert not header.any()                                         # ticket counters are back at zero


def test_timeout_status_is_reported_and_the_workspace_recovered(cuda_device):
    """What the host sees after a launch whose bounded wait expired, made on the host: the status word and
    a ticket counter of a prepared call's workspace are set by hand (no kernel is made to time out).
    ``check()`` must raise with the timeout status and leave the workspace zero-filled, and the next launch
    must give the right result again."""
    x, p, s = ib.workloads.w4a16_inputs(4, 4096, 256, dtype=torch.float16, seed=6)
    xd, pd, sd = x.to(cuda_device), p.to(cuda_device), s.to(cuda_device)
    artifact = _compile("f16", 128, 8, "gemv")
    call = artifact.prepare(xd, pd, sd)
    call.launch()
    call.check()                                                  # a clean launch: nothing to report
    expected = call.result().clone()
    (workspace,) = call._workspace
    words = workspace.view(torch.int32)
    words[0] = 4                                                  # INTENT_B200_ERR_TIMEOUT
    words[64 + 1] = 3                                             # an abandoned ticket counter (offset 256 bytes)
    with pytest.raises(ib.CompilationStageError) as info:
        call.check()
    assert info.value.stage == "provider_invocation" and info.value.status == 4
    assert not workspace.any()                                    # cleared for reuse
    call.check()
    call.result().zero_()
    call.launch()
    call.check()
    assert torch.equal(call.result(), expected)
    # the unprepared path reuses one workspace per stream: artifact.check() covers it
    y = artifact.run(xd, pd, sd)
    artifact.check()
    assert torch.equal(y, expected)
    cached = next(iter(artifact.runtime._stream_workspaces.values()))
    cached.view(torch.int32)[0] = 4
    with pytest.raises(ib.CompilationStageError):
        artifact.check()
    assert not cached.any()
    assert torch.equal(artifact.run(xd, pd, sd), expected)


def test_call_modes_prepare_launch_graph_and_torch_op(cuda_device):
    x, p, s = ib.workloads.w4a16_inputs(4, 1024, 256, dtype=torch.float16, seed=2)
    xd, pd, sd = x.to(cuda_device), p.to(cuda_device), s.to(cuda_device)
    artifact = _compile()
    expected = artifact.run(xd, pd, sd)
    # explicit outputs
    out = torch.zeros_like(expected)
    assert artifact(xd, pd, sd, out) is None
    assert torch.equal(out, expected)
    # prepared call: no launch at prepare/compile/result, replayable, graph-capturable
    call = artifact.prepare(xd, pd, sd)
    call.compile()
    held = call.result()
    held.zero_()
    call.launch()
    torch.cuda.synchronize()
    assert torch.equal(held, expected)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        call.launch()                      # warm up on the side stream before capture
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    held.zero_()
    with torch.cuda.graph(graph, stream=side):
        call.launch()
    held.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(held, expected)
    assert artifact.observation is not None and artifact.observation.status == 0
    # resource facts of the selected kernel instance (from a dry run of the same slots; nothing is launched)
    seen = call.observation
    # four rows: the entry runs the problem as a table of one in the ride-along kernel
    assert seen.kernel.startswith("w4a16_ride_kernel") and seen.threads == 1024 and seen.grid >= 1
    assert 0 < seen.registers <= 64 and seen.shared_dynamic > 0 and seen.cluster == 1
    # one row: the single-problem bandwidth kernel
    one = artifact.prepare(xd[:1].contiguous(), pd, sd)
    one.launch()
    torch.cuda.synchronize()
    assert one.observation.kernel.startswith("w4a16_stream_kernel") and one.observation.threads in (512, 1024)
    assert one.observation.spill_bytes == 0
    # (the two kernels add in different orders: equal up to rounding, not bit for bit)
    assert (one.result().float() - expected[:1].float()).abs().max() <= 2e-2 * expected.float().abs().max()
    # torch custom operator with a fake implementation
    op = artifact.as_torch_op("intent_b200_test::w4a16")
    assert torch.equal(op(xd, pd, sd), expected)
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        fake = op(torch.empty((4, 1024), dtype=torch.float16, device="cuda"),
                  torch.empty((128, 256), dtype=torch.int32, device="cuda"),
                  torch.empty((8, 256), dtype=torch.float16, device="cuda"))
        assert fake.shape == (4, 256) and fake.dtype == torch.float16


def test_errors_and_edges_on_device(cuda_device):
    artifact = _compile()
    x, p, s = ib.workloads.w4a16_inputs(2, 256, 64, dtype=torch.float16)
    xd, pd, sd = x.to(cuda_device), p.to(cuda_device), s.to(cuda_device)
    with pytest.raises(TypeError):
        artifact.run(xd.float(), pd, sd)
    with pytest.raises(ValueError):
        artifact.run(xd, pd, sd.cpu())
    # zero rows: nothing is launched, an empty result comes back
    empty = artifact.run(xd[:0], pd, sd)
    assert empty.shape == (0, 64)
    # an unsupported column count is reported by the C entry as a status, not a crash
    x2, p2, s2 = ib.workloads.w4a16_inputs(2, 256, 68, dtype=torch.float16)
    with pytest.raises(ib.CompilationStageError) as info:
        artifact.run(x2.to(cuda_device), p2.to(cuda_device), s2.to(cuda_device))
    assert info.value.stage == "provider_invocation" and info.value.status == 3
