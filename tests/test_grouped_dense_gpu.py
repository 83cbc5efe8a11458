"""Ragged grouped contractions with dense 16-bit weights (tcgen05 kernel) against the
oracle, the reference's golden outputs and, at the reference's own problem size, a
per-group library matmul.  Tolerances are the reference's
(experiments/cpu/providers/mojo/ragged.py:43-111,174-257: grouped GEMM atol 5e-2, routed
projection atol 1e-1 / rtol 5e-2, MoE FFN atol 2e-3) and the benchmark's
max|y - ref| <= 2e-2 * max|ref|."""
import pytest
import torch

import intent_b200 as ib
import oracle
from intent_b200.runtime import native
from conftest import load_golden, max_abs_rel

pytestmark = pytest.mark.gpu


def _status():
    return native.library().intent_b200_grouped_gemm16_device_status()


def _ragged_case(rows, K, N, sizes, dtype, seed, lead=0):
    gen = torch.Generator().manual_seed(seed)
    x = (torch.randn((rows, K), generator=gen) * 0.5).to(dtype)
    w = (torch.randn((len(sizes), K, N), generator=gen) / K ** 0.5).to(dtype)
    offsets = torch.tensor([lead] + [lead + sum(sizes[:i + 1]) for i in range(len(sizes))], dtype=torch.int32)
    assert int(offsets[-1]) <= rows
    return x, offsets, w


def test_ragged_grouped_gemm_golden(cuda_device):
    g = load_golden("ragged_grouped_gemm")
    artifact = ib.compile(ib.programs.ragged_grouped_gemm, target=ib.B200Target(0))
    y = artifact.run(g["x"].to(cuda_device), g["offsets"].to(cuda_device), g["weight"].to(cuda_device))
    torch.cuda.synchronize()
    assert _status() == 0
    assert torch.allclose(y.cpu().float(), g["output"].float(), atol=5e-2, rtol=0)
    assert max_abs_rel(y.cpu(), g["output"]) <= 2e-2


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,K,N,sizes,lead", [
    (1000, 520, 264, (300, 0, 1, 129, 500), 30),     # K and N tails, an empty group, a single row, untouched rows
    (640, 64, 8, (128, 128, 256, 128), 0),           # whole blocks, one narrow column tile
    (77, 4096, 512, (77,), 0),                       # one group shorter than a tile, long K
    (2048, 1024, 1280, tuple([32] * 64), 0),         # many small groups
])
def test_ragged_grouped_gemm_matches_oracle(cuda_device, dtype, rows, K, N, sizes, lead):
    x, offsets, w = _ragged_case(rows, K, N, sizes, dtype, seed=rows + K + N, lead=lead)
    program = ib.programs.ragged_grouped_gemm if dtype is torch.float16 else ib.programs.ragged_grouped_gemm_bf16
    artifact = ib.compile(program, target=ib.B200Target(0))
    y = torch.full((rows, N), 7.0, dtype=dtype, device=cuda_device)
    artifact.launch(x.to(cuda_device), offsets.to(cuda_device), w.to(cuda_device), y)
    torch.cuda.synchronize()
    assert _status() == 0
    reference = oracle.ragged_grouped_gemm(x, offsets, w)
    begin, end = int(offsets[0]), int(offsets[-1])
    assert max_abs_rel(y.cpu()[begin:end], reference[begin:end]) <= 2e-2
    ulp = 2.0 ** -7 if dtype is torch.bfloat16 else 2.0 ** -10
    assert torch.allclose(y.cpu()[begin:end].float(), reference[begin:end].float(), rtol=2 * ulp, atol=1e-3)
    # rows outside every group are not written
    assert torch.all(y.cpu()[:begin] == 7.0) and torch.all(y.cpu()[end:] == 7.0)


def test_ragged_offsets_are_clamped(cuda_device):
    """Offsets beyond the row count must not cause writes past the output."""
    x, offsets, w = _ragged_case(256, 64, 64, (100, 156), torch.float16, seed=3)
    offsets = torch.tensor([0, 100, 900], dtype=torch.int32)
    artifact = ib.compile(ib.programs.ragged_grouped_gemm, target=ib.B200Target(0))
    guard = torch.full((512, 64), 7.0, dtype=torch.float16, device=cuda_device)
    artifact.launch(x.to(cuda_device), offsets.to(cuda_device), w.to(cuda_device), guard[:256])
    torch.cuda.synchronize()
    assert _status() == 0
    assert torch.all(guard[256:] == 7.0)
    reference = oracle.ragged_grouped_gemm(x, torch.tensor([0, 100, 256], dtype=torch.int32), w)
    assert max_abs_rel(guard[:256].cpu(), reference) <= 2e-2


def _routing(tokens, experts, top_k, seed):
    gen = torch.Generator().manual_seed(seed)
    ids = torch.stack([torch.randperm(experts, generator=gen)[:top_k] for _ in range(tokens)]).to(torch.int32)
    flat = ids.reshape(-1)
    member_routes = torch.argsort(flat, stable=True).to(torch.int32)
    counts = torch.bincount(flat.long(), minlength=experts)
    offsets = torch.cat((torch.zeros(1, dtype=torch.long), counts.cumsum(0))).to(torch.int32)
    return ids, member_routes, offsets


def test_routed_expert_projection_golden(cuda_device):
    g = load_golden("routed_expert_projection_bf16")
    artifact = ib.compile(ib.programs.routed_expert_projection_bf16, target=ib.B200Target(0),
                          constexprs={"TOP_K": 2})
    out = artifact.run(*(g[k].to(cuda_device) for k in ("x", "offsets", "member_routes", "weight")))
    torch.cuda.synchronize()
    assert _status() == 0
    assert out.shape == g["output"].shape
    assert torch.allclose(out.cpu().float(), g["output"].float(), atol=1e-1, rtol=5e-2)
    assert max_abs_rel(out.cpu(), g["output"]) <= 2e-2


@pytest.mark.parametrize("tokens,experts,top_k,K,N", [(300, 6, 2, 136, 72), (1024, 8, 2, 512, 768),
                                                      (130, 3, 3, 64, 256)])
def test_routed_expert_projection_matches_oracle(cuda_device, tokens, experts, top_k, K, N):
    _, member_routes, offsets = _routing(tokens, experts, top_k, seed=tokens + K)
    gen = torch.Generator().manual_seed(K + N)
    x = (torch.randn((tokens, K), generator=gen) * 0.5).bfloat16()
    w = (torch.randn((experts, N, K), generator=gen) / K ** 0.5).bfloat16()
    artifact = ib.compile(ib.programs.routed_expert_projection_bf16, target=ib.B200Target(0),
                          constexprs={"TOP_K": top_k})
    out = artifact.run(x.to(cuda_device), offsets.to(cuda_device), member_routes.to(cuda_device), w.to(cuda_device))
    torch.cuda.synchronize()
    assert _status() == 0
    reference = oracle.routed_expert_projection(x, offsets, member_routes, w)
    assert out.shape == (tokens, top_k, N)
    assert max_abs_rel(out.cpu(), reference) <= 2e-2
    assert torch.allclose(out.cpu().float(), reference.float(), rtol=2.0 ** -6, atol=1e-3)


def test_moe_expert_ffn_golden(cuda_device):
    g = load_golden("moe_expert_ffn")
    artifact = ib.compile(ib.programs.moe_expert_ffn, target=ib.B200Target(0))
    y = torch.zeros(g["y"].shape, dtype=torch.float32, device=cuda_device)
    artifact.run(*(g[k].to(cuda_device) for k in ("x", "route_offsets", "member_routes", "route_token",
                                                   "route_weights", "w1", "w2")), y)
    torch.cuda.synchronize()
    assert _status() == 0
    assert torch.allclose(y.cpu(), g["y"], atol=2e-3, rtol=0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("tokens,experts,D,F", [(200, 5, 128, 264), (1024, 8, 512, 1024)])
def test_moe_expert_ffn_matches_oracle(cuda_device, dtype, tokens, experts, D, F):
    top_k = 2
    _, member_routes, offsets = _routing(tokens, experts, top_k, seed=tokens + D)
    gen = torch.Generator().manual_seed(D + F)
    x = (torch.randn((tokens, D), generator=gen) / D ** 0.5).to(dtype)
    w1 = (torch.randn((experts, D, F), generator=gen) / D ** 0.5).to(dtype)
    w2 = (torch.randn((experts, F, D), generator=gen) / F ** 0.5).to(dtype)
    routes = tokens * top_k
    route_token = (torch.arange(routes) // top_k).to(torch.int32)
    route_weights = torch.rand((routes,), generator=gen)
    y0 = torch.randn((tokens, D), generator=gen) * 0.01       # InOut: accumulated into, not overwritten
    artifact = ib.compile(ib.programs.moe_expert_ffn, target=ib.B200Target(0),
                          constexprs={"DTYPE": "f16" if dtype is torch.float16 else "bf16"})
    y = y0.clone().to(cuda_device)
    result = artifact.run(x.to(cuda_device), offsets.to(cuda_device), member_routes.to(cuda_device),
                          route_token.to(cuda_device), route_weights.to(cuda_device), w1.to(cuda_device),
                          w2.to(cuda_device), y)
    torch.cuda.synchronize()
    assert result is None and _status() == 0
    reference = oracle.moe_expert_ffn(x, offsets, member_routes, route_token, route_weights, w1, w2, y0.clone(),
                                      round_hidden=True)
    assert max_abs_rel(y.cpu(), reference) <= (2e-3 if dtype is torch.float16 else 2e-2)
    loose = oracle.moe_expert_ffn(x, offsets, member_routes, route_token, route_weights, w1, w2, y0.clone())
    assert max_abs_rel(y.cpu(), loose) <= 2e-2


def test_ragged_grouped_gemm_reference_size(cuda_device):
    """The reference's own case (8192 rows, 8 groups, K = N = 4096) against per-group library products."""
    sizes = (1024, 512, 2048, 256, 1536, 1024, 1000, 792)
    x, offsets, w = _ragged_case(8192, 4096, 4096, sizes, torch.bfloat16, seed=11)
    xg, wg = x.to(cuda_device), w.to(cuda_device)
    artifact = ib.compile(ib.programs.ragged_grouped_gemm_bf16, target=ib.B200Target(0))
    y = artifact.run(xg, offsets.to(cuda_device), wg)
    torch.cuda.synchronize()
    assert _status() == 0
    for g in range(len(sizes)):
        b, e = int(offsets[g]), int(offsets[g + 1])
        reference = (xg[b:e].float() @ wg[g].float())
        assert max_abs_rel(y[b:e].cpu(), reference.cpu()) <= 2e-2


def test_dense_grouped_rejects_unsupported(cuda_device):
    artifact = ib.compile(ib.programs.ragged_grouped_gemm, target=ib.B200Target(0))
    x, offsets, w = _ragged_case(64, 36, 64, (64,), torch.float16, seed=1)
    with pytest.raises(ValueError):
        artifact.run(x.to(cuda_device), offsets.to(cuda_device), w.to(cuda_device))   # K % 8
    x, offsets, w = _ragged_case(64, 64, 64, (32, 32), torch.float16, seed=1)
    with pytest.raises(ValueError):
        artifact.run(x.to(cuda_device), offsets[:2].contiguous().to(cuda_device), w.to(cuda_device))  # G + 1 offsets
