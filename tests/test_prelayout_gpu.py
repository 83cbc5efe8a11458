"""Tiled weight copies (intent_b200.prelayout): the tiled layout itself, bit equality of the tensor-core
kernels on either layout (same arithmetic, different fetch), the PRELAYOUT cache, and persistence."""
import pytest
import torch

import intent_b200 as ib
import oracle
from intent_b200 import prelayout
from intent_b200.moe import MoEW4A16FFN
from conftest import max_abs_rel

pytestmark = pytest.mark.gpu


def _tiled_reference(packed: torch.Tensor) -> torch.Tensor:
    """tiled[n / 128][k / 64][(k % 64) / 32][n % 128][4 words] built with plain indexing on the CPU."""
    rows, N = packed.shape
    k_blocks, column_blocks = (rows + 7) // 8, (N + 127) // 128
    padded = torch.zeros((k_blocks * 8, column_blocks * 128), dtype=torch.int32)
    padded[:rows, :N] = packed
    # [kb, part, word, cb, column] -> [cb, kb, part, column, word]
    return padded.reshape(k_blocks, 2, 4, column_blocks, 128).permute(3, 0, 1, 4, 2).reshape(-1).contiguous()


@pytest.mark.parametrize("K,N", [(128, 8), (256, 72), (512, 200), (1024, 256), (4096, 1000)])
def test_tiled_layout_is_the_documented_permutation(cuda_device, K, N):
    packed = torch.randint(-2 ** 31, 2 ** 31, (K // 8, N), dtype=torch.int64).to(torch.int32)
    tiled = prelayout.tile(packed.to(cuda_device))
    assert (tiled.K, tiled.N) == (K, N) and tiled.tensor.numel() == prelayout.words(K, N)
    assert torch.equal(tiled.tensor.cpu(), _tiled_reference(packed))
    grouped = prelayout.tile(torch.stack([packed, packed.flip(0)]).to(cuda_device))
    assert grouped.experts == 2
    assert torch.equal(grouped.tensor[1].cpu(), _tiled_reference(packed.flip(0)))


@pytest.mark.parametrize("dtype,M,K,N,group", [
    (torch.bfloat16, 128, 256, 256, 128), (torch.float16, 77, 1024, 520, 64), (torch.bfloat16, 300, 384, 264, 32),
    (torch.bfloat16, 1100, 1024, 776, 128),        # CTA pairs with ragged tiles
    (torch.bfloat16, 2048, 2048, 2048, 128)])
def test_gemm_on_tiled_weight_equals_reference_layout(cuda_device, dtype, M, K, N, group):
    x, p, s = ib.workloads.w4a16_inputs(M, K, N, dtype=dtype, group_size=group, seed=31)
    xd, pd, sd = x.to(cuda_device), p.to(cuda_device), s.to(cuda_device)
    name = "f16" if dtype == torch.float16 else "bf16"
    constants = {"GROUP_SIZE": group, "ZERO_POINT": 8, "ACT_DTYPE": name, "KERNEL": "gemm"}
    plain = ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(0), constexprs=constants)
    tiled = ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(0),
                       constexprs=dict(constants, WEIGHT_LAYOUT="tiled"))
    expected = plain.run(xd, pd, sd)
    got = tiled.run(xd, prelayout.tile(pd).tensor, sd)
    torch.cuda.synchronize()
    tiled.check()
    assert torch.equal(got, expected)                  # same arithmetic in the same order: only the fetch differs
    ref = oracle.weight_only_int4_matmul(x, p, s, group_size=group, zero_point=8)
    assert max_abs_rel(got.cpu(), ref) <= 2e-2
    with pytest.raises(ValueError):
        tiled.run(xd, prelayout.tile(pd).tensor[:-4], sd)             # not the tiled copy of this shape


def test_prelayout_cache_and_persistence(cuda_device, tmp_path):
    """PRELAYOUT=True keeps the reference's call surface: one tiled copy per weight tensor, a new one when the
    tensor is modified through torch, small batches straight to the bandwidth kernel; save / load carries the
    copies (matched to a weight by its content key, so nothing is re-tiled after a load)."""
    x, p, s = ib.workloads.w4a16_inputs(512, 1024, 768, dtype=torch.bfloat16, group_size=128, seed=5)
    xd, pd, sd = x.to(cuda_device), p.to(cuda_device), s.to(cuda_device)
    constants = {"GROUP_SIZE": 128, "ZERO_POINT": 8, "ACT_DTYPE": "bf16"}
    plain = ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(0), constexprs=constants)
    cached = ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(0),
                        constexprs=dict(constants, PRELAYOUT=True))
    expected = plain.run(xd, pd, sd)
    assert torch.equal(cached.run(xd, pd, sd), expected)
    assert torch.equal(cached.run(xd, pd, sd), expected)
    call = cached.prepare(xd, pd, sd)
    call.launch()
    assert torch.equal(call.result(), expected)
    assert cached.runtime.cache.repacks == 1
    assert cached.observation.entry.endswith("gemm_tiled_bf16")
    small = cached.run(xd[:4], pd, sd)                                 # at most 16 rows: the bandwidth kernel
    assert torch.equal(small, plain.run(xd[:4], pd, sd)) and cached.runtime.cache.repacks == 1
    saved = cached.save(tmp_path / "artifact")
    assert (saved / "prelayout").is_dir()
    restored = ib.load(saved, target=ib.B200Target(0))
    assert torch.equal(restored.run(xd, pd.clone(), sd), expected)      # another tensor with the same contents
    assert restored.runtime.cache.repacks == 0                          # served by the stored copy
    pd.add_(1)                                                          # modified through torch: a new copy
    again = cached.run(xd, pd, sd)
    assert cached.runtime.cache.repacks == 2
    assert torch.equal(again, plain.run(xd, pd, sd))
    with pytest.raises(TypeError):
        cached.run(xd.float(), pd, sd)                                  # errors still name the caller's arguments
    weight = prelayout.tile(pd)
    weight.save(tmp_path / "weight")
    back = prelayout.TiledInt4Weight.load(tmp_path / "weight", cuda_device)
    assert torch.equal(back.tensor, weight.tensor) and (back.K, back.N) == (1024, 768)


def test_moe_ffn_on_tiled_expert_weights(cuda_device):
    tokens, hidden, inter, experts = 1024, 1024, 384, 16
    data = ib.workloads.moe_inputs(tokens, hidden, experts, inter, dtype=torch.bfloat16, seed=11)
    dev = {k: v.to(cuda_device) for k, v in data.items()}
    plain = MoEW4A16FFN(tokens=tokens, hidden=hidden, intermediate=inter, experts=experts, target=ib.B200Target(0))
    tiled = MoEW4A16FFN(tokens=tokens, hidden=hidden, intermediate=inter, experts=experts, target=ib.B200Target(0),
                        prelayout=True)
    ids, weights = plain.route(dev["logits"])
    args = (dev["x"], ids, weights, dev["up_gate_packed"], dev["up_gate_scales"], dev["down_packed"], dev["down_scales"])
    expected = plain(*args)
    assert torch.equal(tiled(*args), expected)
    y = torch.empty_like(expected)
    call = tiled.prepare(*args, y)
    call.launch()
    call.launch()
    assert torch.equal(y, expected) and tiled.prelayout.repacks == 2   # up|gate and down, once each
