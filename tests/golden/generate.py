"""Generate the golden vectors under tests/golden/ from the reference's own
torch-CPU implementations.

Run once in a checkout that has the reference tree next to it:

    python tests/golden/generate.py /path/to/reference

The reference module ``experiments/cpu/baselines/pytorch/cpu_runtime.py`` is
imported UNMODIFIED by path; every output stored below is what that module
returned for the stored inputs.  Input recipes follow the reference's case
definitions (experiments/cpu/providers/mojo/contraction.py:190-198,
routing.py:45-54, ragged.py:43-69,174-206, sorting.py:15-18,
experiments/cpu/providers/weft/matrix.py:78-83) at sizes small enough to commit.
The files are consumed by the CPU tests (oracle vs. golden) and by the GPU
tests (CUDA kernels vs. golden); nothing reads the reference tree at test time.
"""
from __future__ import annotations

import importlib.util
import math
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_reference(root: Path):
    path = root / "experiments/cpu/baselines/pytorch/cpu_runtime.py"
    spec = importlib.util.spec_from_file_location("intent_reference_cpu_runtime", path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def to_numpy(value: torch.Tensor) -> np.ndarray:
    if value.dtype == torch.bfloat16:   # store the bit pattern; the name carries the type
        return value.view(torch.int16).numpy()
    return value.numpy()


def save(name: str, **tensors) -> None:
    arrays = {}
    for key, value in tensors.items():
        suffix = "__bf16" if value.dtype == torch.bfloat16 else ""
        arrays[key + suffix] = to_numpy(value.contiguous())
    np.savez_compressed(HERE / f"{name}.npz", **arrays)
    print(f"{name}: " + ", ".join(f"{k}{tuple(v.shape)}" for k, v in arrays.items()))


def pack(logical: torch.Tensor) -> torch.Tensor:
    packed = torch.zeros((logical.shape[0] // 8, logical.shape[1]), dtype=torch.int32)
    for lane in range(8):
        packed |= (logical[lane::8] & 15) << (4 * lane)
    return packed


def main(root: Path) -> None:
    ref = load_reference(root)
    torch.manual_seed(0)

    # --- weight_only_int4_matmul (group 64 and signed nibbles are fixed in the reference) ---
    for tag, (M, K, N) in {"small": (8, 256, 64), "ragged_m": (5, 512, 96), "wide": (33, 1024, 256)}.items():
        activation = torch.randn((M, K), dtype=torch.float16) * 0.05
        logical = torch.randint(-8, 8, (K, N), dtype=torch.int32)
        packed = pack(logical)
        scales = 0.01 + 0.02 * torch.rand((K // 64, N), dtype=torch.float16)
        output = ref.weight_only_int4_matmul(activation, packed, scales)
        save(f"w4a16_{tag}", activation=activation, packed=packed, scales=scales, output=output)

    # --- i8 GEMM with bias: the reference's exact f64 recipe ---
    generator = torch.Generator().manual_seed(0)
    for tag, (M, K, N) in {"small": (16, 256, 64), "odd": (37, 384, 136)}.items():
        a = torch.randint(-128, 128, (M, K), dtype=torch.int8, generator=generator)
        b = torch.randint(-128, 128, (K, N), dtype=torch.int8, generator=generator)
        bias = torch.randint(-1024, 1024, (N,), dtype=torch.int32, generator=generator)
        reference = (a.to(torch.float64) @ b.to(torch.float64) + bias).to(torch.int32)
        save(f"gemm_i8_{tag}", a=a, b=b, bias=bias, output=reference)

    # --- w4a8 packed matmul (exact) ---
    activation = torch.randint(-128, 128, (24, 128), dtype=torch.int8)
    packed_u8 = torch.randint(0, 256, (40, 64), dtype=torch.uint8)
    save("w4a8_small", activation=activation, packed=packed_u8,
         output=ref.w4a8_packed_matmul(activation, packed_u8))

    # --- moe alignment ---
    for tag, (tokens, experts, block) in {"ref_pattern": (4096, 64, 128), "small": (50, 8, 16)}.items():
        if tag == "ref_pattern":
            ids = torch.arange(tokens * 2, dtype=torch.int32).remainder(experts).reshape(tokens, 2).contiguous()
        else:
            ids = torch.randint(0, experts, (tokens, 2), dtype=torch.int32)
            ids[:, 1] = (ids[:, 0] + 1 + torch.randint(0, experts - 1, (tokens,), dtype=torch.int32)) % experts
            ids[ids == 3] = 4     # leave one expert empty
        sorted_ids, expert_ids, total = ref.moe_align_block_size(ids, block, experts)
        blocks = int(total) // block
        counts = ref.moe_count_routes(ids, torch.zeros((experts,), dtype=torch.int32))
        save(f"moe_align_{tag}", topk_ids=ids, sorted_ids=sorted_ids, expert_ids=expert_ids[:blocks],
             total=total, counts=counts, block=torch.tensor([block]), experts=torch.tensor([experts]))

    # --- insertion top-k (k is 8 in the reference) and softmax ---
    logits = torch.randn((32, 67), dtype=torch.float32)
    logits[3, 10] = logits[3, 50] = logits[3].max() + 1.0       # exact ties: lower index must win
    logits[7, :] = 0.25
    values, indices = ref.insertion_top_k(logits)
    save("insertion_top_k", logits=logits, values=values, indices=indices)
    x = torch.randn((16, 64), dtype=torch.float32) * 3
    save("softmax_f32", x=x, output=ref.softmax(x))

    # --- SiLU gate ---
    packed_act = torch.randn((8, 64), dtype=torch.bfloat16)
    save("silu_and_mul_packed", packed=packed_act, output=ref.silu_and_mul_packed(packed_act))

    # --- ragged grouped GEMM, routed projection, MoE FFN ---
    rows, K, N, groups = 96, 64, 48, 4
    x = torch.randn((rows, K), dtype=torch.float16) / math.sqrt(K)
    offsets = torch.tensor([0, 8, 8, 40, 96], dtype=torch.int32)      # one empty group
    weight = torch.randn((groups, K, N), dtype=torch.float16)
    save("ragged_grouped_gemm", x=x, offsets=offsets, weight=weight,
         output=ref.ragged_grouped_gemm(x, offsets, weight))

    tokens, top_k, experts = 24, 2, 4
    xb = torch.randn((tokens, K), dtype=torch.bfloat16) / math.sqrt(K)
    ids = torch.randint(0, experts, (tokens, top_k))
    member_routes = torch.argsort(ids.flatten(), stable=True).to(torch.int32)
    counts = torch.bincount(ids.flatten(), minlength=experts)
    expert_offsets = torch.cat((torch.zeros(1, dtype=torch.int64), counts.cumsum(0))).to(torch.int32)
    wb = torch.randn((experts, N, K), dtype=torch.bfloat16)
    save("routed_expert_projection_bf16", x=xb, offsets=expert_offsets, member_routes=member_routes, weight=wb,
         output=ref.routed_expert_projection_bf16(xb, expert_offsets, member_routes, wb))

    D, F = 64, 96
    xf = torch.randn((tokens, D), dtype=torch.float16) / math.sqrt(D)
    route_token = torch.arange(tokens, dtype=torch.int32).repeat_interleave(top_k)
    route_weights = torch.rand((tokens * top_k,), dtype=torch.float32)
    w1 = torch.randn((experts, D, F), dtype=torch.float16) / math.sqrt(D)
    w2 = torch.randn((experts, F, D), dtype=torch.float16) / math.sqrt(F)
    y = ref.moe_expert_ffn(xf, expert_offsets, member_routes, route_token, route_weights, w1, w2,
                           torch.zeros((tokens, D), dtype=torch.float32))
    save("moe_expert_ffn", x=xf, route_offsets=expert_offsets, member_routes=member_routes,
         route_token=route_token, route_weights=route_weights, w1=w1, w2=w2, y=y)

    # --- interleaved int2 ("bitnet") and fp4 -> bf16 packed weights; recipes of
    # experiments/cpu/providers/mojo/contraction.py:209-224 at small sizes.  Appended last so the
    # random stream of the fixtures above is unchanged.
    generator = torch.Generator().manual_seed(7)
    for tag, (M, N, K, high) in {"small": (3, 40, 128, 2), "full_range": (24, 72, 192, 4)}.items():
        activation = torch.randint(-8, 8, (M, K), dtype=torch.int8, generator=generator)
        logical = torch.randint(0, high, (N, K), dtype=torch.int8, generator=generator).reshape(N, K // 16, 4, 4)
        packed = torch.zeros((N, K // 16, 4), dtype=torch.uint8)
        for lane in range(4):
            packed |= logical[:, :, lane, :].to(torch.uint8) << (lane * 2)
        packed = packed.flatten(1)
        save(f"bitnet_int2_{tag}", activation=activation, packed=packed,
             output=ref.bitnet_int2_matmul(activation, packed))
    for tag, (M, N, K) in {"small": (8, 40, 128), "all_codes": (16, 128, 256)}.items():
        activation = (torch.randn((M, K), generator=generator) * 0.125).bfloat16()
        packed = torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, generator=generator)
        if tag == "all_codes":      # every 16-bit word value's high and low byte patterns appear
            packed[:, 0::2] = torch.arange(N * K // 4, dtype=torch.int32).reshape(N, K // 4).remainder(256).to(torch.uint8)
        save(f"dequant_bf16_fp4_{tag}", activation=activation, packed=packed,
             output=ref.dequant_bf16_fp4_matmul(activation, packed))

    # quantized_gemm, recipe of experiments/cpu/providers/mojo/contraction.py:177-186 at a small size
    M, K, N = 48, 256, 136
    lhs = (torch.randn((M, K), generator=generator) / math.sqrt(K)).half()
    rhs = torch.randn((K, N), generator=generator).half()
    bias = torch.randn((N,), generator=generator) * 0.25
    residual = (torch.randn((M, N), generator=generator) * 0.25).half()
    scale = torch.linspace(1.0 / 48.0, 1.0 / 24.0, N, dtype=torch.float32)
    save("quantized_gemm_small", a=lhs, b=rhs, bias=bias, residual=residual, scale=scale,
         output=ref.quantized_gemm(lhs, rhs, bias, residual, scale))


def reference_case_inputs():
    """The reference's own W4A16 case at its own size (M512 K2048 N4096, group 64, signed nibbles, f16;
    recipe of experiments/cpu/providers/mojo/contraction.py:190-198), drawn from a private generator so
    the tests can rebuild the same tensors from the seed instead of storing 8 MiB of them."""
    generator = torch.Generator().manual_seed(190)
    M, K, N = 512, 2048, 4096
    activation = (torch.randn((M, K), generator=generator) * 0.05).half()
    logical = torch.randint(-8, 8, (K, N), dtype=torch.int32, generator=generator)
    scales = (0.01 + 0.02 * torch.rand((K // 64, N), generator=generator)).half()
    return activation, pack(logical), scales


def digest(tensor: torch.Tensor) -> torch.Tensor:
    """Order-sensitive 64-bit checksum of a tensor's bytes (so a test can tell that it rebuilt the stored
    inputs exactly)."""
    raw = torch.from_numpy(tensor.contiguous().view(torch.uint8).numpy().reshape(-1).copy()).to(torch.int64)
    weights = (torch.arange(raw.numel(), dtype=torch.int64) % 65521) + 1
    return torch.tensor([int((raw * weights).sum()), int(raw.sum())], dtype=torch.int64)


def reference_case(root: Path) -> None:
    """Stored: 16 output rows of the reference module spread over the row tiles, and checksums of the
    seeded inputs.  Kept apart from main() so the random stream of the other fixtures is untouched."""
    ref = load_reference(root)
    activation, packed, scales = reference_case_inputs()
    output = ref.weight_only_int4_matmul(activation, packed, scales)
    rows = torch.tensor([0, 1, 63, 127, 128, 200, 255, 256, 300, 383, 384, 420, 447, 448, 500, 511])
    save("w4a16_reference_case_rows", rows=rows.to(torch.int32), output_rows=output[rows],
         activation_digest=digest(activation), packed_digest=digest(packed), scales_digest=digest(scales))


if __name__ == "__main__":
    if len(sys.argv) == 3 and sys.argv[2] == "reference_case":
        reference_case(Path(sys.argv[1]))
    elif len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/generate.py /path/to/reference [reference_case]")
    else:
        main(Path(sys.argv[1]))
        reference_case(Path(sys.argv[1]))
