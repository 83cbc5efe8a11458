"""Q4_K x Q8_K quantized projection against the oracle's restatement of the published record
arithmetic (doc/dsl/quantized-operations.en.md sections 2-4).  The integer sums are exact and the
float roundings are prescribed one by one, so the comparison is bit for bit.  The reference holds no
golden vectors for this program (its own comparison runs on a remote RISC-V host with
Tolerance(1e-4, 2e-3): experiments/cpu/providers/weft/contraction.py:113-117)."""
import numpy as np
import pytest
import torch

import intent_b200 as ib
import oracle

pytestmark = pytest.mark.gpu


def _case(rows, records, seed, scale=1.0):
    rng = np.random.default_rng(seed)
    weights = rng.integers(0, 256, (rows, records, 144), dtype=np.uint8)
    d = rng.uniform(0.001, 0.05, (rows, records)).astype(np.float16)
    dmin = rng.uniform(0.001, 0.05, (rows, records)).astype(np.float16)
    weights[:, :, 0:2] = d.view(np.uint8).reshape(rows, records, 2)
    weights[:, :, 2:4] = dmin.view(np.uint8).reshape(rows, records, 2)
    activation = (rng.standard_normal((records, 256)) * scale).astype(np.float32)
    return weights, activation


@pytest.mark.parametrize("rows,records,seed", [(8, 1, 0), (64, 4, 1), (300, 16, 2), (4096, 16, 3)])
def test_quantized_projection_bit_exact(cuda_device, rows, records, seed):
    weights, activation = _case(rows, records, seed)
    if seed == 1:
        activation[2] = 0.0                    # an all-zero block: ds = +0, q = 0
        activation[3, 5] = -activation[3].max()  # a tie between the extremes: the minimum wins
    artifact = ib.compile(ib.programs.quantized_projection, target=ib.B200Target(0))
    out = artifact.run(torch.from_numpy(weights).to(cuda_device), torch.from_numpy(activation).to(cuda_device))
    torch.cuda.synchronize()
    check = slice(0, rows) if rows <= 300 else slice(0, rows, 37)     # the oracle is a Python loop
    reference = oracle.quantized_projection(weights[check], activation)
    assert out.dtype == torch.float32 and out.shape == (rows,)
    assert np.array_equal(out.cpu().numpy()[check].view(np.uint32), reference.view(np.uint32))


def test_quantized_projection_interface(cuda_device):
    artifact = ib.compile(ib.programs.quantized_projection, target=ib.B200Target(0))
    weights = torch.zeros((4, 2, 144), dtype=torch.uint8, device=cuda_device)
    with pytest.raises(ValueError):
        artifact.run(weights, torch.zeros((3, 256), device=cuda_device))          # record counts differ
    with pytest.raises(ValueError):
        artifact.run(weights[:, :, :100].contiguous(), torch.zeros((2, 256), device=cuda_device))  # 144-byte records
    out = artifact.run(weights, torch.randn((2, 256), device=cuda_device))
    assert torch.all(out == 0)                                                     # d = dmin = 0
