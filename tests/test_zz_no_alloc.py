"""The W4A16 entry that takes no workspace.

Some users of the library cannot allocate device memory for it: a serving
process with a frozen memory pool, a plugin interface that only passes an
operator's inputs and outputs, or code running inside a stream capture where
cudaMalloc is forbidden.  For them `intent_b200_w4a16_gemv_f16_builtin_scratch`
keeps the kernel's scratch in a fixed 8 MiB device array inside the library.
This test calls it through the C ABI, twice in a row (the array keeps the
previous call's contents), and checks the result against the workspace entry.
It is collected last on purpose, and it also passes when run on its own.
"""
import ctypes

import pytest
import torch

import intent_b200 as ib
from intent_b200.runtime import native
from conftest import max_abs_rel

pytestmark = pytest.mark.gpu

VIEW2 = [ctypes.c_void_p] + [ctypes.c_int64] * 4


def _slots(t):
    return [ctypes.c_void_p(t.data_ptr()), *[ctypes.c_int64(int(v)) for v in t.shape],
            *[ctypes.c_int64(int(v)) for v in t.stride()]]


def _entries():
    lib = native.library()
    plain = lib.intent_b200_w4a16_gemv_f16
    plain.restype = ctypes.c_int
    plain.argtypes = VIEW2 * 4 + [ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
    builtin = lib.intent_b200_w4a16_gemv_f16_builtin_scratch
    builtin.restype = ctypes.c_int
    builtin.argtypes = VIEW2 * 4 + [ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    query = lib.intent_b200_w4a16_gemv_workspace_bytes
    query.restype = ctypes.c_int64
    query.argtypes = [ctypes.c_int64] * 3
    return plain, builtin, query


@pytest.mark.parametrize("M,K,N", [(1, 4096, 14336), (4, 14336, 4096), (3, 512, 200)])
def test_builtin_scratch_matches_workspace_entry_twice(cuda_device, M, K, N):
    plain, builtin, query = _entries()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    outputs = []
    for call in range(2):                      # second call reuses the array the first one left behind
        x, p, s = ib.workloads.w4a16_inputs(M, K, N, dtype=torch.float16, seed=10 + call)
        xd, pd, sd = x.to(cuda_device), p.to(cuda_device), s.to(cuda_device)
        expected = torch.empty((M, N), dtype=torch.float16, device=cuda_device)
        workspace = torch.zeros(int(query(M, K, N)), dtype=torch.uint8, device=cuda_device)
        status = plain(*_slots(xd), *_slots(pd), *_slots(sd), *_slots(expected), 128, 8,
                       ctypes.c_void_p(workspace.data_ptr()), workspace.numel(), stream)
        assert status == 0
        got = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
        status = builtin(*_slots(xd), *_slots(pd), *_slots(sd), *_slots(got), 128, 8, stream)
        assert status == 0
        torch.cuda.synchronize()
        # same kernel, same summation order: the benchmark tolerance holds trivially, the bits agree
        assert max_abs_rel(got.cpu(), expected.cpu()) <= 2e-2
        assert torch.equal(got, expected)
        # no bounded wait gave up inside the call (the word lives in the built-in array and is only valid
        # until the next call of the entry clears it)
        reader = native.library().intent_b200_w4a16_gemv_builtin_scratch_status
        reader.restype, reader.argtypes = ctypes.c_int, [ctypes.c_void_p]
        assert reader(stream) == 0
        outputs.append(got)
    assert not torch.equal(outputs[0], outputs[1])      # the two calls really had different inputs


def test_builtin_scratch_rejects_oversized_problem(cuda_device):
    _, builtin, query = _entries()
    M, K, N = 16, 8192, 16384                           # needs more than the 8 MiB array
    assert query(M, K, N) > 8 << 20
    x = torch.zeros((M, K), dtype=torch.float16, device=cuda_device)
    p = torch.zeros((K // 8, N), dtype=torch.int32, device=cuda_device)
    s = torch.zeros((K // 128, N), dtype=torch.float16, device=cuda_device)
    y = torch.zeros((M, N), dtype=torch.float16, device=cuda_device)
    status = builtin(*_slots(x), *_slots(p), *_slots(s), *_slots(y), 128, 8,
                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert status == 7
    assert "built-in scratch" in native.status_string(status)
