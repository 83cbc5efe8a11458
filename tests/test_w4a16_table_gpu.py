"""Tables of W4A16 decode projections in one persistent launch (intent_b200.table): parity with the oracle
at the benchmark tolerance  max|y - ref| <= 2e-2 * max|ref|  (and the tighter error the kernel really
achieves), bitwise reproducibility, workspace hygiene, and the fallback for problems outside its coverage."""
import ctypes

import pytest
import torch

import intent_b200 as ib
import oracle
from intent_b200.runtime import native
from intent_b200.table import W4A16Table
from conftest import load_golden, max_abs_rel

pytestmark = pytest.mark.gpu

BENCH_TOL = 2e-2


def _problems(shapes, dtype, group, device, seed=0):
    host, dev = [], []
    for index, (M, K, N) in enumerate(shapes):
        x, p, s = ib.workloads.w4a16_inputs(M, K, N, dtype=dtype, group_size=group, seed=seed + index)
        host.append((x, p, s))
        dev.append((x.to(device), p.to(device), s.to(device)))
    return host, dev


def _check(call, host, group, zero_point, dtype):
    call.launch()
    call.check()
    first = [y.clone() for y in call.results()]
    for y, (x, p, s) in zip(first, host):
        ref = oracle.weight_only_int4_matmul(x, p, s, group_size=group, zero_point=zero_point)
        assert y.dtype == dtype and y.shape == ref.shape
        if ref.numel():
            assert max_abs_rel(y.cpu(), ref) <= BENCH_TOL
            assert max_abs_rel(y.cpu(), ref) <= (2e-3 if dtype == torch.float16 else 1.6e-2)
    for y in call.results():
        y.fill_(float("nan"))
    call.launch()                      # same workspace, left clean by the first launch
    call.check()
    for y, again in zip(first, call.results()):
        assert torch.equal(y, again)   # fixed summation order: the same bits
    return first


@pytest.mark.parametrize("M", [1, 4, 8])
def test_decode_step_table(cuda_device, M):
    """Benchmark configuration 1: up and down projection of one decode step in one launch."""
    shapes = [(M, 4096, 14336), (M, 14336, 4096)]
    host, dev = _problems(shapes, torch.float16, 128, cuda_device)
    table = W4A16Table(group_size=128, zero_point=8, act_dtype="f16", target=ib.B200Target(0))
    call = table.prepare(dev)
    assert call.single_launch
    before = native.launch_count()
    call.launch()
    assert native.launch_count() - before == 1
    _check(call, host, 128, 8, torch.float16)


@pytest.mark.parametrize("dtype,group", [(torch.float16, 128), (torch.bfloat16, 128), (torch.float16, 64),
                                         (torch.bfloat16, 32)])
def test_mixed_table_matches_oracle(cuda_device, dtype, group):
    """Ragged and tiny problems next to large ones, different row counts, in one table (and, with ten
    problems, more than one launch)."""
    shapes = [(1, 4096, 4096), (3, 256, 72), (8, 128, 8), (5, 512, 200), (1, 1024, 64), (2, 2048, 1000),
              (7, 768, 328), (4, 14336, 4096), (1, 128, 8), (6, 8192, 512)]
    host, dev = _problems(shapes, dtype, group, cuda_device, seed=20)
    table = W4A16Table(group_size=group, zero_point=8, act_dtype="f16" if dtype == torch.float16 else "bf16",
                       target=ib.B200Target(0))
    call = table.prepare(dev)
    assert call.single_launch
    before = native.launch_count()
    call.launch()
    # ten problems: the one- and two-row ones in one launch, the staged ones in as few as fit together
    assert 2 <= native.launch_count() - before <= 4
    _check(call, host, group, 8, dtype)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_both_forms_of_the_table_kernel(cuda_device, dtype):
    """Problems of one or two rows run in the barrier-free form (every unit brings its activations); the
    staged form can be forced for them.  Both must meet the oracle, and a long table must keep the per-problem
    partial areas apart (eight problems per launch alternate between two buffers)."""
    from intent_b200 import table as table_module

    shapes = [(1, 4096, 14336), (2, 14336, 4096), (1, 4096, 4096), (2, 256, 72), (1, 14336, 4096), (1, 1024, 64),
              (2, 4096, 14336), (1, 128, 8), (1, 11008, 4096)]
    host, dev = _problems(shapes, dtype, 128, cuda_device, seed=40)
    table = W4A16Table(group_size=128, zero_point=8, act_dtype="f16" if dtype == torch.float16 else "bf16",
                       target=ib.B200Target(0))
    try:
        table_module.set_ride_along(False)
        staged = _check(table.prepare(dev), host, 128, 8, dtype)
    finally:
        table_module.set_ride_along(True)
    riding = _check(table.prepare(dev), host, 128, 8, dtype)
    for a, b in zip(staged, riding):
        assert max_abs_rel(a.cpu(), b.cpu()) <= (2e-3 if dtype == torch.float16 else 1.6e-2)


def test_table_agrees_with_single_problem_entry(cuda_device):
    """The table kernel and the single-problem kernel implement one program: same inputs, results within a
    few units in the last place of each other (both are inside the tolerance against the oracle)."""
    shapes = [(1, 4096, 14336), (2, 14336, 4096), (8, 4096, 4096), (16, 1024, 512)]
    host, dev = _problems(shapes, torch.float16, 128, cuda_device, seed=3)
    table = W4A16Table(group_size=128, zero_point=8, act_dtype="f16", target=ib.B200Target(0))
    call = table.prepare(dev)
    results = _check(call, host, 128, 8, torch.float16)
    for (x, p, s), y in zip(dev, results):
        single = table.artifact.run(x, p, s)
        assert max_abs_rel(y.cpu(), single.cpu()) <= 2e-3


def test_reference_layout_golden_through_the_table(cuda_device):
    """The reference's own constants (group 64, two's-complement nibbles, f16) on its golden vectors."""
    goldens = [load_golden(f"w4a16_{tag}") for tag in ("small", "ragged_m")]
    table = W4A16Table(target=ib.B200Target(0))                    # defaults = the reference's constants
    call = table.prepare([(g["activation"].to(cuda_device), g["packed"].to(cuda_device), g["scales"].to(cuda_device))
                          for g in goldens])
    call.launch()
    call.check()
    for g, y in zip(goldens, call.results()):
        assert (y.cpu().float() - g["output"].float()).abs().max() <= 4e-2      # the reference's own tolerance
        assert max_abs_rel(y.cpu(), g["output"]) <= 2e-3


def test_explicit_outputs_empty_problems_and_validation(cuda_device):
    host, dev = _problems([(2, 256, 64), (0, 256, 64), (3, 512, 96)], torch.float16, 128, cuda_device, seed=8)
    table = W4A16Table(group_size=128, zero_point=8, act_dtype="f16", target=ib.B200Target(0))
    outputs = [torch.full((x.shape[0], p.shape[1]), float("nan"), dtype=torch.float16, device=cuda_device)
               for x, p, _ in dev]
    call = table.prepare(dev, outputs=outputs)
    assert all(a.data_ptr() == b.data_ptr() for a, b in zip(call.results(), outputs))
    _check(call, host, 128, 8, torch.float16)
    with pytest.raises(TypeError):
        table.prepare([(dev[0][0].float(), dev[0][1], dev[0][2])])                 # dtype mismatch: never coerced
    with pytest.raises(ValueError):
        table.prepare([(dev[0][0], dev[0][1], dev[0][2].cpu())])                   # wrong device
    with pytest.raises(ValueError):
        table.prepare([(dev[0][0], dev[2][1], dev[0][2])])                         # K/8 disagrees with the packed rows
    with pytest.raises(TypeError):
        table.prepare([dev[0][:2]])


def test_problems_outside_the_table_kernel_fall_back(cuda_device):
    """Sixteen rows against a long K do not fit the table kernel's shared memory: prepare() falls back to one
    single-problem launch per entry, with the same results contract."""
    shapes = [(16, 4096, 14336), (1, 4096, 4096)]
    host, dev = _problems(shapes, torch.float16, 128, cuda_device, seed=12)
    table = W4A16Table(group_size=128, zero_point=8, act_dtype="f16", target=ib.B200Target(0))
    call = table.prepare(dev)
    assert not call.single_launch
    _check(call, host, 128, 8, torch.float16)


def test_table_entry_through_raw_c_abi(cuda_device):
    """The C entry itself: a host array of problem records, device pointers, a zero-filled workspace."""
    class Problem(ctypes.Structure):
        _fields_ = [("x", ctypes.c_void_p), ("packed", ctypes.c_void_p), ("scales", ctypes.c_void_p),
                    ("y", ctypes.c_void_p), ("M", ctypes.c_int64), ("K", ctypes.c_int64), ("N", ctypes.c_int64)]

    lib = native.library()
    host, dev = _problems([(1, 4096, 14336), (1, 14336, 4096)], torch.float16, 128, cuda_device, seed=0)
    ys = [torch.empty((1, p.shape[1]), dtype=torch.float16, device=cuda_device) for _, p, _ in dev]
    rows = (Problem * 2)()
    for row, (x, p, s), y in zip(rows, dev, ys):
        row.x, row.packed, row.scales, row.y = x.data_ptr(), p.data_ptr(), s.data_ptr(), y.data_ptr()
        row.M, row.K, row.N = x.shape[0], x.shape[1], p.shape[1]
    query = lib.intent_b200_w4a16_gemv_table_workspace_bytes
    query.restype, query.argtypes = ctypes.c_int64, [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32]
    need = query(rows, 2, 128)
    assert need > 0
    entry = lib.intent_b200_w4a16_gemv_table_f16
    entry.restype = ctypes.c_int
    entry.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p,
                      ctypes.c_int64, ctypes.c_void_p]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    small = torch.zeros((need - 16,), dtype=torch.uint8, device=cuda_device)
    assert entry(rows, 2, 128, 8, ctypes.c_void_p(small.data_ptr()), small.numel(), stream) == 5     # workspace too small
    workspace = torch.zeros((need,), dtype=torch.uint8, device=cuda_device)
    assert entry(rows, 2, 128, 8, ctypes.c_void_p(workspace.data_ptr()), need, stream) == 0
    torch.cuda.synchronize()
    for (x, p, s), y in zip(host, ys):
        ref = oracle.weight_only_int4_matmul(x, p, s, group_size=128, zero_point=8)
        assert max_abs_rel(y.cpu(), ref) <= 2e-3
    assert int(workspace[:4].view(torch.int32)[0]) == 0                                               # status word
    rows[1].K = 14336 + 8                                                                             # not a multiple of the group
    assert entry(rows, 2, 128, 8, ctypes.c_void_p(workspace.data_ptr()), need, stream) == 3


def test_ring_probe_entry(cuda_device):
    """The measurement entry behind the decode kernels' design notes: streams matrices through the bare slot
    ring and returns a time; its bounded waits leave the status word at zero."""
    import ctypes

    from intent_b200.runtime import native
    probe = native.library().intent_b200_ring_probe_ms
    probe.restype = ctypes.c_double
    probe.argtypes = [ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                      ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p, ctypes.c_void_p]
    sms = torch.cuda.get_device_properties(cuda_device).multi_processor_count
    matrices = torch.randint(0, 2 ** 31 - 1, (3, 96, 512), dtype=torch.int32, device=cuda_device)
    scratch = torch.zeros(8192 + sms * 8192, dtype=torch.uint8, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    for slots, mode in ((16, 0), (32, 3), (48, 2), (32, 1), (16, 5), (32, 4)):
        ms = probe(matrices.data_ptr(), 3, 96, 512, slots, mode, 2, scratch.data_ptr(), stream)
        assert ms > 0
        assert int(scratch[:4].view(torch.int32).item()) == 0
    assert probe(matrices.data_ptr(), 3, 96, 500, 16, 0, 2, scratch.data_ptr(), stream) < 0     # cols not a multiple of 32
    assert probe(matrices.data_ptr(), 3, 96, 512, 24, 0, 2, scratch.data_ptr(), stream) < 0      # slots not a multiple of 16
    assert probe(None, 3, 96, 512, 16, 0, 2, scratch.data_ptr(), stream) < 0


@pytest.mark.parametrize("M,dtype,group", [(1, torch.float16, 128), (3, torch.bfloat16, 64), (8, torch.float16, 32)])
def test_many_short_segments_recycle_the_chain_sets(cuda_device, M, dtype, group):
    """Short K and very wide N: every unit (or every second one) is a segment of its own and a CTA meets far
    more segments per launch than its ring of chain sets holds, so the sets are reused through their generation
    counters; ragged N and K exercise the zero-filled edges of the TMA boxes."""
    shapes = [(M, 256, 81920), (M, 384, 70008), (M, 512, 40000), (M, 4096, 14336), (M, 640, 33000), (M, 256, 8)]
    host, dev = _problems(shapes, dtype, group, cuda_device, seed=40)
    table = W4A16Table(group_size=group, zero_point=8, act_dtype="f16" if dtype == torch.float16 else "bf16",
                       target=ib.B200Target(0))
    call = table.prepare(dev)
    assert call.single_launch
    _check(call, host, group, 8, dtype)


def test_eight_step_table_matches_per_step_tables(cuda_device):
    """Sixteen problems in one call (two launches of eight) give, problem by problem, the bits of eight
    two-problem calls: a problem's sums do not depend on its neighbours in the table."""
    shapes = [(1, 4096, 14336), (1, 14336, 4096)] * 8
    host, dev = _problems(shapes, torch.float16, 128, cuda_device, seed=7)
    table = W4A16Table(group_size=128, zero_point=8, act_dtype="f16", target=ib.B200Target(0))
    whole = table.prepare(dev)
    before = native.launch_count()
    whole.launch()
    whole.check()
    assert native.launch_count() - before == 2
    for step in range(8):
        pair = table.prepare(dev[2 * step:2 * step + 2])
        pair.launch()
        pair.check()
        for y, expected in zip(pair.results(), whole.results()[2 * step:2 * step + 2]):
            assert torch.equal(y, expected)
