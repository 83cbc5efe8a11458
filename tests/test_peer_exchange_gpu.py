"""Expert-parallel MoE over peer memory.

On one GPU the ranks are emulated in sequence: every rank's buffers are plain local tensors,
the address tables point at them, and the phases run rank after rank (no kernel waits on
another one).  The result must equal the single-GPU FFN over all tokens bit for bit.  The
two-process test (skipped on a single GPU) does the same through symmetric memory and NCCL."""
import os
import socket

import pytest
import torch

import intent_b200 as ib
from intent_b200.moe import MoEW4A16FFN
from intent_b200.peer import PeerExchangeRank

pytestmark = pytest.mark.gpu


def _slices(data, device, rank, world, tokens, experts):
    t_local, e_local = tokens // world, experts // world
    rows, ex = slice(rank * t_local, (rank + 1) * t_local), slice(rank * e_local, (rank + 1) * e_local)
    return (data["logits"][rows].contiguous().to(device), data["x"][rows].contiguous().to(device),
            [data[k][ex].contiguous().to(device) for k in ("up_gate_packed", "up_gate_scales", "down_packed",
                                                            "down_scales")])


@pytest.mark.parametrize("world,tokens,hidden,inter,experts", [(2, 512, 512, 256, 8), (4, 1024, 256, 128, 16),
                                                               (1, 300, 256, 128, 4)])
def test_peer_exchange_emulated_ranks(cuda_device, world, tokens, hidden, inter, experts):
    data = ib.workloads.moe_inputs(tokens, hidden, experts, inter, dtype=torch.bfloat16, seed=5)
    target = ib.B200Target(0)
    full = MoEW4A16FFN(tokens=tokens, hidden=hidden, intermediate=inter, experts=experts, target=target)
    dev = {k: v.to(cuda_device) for k, v in data.items()}
    ids, weights = full.route(dev["logits"])
    expected = full(dev["x"], ids, weights, dev["up_gate_packed"], dev["up_gate_scales"], dev["down_packed"],
                    dev["down_scales"])

    t_local = tokens // world
    sides = [PeerExchangeRank(rank=r, world=world, tokens=t_local, hidden=hidden, intermediate=inter,
                              experts=experts, target=target) for r in range(world)]
    (rows_shape, rows_dtype), (out_shape, out_dtype) = sides[0].buffer_shapes()
    rows = [torch.zeros(rows_shape, dtype=rows_dtype, device=cuda_device) for _ in range(world)]
    out = [torch.zeros(out_shape, dtype=out_dtype, device=cuda_device) for _ in range(world)]
    peer_rows = torch.tensor([t.data_ptr() for t in rows], dtype=torch.int64, device=cuda_device)
    peer_out = torch.tensor([t.data_ptr() for t in out], dtype=torch.int64, device=cuda_device)
    counts_all = torch.zeros((world, experts), dtype=torch.int32, device=cuda_device)
    ys, steps = [], []
    for r, side in enumerate(sides):
        logits, x, w = _slices(data, cuda_device, r, world, tokens, experts)
        y = torch.full((t_local, hidden), 3.0, dtype=torch.float32, device=cuda_device)
        ys.append(y)
        steps.append(side.prepare(logits, x, *w, y, rows=rows[r], out=out[r], peer_rows=peer_rows,
                                  peer_out=peer_out, counts_all=counts_all))
    # the ranks' sync points: every rank has its own flag array and its own view of the count matrix
    from intent_b200.peer import PeerSignals

    flags = [torch.zeros((PeerSignals.CHANNELS, world), dtype=torch.int32, device=cuda_device) for _ in range(world)]
    tables = [counts_all] + [torch.zeros_like(counts_all) for _ in range(world - 1)]   # rank 0's is the bound one
    peer_flags = torch.tensor([t.data_ptr() for t in flags], dtype=torch.int64, device=cuda_device)
    peer_tables = torch.tensor([t.data_ptr() for t in tables], dtype=torch.int64, device=cuda_device)
    signals = [PeerSignals(rank=r, world=world, flags=flags[r], peer_flags=peer_flags, peer_tables=peer_tables,
                           counts=steps[r].counts, target=target) for r in range(world)]
    for repeat in range(2):          # the second pass runs over buffers that hold the first pass's rows
        for step in steps:
            step.route()
        if repeat == 0:              # counts by hand
            for r, step in enumerate(steps):
                counts_all[r].copy_(step.counts)
        else:                        # counts through the signalling kernels: all ranks post, then all wait
            counts_all.zero_()
            for s in signals:
                s.post(0)
            for s in signals:
                s.wait(0)
            assert all(torch.equal(t, counts_all) for t in tables)
        for step in steps:
            step.dispatch_rows()
        for channel in (1, 2):
            for s in signals:
                s.post(channel)
            for s in signals:
                s.wait(channel)
        for step in steps:
            step.experts()
        for step in steps:
            step.combine()
        torch.cuda.synchronize()
        for s in signals:
            s.check()
        assert torch.equal(torch.cat(ys), expected), f"pass {repeat}"
    # every route was placed: owners and positions are in range, positions are unique per owner
    placed = torch.cat([s.route_dest for s in steps]).cpu()
    assert placed[:, 0].min() >= 0 and placed[:, 0].max() < world
    keys = placed[:, 0].long() * sides[0].capacity_rows + placed[:, 1].long()
    assert keys.unique().numel() == keys.numel()
    assert int(counts_all.sum()) == tokens * 2


def test_peer_wait_gives_up(cuda_device):
    """A sync point that one rank never reaches: the wait must return with a timeout status instead of
    hanging (a flag that nothing sets; the context stays usable)."""
    from intent_b200.peer import PeerSignals

    world = 2
    flags = torch.zeros((PeerSignals.CHANNELS, world), dtype=torch.int32, device=cuda_device)
    other = torch.zeros_like(flags)
    peer_flags = torch.tensor([flags.data_ptr(), other.data_ptr()], dtype=torch.int64, device=cuda_device)
    table = torch.zeros((world, 8), dtype=torch.int32, device=cuda_device)
    peer_tables = torch.tensor([table.data_ptr(), table.data_ptr()], dtype=torch.int64, device=cuda_device)
    counts = torch.arange(8, dtype=torch.int32, device=cuda_device)
    signals = PeerSignals(rank=0, world=world, flags=flags, peer_flags=peer_flags, peer_tables=peer_tables,
                          counts=counts, target=ib.B200Target(0), max_polls=2000)
    signals.post(1)
    signals.wait(1)                      # rank 1 never posts
    torch.cuda.synchronize()
    assert flags[1].tolist() == [1, 0] and other[1].tolist() == [1, 0]
    with pytest.raises(RuntimeError, match="expired"):
        signals.check()
    signals.check()                      # the status is cleared by the failed check
    other_side = torch.tensor([2, 2], dtype=torch.int32, device=cuda_device)
    flags[1].copy_(other_side)           # "rank 1" arrives (and is already one step ahead)
    signals.post(1)
    signals.wait(1)
    torch.cuda.synchronize()
    signals.check()
    assert torch.equal(torch.ones(1, device=cuda_device), torch.ones(1, device=cuda_device))   # context is usable


def test_second_prepared_step_still_waits(cuda_device):
    """Two steps bound one after the other to the same flag array must continue one sequence: the flags keep
    the first step's numbers, so counters that restarted at zero would let every wait of the second step pass
    at once.  With the shared counters the second step's wait runs out when the other rank has not posted
    again (bounded wait, a flag that nothing sets)."""
    from intent_b200.peer import PeerSignals

    world = 2
    flags = torch.zeros((PeerSignals.CHANNELS, world), dtype=torch.int32, device=cuda_device)
    other = torch.zeros_like(flags)
    peer_flags = torch.tensor([flags.data_ptr(), other.data_ptr()], dtype=torch.int64, device=cuda_device)
    table = torch.zeros((world, 8), dtype=torch.int32, device=cuda_device)
    peer_tables = torch.tensor([table.data_ptr(), table.data_ptr()], dtype=torch.int64, device=cuda_device)
    counts = torch.arange(8, dtype=torch.int32, device=cuda_device)
    sequence, status = PeerSignals.counters(cuda_device)
    common = dict(rank=0, world=world, flags=flags, peer_flags=peer_flags, peer_tables=peer_tables, counts=counts,
                  target=ib.B200Target(0), max_polls=2000, sequence=sequence, status=status)
    first = PeerSignals(**common)
    flags[:, 1] = 1                      # "rank 1" posts its first step on every channel
    for channel in range(PeerSignals.CHANNELS):
        first.post(channel)
        first.wait(channel)
    torch.cuda.synchronize()
    first.check()
    second = PeerSignals(**common)       # what a second prepare() on the same exchange builds
    assert second.sequence.data_ptr() == first.sequence.data_ptr()
    second.post(1)
    second.wait(1)                       # rank 1 has not posted its second step
    torch.cuda.synchronize()
    assert sequence.tolist() == [1, 1, 2, 2, 1, 1]
    with pytest.raises(RuntimeError, match="expired"):
        second.check()
    flags[1, 1] = 2                      # now it has
    second.post(1)                       # (a retry after the failure: number 3 here, rank 1 must follow)
    flags[1, 1] = 3
    second.wait(1)
    torch.cuda.synchronize()
    second.check()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _peer_worker(rank, world, port, results):
    import torch.distributed as dist

    from intent_b200.peer import PeerExpertParallelMoE

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        tokens, hidden, inter, experts = 512, 512, 256, 8
        data = ib.workloads.moe_inputs(tokens, hidden, experts, inter, dtype=torch.bfloat16, seed=21)
        target = ib.B200Target(rank)
        full = MoEW4A16FFN(tokens=tokens, hidden=hidden, intermediate=inter, experts=experts, target=target)
        dev = {k: v.to(device) for k, v in data.items()}
        ids, weights = full.route(dev["logits"])
        expected = full(dev["x"], ids, weights, dev["up_gate_packed"], dev["up_gate_scales"], dev["down_packed"],
                        dev["down_scales"])
        logits, x, w = _slices(data, device, rank, world, tokens, experts)
        ok = True
        for signals in ("peer", "nccl"):
            ep = PeerExpertParallelMoE(tokens=tokens // world, hidden=hidden, intermediate=inter, experts=experts,
                                       target=target, signals=signals)
            call = ep.prepare(logits, x, *w)
            for _ in range(3):
                call.launch()
                torch.cuda.synchronize()
                call.check()
                t_local = tokens // world
                ok = ok and bool(torch.equal(call.y, expected[rank * t_local:(rank + 1) * t_local]))
            # a second bound step and the unprepared call share the exchange's flags and counters
            again = ep.prepare(logits, x, *w)
            again.launch()
            torch.cuda.synchronize()
            again.check()
            ok = ok and bool(torch.equal(again.y, expected[rank * t_local:(rank + 1) * t_local]))
            for _ in range(2):
                y = ep(logits, x, *w)
                torch.cuda.synchronize()
                ok = ok and bool(torch.equal(y, expected[rank * t_local:(rank + 1) * t_local]))
        results[rank] = ok
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_peer_exchange_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_peer_worker, args=(2, _free_port(), results), nprocs=2, join=True)
    assert dict(results) == {0: True, 1: True}
