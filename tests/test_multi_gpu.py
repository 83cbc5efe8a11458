"""Two-rank GPU checks (skipped on a single GPU): the expert-parallel MoE must reproduce the
single-GPU result bit for bit (f32 rows travel, the combine order is fixed), and a column shard of
the dense prefill must equal the same columns of the unsharded product."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ep_worker(rank, world, port, results):
    import torch.distributed as dist

    import intent_b200 as ib
    from intent_b200.distributed import ExpertParallelMoE, column_shard
    from intent_b200.moe import MoEW4A16FFN

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        tokens, hidden, inter, experts = 512, 512, 256, 8
        data = ib.workloads.moe_inputs(tokens, hidden, experts, inter, dtype=torch.bfloat16, seed=21)
        target = ib.B200Target(rank)
        # single-GPU result on every rank (all experts local)
        full = MoEW4A16FFN(tokens=tokens, hidden=hidden, intermediate=inter, experts=experts, target=target)
        dev = {k: v.to(device) for k, v in data.items()}
        ids, weights = full.route(dev["logits"])
        expected = full(dev["x"], ids, weights, dev["up_gate_packed"], dev["up_gate_scales"], dev["down_packed"],
                        dev["down_scales"])
        # expert parallel: this rank's tokens and experts
        t_local, e_local = tokens // world, experts // world
        rows = slice(rank * t_local, (rank + 1) * t_local)
        ex = slice(rank * e_local, (rank + 1) * e_local)
        ep = ExpertParallelMoE(tokens=t_local, hidden=hidden, intermediate=inter, experts=experts, target=target)
        y = ep(dev["logits"][rows].contiguous(), dev["x"][rows].contiguous(),
               dev["up_gate_packed"][ex].contiguous(), dev["up_gate_scales"][ex].contiguous(),
               dev["down_packed"][ex].contiguous(), dev["down_scales"][ex].contiguous())
        torch.cuda.synchronize()
        moe_ok = bool(torch.equal(y, expected[rows]))
        # fixed-capacity exchange: asynchronous, same bits while nothing overflows
        capped = ExpertParallelMoE(tokens=t_local, hidden=hidden, intermediate=inter, experts=experts,
                                   capacity_factor=1.5, target=target)
        y_capped = capped(dev["logits"][rows].contiguous(), dev["x"][rows].contiguous(),
                          dev["up_gate_packed"][ex].contiguous(), dev["up_gate_scales"][ex].contiguous(),
                          dev["down_packed"][ex].contiguous(), dev["down_scales"][ex].contiguous())
        capped.check_overflow()
        moe_ok = moe_ok and bool(torch.equal(y_capped, expected[rows]))
        # the same step bound once to fixed buffers and replayed twice
        prepared = capped.prepare(dev["logits"][rows].contiguous(), dev["x"][rows].contiguous(),
                                  dev["up_gate_packed"][ex].contiguous(), dev["up_gate_scales"][ex].contiguous(),
                                  dev["down_packed"][ex].contiguous(), dev["down_scales"][ex].contiguous())
        prepared.launch()
        y_prepared = prepared.launch()
        capped.check_overflow()
        moe_ok = moe_ok and bool(torch.equal(y_prepared, expected[rows]))
        # a capacity that is too small is reported, not silently wrong
        tiny = ExpertParallelMoE(tokens=t_local, hidden=hidden, intermediate=inter, experts=experts,
                                 capacity_factor=0.5, target=target)
        tiny(dev["logits"][rows].contiguous(), dev["x"][rows].contiguous(),
             dev["up_gate_packed"][ex].contiguous(), dev["up_gate_scales"][ex].contiguous(),
             dev["down_packed"][ex].contiguous(), dev["down_scales"][ex].contiguous())
        try:
            tiny.check_overflow()
            moe_ok = False
        except RuntimeError:
            pass

        # column-sharded dense prefill
        x, p, s = ib.workloads.w4a16_inputs(256, 1024, 1024, dtype=torch.bfloat16, seed=3)
        artifact = ib.compile(ib.programs.weight_only_int4_matmul, target=target,
                              constexprs={"GROUP_SIZE": 128, "ZERO_POINT": 8, "ACT_DTYPE": "bf16"})
        whole = artifact.run(x.to(device), p.to(device), s.to(device))
        cols = column_shard(1024, world, rank)
        part = artifact.run(x.to(device), p[:, cols].contiguous().to(device), s[:, cols].contiguous().to(device))
        torch.cuda.synchronize()
        results[rank] = (moe_ok, bool(torch.equal(part, whole[:, cols])))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_and_column_shard_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_ep_worker, args=(2, _free_port(), results), nprocs=2, join=True)
    assert dict(results) == {0: (True, True), 1: (True, True)}
