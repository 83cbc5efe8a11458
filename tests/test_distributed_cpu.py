"""Multi-rank host logic on CPU (gloo, world size 2): the row exchange of the expert-parallel
MoE and the column sharding of the dense contractions."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from intent_b200.distributed import (column_shard, dispatch_rows, exchange_counts, return_rows)


def test_column_shard_covers_columns_once():
    for columns, world, multiple in [(8192, 8, 256), (8192, 4, 256), (14336, 8, 256), (1000, 3, 128), (256, 4, 256)]:
        blocks = [column_shard(columns, world, rank, multiple) for rank in range(world)]
        assert blocks[0].start == 0 and blocks[-1].stop == columns
        for left, right in zip(blocks, blocks[1:]):
            assert left.stop == right.start
        assert all(b.start % multiple == 0 for b in blocks)
    with pytest.raises(ValueError):
        column_shard(10, 2, 2)


def test_pipeline_piece_rows_cover_the_rows_once():
    """Piece sizes of the host-to-host pipeline of the column-sharded programs: every rank's rows exactly once,
    the outermost pieces a quarter of a full one."""
    from intent_b200.distributed import ColumnShardedRows
    assert ColumnShardedRows.piece_rows(8192, 1, 8) == [256, 768, 1024, 1024, 1024, 1024, 1024, 1024, 768, 256]
    assert ColumnShardedRows.piece_rows(8192, 2, 8) == [128, 384, 512, 512, 512, 512, 512, 512, 384, 128]
    assert ColumnShardedRows.piece_rows(8192, 1, 8, taper=False) == [1024] * 8
    assert ColumnShardedRows.piece_rows(4096, 8, 8) == [32, 96, 128, 128, 96, 32]   # (256 gathered rows at the ends)
    assert ColumnShardedRows.piece_rows(384, 1, 8) == [128] * 3                      # too few pieces to taper
    for rows, world, chunks in [(8192, 1, 8), (8192, 4, 8), (4096, 1, 16), (1000, 1, 8), (8192, 8, 3), (384, 1, 8)]:
        sizes = ColumnShardedRows.piece_rows(rows, world, chunks)
        assert sum(sizes) == rows // world and min(sizes) > 0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _expert_fn(rows, experts):
    # stand-in for the expert FFN: depends on the row and on the (local) expert it was sent to
    return rows.float() * (experts.float() + 1.0)


def _worker(rank, world, port, tokens, hidden, experts, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        local_experts = experts // world
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn((tokens, hidden), generator=g)
        ids = torch.randint(0, experts, (tokens, 2), generator=g, dtype=torch.int32)
        if rank == 1:
            ids[:] = ids % local_experts        # rank 1 sends everything to rank 0: ragged and empty splits
        weights = torch.rand((tokens, 2), generator=g)
        destination = (ids // local_experts).flatten()
        order = torch.argsort(destination, stable=True)
        counts = torch.bincount(destination, minlength=world)
        plan = exchange_counts(counts)
        assert sum(plan.send) == tokens * 2
        received = dispatch_rows(x[order // 2], plan)
        received_experts = dispatch_rows((ids.flatten()[order] % local_experts).unsqueeze(1), plan)
        assert received.shape[0] == plan.received_rows == received_experts.shape[0]
        outputs = _expert_fn(received, received_experts + rank * local_experts)
        returned = return_rows(outputs, plan)
        position = torch.empty_like(order)
        position[order] = torch.arange(order.numel())
        y = (weights.flatten()[:, None] * returned[position]).reshape(tokens, 2, hidden).sum(dim=1)
        expected = (weights[:, :, None] * _expert_fn(x[:, None, :].expand(-1, 2, -1), ids[:, :, None])).sum(dim=1)
        results[rank] = bool(torch.allclose(y, expected, rtol=1e-6, atol=1e-6))
    finally:
        dist.destroy_process_group()


def test_expert_parallel_exchange_two_ranks():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), 37, 16, 8, results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}
