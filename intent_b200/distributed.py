"""Multi-GPU forms of the programs: one process per GPU, ``torch.distributed``.

The reference is single-device (each artifact binds one CUDA device,
python/intent/runtime/artifact.py:216-237); what is here is the sharding the
benchmark configurations ask for.

  * Dense W4A16 prefill and W8A8 shard over output columns: rank r owns a
    contiguous block of columns of the weight (and of its scales), activations are
    replicated, every rank writes its own block of Y.  No collective on the path.
  * MoE is expert-parallel: rank r owns experts [r*E/g, (r+1)*E/g).  Tokens are
    routed where they live, token rows travel to the owners of their experts with
    one all-to-all, the expert FFN runs on the received rows, the f32 result rows
    travel back with the reverse all-to-all and are combined per token.  The rows a
    kernel reads are always in local memory.
"""
from __future__ import annotations

from dataclasses import dataclass


def column_shard(columns: int, world: int, rank: int, multiple: int = 256) -> slice:
    """Contiguous block of output columns owned by ``rank``; block edges are multiples of
    ``multiple`` (one kernel tile) except the last edge."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError("rank must be in [0, world)")
    tiles = -(-columns // multiple)
    first = (tiles * rank) // world * multiple
    last = min(columns, (tiles * (rank + 1)) // world * multiple)
    return slice(first, max(first, last))


@dataclass
class RowAligned:
    """Marks a resident operand of :class:`ColumnShardedRows` that has one entry per activation row (the
    per-token scales of W8A8): every piece gets the entries of its own rows."""

    tensor: object


class ColumnShardedRows:
    """End-to-end form of a column-sharded dense program (W4A16 prefill, W8A8): the activation rows start in
    pinned HOST memory and the result block ends there, with the copies overlapped with the contraction.

    ``artifact`` is a compiled dense program whose first parameter is the row operand ``[M, K]`` and whose
    single Out is ``[M, n_local]``; ``resident`` are its remaining inputs, already on the device (this rank's
    column shard of the weights; an operand with one entry per row is wrapped in :class:`RowAligned`).  One call of :meth:`run` computes ``Y[:, shard] = program(X, resident)``:

      * rank r uploads only ITS rows ``[r*M/world, (r+1)*M/world)`` of X, in ``chunks`` pieces on a copy
        stream (plain ``cudaMemcpyAsync`` from pinned memory);
      * with more than one rank every piece is all-gathered over NVLink (NCCL) into a local buffer, so each
        row crosses PCIe once on the whole node and the contraction reads local memory only;
      * the contraction of piece i runs on the compute stream while piece i+1 uploads and the result of
        piece i-1 downloads on a third stream (PCIe is full duplex);
      * the first and the last pieces are smaller than the rest (``taper``): the pipeline is bound by the
        uploads, and what it adds to them is the upload of the first piece plus the contraction and the
        download of the last one.

    Gathered pieces hold rows ``{r*M/world + i*piece .. }`` of every rank r; the result rows are copied back
    to exactly those rows of the pinned output.  Every buffer and prepared call is built once here; ``run``
    neither allocates nor validates.  Nothing here runs on one GPU only: no load is a multicast load.
    """

    @staticmethod
    def piece_rows(rows: int, world: int, chunks: int, taper: bool = True) -> list:
        """Rows of every piece PER RANK.  ``chunks`` sets the size of a full piece (rows / chunks over all
        ranks); with ``taper`` the first and the last full piece are each cut into a quarter and three quarters,
        the quarter outermost (8192 rows, 8 chunks: 256, 768, 1024 x 6, 768, 256)."""
        local = rows // world
        chunks = max(1, min(chunks, local // 128 or 1))
        while local % chunks:
            chunks -= 1
        piece = local // chunks
        if not taper or chunks < 4 or piece % 4:
            return [piece] * chunks
        return [piece // 4, piece - piece // 4] + [piece] * (chunks - 2) + [piece - piece // 4, piece // 4]

    def __init__(self, artifact, resident: tuple, *, rows: int, width: int, n_local: int, in_dtype, out_dtype,
                 device, chunks: int = 8, group=None, taper: bool = True):
        import torch
        import torch.distributed as dist

        self.world = dist.get_world_size(group) if (dist.is_available() and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.group, self._dist = group, dist
        if rows % self.world:
            raise ValueError("the row count must be a multiple of the number of ranks")
        self.rows, self.width, self.n_local = rows, width, n_local
        self.local_rows = rows // self.world
        self.sizes = self.piece_rows(rows, self.world, chunks, taper)
        self.starts = [sum(self.sizes[:i]) for i in range(len(self.sizes))]
        self.chunks = chunks = len(self.sizes)
        self.device = device
        self._mine = [torch.empty((size, width), dtype=in_dtype, device=device) for size in self.sizes]
        self._x = (self._mine if self.world == 1 else
                   [torch.empty((size * self.world, width), dtype=in_dtype, device=device) for size in self.sizes])
        self._y = [torch.empty((size * self.world, n_local), dtype=out_dtype, device=device) for size in self.sizes]
        self._calls = []
        for i, (x, y) in enumerate(zip(self._x, self._y)):
            # rows of piece i, in the order the gathered buffer holds them: rank 0's rows first
            index = torch.cat([torch.arange(r * self.local_rows + self.starts[i],
                                            r * self.local_rows + self.starts[i] + self.sizes[i])
                               for r in range(self.world)])
            operands = [o.tensor[index.to(o.tensor.device)].contiguous() if isinstance(o, RowAligned) else o
                        for o in resident]
            self._calls.append(artifact.prepare(x, *operands, outputs=(y,)))
        self._upload, self._download = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self._uploaded = [torch.cuda.Event() for _ in range(chunks)]
        self._computed = [torch.cuda.Event() for _ in range(chunks)]
        self._released = [torch.cuda.Event() for _ in range(chunks)]     # result buffer i may be overwritten
        self._used = [torch.cuda.Event() for _ in range(chunks)]         # upload buffer i may be overwritten
        self._first = True

    @property
    def h2d_bytes(self) -> int:
        return self.local_rows * self.width * self._mine[0].element_size()

    @property
    def d2h_bytes(self) -> int:
        return self.rows * self.n_local * self._y[0].element_size()

    def run(self, host_x, host_y) -> None:
        """``host_x`` [M, K] and ``host_y`` [M, n_local]: pinned host tensors.  Returns after queueing; the
        caller synchronises (``torch.cuda.synchronize``) before reading ``host_y``."""
        import torch

        compute = torch.cuda.current_stream(self.device)
        first_row = self.rank * self.local_rows
        self._upload.wait_stream(compute)
        for i in range(self.chunks):
            begin, size = first_row + self.starts[i], self.sizes[i]
            with torch.cuda.stream(self._upload):
                if not self._first:
                    self._upload.wait_event(self._used[i])
                self._mine[i].copy_(host_x[begin:begin + size], non_blocking=True)
                self._uploaded[i].record(self._upload)
            compute.wait_event(self._uploaded[i])
            if self.world > 1:
                self._dist.all_gather_into_tensor(self._x[i], self._mine[i], group=self.group)
            if not self._first:
                compute.wait_event(self._released[i])
            self._calls[i].launch()
            self._computed[i].record(compute)
            self._used[i].record(compute)
            with torch.cuda.stream(self._download):
                self._download.wait_event(self._computed[i])
                for r in range(self.world):
                    row = r * self.local_rows + self.starts[i]
                    host_y[row:row + size].copy_(self._y[i][r * size:(r + 1) * size], non_blocking=True)
                self._released[i].record(self._download)
        compute.wait_stream(self._download)
        self._first = False


@dataclass
class ExchangePlan:
    """Row counts of one all-to-all: what this rank sends to / receives from every rank."""

    send: list
    receive: list

    @property
    def received_rows(self) -> int:
        return int(sum(self.receive))


def exchange_counts(send_counts, group=None) -> ExchangePlan:
    """All ranks tell each other how many rows they will send (one small all-to-all);
    the counts come back to the host because the collective needs them as split sizes."""
    import torch
    import torch.distributed as dist

    send = send_counts.to(torch.int64)
    received = torch.empty_like(send)
    dist.all_to_all_single(received, send, group=group)
    return ExchangePlan([int(v) for v in send.cpu()], [int(v) for v in received.cpu()])


def dispatch_rows(rows, plan: ExchangePlan, group=None):
    """rows sorted by destination rank [sum(send), ...] -> rows received, grouped by source rank."""
    import torch
    import torch.distributed as dist

    out = torch.empty((plan.received_rows, *rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=plan.receive, input_split_sizes=plan.send,
                           group=group)
    return out


def return_rows(rows, plan: ExchangePlan, group=None):
    """Inverse of :func:`dispatch_rows`: results for received rows go back to their senders and
    arrive in the order the rows were sent."""
    import torch
    import torch.distributed as dist

    out = torch.empty((int(sum(plan.send)), *rows.shape[1:]), dtype=rows.dtype, device=rows.device)
    dist.all_to_all_single(out, rows.contiguous(), output_split_sizes=plan.send, input_split_sizes=plan.receive,
                           group=group)
    return out


class ExpertParallelMoE:
    """Expert-parallel SiLU-gated int4 MoE FFN.  ``experts`` is the global expert count,
    ``tokens`` the number of tokens routed by THIS rank per call; every rank holds the weights of
    its own ``experts // world`` experts.

    Two exchange modes:

    * exact (default): rows travel with their true per-rank counts.  The counts have to reach the
      host as split sizes of the collective, which costs one device -> host read per step.
    * ``capacity_factor=f``: every rank sends a fixed ``cap = ceil(f * routes / world)`` rows to every
      rank (unused slots are zero rows), so nothing is read back and the whole step is
      asynchronous.  If a rank ever gets more than ``cap`` routes for one destination the step's
      result is incomplete; that is recorded on the device and :meth:`check_overflow` raises.
    """

    def __init__(self, *, tokens, hidden, intermediate, experts, top_k=2, group_size=128, zero_point=8,
                 act_dtype="bf16", capacity_rows=None, capacity_factor=None, block_size=128, target=None,
                 group=None):
        import torch
        import torch.distributed as dist

        from . import programs
        from .compiler import compile as _compile
        from .moe import MoEAlignment, MoEW4A16FFN

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if experts % self.world:
            raise ValueError("the expert count must be a multiple of the number of ranks")
        self.local_experts = experts // self.world
        self.tokens, self.hidden, self.top_k = tokens, hidden, top_k
        self.routes = tokens * top_k
        self.capacity_factor = capacity_factor
        if capacity_factor is None:
            self.slot_rows = 1                           # spans are exactly as long as their counts
            self.capacity = capacity_rows or self.routes * self.world
        else:
            self.slot_rows = -(-int(capacity_factor * self.routes) // self.world)
            self.capacity = self.slot_rows * self.world   # rows sent and received per step, fixed
        self.router = _compile(programs.moe_route_top2, target=target)
        # sorting routes by destination rank is the same stable partition as the expert alignment
        self.by_rank = MoEAlignment.build(tokens=tokens, top_k=top_k, experts=self.world,
                                          block_size=self.slot_rows, target=target)
        rank_constexprs = {"TOKENS": tokens, "TOP_K": top_k, "EXPERTS": self.world, "BLOCK_SIZE": self.slot_rows}
        self.send_positions = _compile(programs.moe_route_positions, target=target, constexprs=rank_constexprs)
        self.gather = _compile(programs.moe_gather_rows, target=target,
                               constexprs={"ACT_DTYPE": act_dtype, "TOP_K": top_k})
        self.local = MoEW4A16FFN(tokens=self.capacity, hidden=hidden, intermediate=intermediate,
                                 experts=self.local_experts, top_k=1, group_size=group_size,
                                 zero_point=zero_point, act_dtype=act_dtype, block_size=block_size, target=target)
        self.combine = _compile(programs.moe_combine, target=target)
        self._overflow = None
        self._torch = torch

    def check_overflow(self) -> None:
        """Capacity mode: raise if any step since the last check had more routes for one rank than
        fit its slot (reads one device word)."""
        if self._overflow is not None and bool(self._overflow.item()):
            self._overflow.zero_()
            raise RuntimeError("expert-parallel exchange overflowed its capacity; raise capacity_factor")

    def _send_experts(self, ids, sorted_routes, rows):
        """Local expert id of every sent row; rows that are padding get an id no expert matches."""
        torch = self._torch
        index = sorted_routes[:rows].long()
        valid = index < self.routes
        chosen = ids.flatten()[index.clamp(max=self.routes - 1)] % self.local_experts
        return torch.where(valid, chosen, torch.full_like(chosen, self.local_experts)).to(torch.int32)

    def forward(self, logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales):
        """logits [T, E] f32 and x [T, H] of this rank's tokens; weights of this rank's experts.
        Returns y [T, H] f32."""
        torch = self._torch
        ids, weights = self.router.run(logits)
        destination = torch.div(ids, self.local_experts, rounding_mode="floor").to(torch.int32)
        call = self.by_rank.prepare(destination)
        call.launch()                                                     # routes grouped by destination rank
        sorted_routes, _, total = call.result()
        if self.capacity_factor is None:
            plan = exchange_counts(call.counts, self.group)               # the one host read of the step
            n_send, n = self.routes, plan.received_rows
            if n > self.capacity:
                raise RuntimeError(f"received {n} rows, capacity is {self.capacity}")
        else:
            plan = ExchangePlan([self.slot_rows] * self.world, [self.slot_rows] * self.world)
            n_send = n = self.capacity
            over = (total != self.capacity).to(torch.int32)
            self._overflow = over if self._overflow is None else torch.maximum(self._overflow, over)
        send_rows = self.gather.run(x, sorted_routes, total)[:n_send]
        send_experts = self._send_experts(ids, sorted_routes, n_send)
        received = dispatch_rows(send_rows, plan, self.group)
        received_experts = dispatch_rows(send_experts.unsqueeze(1), plan, self.group)
        results = torch.zeros((n, self.hidden), dtype=torch.float32, device=x.device)
        if n:
            rows, positions = self.local.experts_forward(received, received_experts.contiguous(), up_gate_packed,
                                                         up_gate_scales, down_packed, down_scales,
                                                         clear_positions=self.capacity_factor is not None)
            ones = torch.ones((n, 1), dtype=torch.float32, device=x.device)
            self.combine.run(rows, positions[:n], ones, results)            # back to arrival order
        returned = return_rows(results, plan, self.group)                   # [rows sent, H] in send order
        send_position = self.send_positions.run(sorted_routes, total)       # route -> slot in send order
        y = torch.zeros((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
        self.combine.run(returned, send_position, weights, y)
        return y

    __call__ = forward

    def prepare(self, logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales):
        """Capacity mode only: bind the whole step to fixed buffers (all shapes are static), so that
        ``launch()`` is a short sequence of pre-bound kernel launches and collectives on those
        buffers.  Returns an object whose ``launch()`` yields y [T, H] f32 (same bits as forward)."""
        if self.capacity_factor is None:
            raise NotImplementedError("prepare() needs the fixed-capacity exchange (capacity_factor=...)")
        return PreparedExpertParallel(self, logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales)


class PreparedExpertParallel:
    def __init__(self, ep: ExpertParallelMoE, logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales):
        import torch

        self.ep = ep
        n, device = ep.capacity, x.device
        self.router = ep.router.prepare(logits)
        self.ids, self.weights = self.router.result()
        self.destination = torch.empty_like(self.ids)
        self.by_rank = ep.by_rank.prepare(self.destination)
        self.sorted_routes, _, self.total = self.by_rank.result()
        self.gather = ep.gather.prepare(x, self.sorted_routes, self.total)
        self.send_rows = self.gather.result()[:n]
        self.received = torch.empty((n, ep.hidden), dtype=x.dtype, device=device)
        self.received_experts = torch.empty((n, 1), dtype=torch.int32, device=device)
        self.results = torch.zeros((n, ep.hidden), dtype=torch.float32, device=device)
        self.local = ep.local.prepare(self.received, self.received_experts,
                                      torch.ones((n, 1), dtype=torch.float32, device=device), up_gate_packed,
                                      up_gate_scales, down_packed, down_scales, self.results, clear_positions=True)
        self.returned = torch.empty((n, ep.hidden), dtype=torch.float32, device=device)
        self.send_position = ep.send_positions.prepare(self.sorted_routes, self.total)
        self.y = torch.zeros((x.shape[0], ep.hidden), dtype=torch.float32, device=device)
        self.combine = ep.combine.prepare(self.returned, self.send_position.result(), self.weights, self.y)
        self.splits = [ep.slot_rows] * ep.world

    def launch(self):
        import torch
        import torch.distributed as dist

        ep = self.ep
        self.router.launch()
        torch.div(self.ids, ep.local_experts, rounding_mode="floor", out=self.destination)
        self.by_rank.launch()
        over = (self.total != ep.capacity).to(torch.int32)
        ep._overflow = over if ep._overflow is None else torch.maximum(ep._overflow, over)
        self.gather.launch()
        send_experts = ep._send_experts(self.ids, self.sorted_routes, ep.capacity).unsqueeze(1)
        dist.all_to_all_single(self.received, self.send_rows, self.splits, self.splits, group=ep.group)
        dist.all_to_all_single(self.received_experts, send_experts, self.splits, self.splits, group=ep.group)
        self.local.launch()                      # zeroes `results`, then un-permutes the expert rows into it
        dist.all_to_all_single(self.returned, self.results, self.splits, self.splits, group=ep.group)
        self.send_position.launch()
        self.y.zero_()
        self.combine.launch()
        return self.y
