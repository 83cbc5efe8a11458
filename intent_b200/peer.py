"""Expert-parallel MoE over peer memory: no collective on the data path.

Every rank writes the token rows of its routes straight into the expert-sorted row buffer
of the rank that owns the expert (NVLink stores), the owners run the grouped int4 FFN on
rows that are already in place, and every rank then reads the finished f32 rows straight
out of the owners' result buffers while it combines them (NVLink loads).  Only real rows
cross the links: there are no padded spans, no staging copy and no second gather.  The
ranks meet at three sync points per step (counts exchanged, rows written, results written):
flag posts and bounded flag waits over peer memory (``PeerSignals``), so the step holds no
collective call, or - ``signals='nccl'`` - an all-gather and two one-word all-reduces.

The owner's layout (experts in local order, spans padded to the tile rows, source rank 0
first inside a span) equals the single-GPU stable alignment over all tokens when the
tokens are split contiguously over the ranks, so the result is bit-identical to one GPU.

``PeerExchangeRank`` is one rank's side with the cross-rank steps left to the caller; the
tests drive several of them on one GPU in sequence (the ranks' buffers are then plain
local tensors).  ``PeerExpertParallelMoE`` binds it to ``torch.distributed``: the buffers
live in symmetric memory so every rank can address every other rank's copy.
"""
from __future__ import annotations

from . import programs
from .compiler import compile as _compile


class PeerExchangeRank:
    def __init__(self, *, rank, world, tokens, hidden, intermediate, experts, top_k=2, group_size=128,
                 zero_point=8, act_dtype="bf16", block_rows=128, target=None):
        if experts % world:
            raise ValueError("the expert count must be a multiple of the number of ranks")
        if block_rows not in (128, 256):
            raise ValueError("block_rows must be 128 or 256")
        self.rank, self.world = rank, world
        self.tokens, self.hidden, self.intermediate = tokens, hidden, intermediate
        self.experts, self.local_experts, self.top_k = experts, experts // world, top_k
        self.routes = tokens * top_k
        self.block_rows = block_rows
        self.act_dtype = act_dtype
        # worst case: every route of every rank goes to this rank's experts
        self.capacity_rows = world * self.routes + self.local_experts * (block_rows - 1)
        send = {"TOKENS": tokens, "TOP_K": top_k, "EXPERTS": experts, "BLOCK_SIZE": 1}
        quant = {"GROUP_SIZE": group_size, "ZERO_POINT": zero_point, "ACT_DTYPE": act_dtype,
                 "BLOCK_ROWS": block_rows}
        self.router = _compile(programs.moe_route_top2, target=target)
        self.count = _compile(programs.moe_count_routes, target=target, constexprs=send)
        self.prefix = _compile(programs.moe_prefix_routes, target=target, constexprs=send)
        self.scatter = _compile(programs.moe_scatter_routes, target=target, constexprs=send)
        self.layout = _compile(programs.moe_peer_layout, target=target,
                               constexprs={"WORLD": world, "EXPERTS": experts, "RANK": rank,
                                           "BLOCK_ROWS": block_rows, "CAPACITY_ROWS": self.capacity_rows})
        self.dispatch = _compile(programs.moe_peer_dispatch, target=target,
                                 constexprs={"ACT_DTYPE": act_dtype, "TOP_K": top_k,
                                             "CAPACITY_ROWS": self.capacity_rows})
        self.up_gate = _compile(programs.moe_grouped_upgate_silu, target=target, constexprs=quant)
        self.down = _compile(programs.moe_grouped_down, target=target, constexprs=quant)
        self.combine = _compile(programs.moe_peer_combine, target=target,
                                constexprs={"CAPACITY_ROWS": self.capacity_rows, "ACCUMULATE": False})
        self.combine_add = _compile(programs.moe_peer_combine, target=target,
                                    constexprs={"CAPACITY_ROWS": self.capacity_rows, "ACCUMULATE": True})

    def buffer_shapes(self):
        """(shape, torch dtype) of the row buffer and of the f32 result buffer every rank exposes."""
        import torch

        rows = torch.bfloat16 if self.act_dtype == "bf16" else torch.float16
        return ((self.capacity_rows, self.hidden), rows), ((self.capacity_rows, self.hidden), torch.float32)

    def prepare(self, logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales, y, *, rows, out,
                peer_rows, peer_out, counts_all):
        """Bind one step to fixed buffers.  ``rows`` / ``out``: this rank's buffers; ``peer_rows`` /
        ``peer_out``: int64 [world] device tensors with every rank's buffer address as seen from
        this device; ``counts_all``: int32 [world, experts] device tensor the caller fills between
        ``route()`` and ``dispatch_rows()`` (this rank's own row is ``step.counts``)."""
        return PeerStep(self, logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales, y, rows, out,
                        peer_rows, peer_out, counts_all)


class PeerStep:
    """The four phases of one bound step; the caller puts the cross-rank steps between them:

        route()          -> exchange ``counts`` into ``counts_all``
        dispatch_rows()  -> barrier (all rows are in their owners' buffers)
        experts()        -> barrier (all result rows are written)
        combine()
    """

    def __init__(self, ep, logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales, y, rows, out,
                 peer_rows, peer_out, counts_all):
        import torch

        device = x.device
        self.ep, self.y = ep, y
        self._counters = torch.zeros((2 * ep.experts,), dtype=torch.int32, device=device)  # cleared together
        self.counts, self.cursors = self._counters[:ep.experts], self._counters[ep.experts:]
        self.sorted_routes = torch.empty((ep.routes,), dtype=torch.int32, device=device)
        self._router = ep.router.prepare(logits)
        self.ids, self.weights = self._router.result()
        self._count = ep.count.prepare(self.ids, self.counts)
        self._prefix = ep.prefix.prepare(self.counts)
        self.send_offsets, _ = self._prefix.result()
        self._scatter = ep.scatter.prepare(self.ids, self.send_offsets, self.cursors, self.sorted_routes)
        self._layout = ep.layout.prepare(counts_all)
        self.dest_base, self.local_offsets, self.total, self.expert_blocks = self._layout.result()
        self._dispatch = ep.dispatch.prepare(x, self.sorted_routes, self.send_offsets, self.dest_base, peer_rows)
        self.route_dest = self._dispatch.result()
        self._up = ep.up_gate.prepare(rows, self.expert_blocks, self.total, up_gate_packed, up_gate_scales)
        self._down = ep.down.prepare(self._up.result(), self.expert_blocks, self.total, down_packed, down_scales,
                                     outputs=(out,))
        self._combine = ep.combine.prepare(peer_out, self.route_dest, self.weights, y)
        self._combine_add = ep.combine_add.prepare(peer_out, self.route_dest, self.weights, y)

    def route(self):
        self._counters.zero_()
        self._router.launch()
        self._count.launch()
        self._prefix.launch()
        self._scatter.launch()

    def dispatch_rows(self):
        self._layout.launch()
        self._dispatch.launch()

    def experts(self):
        self._up.launch()
        self._down.launch()

    def combine(self, accumulate=False):
        (self._combine_add if accumulate else self._combine).launch()


class PeerSignals:
    """One rank's sync points over peer memory: ``flags`` [3, world] is this rank's flag array,
    ``peer_flags`` the int64 table of every rank's array, ``peer_tables`` the table of every rank's count
    matrix.  Channel 0 carries the per-expert counts, channels 1 and 2 are plain barriers.  The waits are
    bounded (``max_polls`` polls about a microsecond apart: the default rides out a rank that is still loading
    its kernels, roughly 20 s); ``status`` holds a timeout code if one gave up.

    The sequence counters must live exactly as long as the flag arrays they are compared with: flags keep the
    numbers of every earlier step, so counters that restart at zero would be behind the flags and every wait
    would pass without waiting.  Whoever owns the flag arrays therefore owns one ``sequence`` (and ``status``)
    tensor and hands the same one to every ``PeerSignals`` built on those flags; a ``PeerSignals`` only binds a
    step's payload (its per-expert counts) to them."""

    CHANNELS = 3

    @classmethod
    def counters(cls, device):
        """(sequence, status) for one flag array: zero exactly when the flags are zero."""
        import torch

        return (torch.zeros((2 * cls.CHANNELS,), dtype=torch.int32, device=device),
                torch.zeros((1,), dtype=torch.int32, device=device))

    def __init__(self, *, rank, world, flags, peer_flags, peer_tables, counts, target=None, max_polls=1 << 24,
                 sequence=None, status=None):
        import torch

        device = flags.device
        if (sequence is None) != (status is None):
            raise ValueError("pass both sequence and status (PeerSignals.counters) or neither")
        if sequence is None:      # a flag array used by this object alone (it must still be all zero)
            sequence, status = self.counters(device)
        self.flags, self.status, self.sequence = flags, status, sequence
        none = torch.empty((0,), dtype=torch.int64, device=device)
        self.posts, self.waits = [], []
        for channel in range(self.CHANNELS):
            post = _compile(programs.moe_peer_post, target=target,
                            constexprs={"RANK": rank, "CHANNEL": channel, "PAYLOAD": channel == 0})
            wait = _compile(programs.moe_peer_wait, target=target,
                            constexprs={"CHANNEL": channel, "MAX_POLLS": max_polls})
            self.posts.append(post.prepare(peer_flags, self.sequence, peer_tables if channel == 0 else none, counts))
            self.waits.append(wait.prepare(flags, self.sequence, self.status))

    def post(self, channel):
        self.posts[channel].launch()

    def wait(self, channel):
        self.waits[channel].launch()

    def check(self):
        """Raise if a wait has given up since the last check (reads one device word)."""
        code = int(self.status.item())
        if code:
            self.status.zero_()
            raise RuntimeError(f"a cross-rank wait expired (status {code}): a rank did not reach the sync point")


class PeerExpertParallelMoE:
    """``PeerExchangeRank`` bound to a process group: symmetric-memory buffers and three sync points per
    step (the first one carries the per-expert route counts), all on the current stream.
    ``signals='peer'``: the sync points are flag writes and bounded flag waits over peer memory;
    ``signals='nccl'``: an all-gather and two one-word all-reduces."""

    def __init__(self, *, tokens, hidden, intermediate, experts, top_k=2, group_size=128, zero_point=8,
                 act_dtype="bf16", block_rows=128, target=None, group=None, signals="peer", max_polls=1 << 24):
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symmetric

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.side = PeerExchangeRank(rank=self.rank, world=self.world, tokens=tokens, hidden=hidden,
                                     intermediate=intermediate, experts=experts, top_k=top_k,
                                     group_size=group_size, zero_point=zero_point, act_dtype=act_dtype,
                                     block_rows=block_rows, target=target)
        device = torch.device("cuda", target.device if target is not None else torch.cuda.current_device())
        (rows_shape, rows_dtype), (out_shape, out_dtype) = self.side.buffer_shapes()
        self.rows = symmetric.empty(rows_shape, dtype=rows_dtype, device=device)
        self.out = symmetric.empty(out_shape, dtype=out_dtype, device=device)
        self.rows.zero_()
        rows_handle = symmetric.rendezvous(self.rows, self.group)
        out_handle = symmetric.rendezvous(self.out, self.group)
        # keep the peer views alive: their storage is the mapping of the peer's buffer
        self._peer_rows = [rows_handle.get_buffer(r, rows_shape, rows_dtype) for r in range(self.world)]
        self._peer_out = [out_handle.get_buffer(r, out_shape, out_dtype) for r in range(self.world)]
        self.peer_rows = torch.tensor([t.data_ptr() for t in self._peer_rows], dtype=torch.int64, device=device)
        self.peer_out = torch.tensor([t.data_ptr() for t in self._peer_out], dtype=torch.int64, device=device)
        if signals not in ("peer", "nccl"):
            raise ValueError("signals must be 'peer' or 'nccl'")
        self.signals = signals
        self._token = torch.zeros((1,), dtype=torch.int32, device=device)
        self._dist = dist
        self._target = target
        if signals == "nccl":
            self.counts_all = torch.zeros((self.world, experts), dtype=torch.int32, device=device)
        else:
            self.counts_all = symmetric.empty((self.world, experts), dtype=torch.int32, device=device)
            self.flags = symmetric.empty((PeerSignals.CHANNELS, self.world), dtype=torch.int32, device=device)
            self.counts_all.zero_()
            self.flags.zero_()
            counts_handle = symmetric.rendezvous(self.counts_all, self.group)
            flags_handle = symmetric.rendezvous(self.flags, self.group)
            self._peer_counts = [counts_handle.get_buffer(r, tuple(self.counts_all.shape), torch.int32)
                                 for r in range(self.world)]
            self._peer_flags = [flags_handle.get_buffer(r, tuple(self.flags.shape), torch.int32)
                                for r in range(self.world)]
            self.peer_counts = torch.tensor([t.data_ptr() for t in self._peer_counts], dtype=torch.int64,
                                            device=device)
            self.peer_flags = torch.tensor([t.data_ptr() for t in self._peer_flags], dtype=torch.int64,
                                           device=device)
            # one pair of counters for the life of the flag arrays: every prepared step continues the same
            # sequence, so a second prepare() (or every __call__) still waits for the other ranks
            self._sequence, self._status = PeerSignals.counters(device)
            self._max_polls = max_polls
        # every rank's buffers are cleared before any rank may write into them
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)

    def barrier(self):
        self._dist.all_reduce(self._token, group=self.group)

    def prepare(self, logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales, y=None):
        import torch

        if y is None:
            y = torch.empty((x.shape[0], self.side.hidden), dtype=torch.float32, device=x.device)
        step = self.side.prepare(logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales, y,
                                 rows=self.rows, out=self.out, peer_rows=self.peer_rows, peer_out=self.peer_out,
                                 counts_all=self.counts_all)
        signals = None
        if self.signals == "peer":
            signals = PeerSignals(rank=self.rank, world=self.world, flags=self.flags, peer_flags=self.peer_flags,
                                  peer_tables=self.peer_counts, counts=step.counts, target=self._target,
                                  max_polls=self._max_polls, sequence=self._sequence, status=self._status)
        return PreparedPeerStep(self, step, signals)

    def __call__(self, logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales):
        call = self.prepare(logits, x, up_gate_packed, up_gate_scales, down_packed, down_scales)
        call.launch()
        return call.y


class PreparedPeerStep:
    def __init__(self, ep: PeerExpertParallelMoE, step: PeerStep, signals: PeerSignals | None = None):
        self.ep, self.step, self.y, self.signals = ep, step, step.y, signals

    def _sync(self, channel):
        if self.signals is not None:
            self.signals.post(channel)
            self.signals.wait(channel)
        elif channel == 0:
            self.ep._dist.all_gather_into_tensor(self.ep.counts_all.view(-1), self.step.counts, group=self.ep.group)
        else:
            self.ep.barrier()

    PHASES = ("route", "sync_counts", "dispatch", "sync_rows", "up_gate", "down", "sync_results", "combine")

    def launch(self, accumulate=False, marks=None):
        """``marks``: an empty list that receives one timing event before the first phase and one after each
        phase of :attr:`PHASES` (for per-phase device times; leave it None otherwise)."""
        step = self.step

        def mark():
            if marks is not None:
                import torch

                event = torch.cuda.Event(enable_timing=True)
                event.record()
                marks.append(event)

        mark()
        step.route()
        mark()
        self._sync(0)         # every rank's per-expert counts are in every rank's count matrix
        mark()
        step.dispatch_rows()
        mark()
        self._sync(1)         # every row of this step is in its owner's buffer
        mark()
        step._up.launch()
        mark()
        step._down.launch()
        mark()
        self._sync(2)         # every result row is written; also fences the row buffers for the next step
        mark()
        step.combine(accumulate)
        mark()

    def check(self):
        if self.signals is not None:
            self.signals.check()
