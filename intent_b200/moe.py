"""Host-side compositions of the MoE programs.

``MoEAlignment`` mirrors the reference's multi-kernel host program
(examples/programs/composition.py:98-174): the same four artifacts, the same
workspace reset, the same ``run`` / ``run_into`` / ``prepare`` results
``(sorted_route_ids, expert_blocks, total_padded)``.

``MoEW4A16FFN`` chains router -> alignment -> row gather -> grouped up|gate
projection with the SiLU gate -> grouped down projection -> weighted combine, the
benchmark's MoE configuration (the reference's dense-weight counterpart is
examples/kernels/ragged/moe.py:12-53).  Everything runs on the current stream;
no step reads a device value back to the host.
"""
from __future__ import annotations

from dataclasses import dataclass

from . import programs
from .compiler import compile as _compile
from .targets import B200Target


_ALIGN_STAGES = ("moe_count_routes", "moe_prefix_routes", "moe_scatter_routes", "moe_mark_expert_blocks")


class MoEAlignmentCall:
    """The four alignment launches bound to fixed buffers.  ``launch()`` clears the per-expert counters,
    refills the route list with the padding sentinel and replays the launches; ``result()`` is
    ``(sorted_route_ids, expert_blocks, total_padded)`` like the unbound forms."""

    def __init__(self, stages, counters, sorted_routes, expert_blocks, total_padded, sentinel):
        self.stages = tuple(stages)
        self._counters = counters                      # counts | cursors in one buffer: one clear per launch
        half = counters.numel() // 2
        self.counts, self.cursors = counters[:half], counters[half:]
        self.sorted_routes, self.expert_blocks, self.total_padded = sorted_routes, expert_blocks, total_padded
        self.routes = sentinel

    def compile(self):
        for stage in self.stages:
            stage.compile()

    def launch(self):
        self._counters.zero_()
        self.sorted_routes.fill_(self.routes)
        for stage in self.stages:
            stage.launch()

    def result(self):
        return self.sorted_routes, self.expert_blocks, self.total_padded


class MoEAlignment:
    """Host composition of the route alignment, with the reference's surface
    (examples/programs/composition.py:98-174: ``build`` / ``run`` / ``run_into`` / ``prepare``, results
    ``(sorted_route_ids, expert_blocks, total_padded)``, padding sentinel = number of routes).  The stages
    are the four alignment programs compiled with this object's token / top-k / expert / block constants
    (the reference fixes them at module level; here they are constructor arguments)."""

    def __init__(self, count, prefix, scatter, mark, tokens=4096, top_k=2, experts=64, block_size=128):
        self.count, self.prefix, self.scatter, self.mark = count, prefix, scatter, mark
        self.tokens, self.top_k, self.experts, self.block_size = tokens, top_k, experts, block_size

    @classmethod
    def build(cls, *, tokens=4096, top_k=2, experts=64, block_size=128, target=None, resolve_target=True):
        constants = {"TOKENS": tokens, "TOP_K": top_k, "EXPERTS": experts, "BLOCK_SIZE": block_size}
        stages = [_compile(getattr(programs, name), target=target, constexprs=constants,
                           resolve_target=resolve_target) for name in _ALIGN_STAGES]
        return cls(*stages, tokens=tokens, top_k=top_k, experts=experts, block_size=block_size)

    @property
    def routes(self) -> int:
        return self.tokens * self.top_k

    @property
    def padded_routes(self) -> int:
        # every expert span may need up to block_size - 1 padding entries
        return self.routes + self.experts * (self.block_size - 1)

    def _check(self, ids):
        if ids.dim() != 2 or ids.shape[1] != self.top_k or ids.shape[0] > self.tokens:
            raise ValueError(f"MoEAlignment requires at most {self.tokens} tokens with top-k {self.top_k}")

    def _buffers(self, device):
        import torch

        counters = torch.empty((2 * self.experts,), dtype=torch.int32, device=device)
        return counters, torch.empty((self.padded_routes,), dtype=torch.int32, device=device)

    def run_into(self, ids, counts, cursors, sorted_routes):
        """Alignment into caller-owned ``counts`` / ``cursors`` [experts] and ``sorted_routes``
        [padded_routes]; all three are reset first."""
        self._check(ids)
        for buffer, value in ((counts, 0), (cursors, 0), (sorted_routes, self.routes)):
            buffer.fill_(value)
        self.count.run(ids, counts)
        offsets, total_padded = self.prefix.run(counts)
        self.scatter.run(ids, offsets, cursors, sorted_routes)
        return sorted_routes, self.mark.run(offsets), total_padded

    def run(self, ids):
        counters, sorted_routes = self._buffers(ids.device)
        return self.run_into(ids, counters[:self.experts], counters[self.experts:], sorted_routes)

    def prepare(self, ids):
        self._check(ids)
        counters, sorted_routes = self._buffers(ids.device)
        counts, cursors = counters[:self.experts], counters[self.experts:]
        count = self.count.prepare(ids, counts)
        prefix = self.prefix.prepare(counts)
        offsets, total_padded = prefix.result()
        scatter = self.scatter.prepare(ids, offsets, cursors, sorted_routes)
        mark = self.mark.prepare(offsets)
        return MoEAlignmentCall((count, prefix, scatter, mark), counters, sorted_routes, mark.result(),
                                total_padded, self.routes)


class MoEW4A16FFN:
    """SiLU-gated MoE FFN with int4 group-quantised expert weights on one GPU.

    ``experts`` is the number of experts held on this GPU; ``tokens`` the number of
    token rows it routes per call (after any expert-parallel exchange this is the
    number of received rows with ``top_k = 1``)."""

    def __init__(self, *, tokens, hidden, intermediate, experts, top_k=2, group_size=128, zero_point=8,
                 act_dtype="bf16", block_size=128, target: B200Target | None = None, prelayout: bool = False):
        """``prelayout``: the expert weights are static model state; the grouped contractions then run on tiled
        copies (intent_b200.prelayout) that are made the first time a weight tensor is seen."""
        self.tokens, self.hidden, self.intermediate = tokens, hidden, intermediate
        self.experts, self.top_k = experts, top_k
        self.alignment = MoEAlignment.build(tokens=tokens, top_k=top_k, experts=experts, block_size=block_size,
                                            target=target)
        align = {"TOKENS": tokens, "TOP_K": top_k, "EXPERTS": experts, "BLOCK_SIZE": block_size}
        if block_size not in (128, 256):
            raise ValueError("block_size must be 128 or 256 (rows of one tile of the grouped contraction)")
        quant = {"GROUP_SIZE": group_size, "ZERO_POINT": zero_point, "ACT_DTYPE": act_dtype}
        self.router = _compile(programs.moe_route_top2, target=target)
        self.positions = _compile(programs.moe_route_positions, target=target, constexprs=align)
        self.gather = _compile(programs.moe_gather_rows, target=target,
                               constexprs={"ACT_DTYPE": act_dtype, "TOP_K": top_k})
        grouped = dict(quant, BLOCK_ROWS=block_size, WEIGHT_LAYOUT="tiled" if prelayout else "reference")
        self.prelayout = None
        if prelayout:
            from .prelayout import PrelayoutCache

            self.prelayout = PrelayoutCache()
        self.up_gate = _compile(programs.moe_grouped_upgate_silu, target=target, constexprs=grouped)
        self.down = _compile(programs.moe_grouped_down, target=target, constexprs=grouped)
        self.combine = _compile(programs.moe_combine, target=target)
        self.combine_overwrite = _compile(programs.moe_combine, target=target, constexprs={"ACCUMULATE": False})
        # With at most two choices per token the weighted combine runs in the down projection's epilogue
        # (relaxed vector atomics on y): on a zeroed y two additions commute exactly, so the result has the same
        # bits as the ordered combine.  More choices keep the ordered combine kernel.
        self.fused_combine = top_k <= 2
        self.down_scatter = _compile(programs.moe_grouped_down_scatter, target=target, constexprs=grouped)

    def route(self, logits):
        """logits [T, E_total] f32 -> (ids [T,2] i32, weights [T,2] f32)."""
        return self.router.run(logits)

    def _weights(self, up_gate_packed, down_packed):
        """The packed expert weights as the grouped programs take them (tiled copies with ``prelayout``)."""
        if self.prelayout is None:
            return up_gate_packed, down_packed
        return self.prelayout.get(up_gate_packed).tensor, self.prelayout.get(down_packed).tensor

    def experts_forward(self, x, topk_ids, up_gate_packed, up_gate_scales, down_packed, down_scales,
                        clear_positions=False):
        """Rows of the down projection in the expert-sorted layout plus the inverse map:
        returns (rows f32 [P, H], route_positions i32 [T*top_k]).  ``clear_positions``: routes whose
        expert id matches no local expert (padding of a fixed-capacity exchange) get position 0."""
        up_gate_packed, down_packed = self._weights(up_gate_packed, down_packed)
        sorted_routes, expert_blocks, total = self.alignment.run(topk_ids)
        if clear_positions:
            import torch

            positions = torch.zeros((self.tokens * self.top_k,), dtype=torch.int32, device=x.device)
            self.positions(sorted_routes, total, positions)
        else:
            positions = self.positions.run(sorted_routes, total)
        rows = self.gather.run(x, sorted_routes, total)
        hidden = self.up_gate.run(rows, expert_blocks, total, up_gate_packed, up_gate_scales)
        out = self.down.run(hidden, expert_blocks, total, down_packed, down_scales)
        return out, positions

    def forward(self, x, topk_ids, topk_weights, up_gate_packed, up_gate_scales, down_packed, down_scales, y=None):
        """y[t] (+)= sum_c topk_weights[t, c] * FFN_{topk_ids[t, c]}(x[t]); y f32 [T, H]."""
        import torch

        if y is None:
            y = torch.zeros((x.shape[0], self.hidden), dtype=torch.float32, device=x.device)
        if self.fused_combine:
            up_gate_packed, down_packed = self._weights(up_gate_packed, down_packed)
            sorted_routes, expert_blocks, total = self.alignment.run(topk_ids)
            rows = self.gather.run(x, sorted_routes, total)
            hidden = self.up_gate.run(rows, expert_blocks, total, up_gate_packed, up_gate_scales)
            self.down_scatter(hidden, expert_blocks, total, down_packed, down_scales, sorted_routes, topk_weights, y)
            return y
        rows, positions = self.experts_forward(x, topk_ids, up_gate_packed, up_gate_scales, down_packed,
                                               down_scales)
        self.combine.run(rows, positions, topk_weights, y)
        return y

    __call__ = forward

    def prepare(self, x, topk_ids, topk_weights, up_gate_packed, up_gate_scales, down_packed, down_scales, y,
                clear_positions=False):
        """Bind the whole chain to fixed buffers once; ``launch()`` then replays it without any
        per-call validation or allocation (same results as :meth:`forward`).  Every launch overwrites
        ``y`` unless ``launch(accumulate=True)``."""
        import torch

        up_gate_packed, down_packed = self._weights(up_gate_packed, down_packed)
        align = self.alignment.prepare(topk_ids)
        sorted_routes, expert_blocks, total = align.result()
        if self.fused_combine and not clear_positions:
            gather_call = self.gather.prepare(x, sorted_routes, total)
            up_call = self.up_gate.prepare(gather_call.result(), expert_blocks, total, up_gate_packed, up_gate_scales)
            scatter_call = self.down_scatter.prepare(up_call.result(), expert_blocks, total, down_packed, down_scales,
                                                     sorted_routes, topk_weights, y)
            return PreparedFusedFFN(align, gather_call, up_call, scatter_call, y)
        positions = torch.zeros((topk_ids.shape[0] * self.top_k,), dtype=torch.int32, device=x.device)
        full_positions = torch.zeros((self.tokens * self.top_k,), dtype=torch.int32, device=x.device)
        position_call = self.positions.prepare(sorted_routes, total, outputs=(full_positions,))
        positions = full_positions[: topk_ids.shape[0] * self.top_k]
        gather_call = self.gather.prepare(x, sorted_routes, total)
        up_call = self.up_gate.prepare(gather_call.result(), expert_blocks, total, up_gate_packed, up_gate_scales)
        down_call = self.down.prepare(up_call.result(), expert_blocks, total, down_packed, down_scales)
        combine_call = self.combine.prepare(down_call.result(), positions, topk_weights, y)
        overwrite_call = self.combine_overwrite.prepare(down_call.result(), positions, topk_weights, y)
        return PreparedFFN(align, position_call, gather_call, up_call, down_call, combine_call, overwrite_call,
                           full_positions, y, clear_positions)


_SIDE_STREAMS: dict = {}


def _side_stream(device):
    """One extra stream per device for work that may overlap a contraction (created on first use)."""
    import torch

    key = torch.device(device).index
    if key not in _SIDE_STREAMS:
        _SIDE_STREAMS[key] = torch.cuda.Stream(device)
    return _SIDE_STREAMS[key]


@dataclass
class PreparedFusedFFN:
    """The chain with the weighted combine inside the down projection's epilogue (top_k <= 2)."""

    align: object
    gather_call: object
    up_call: object
    scatter_call: object
    y: object

    PHASES = ("align", "gather", "up_gate", "down_combine")

    def launch(self, accumulate: bool = False, marks=None):
        """Overwrites ``y`` (it is cleared first) unless ``accumulate``; ``marks`` as in :class:`PreparedFFN`."""
        def mark():
            if marks is not None:
                import torch

                event = torch.cuda.Event(enable_timing=True)
                event.record()
                marks.append(event)

        import torch

        side = None
        if not accumulate:
            # y is cleared on a second stream while the alignment, the gather and the up|gate contraction run:
            # the fill is bound by HBM writes, the contraction by the tensor pipe (works inside a stream capture)
            current = torch.cuda.current_stream(self.y.device)
            side = _side_stream(self.y.device)
            side.wait_stream(current)
            with torch.cuda.stream(side):
                self.y.zero_()
        mark()
        self.align.launch()
        mark()
        self.gather_call.launch()
        mark()
        self.up_call.launch()
        if side is not None:
            current.wait_stream(side)
        mark()
        self.scatter_call.launch()
        mark()
        return self.y


@dataclass
class PreparedFFN:
    align: object
    position_call: object
    gather_call: object
    up_call: object
    down_call: object
    combine_call: object
    overwrite_call: object
    positions: object
    y: object
    clear_positions: bool

    PHASES = ("align", "gather", "up_gate", "down", "combine")

    def launch(self, accumulate: bool = False, marks=None):
        """``marks``: an empty list that receives one timing event before the first phase and one after each
        phase of :attr:`PHASES` (for per-phase device times; leave it None otherwise)."""
        def mark():
            if marks is not None:
                import torch

                event = torch.cuda.Event(enable_timing=True)
                event.record()
                marks.append(event)

        mark()
        self.align.launch()
        if self.clear_positions:
            self.positions.zero_()
        self.position_call.launch()
        mark()
        self.gather_call.launch()
        mark()
        self.up_call.launch()
        mark()
        self.down_call.launch()
        mark()
        (self.combine_call if accumulate else self.overwrite_call).launch()   # overwrite: y is not read or cleared
        mark()
        return self.y


class HostPipelinedFFN:
    """The MoE FFN for inputs and results that live in (pinned) host memory: the tokens are cut into ``chunks``
    pieces and, for every piece, the upload of its rows and logits, the routed FFN and the download of its f32
    result run on three streams, so that the copies of neighbouring pieces overlap the contractions.  Tokens are
    independent of one another in this FFN (every row meets its experts' weights alone), so every piece gives the
    bits the whole batch gives.

    ``run(logits, x, out)`` takes host tensors ``logits [T, E] f32``, ``x [T, H]`` and ``out [T, H] f32`` (pinned
    for the copies to be asynchronous) and returns after the last piece has arrived in ``out``."""

    def __init__(self, *, tokens, hidden, intermediate, experts, chunks=4, top_k=2, group_size=128, zero_point=8,
                 act_dtype="bf16", block_size=128, target: B200Target | None = None):
        import torch

        if chunks < 1 or tokens % chunks:
            raise ValueError("the token count must be a multiple of the number of pieces")
        self.tokens, self.chunks, self.piece = tokens, chunks, tokens // chunks
        self.hidden, self.experts = hidden, experts
        self.ffn = MoEW4A16FFN(tokens=self.piece, hidden=hidden, intermediate=intermediate, experts=experts,
                               top_k=top_k, group_size=group_size, zero_point=zero_point, act_dtype=act_dtype,
                               block_size=block_size, target=target)
        self.device = torch.device("cuda", (target or B200Target()).device)
        self._rows = torch.bfloat16 if act_dtype == "bf16" else torch.float16
        self._bound = None

    def bind(self, up_gate_packed, up_gate_scales, down_packed, down_scales):
        """Bind the expert weights and allocate the pieces' device buffers (once)."""
        import torch

        pieces = []
        for _ in range(self.chunks):
            logits = torch.empty((self.piece, self.experts), dtype=torch.float32, device=self.device)
            x = torch.empty((self.piece, self.hidden), dtype=self._rows, device=self.device)
            y = torch.empty((self.piece, self.hidden), dtype=torch.float32, device=self.device)
            router = self.ffn.router.prepare(logits)
            ids, weights = router.result()
            chain = self.ffn.prepare(x, ids, weights, up_gate_packed, up_gate_scales, down_packed, down_scales, y)
            pieces.append({"logits": logits, "x": x, "y": y, "router": router, "chain": chain,
                           "uploaded": torch.cuda.Event(), "computed": torch.cuda.Event(),
                           "downloaded": torch.cuda.Event(), "used": False})
        self._bound = pieces
        self._upload, self._download = torch.cuda.Stream(self.device), torch.cuda.Stream(self.device)
        return self

    def run(self, logits, x, out):
        import torch

        if self._bound is None:
            raise RuntimeError("bind() the expert weights first")
        if logits.shape[0] != self.tokens or x.shape[0] != self.tokens or out.shape[0] != self.tokens:
            raise ValueError(f"expected {self.tokens} token rows")
        compute = torch.cuda.current_stream(self.device)
        for index, piece in enumerate(self._bound):
            rows = slice(index * self.piece, (index + 1) * self.piece)
            with torch.cuda.stream(self._upload):
                if piece["used"]:
                    self._upload.wait_event(piece["computed"])       # the previous run no longer reads these inputs
                piece["logits"].copy_(logits[rows], non_blocking=True)
                piece["x"].copy_(x[rows], non_blocking=True)
                piece["uploaded"].record(self._upload)
            compute.wait_event(piece["uploaded"])
            if piece["used"]:
                compute.wait_event(piece["downloaded"])              # the previous result has left y
            piece["router"].launch()
            piece["chain"].launch()
            piece["computed"].record(compute)
            with torch.cuda.stream(self._download):
                self._download.wait_event(piece["computed"])
                out[rows].copy_(piece["y"], non_blocking=True)
                piece["downloaded"].record(self._download)
            piece["used"] = True
        self._download.synchronize()
        return out

    def check(self) -> None:
        for piece in self._bound or ():
            piece["chain"].up_call.check()
