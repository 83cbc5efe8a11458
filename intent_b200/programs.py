"""The shipped programs (kernel definitions).

Each definition carries the reference program's name and parameter order, so
code written against the reference's examples binds the same way:

    artifact = intent_b200.compile(programs.weight_only_int4_matmul,
                                   target=B200Target(device=0),
                                   constexprs={"GROUP_SIZE": 128, "ZERO_POINT": 8})
    y = artifact.run(x, packed, scales)
"""
from __future__ import annotations

from . import dtypes
from .compiler import KernelDefinition
from .errors import CompilationStageError
from .runtime.artifact import NativeProgram
from .runtime.interface import PublicInterface, ScalarParameter, ViewKind, ViewParameter

IN, OUT, INOUT = ViewKind.IN, ViewKind.OUT, ViewKind.INOUT


def _act_dtype(constants, name="ACT_DTYPE"):
    element = dtypes.dtype(constants[name])
    if element not in (dtypes.f16, dtypes.bf16):
        raise CompilationStageError("provider_native_compilation",
                                    f"{name} must be f16 or bf16, got {element}")
    return element


def _rule(condition, message):
    def check(d):
        if not condition(d):
            raise ValueError(message(d) if callable(message) else message)
    return check


# ---------------------------------------------------------------------------------
# weight_only_int4_matmul (W4A16)
# ---------------------------------------------------------------------------------
def _lower_w4a16(constants, device):
    act = _act_dtype(constants)
    group = int(constants["GROUP_SIZE"])
    if group not in (32, 64, 128):
        raise CompilationStageError("provider_native_compilation",
                                    f"GROUP_SIZE {group} has no kernel specialisation (32, 64, 128)")
    zero_point = constants["ZERO_POINT"]
    if zero_point in ("twos_complement", None, -1):
        zp = -1
    elif zero_point == 8:
        zp = 8
    else:
        raise CompilationStageError("provider_native_compilation",
                                    "ZERO_POINT must be 'twos_complement' or 8")
    kernel = constants["KERNEL"]
    stem = {"auto": "weight_only_int4_matmul", "gemv": "w4a16_gemv", "gemm": "w4a16_gemm"}.get(kernel)
    if stem is None:
        raise CompilationStageError("frontend_kir", "KERNEL must be 'auto', 'gemv' or 'gemm'")
    layout = constants.get("WEIGHT_LAYOUT", "reference")
    if layout not in ("reference", "tiled"):
        raise CompilationStageError("frontend_kir", "WEIGHT_LAYOUT must be 'reference' or 'tiled'")
    if layout == "tiled":
        # packed_weight is the tiled copy made by intent_b200.prelayout.tile: tensor-core kernels only
        if kernel == "gemv":
            raise CompilationStageError("provider_native_compilation",
                                        "the bandwidth kernel reads the reference layout; WEIGHT_LAYOUT='tiled' "
                                        "needs KERNEL 'auto' or 'gemm'")
        from . import prelayout

        tiled_interface = PublicInterface((
            ViewParameter(0, "activation", act, ("M", "K"), IN),
            ViewParameter(1, "packed_weight", dtypes.i32, ("W",), IN),
            ViewParameter(2, "scales", act, ("G", "N"), IN),
            ViewParameter(3, "output", act, ("M", "N"), OUT),
        ), dimension_rules=(
            _rule(lambda d: d["K"] % group == 0 and d["G"] * group == d["K"],
                  lambda d: f"scales.shape[0] must be K/GROUP_SIZE with K a multiple of {group}"),
            _rule(lambda d: d["W"] == prelayout.words(d["K"], d["N"]),
                  lambda d: f"packed_weight must hold the {prelayout.words(d['K'], d['N'])} words of the tiled copy "
                            f"of a [{d['K'] // 8}, {d['N']}] weight, got {d['W']}"),
        ))
        return NativeProgram(interface=tiled_interface, entry_name=f"intent_b200_w4a16_gemm_tiled_{act.name}",
                             constants=(group, zp), device=device, empty=lambda d: d["M"] == 0 or d["N"] == 0)
    interface = PublicInterface((
        ViewParameter(0, "activation", act, ("M", "K"), IN),
        ViewParameter(1, "packed_weight", dtypes.i32, ("P", "N"), IN),
        ViewParameter(2, "scales", act, ("G", "N"), IN),
        ViewParameter(3, "output", act, ("M", "N"), OUT),
    ), dimension_rules=(
        _rule(lambda d: d["P"] * 8 == d["K"],
              lambda d: f"packed_weight.shape[0] must be K/8 = {d['K'] // 8}, got {d['P']}"),
        _rule(lambda d: d["K"] % group == 0 and d["G"] * group == d["K"],
              lambda d: f"scales.shape[0] must be K/GROUP_SIZE with K a multiple of {group}"),
    ))
    def workspace_bytes(d):
        import ctypes

        from .runtime import native

        query = native.library().intent_b200_weight_only_int4_matmul_workspace_bytes
        query.restype = ctypes.c_int64
        query.argtypes = [ctypes.c_int64] * 3
        rows = d["M"] if kernel != "gemm" else 1 << 30
        return int(query(rows, d["K"], d["N"])) if kernel != "gemm" else 0

    program = NativeProgram(interface=interface, entry_name=f"intent_b200_{stem}_{act.name}",
                            constants=(group, zp), device=device, workspace=workspace_bytes,
                            empty=lambda d: d["M"] == 0 or d["N"] == 0,
                            workspace_status="intent_b200_w4a16_gemv_workspace_status",
                            device_status=() if kernel == "gemv" else ("intent_b200_w4a16_gemm_device_status",))
    if constants.get("PRELAYOUT"):
        if kernel == "gemv":
            raise CompilationStageError("provider_native_compilation", "PRELAYOUT applies to the tensor-core kernels")
        tiled = _lower_w4a16({**constants, "WEIGHT_LAYOUT": "tiled", "PRELAYOUT": False, "KERNEL": "gemm"}, device)
        return PrelayoutProgram(program, tiled)
    return program


class PrelayoutProgram:
    """``weight_only_int4_matmul`` with ``PRELAYOUT=True``: the call surface and the weight format are the
    reference's, but the weights are taken to be static model state.  Calls with more than 16 activation rows
    run on a tiled copy of the weight that is made the first time a weight tensor is seen and kept in a
    :class:`intent_b200.prelayout.PrelayoutCache`; calls with at most 16 rows go to the bandwidth kernel, which
    reads the reference layout directly."""

    SKINNY_ROWS = 16

    def __init__(self, reference: NativeProgram, tiled: NativeProgram):
        from .prelayout import PrelayoutCache

        self.reference, self.tiled = reference, tiled
        self.cache = PrelayoutCache()
        self.interface = reference.interface
        self.device = reference.device
        self.entry_name = tiled.entry_name
        self.constants = reference.constants
        self._last = reference

    @property
    def observation(self):
        return self._last.observation

    def _route(self, arguments: tuple):
        """(program, arguments) with the packed weight swapped for its tiled copy when the call is a GEMM."""
        import torch

        if (len(arguments) >= 3 and all(isinstance(a, torch.Tensor) for a in arguments[:3]) and
                arguments[0].dim() == 2 and arguments[0].shape[0] > self.SKINNY_ROWS and arguments[1].is_cuda):
            # validate against the reference interface first: errors name the caller's own arguments
            self.reference.interface.bind(tuple(arguments[:3]), device=self.reference._torch_device, abstract=True)
            tiled = self.cache.get(arguments[1])
            self._last = self.tiled
            return self.tiled, (arguments[0], tiled.tensor, *arguments[2:])
        self._last = self.reference
        return self.reference, arguments

    def run(self, *arguments):
        program, routed = self._route(arguments)
        return program.run(*routed)

    def launch(self, *arguments) -> None:
        program, routed = self._route(arguments)
        program.launch(*routed)

    def prepare(self, *arguments, outputs=None, explicit_outputs=False):
        program, routed = self._route(arguments)
        return program.prepare(*routed, outputs=outputs, explicit_outputs=explicit_outputs)

    def prepare_call(self, arguments: tuple, *, outputs=None):
        return self.prepare(*arguments, outputs=outputs)

    def infer_outputs(self, arguments: tuple):
        return self.reference.infer_outputs(arguments)

    def check(self, workspace=None) -> None:
        self.reference.check(workspace)
        self.tiled.check(None)



weight_only_int4_matmul = KernelDefinition(
    name="weight_only_int4_matmul",
    constexprs={"GROUP_SIZE": 64, "ZERO_POINT": "twos_complement", "ACT_DTYPE": "f16", "KERNEL": "auto",
                "WEIGHT_LAYOUT": "reference", "PRELAYOUT": False},
    lower=_lower_w4a16,
    reference="examples/kernels/contraction/weight_only_int4.py:18-51",
    summary="Y = X @ dequant(int4 packed along K, per-group scales); f32 accumulation",
)



# ---------------------------------------------------------------------------------
# gemm_i8 and the scaled W8A8 form
# ---------------------------------------------------------------------------------
def _i8_rules():
    return (
        _rule(lambda d: d["K"] % 16 == 0 and d["N"] % 16 == 0,
              "this backend requires K and N to be multiples of 16 for int8 operands"),
    )


def _lower_gemm_i8(constants, device):
    interface = PublicInterface((
        ViewParameter(0, "a", dtypes.i8, ("M", "K"), IN),
        ViewParameter(1, "b", dtypes.i8, ("K", "N"), IN),
        ViewParameter(2, "bias", dtypes.i32, ("N",), IN),
        ViewParameter(3, "c", dtypes.i32, ("M", "N"), OUT),
    ), dimension_rules=_i8_rules())
    return NativeProgram(interface=interface, entry_name="intent_b200_gemm_i8", device=device,
                         empty=lambda d: d["M"] == 0 or d["N"] == 0)


gemm_i8 = KernelDefinition(
    name="gemm_i8", constexprs={}, lower=_lower_gemm_i8,
    reference="examples/kernels/contraction/gemm.py:29-39",
    summary="C = i32(A @ B) + bias, exact wrapping integers",
)


def _lower_w8a8(constants, device):
    if dtypes.dtype(constants["OUT_DTYPE"]) is not dtypes.bf16:
        raise CompilationStageError("provider_native_compilation", "OUT_DTYPE must be bf16")
    interface = PublicInterface((
        ViewParameter(0, "a", dtypes.i8, ("M", "K"), IN),
        ViewParameter(1, "b", dtypes.i8, ("K", "N"), IN),
        ViewParameter(2, "a_scales", dtypes.f32, ("M",), IN),
        ViewParameter(3, "b_scales", dtypes.f32, ("N",), IN),
        ViewParameter(4, "output", dtypes.bf16, ("M", "N"), OUT),
    ), dimension_rules=_i8_rules())
    return NativeProgram(interface=interface, entry_name="intent_b200_w8a8_gemm_bf16", device=device,
                         empty=lambda d: d["M"] == 0 or d["N"] == 0)


w8a8_gemm = KernelDefinition(
    name="w8a8_gemm", constexprs={"OUT_DTYPE": "bf16"}, lower=_lower_w8a8,
    reference="examples/kernels/contraction/gemm.py:29-39 (+ per-channel scale precedent :83-106)",
    summary="Y = bf16((i32(A @ B) * sa[m]) * sb[n])",
)

ALL = {d.name: d for d in (weight_only_int4_matmul, gemm_i8, w8a8_gemm)}


# ---------------------------------------------------------------------------------
# MoE routing and route alignment.  The reference fixes TOKENS / TOP_K / EXPERTS /
# BLOCK_SIZE as module constants (examples/kernels/routing/moe_align.py:5-11); here
# they are compile-time constants of each program.
# ---------------------------------------------------------------------------------
from .runtime.interface import Derived  # noqa: E402

_ALIGN_CONSTEXPRS = {"TOKENS": 4096, "TOP_K": 2, "EXPERTS": 64, "BLOCK_SIZE": 128}


def _align_sizes(c):
    tokens, top_k, experts, block = (int(c[k]) for k in ("TOKENS", "TOP_K", "EXPERTS", "BLOCK_SIZE"))
    if min(tokens, top_k, experts, block) <= 0:
        raise CompilationStageError("frontend_kir", "TOKENS, TOP_K, EXPERTS and BLOCK_SIZE must be positive")
    routes = tokens * top_k
    padded = routes + experts * (block - 1)
    return tokens, top_k, experts, block, routes, padded, padded // block + 1


def _lower_count(c, device):
    tokens, top_k, experts, *_ = _align_sizes(c)
    interface = PublicInterface((
        ViewParameter(0, "topk_ids", dtypes.i32, ("T", top_k), IN, alignment=4),
        ViewParameter(1, "expert_counts", dtypes.i32, (experts,), INOUT, alignment=4),
    ), dimension_rules=(_rule(lambda d: d["T"] <= tokens, f"at most {tokens} tokens (TOKENS constexpr)"),))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_count_routes", device=device)


def _lower_prefix(c, device):
    _, _, experts, block, *_ = _align_sizes(c)
    interface = PublicInterface((
        ViewParameter(0, "expert_counts", dtypes.i32, (experts,), IN, alignment=4),
        ViewParameter(1, "expert_offsets", dtypes.i32, (experts + 1,), OUT, alignment=4),
        ViewParameter(2, "total_padded", dtypes.i32, (1,), OUT, alignment=4),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_prefix_routes", constants=(block,),
                         device=device)


def _lower_scatter(c, device):
    tokens, top_k, experts, _, _, padded, _ = _align_sizes(c)
    interface = PublicInterface((
        ViewParameter(0, "topk_ids", dtypes.i32, ("T", top_k), IN, alignment=4),
        ViewParameter(1, "expert_offsets", dtypes.i32, (experts + 1,), IN, alignment=4),
        ViewParameter(2, "expert_cursors", dtypes.i32, (experts,), INOUT, alignment=4),
        ViewParameter(3, "sorted_route_ids", dtypes.i32, (padded,), INOUT, alignment=4),
    ), dimension_rules=(_rule(lambda d: d["T"] <= tokens, f"at most {tokens} tokens (TOKENS constexpr)"),))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_scatter_routes", device=device)


def _lower_mark(c, device):
    _, _, experts, block, _, _, blocks = _align_sizes(c)
    interface = PublicInterface((
        ViewParameter(0, "expert_offsets", dtypes.i32, (experts + 1,), IN, alignment=4),
        ViewParameter(1, "expert_blocks", dtypes.i32, (blocks,), OUT, alignment=4),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_mark_expert_blocks", constants=(block,),
                         device=device)


def _lower_positions(c, device):
    _, _, _, _, routes, padded, _ = _align_sizes(c)
    interface = PublicInterface((
        ViewParameter(0, "sorted_route_ids", dtypes.i32, (padded,), IN, alignment=4),
        ViewParameter(1, "total_padded", dtypes.i32, (1,), IN, alignment=4),
        ViewParameter(2, "route_positions", dtypes.i32, (routes,), OUT, alignment=4),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_route_positions", device=device)


_MOE_ALIGN_REF = "examples/kernels/routing/moe_align.py"
moe_count_routes = KernelDefinition("moe_count_routes", dict(_ALIGN_CONSTEXPRS), _lower_count,
                                    f"{_MOE_ALIGN_REF}:14-29", "counts[e] += routes to e")
moe_prefix_routes = KernelDefinition("moe_prefix_routes", dict(_ALIGN_CONSTEXPRS), _lower_prefix,
                                     f"{_MOE_ALIGN_REF}:32-49", "block-padded exclusive offsets and padded total")
moe_scatter_routes = KernelDefinition("moe_scatter_routes", dict(_ALIGN_CONSTEXPRS), _lower_scatter,
                                      f"{_MOE_ALIGN_REF}:52-73", "stable partition of route ids by expert")
moe_mark_expert_blocks = KernelDefinition("moe_mark_expert_blocks", dict(_ALIGN_CONSTEXPRS), _lower_mark,
                                          f"{_MOE_ALIGN_REF}:76-86", "expert of every padded block")
moe_route_positions = KernelDefinition("moe_route_positions", dict(_ALIGN_CONSTEXPRS), _lower_positions,
                                       "examples/kernels/ragged/moe.py:24-33 (member_routes indirection, inverted)",
                                       "slot of every route in the sorted layout")


def _lower_route_top2(c, device):
    interface = PublicInterface((
        ViewParameter(0, "logits", dtypes.f32, ("T", "E"), IN, alignment=4),
        ViewParameter(1, "topk_ids", dtypes.i32, ("T", 2), OUT, alignment=4),
        ViewParameter(2, "topk_weights", dtypes.f32, ("T", 2), OUT, alignment=4),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_route_top2", device=device,
                         empty=lambda d: d["T"] == 0)


moe_route_top2 = KernelDefinition(
    "moe_route_top2", {}, _lower_route_top2,
    "examples/kernels/sampling/top_k.py:10-33, examples/kernels/normalization/softmax.py:23-37",
    "top-2 experts by logit (ties: lower id) and their softmax probabilities")


# ---------------------------------------------------------------------------------
# MoE data path: row gather, grouped W4A16 projections, weighted combine
# ---------------------------------------------------------------------------------
def _lower_gather(c, device):
    act = _act_dtype(c)
    interface = PublicInterface((
        ViewParameter(0, "x", act, ("T", "H"), IN),
        ViewParameter(1, "sorted_route_ids", dtypes.i32, ("P",), IN, alignment=4),
        ViewParameter(2, "total_padded", dtypes.i32, (1,), IN, alignment=4),
        ViewParameter(3, "rows", act, ("P", "H"), OUT),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_gather_rows",
                         constants=(int(c["TOP_K"]),), device=device)


moe_gather_rows = KernelDefinition("moe_gather_rows", {"ACT_DTYPE": "bf16", "TOP_K": 2}, _lower_gather,
                                   "examples/kernels/ragged/moe.py:34-36 (I.gather of token rows)",
                                   "rows[p] = x[sorted[p] // TOP_K], zero rows for padding")


def _grouped_constants(c):
    group = int(c["GROUP_SIZE"])
    if group not in (32, 64, 128):
        raise CompilationStageError("provider_native_compilation", f"GROUP_SIZE {group} has no kernel specialisation")
    zero_point = c["ZERO_POINT"]
    zp = -1 if zero_point in ("twos_complement", None, -1) else zero_point
    if zp not in (-1, 8):
        raise CompilationStageError("provider_native_compilation", "ZERO_POINT must be 'twos_complement' or 8")
    return group, zp


def _lower_grouped(c, device, *, gated):
    act = _act_dtype(c)
    group, zp = _grouped_constants(c)
    block = int(c["BLOCK_ROWS"])
    if block not in (128, 256):
        raise CompilationStageError("provider_native_compilation", "BLOCK_ROWS must be 128 or 256")
    out_cols = Derived("I", lambda d: d["WN"] // 2) if gated else "WN"
    weight, weight_rule, suffix = _grouped_weight(c, group)
    interface = PublicInterface((
        ViewParameter(0, "rows", act, ("P", "K"), IN),
        ViewParameter(1, "expert_blocks", dtypes.i32, ("B",), IN, alignment=4),
        ViewParameter(2, "total_padded", dtypes.i32, (1,), IN, alignment=4),
        weight,
        ViewParameter(4, "scales", act, ("E", "KG", "WN"), IN),
        ViewParameter(5, "output", act if gated else dtypes.f32, ("P", out_cols), OUT),
    ), dimension_rules=(
        weight_rule,
        _rule(lambda d: d["B"] * block >= d["P"], f"expert_blocks must cover every {block}-row block of rows"),
    ))
    stem = "upgate_silu" if gated else "down_f32"
    return NativeProgram(interface=interface, entry_name=f"intent_b200_moe_grouped_w4a16_{stem}{suffix}_{act.name}",
                         constants=(group, zp, block), device=device)


def _grouped_weight(c, group):
    """Parameter 3 of the grouped int4 programs, its shape rule and the entry-name suffix: the reference layout
    ``[E, K/8, WN]`` or, with ``WEIGHT_LAYOUT='tiled'``, the tiled copies ``[E, words]``
    (intent_b200.prelayout.tile of the same tensor)."""
    layout = c.get("WEIGHT_LAYOUT", "reference")
    if layout == "reference":
        return (ViewParameter(3, "packed_weight", dtypes.i32, ("E", "KP", "WN"), IN),
                _rule(lambda d: d["KP"] * 8 == d["K"] and d["KG"] * group == d["K"],
                      "packed_weight / scales do not match K and GROUP_SIZE"), "")
    if layout != "tiled":
        raise CompilationStageError("frontend_kir", "WEIGHT_LAYOUT must be 'reference' or 'tiled'")
    from . import prelayout

    return (ViewParameter(3, "packed_weight", dtypes.i32, ("E", "W"), IN),
            _rule(lambda d: d["KG"] * group == d["K"] and d["W"] == prelayout.words(d["K"], d["WN"]),
                  "packed_weight must hold the tiled copy of every expert's [K/8, WN] weight"), "_tiled")


_GROUPED_CONSTEXPRS = {"GROUP_SIZE": 128, "ZERO_POINT": 8, "ACT_DTYPE": "bf16", "BLOCK_ROWS": 128,
                       "WEIGHT_LAYOUT": "reference"}
moe_grouped_upgate_silu = KernelDefinition(
    "moe_grouped_upgate_silu", dict(_GROUPED_CONSTEXPRS), lambda c, d: _lower_grouped(c, d, gated=True),
    "examples/kernels/ragged/grouped_gemm.py:42-70, examples/kernels/ragged/moe.py:37-42, "
    "examples/kernels/activation/swiglu.py:27-46",
    "hidden = silu(rows @ Wgate[e]) * (rows @ Wup[e]) per expert block, int4 weights")
moe_grouped_down = KernelDefinition(
    "moe_grouped_down", dict(_GROUPED_CONSTEXPRS), lambda c, d: _lower_grouped(c, d, gated=False),
    "examples/kernels/ragged/grouped_gemm.py:42-70, examples/kernels/ragged/moe.py:43-47",
    "out = hidden @ Wdown[e] per expert block, f32 rows")


def _lower_down_scatter(c, device):
    act = _act_dtype(c)
    group, zp = _grouped_constants(c)
    block = int(c["BLOCK_ROWS"])
    if block not in (128, 256):
        raise CompilationStageError("provider_native_compilation", "BLOCK_ROWS must be 128 or 256")
    weight, weight_rule, suffix = _grouped_weight(c, group)
    interface = PublicInterface((
        ViewParameter(0, "rows", act, ("P", "K"), IN),
        ViewParameter(1, "expert_blocks", dtypes.i32, ("B",), IN, alignment=4),
        ViewParameter(2, "total_padded", dtypes.i32, (1,), IN, alignment=4),
        weight,
        ViewParameter(4, "scales", act, ("E", "KG", "WN"), IN),
        ViewParameter(5, "sorted_route_ids", dtypes.i32, ("S",), IN, alignment=4),
        ViewParameter(6, "route_weights", dtypes.f32, ("T", "TOP_K"), IN, alignment=4),
        ViewParameter(7, "y", dtypes.f32, ("T", "WN"), INOUT),
    ), dimension_rules=(
        weight_rule,
        _rule(lambda d: d["B"] * block >= d["P"], f"expert_blocks must cover every {block}-row block of rows"),
        _rule(lambda d: d["S"] >= d["P"], "sorted_route_ids must cover every row"),
    ))
    return NativeProgram(interface=interface,
                         entry_name=f"intent_b200_moe_grouped_w4a16_down_scatter{suffix}_{act.name}",
                         constants=(group, zp, block), device=device)


moe_grouped_down_scatter = KernelDefinition(
    "moe_grouped_down_scatter", dict(_GROUPED_CONSTEXPRS), _lower_down_scatter,
    "examples/kernels/ragged/moe.py:43-53 (down projection + weighted scatter_reduce add)",
    "y[route // TOP_K] += weight[route] * (hidden[r] @ Wdown[e]) per expert-sorted row r, relaxed atomics")


def _lower_combine(c, device):
    interface = PublicInterface((
        ViewParameter(0, "rows", dtypes.f32, ("P", "H"), IN),
        ViewParameter(1, "route_positions", dtypes.i32, ("R",), IN, alignment=4),
        ViewParameter(2, "route_weights", dtypes.f32, ("T", "TOP_K"), IN, alignment=4),
        ViewParameter(3, "y", dtypes.f32, ("T", "H"), INOUT),
    ), dimension_rules=(_rule(lambda d: d["R"] == d["T"] * d["TOP_K"], "route_positions must have T * TOP_K entries"),))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_combine",
                         constants=(1 if c["ACCUMULATE"] else 0,), device=device)


moe_combine = KernelDefinition("moe_combine", {"ACCUMULATE": True}, _lower_combine,
                               "examples/kernels/ragged/moe.py:48-53 (weighted scatter_reduce add)",
                               "y[t] += sum_c weight[t,c] * rows[position[t,c]] in choice order")

ALL.update({d.name: d for d in (moe_count_routes, moe_prefix_routes, moe_scatter_routes, moe_mark_expert_blocks,
                                moe_route_positions, moe_route_top2, moe_gather_rows, moe_grouped_upgate_silu,
                                moe_grouped_down, moe_grouped_down_scatter, moe_combine)})


# ---------------------------------------------------------------------------------
# Ragged grouped contractions with dense 16-bit weights
# ---------------------------------------------------------------------------------
def _align256(count):
    return (int(count) + 255) & ~255


_DENSE_RULES = (
    _rule(lambda d: d["K"] % 8 == 0 and d["N"] % 8 == 0,
          "this backend requires K and N to be multiples of 8 for 16-bit operands"),
)


def _lower_ragged(c, device, element):
    interface = PublicInterface((
        ViewParameter(0, "x", element, ("R", "K"), IN),
        ViewParameter(1, "group_offsets", dtypes.i32, ("G_PLUS_1",), IN, alignment=4),
        ViewParameter(2, "weight", element, ("G", "K", "N"), IN),
        ViewParameter(3, "y", element, ("R", "N"), OUT),
    ), dimension_rules=_DENSE_RULES + (
        _rule(lambda d: d["G_PLUS_1"] == d["G"] + 1, "group_offsets must have G + 1 entries"),
        _rule(lambda d: d["G"] <= 1024, "at most 1024 groups"),
    ))
    return NativeProgram(interface=interface, entry_name=f"intent_b200_ragged_grouped_gemm_{element.name}",
                         device=device, empty=lambda d: d["R"] == 0 or d["N"] == 0 or d["G"] == 0)


ragged_grouped_gemm = KernelDefinition(
    "ragged_grouped_gemm", {}, lambda c, d: _lower_ragged(c, d, dtypes.f16),
    "examples/kernels/ragged/grouped_gemm.py:11-39",
    "rows offsets[g]:offsets[g+1] of X times W[g], f16, f32 accumulation")
ragged_grouped_gemm_bf16 = KernelDefinition(
    "ragged_grouped_gemm_bf16", {}, lambda c, d: _lower_ragged(c, d, dtypes.bf16),
    "examples/kernels/ragged/grouped_gemm.py:42-70",
    "rows offsets[g]:offsets[g+1] of X times W[g], bf16, f32 accumulation")


def _lower_routed(c, device):
    element = _act_dtype(c, "DTYPE")
    top_k = int(c["TOP_K"])
    if top_k <= 0:
        raise CompilationStageError("frontend_kir", "TOP_K must be positive")
    interface = PublicInterface((
        ViewParameter(0, "x", element, ("T", "K"), IN),
        ViewParameter(1, "expert_offsets", dtypes.i32, ("E_PLUS_1",), IN, alignment=4),
        ViewParameter(2, "member_routes", dtypes.i32, ("R",), IN, alignment=4),
        ViewParameter(3, "weight", element, ("E", "N", "K"), IN),
        ViewParameter(4, "output", element, ("T", top_k, "N"), OUT),
    ), dimension_rules=_DENSE_RULES + (
        _rule(lambda d: d["E_PLUS_1"] == d["E"] + 1, "expert_offsets must have E + 1 entries"),
        _rule(lambda d: d["E"] <= 1024, "at most 1024 experts"),
    ))
    return NativeProgram(interface=interface, entry_name=f"intent_b200_routed_expert_projection_{element.name}",
                         constants=(top_k,), device=device,
                         workspace=lambda d: _align256(d["R"] * d["K"] * 2),
                         empty=lambda d: d["R"] == 0 or d["N"] == 0 or d["E"] == 0 or d["T"] == 0)


routed_expert_projection_bf16 = KernelDefinition(
    "routed_expert_projection_bf16", {"TOP_K": 2, "DTYPE": "bf16"}, _lower_routed,
    "examples/kernels/ragged/grouped_gemm.py:101-138",
    "out[token, slot] = x[token] @ W[e].T for the routes member_routes lists per expert")


def _lower_expert_ffn(c, device):
    element = _act_dtype(c, "DTYPE")
    interface = PublicInterface((
        ViewParameter(0, "x", element, ("T", "D"), IN),
        ViewParameter(1, "route_offsets", dtypes.i32, ("E_PLUS_1",), IN, alignment=4),
        ViewParameter(2, "member_routes", dtypes.i32, ("R",), IN, alignment=4),
        ViewParameter(3, "route_token", dtypes.i32, ("NR",), IN, alignment=4),
        ViewParameter(4, "route_weights", dtypes.f32, ("NR",), IN, alignment=4),
        ViewParameter(5, "w1", element, ("E", "D", "F"), IN),
        ViewParameter(6, "w2", element, ("E", "F", "D"), IN),
        ViewParameter(7, "y", dtypes.f32, ("T", "D"), INOUT),
    ), dimension_rules=(
        _rule(lambda d: d["D"] % 8 == 0 and d["F"] % 8 == 0,
              "this backend requires D and F to be multiples of 8 for 16-bit operands"),
        _rule(lambda d: d["E_PLUS_1"] == d["E"] + 1, "route_offsets must have E + 1 entries"),
        _rule(lambda d: d["E"] <= 1024, "at most 1024 experts"),
    ))
    return NativeProgram(interface=interface, entry_name=f"intent_b200_moe_expert_ffn_{element.name}", device=device,
                         workspace=lambda d: _align256(d["R"] * d["D"] * 2) + _align256(d["R"] * d["F"] * 2),
                         empty=lambda d: d["R"] == 0 or d["D"] == 0 or d["E"] == 0 or d["T"] == 0 or d["F"] == 0)


moe_expert_ffn = KernelDefinition(
    "moe_expert_ffn", {"DTYPE": "f16"}, _lower_expert_ffn,
    "examples/kernels/ragged/moe.py:12-53",
    "y[token] += w[route] * (relu(x[token] @ W1[e]) @ W2[e]) over the routes of every expert")

ALL.update({d.name: d for d in (ragged_grouped_gemm, ragged_grouped_gemm_bf16, routed_expert_projection_bf16,
                                moe_expert_ffn)})


# ---------------------------------------------------------------------------------
# Packed-weight contractions next to weight_only_int4_matmul: decode once into a workspace,
# then the dense tensor-core kernels
# ---------------------------------------------------------------------------------
def _lower_w4a8(c, device):
    interface = PublicInterface((
        ViewParameter(0, "activation", dtypes.i8, ("M", "K"), IN),
        ViewParameter(1, "packed_weight", dtypes.u8, ("N", "P"), IN),
        ViewParameter(2, "output", dtypes.i32, ("N", "M"), OUT),
    ), dimension_rules=(
        _rule(lambda d: d["P"] * 2 == d["K"], lambda d: f"packed_weight.shape[1] must be K/2 = {d['K'] // 2}"),
        _rule(lambda d: d["K"] % 32 == 0 and d["M"] % 16 == 0,
              "this backend requires K to be a multiple of 32 and M a multiple of 16"),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_w4a8_packed_matmul", device=device,
                         workspace=lambda d: _align256(d["N"] * d["K"]),
                         empty=lambda d: d["M"] == 0 or d["N"] == 0)


w4a8_packed_matmul = KernelDefinition(
    "w4a8_packed_matmul", {}, _lower_w4a8, "examples/kernels/contraction/weight_only_int4.py:54-91",
    "out[N,M] = i32(int4(W)[N,K] @ A[M,K].T), two nibbles per byte, exact")


def _lower_bitnet(c, device):
    interface = PublicInterface((
        ViewParameter(0, "activation", dtypes.i8, ("M", "K"), IN),
        ViewParameter(1, "packed_weight", dtypes.u8, ("N", "P"), IN),
        ViewParameter(2, "output", dtypes.i32, ("M", "N"), OUT),
    ), dimension_rules=(
        _rule(lambda d: d["P"] * 4 == d["K"], lambda d: f"packed_weight.shape[1] must be K/4 = {d['K'] // 4}"),
        _rule(lambda d: d["K"] % 16 == 0 and d["N"] % 16 == 0,
              "this backend requires K and N to be multiples of 16"),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_bitnet_int2_matmul", device=device,
                         workspace=lambda d: _align256(d["N"] * d["K"]),
                         empty=lambda d: d["M"] == 0 or d["N"] == 0)


bitnet_int2_matmul = KernelDefinition(
    "bitnet_int2_matmul", {}, _lower_bitnet, "examples/kernels/contraction/weight_only_int4.py:94-123",
    "out[M,N] = i32(A[M,K] @ int2(W)[N,K].T), interleaved 16-value words, exact")


def _lower_fp4(c, device):
    interface = PublicInterface((
        ViewParameter(0, "activation", dtypes.bf16, ("M", "K"), IN),
        ViewParameter(1, "packed_weight", dtypes.u8, ("N", "P"), IN),
        ViewParameter(2, "output", dtypes.bf16, ("M", "N"), OUT),
    ), dimension_rules=(
        _rule(lambda d: d["P"] * 2 == d["K"], lambda d: f"packed_weight.shape[1] must be K/2 = {d['K'] // 2}"),
        _rule(lambda d: d["K"] % 8 == 0 and d["N"] % 8 == 0, "this backend requires K and N to be multiples of 8"),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_dequant_bf16_fp4_matmul", device=device,
                         workspace=lambda d: _align256(d["N"] * d["K"] * 2) + 256,
                         empty=lambda d: d["M"] == 0 or d["N"] == 0)


dequant_bf16_fp4_matmul = KernelDefinition(
    "dequant_bf16_fp4_matmul", {}, _lower_fp4, "examples/kernels/contraction/weight_only_int4.py:126-175",
    "out[M,N] = bf16(A[M,K] @ e2m1(W)[N,K].T), four fp4 codes per 16-bit word")

ALL.update({d.name: d for d in (w4a8_packed_matmul, bitnet_int2_matmul, dequant_bf16_fp4_matmul)})


# ---------------------------------------------------------------------------------
# Dense 16-bit GEMMs of the reference's gemm.py on the ragged kernel (one row group)
# ---------------------------------------------------------------------------------
def _dense_interface(element, out):
    return PublicInterface((
        ViewParameter(0, "a", element, ("M", "K"), IN),
        ViewParameter(1, "b", element, ("K", "N"), IN),
        ViewParameter(2, "c", out, ("M", "N"), OUT),
    ), dimension_rules=_DENSE_RULES)


def _lower_gemm(c, device):
    activation = c["ACTIVATION"]
    code = {"none": 0, "NONE": 0, 0: 0, "relu": 1, "RELU": 1, 1: 1}.get(getattr(activation, "name", activation))
    if code is None:
        raise CompilationStageError("frontend_kir", "ACTIVATION must be 'none' (0) or 'relu' (1)")
    return NativeProgram(interface=_dense_interface(dtypes.f16, dtypes.f16), entry_name="intent_b200_gemm_f16",
                         constants=(code,), device=device, empty=lambda d: d["M"] == 0 or d["N"] == 0)


gemm = KernelDefinition("gemm", {"ACTIVATION": "none"}, _lower_gemm,
                        "examples/kernels/contraction/gemm.py:40-61", "C = f16(act(A @ B)), f32 accumulation")
bf16_gemm = KernelDefinition(
    "bf16_gemm", {},
    lambda c, device: NativeProgram(interface=_dense_interface(dtypes.bf16, dtypes.bf16),
                                    entry_name="intent_b200_bf16_gemm", device=device,
                                    empty=lambda d: d["M"] == 0 or d["N"] == 0),
    "examples/kernels/contraction/gemm.py:64-80", "C = bf16(A @ B), f32 accumulation")


def _lower_quantized_gemm(c, device):
    interface = PublicInterface((
        ViewParameter(0, "a", dtypes.f16, ("M", "K"), IN),
        ViewParameter(1, "b", dtypes.f16, ("K", "N"), IN),
        ViewParameter(2, "bias", dtypes.f32, ("N",), IN),
        ViewParameter(3, "residual", dtypes.f16, ("M", "N"), IN),
        ViewParameter(4, "output_scale", dtypes.f32, ("N",), IN),
        ViewParameter(5, "output", dtypes.i8, ("M", "N"), OUT),
    ), dimension_rules=_DENSE_RULES)
    return NativeProgram(interface=interface, entry_name="intent_b200_quantized_gemm_f16", device=device,
                         empty=lambda d: d["M"] == 0 or d["N"] == 0)


quantized_gemm = KernelDefinition(
    "quantized_gemm", {}, _lower_quantized_gemm, "examples/kernels/contraction/gemm.py:83-106",
    "i8(clamp((relu(A @ B + bias) + residual) / scale)), truncating cast")

ALL.update({d.name: d for d in (gemm, bf16_gemm, quantized_gemm)})


# ---------------------------------------------------------------------------------
# Expert-parallel exchange over peer memory
# ---------------------------------------------------------------------------------
def _lower_peer_layout(c, device):
    world, experts, rank, block = (int(c[k]) for k in ("WORLD", "EXPERTS", "RANK", "BLOCK_ROWS"))
    capacity = int(c["CAPACITY_ROWS"])
    if world <= 0 or experts % world or not 0 <= rank < world or block <= 0 or capacity < 0:
        raise CompilationStageError("frontend_kir", "EXPERTS must be a multiple of WORLD and 0 <= RANK < WORLD")
    interface = PublicInterface((
        ViewParameter(0, "counts", dtypes.i32, (world, experts), IN, alignment=4),
        ViewParameter(1, "dest_base", dtypes.i32, (experts,), OUT, alignment=4),
        ViewParameter(2, "local_offsets", dtypes.i32, (experts // world + 1,), OUT, alignment=4),
        ViewParameter(3, "total_padded", dtypes.i32, (1,), OUT, alignment=4),
        ViewParameter(4, "expert_blocks", dtypes.i32, (capacity // block + 1,), OUT, alignment=4),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_peer_layout", constants=(rank, block),
                         device=device)


moe_peer_layout = KernelDefinition(
    "moe_peer_layout", {"WORLD": 1, "EXPERTS": 64, "RANK": 0, "BLOCK_ROWS": 128, "CAPACITY_ROWS": 0},
    _lower_peer_layout,
    "examples/kernels/routing/moe_align.py:32-49 (padded offsets), over the ranks' count matrix",
    "where this rank's routes start inside every owner's expert-sorted row buffer")


def _lower_peer_dispatch(c, device):
    act = _act_dtype(c)
    top_k, capacity = int(c["TOP_K"]), int(c["CAPACITY_ROWS"])
    interface = PublicInterface((
        ViewParameter(0, "x", act, ("T", "H"), IN),
        ViewParameter(1, "sorted_routes", dtypes.i32, ("R",), IN, alignment=4),
        ViewParameter(2, "send_offsets", dtypes.i32, ("E_PLUS_1",), IN, alignment=4),
        ViewParameter(3, "dest_base", dtypes.i32, ("E",), IN, alignment=4),
        ViewParameter(4, "peer_rows", dtypes.i64, ("W",), IN, alignment=8),
        ViewParameter(5, "route_dest", dtypes.i32, ("R", 2), OUT, alignment=4),
    ), dimension_rules=(
        _rule(lambda d: d["R"] == d["T"] * top_k, "sorted_routes must have T * TOP_K entries"),
        _rule(lambda d: d["E_PLUS_1"] == d["E"] + 1 and d["E"] % d["W"] == 0,
              "send_offsets needs E + 1 entries and E must be a multiple of the rank count"),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_peer_dispatch",
                         constants=(top_k, capacity), device=device)


moe_peer_dispatch = KernelDefinition(
    "moe_peer_dispatch", {"ACT_DTYPE": "bf16", "TOP_K": 2, "CAPACITY_ROWS": 0}, _lower_peer_dispatch,
    "examples/kernels/ragged/moe.py:34-36 (I.gather of token rows), written into the owner rank's buffer",
    "rows[owner][position] = x[route // TOP_K] over peer memory")


def _lower_peer_combine(c, device):
    capacity = int(c["CAPACITY_ROWS"])
    interface = PublicInterface((
        ViewParameter(0, "peer_out", dtypes.i64, ("W",), IN, alignment=8),
        ViewParameter(1, "route_dest", dtypes.i32, ("R", 2), IN, alignment=4),
        ViewParameter(2, "route_weights", dtypes.f32, ("T", "TOP_K"), IN, alignment=4),
        ViewParameter(3, "y", dtypes.f32, ("T", "H"), INOUT),
    ), dimension_rules=(_rule(lambda d: d["R"] == d["T"] * d["TOP_K"], "route_dest must have T * TOP_K rows"),))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_peer_combine",
                         constants=(capacity, 1 if c["ACCUMULATE"] else 0), device=device)


moe_peer_combine = KernelDefinition(
    "moe_peer_combine", {"CAPACITY_ROWS": 0, "ACCUMULATE": True}, _lower_peer_combine,
    "examples/kernels/ragged/moe.py:48-53 (weighted scatter_reduce add), reading the owners' result rows",
    "y[t] += sum_c weight[t,c] * out[owner(t,c)][position(t,c)] over peer memory")

ALL.update({d.name: d for d in (moe_peer_layout, moe_peer_dispatch, moe_peer_combine)})


# ---------------------------------------------------------------------------------
# Q4_K x Q8_K quantized projection (a second bandwidth-bound GEMV format)
# ---------------------------------------------------------------------------------
def _lower_quantized_projection(c, device):
    interface = PublicInterface((
        ViewParameter(0, "weights", dtypes.u8, ("N", "G", 144), IN),
        ViewParameter(1, "activation", dtypes.f32, ("G", 256), IN),
        ViewParameter(2, "output", dtypes.f32, ("N",), OUT, alignment=4),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_quantized_projection", device=device,
                         workspace=lambda d: _align256(d["G"] * 292), empty=lambda d: d["N"] == 0)


quantized_projection = KernelDefinition(
    "quantized_projection", {}, _lower_quantized_projection,
    "examples/kernels/quantization/quantized_projection.py:5-19",
    "out[n] = sum over records of quantized_dot(Q4_K weights[n], Q8_K(activation))")

ALL.update({quantized_projection.name: quantized_projection})


def _lower_peer_post(c, device):
    rank, channel, payload = int(c["RANK"]), int(c["CHANNEL"]), bool(c["PAYLOAD"])
    interface = PublicInterface((
        ViewParameter(0, "peer_flags", dtypes.i64, ("W",), IN, alignment=8),
        ViewParameter(1, "sequence", dtypes.i32, ("S",), INOUT, alignment=4),
        ViewParameter(2, "peer_tables", dtypes.i64, ("W",) if payload else (0,), IN, alignment=8),
        ViewParameter(3, "payload", dtypes.i32, ("C",), IN, alignment=4),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_peer_post", constants=(rank, channel),
                         device=device)


def _lower_peer_wait(c, device):
    channel, polls = int(c["CHANNEL"]), int(c["MAX_POLLS"])
    interface = PublicInterface((
        ViewParameter(0, "flags", dtypes.i32, ("CHANNELS", "W"), IN, alignment=4),
        ViewParameter(1, "sequence", dtypes.i32, ("S",), INOUT, alignment=4),
        ViewParameter(2, "status", dtypes.i32, (1,), INOUT, alignment=4),
    ))
    return NativeProgram(interface=interface, entry_name="intent_b200_moe_peer_wait", constants=(channel, polls),
                         device=device)


moe_peer_post = KernelDefinition(
    "moe_peer_post", {"RANK": 0, "CHANNEL": 0, "PAYLOAD": False}, _lower_peer_post,
    "no counterpart in the reference (it has no multi-GPU path)",
    "announce this rank at a sync point (optionally with its per-expert counts) in every rank's flag array")
moe_peer_wait = KernelDefinition(
    "moe_peer_wait", {"CHANNEL": 0, "MAX_POLLS": 1 << 24}, _lower_peer_wait,
    "no counterpart in the reference (it has no multi-GPU path)",
    "bounded wait until every rank has announced itself at the sync point")

ALL.update({d.name: d for d in (moe_peer_post, moe_peer_wait)})
