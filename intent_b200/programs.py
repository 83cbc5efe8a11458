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

    return NativeProgram(interface=interface, entry_name=f"intent_b200_{stem}_{act.name}",
                         constants=(group, zp), device=device, workspace=workspace_bytes,
                         empty=lambda d: d["M"] == 0 or d["N"] == 0)


weight_only_int4_matmul = KernelDefinition(
    name="weight_only_int4_matmul",
    constexprs={"GROUP_SIZE": 64, "ZERO_POINT": "twos_complement", "ACT_DTYPE": "f16", "KERNEL": "auto"},
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
