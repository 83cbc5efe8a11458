"""Several W4A16 decode projections in one persistent launch.

``weight_only_int4_matmul`` (reference kernel body examples/kernels/contraction/weight_only_int4.py:18-51)
is one contraction per artifact call in the reference.  A decode step's projections are each a few tens
of megabytes of weights, small enough that a launch's ramp-up and drain cost as much as its weight
stream, so this host composition (in the manner of the reference's multi-kernel host programs,
examples/programs/composition.py) binds a TABLE of independent contractions to one launch of
``intent_b200_w4a16_gemv_table_*``: the weight stream of one problem starts while the previous one is
still being reduced.  Numerics and tolerances are those of the single-problem program.

    table = W4A16Table(group_size=128, zero_point=8, act_dtype="f16", target=B200Target(0))
    call = table.prepare([(x_up, packed_up, scales_up), (x_down, packed_down, scales_down)])
    call.launch()                  # asynchronous on torch's current stream; no allocation, no sync
    y_up, y_down = call.results()

The problems of one table must be independent (no problem reads another's output).  Problems the table
kernel does not cover (more than 16 rows is rejected; 9..16 rows with a long K may not fit its shared
memory) make ``prepare`` fall back to one single-problem launch each, through the same artifact.
"""
from __future__ import annotations

import ctypes

from . import dtypes, programs
from .compiler import compile as _compile
from .errors import CompilationStageError
from .runtime import native


class _Problem(ctypes.Structure):
    _fields_ = [("x", ctypes.c_void_p), ("packed", ctypes.c_void_p), ("scales", ctypes.c_void_p),
                ("y", ctypes.c_void_p), ("M", ctypes.c_int64), ("K", ctypes.c_int64), ("N", ctypes.c_int64)]


class W4A16Table:
    def __init__(self, *, group_size: int = 64, zero_point="twos_complement", act_dtype="f16", target=None):
        self.artifact = _compile(programs.weight_only_int4_matmul, target=target,
                                 constexprs={"GROUP_SIZE": group_size, "ZERO_POINT": zero_point,
                                             "ACT_DTYPE": act_dtype, "KERNEL": "gemv"})
        self.group_size = int(group_size)
        self.zero_point = -1 if zero_point in ("twos_complement", None, -1) else int(zero_point)
        self.element = dtypes.dtype(act_dtype)
        self.device = self.artifact.device
        suffix = self.element.name
        library = native.library()
        self._entry = getattr(library, f"intent_b200_w4a16_gemv_table_{suffix}")
        self._entry.restype = ctypes.c_int
        self._entry.argtypes = [ctypes.POINTER(_Problem), ctypes.c_int32, ctypes.c_int32, ctypes.c_int32,
                                ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        self._query = library.intent_b200_w4a16_gemv_table_workspace_bytes
        self._query.restype = ctypes.c_int64
        self._query.argtypes = [ctypes.POINTER(_Problem), ctypes.c_int32, ctypes.c_int32]

    def prepare(self, problems, outputs=None) -> "PreparedTable":
        """``problems``: sequence of ``(activation [M,K], packed_weight [K/8,N] i32, scales [K/G,N])``;
        ``outputs``: optional sequence of ``[M,N]`` buffers (allocated with ``torch.empty`` otherwise).
        Arguments are validated like the single-problem artifact's (raise, never coerce)."""
        import torch

        problems = [tuple(problem) for problem in problems]
        if outputs is not None and len(outputs) != len(problems):
            raise TypeError(f"expected {len(problems)} outputs, got {len(outputs)}")
        interface = self.artifact.interface
        device = torch.device("cuda", self.device)
        bound = []
        for index, problem in enumerate(problems):
            if len(problem) != 3:
                raise TypeError(f"problem {index} must be (activation, packed_weight, scales)")
            arguments = problem if outputs is None else interface.explicit_arguments(problem, (outputs[index],))
            # the artifact's own binder: dtype / device / rank / shape relations / layout / alignment
            bound.append(interface.bind(tuple(arguments), device=device, explicit_outputs=outputs is not None))
        return PreparedTable(self, bound)


class PreparedTable:
    def __init__(self, table: W4A16Table, bound: list):
        import torch

        self.table, self._bound = table, bound
        self._rows = (_Problem * max(1, len(bound)))()
        self._count = 0
        for invocation in bound:
            x, packed, scales, y = invocation.arguments
            if x.shape[0] == 0 or packed.shape[1] == 0:
                continue                                   # nothing to compute for this problem
            row = self._rows[self._count]
            row.x, row.packed, row.scales, row.y = x.data_ptr(), packed.data_ptr(), scales.data_ptr(), y.data_ptr()
            row.M, row.K, row.N = x.shape[0], x.shape[1], packed.shape[1]
            self._count += 1
        self._fallback = None
        self._workspace = None
        if self._count:
            need = int(table._query(self._rows, self._count, table.group_size))
            if need > 0:
                self._workspace = torch.zeros((need,), dtype=torch.uint8, device=torch.device("cuda", table.device))
            else:   # outside the table kernel's coverage: one single-problem launch each
                self._fallback = [table.artifact.prepare(*inv.arguments[:3], outputs=(inv.arguments[3],))
                                  for inv in bound]

    @property
    def single_launch(self) -> bool:
        """True when the whole table runs through the table kernel (otherwise: one launch per problem)."""
        return self._fallback is None

    def results(self) -> tuple:
        return tuple(invocation.arguments[3] for invocation in self._bound)

    def launch(self) -> None:
        import torch

        if self._fallback is not None:
            for call in self._fallback:
                call.launch()
            return
        if not self._count:
            return
        table = self.table
        with torch.cuda.device(table.device):
            stream = torch.cuda.current_stream(table.device).cuda_stream
            status = table._entry(self._rows, self._count, table.group_size, table.zero_point,
                                  ctypes.c_void_p(self._workspace.data_ptr()), self._workspace.numel(),
                                  ctypes.c_void_p(stream))
        native.check(status, table._entry.__name__ if hasattr(table._entry, "__name__") else "w4a16_gemv_table")

    __call__ = launch

    def check(self) -> None:
        """Synchronise the current stream and raise if a bounded device-side wait of an earlier launch gave
        up; a workspace left dirty by such a launch is cleared for reuse."""
        import torch

        if self._fallback is not None:
            for call in self._fallback:
                call.check()
            return
        if self._workspace is None:
            return
        reader = native.library().intent_b200_w4a16_gemv_workspace_status
        reader.restype = ctypes.c_int
        reader.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
        with torch.cuda.device(self.table.device):
            stream = torch.cuda.current_stream(self.table.device).cuda_stream
            status = int(reader(ctypes.c_void_p(self._workspace.data_ptr()), self._workspace.numel(),
                                ctypes.c_void_p(stream)))
        native.check(status, "intent_b200_w4a16_gemv_table")


def set_launch_overlap(enabled: bool) -> None:
    """Process-wide: a table launch may start requesting its packed weights while the kernel before it on
    the stream is still running (programmatic dependent launch).  Only valid when the weights are not
    written by that kernel (static model weights in a decode loop)."""
    native.check(native.library().intent_b200_w4a16_gemv_table_overlap(1 if enabled else 0),
                 "intent_b200_w4a16_gemv_table_overlap")


def set_ride_along(enabled: bool) -> None:
    """Process-wide: problems of at most eight rows run in the ride-along kernel, in which every unit brings
    its own activations and no CTA-wide barrier separates the problems (the default); False forces the staged
    kernel for them too.  For measurement and tests; set it before ``prepare`` (the workspace layout depends
    on it)."""
    native.check(native.library().intent_b200_w4a16_gemv_table_ride(1 if enabled else 0),
                 "intent_b200_w4a16_gemv_table_ride")
