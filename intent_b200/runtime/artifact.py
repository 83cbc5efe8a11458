"""The callable artifact: same call surface as the reference's
``CompiledArtifact`` / ``PreparedCall`` (python/intent/runtime/artifact.py:22-53,
98-237; GPU program python/intent/runtime/gpu/program.py:33-131).

  artifact.run(*inputs)            allocate Out buffers, launch, return None / Out / tuple
  artifact(*all) / .launch(*all)   every parameter supplied, returns None
  artifact.prepare(*inputs, outputs=...) -> PreparedCall(.compile/.launch/.result)
  artifact.as_torch_op("ns::name") -> torch.library.CustomOpDef

Launches are asynchronous on torch's current CUDA stream of the artifact's
device.  ``PreparedCall.launch`` neither allocates nor synchronises, so it can
be captured in a CUDA graph.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

from ..errors import CompilationStageError
from . import native
from .interface import BoundArguments, PublicInterface, ScalarParameter, ViewParameter


@dataclass(frozen=True, slots=True)
class NativeObservation:
    """Facts about the latest invocation of an entry (never an estimate).  The resource fields are what the
    reference's observation reports for a native call (registers, spills, shared memory, the selected
    configuration: python/intent/runtime/diagnostics.py:119-137); they come from the library's dry-run
    observation of the same slots and are None for entries whose kernels do not take part in it."""

    provider: str
    entry: str
    stage: str
    constants: tuple
    arguments: tuple          # per view: (name, shape, strides)
    workspace_bytes: int
    status: int
    kernel: str | None = None            # kernel family and the launch plan's choice
    registers: int | None = None         # per thread
    spill_bytes: int | None = None       # per-thread local memory
    shared_static: int | None = None     # bytes
    shared_dynamic: int | None = None    # bytes
    threads: int | None = None           # per CTA
    grid: int | None = None              # CTAs
    cluster: int | None = None           # CTAs per cluster


class _LaunchFacts(ctypes.Structure):
    _fields_ = [("valid", ctypes.c_int32), ("registers", ctypes.c_int32), ("local_bytes", ctypes.c_int32),
                ("static_smem", ctypes.c_int32), ("dynamic_smem", ctypes.c_int32), ("threads", ctypes.c_int32),
                ("grid", ctypes.c_int32), ("cluster", ctypes.c_int32), ("kernel", ctypes.c_char * 64)]


# entries made only of kernels that honour the dry-run observation
_OBSERVABLE = ("intent_b200_weight_only_int4_matmul", "intent_b200_w4a16_gemv", "intent_b200_w4a16_gemm",
               "intent_b200_gemm_i8", "intent_b200_w8a8_gemm", "intent_b200_ragged_grouped_gemm",
               "intent_b200_routed_expert_projection", "intent_b200_moe_expert_ffn", "intent_b200_gemm_f16",
               "intent_b200_bf16_gemm", "intent_b200_quantized_gemm", "intent_b200_moe_grouped_w4a16")


class PreparedCall:
    """Arguments bound to one C entry; ``launch`` replays the same call."""

    def __init__(self, program: "NativeProgram", bound: BoundArguments, workspace: tuple | None = None) -> None:
        self.program = program
        self.invocation = bound
        self._workspace = program.allocate_workspace(bound) if workspace is None else workspace
        self._slots = program.marshal(bound, self._workspace)
        self._observation: NativeObservation | None = None
        self._skip = program.is_empty(bound)
        self._facts: dict | None = None     # resource facts of this binding, observed once

    @property
    def outputs(self) -> tuple:
        return self.invocation.outputs

    def result(self):
        return self.invocation.result()

    @property
    def observation(self) -> NativeObservation | None:
        return self._observation

    def inspect_configurations(self):
        raise NotImplementedError("this provider does not export structured tuning configurations")

    def compile(self) -> None:
        """Nothing is compiled at run time; this resolves the exported symbol."""
        self.program.function()

    def check(self) -> None:
        """Synchronise the current stream and raise ``CompilationStageError('provider_invocation')`` if a
        bounded device-side wait of an earlier launch of this call gave up (its output is then incomplete).
        A workspace that such a launch left dirty is cleared, so the call can be launched again."""
        self.program.check(self._workspace)

    def launch(self) -> None:
        import torch

        program = self.program
        if self._skip:
            return
        if torch.cuda.current_device() != program.device:
            with torch.cuda.device(program.device):
                self._invoke()
        else:
            self._invoke()

    __call__ = launch

    def _observe(self, stream: int) -> dict:
        """The same slots once more in the library's dry-run mode: nothing is launched, the entry reports the
        kernel instance it selects for them and that instance's resource usage."""
        program = self.program
        if not program.entry_name.startswith(_OBSERVABLE):
            return {}
        library = native.library()
        facts = _LaunchFacts()
        if library.intent_b200_observe_begin(ctypes.byref(facts)) != 0:
            return {}
        try:
            status = program.function()(*self._slots, ctypes.c_void_p(stream))
        finally:
            library.intent_b200_observe_end()
        if status != 0 or not facts.valid:
            return {}
        return {"kernel": facts.kernel.decode(), "registers": facts.registers, "spill_bytes": facts.local_bytes,
                "shared_static": facts.static_smem, "shared_dynamic": facts.dynamic_smem, "threads": facts.threads,
                "grid": facts.grid, "cluster": facts.cluster}

    def _invoke(self) -> None:
        import torch

        program = self.program
        stream = torch.cuda.current_stream(program.device).cuda_stream
        status = program.function()(*self._slots, ctypes.c_void_p(stream))
        if self._facts is None:
            self._facts = self._observe(stream) if status == 0 else {}
        observation = NativeObservation(
            "b200", program.entry_name, "launched" if status == 0 else "failed", program.constants,
            tuple((p.name, f.shape, f.strides) for p, f in zip(program.interface.parameters, self.invocation.views)
                  if f is not None),
            sum(w.numel() * w.element_size() for w in self._workspace), int(status), **self._facts)
        self._observation = observation
        program._observation = observation
        native.check(status, program.entry_name, observation)


# Which process-wide status word the tensor-core kernels behind an entry write when a bounded wait gives up
# (entry-name prefix -> C reader).  The bandwidth kernel keeps its word in the caller's workspace instead.
_W4, _I8, _DENSE = ("intent_b200_w4a16_gemm_device_status", "intent_b200_i8_gemm_device_status",
                    "intent_b200_grouped_gemm16_device_status")
_STATUS_READERS = (
    ("intent_b200_weight_only_int4_matmul", (_W4,)), ("intent_b200_w4a16_gemm", (_W4,)),
    ("intent_b200_moe_grouped_w4a16", (_W4,)),
    ("intent_b200_gemm_i8", (_I8,)), ("intent_b200_w8a8_gemm", (_I8,)), ("intent_b200_w4a8_packed", (_I8,)),
    ("intent_b200_bitnet_int2", (_I8,)),
    ("intent_b200_ragged_grouped_gemm", (_DENSE,)), ("intent_b200_routed_expert_projection", (_DENSE,)),
    ("intent_b200_moe_expert_ffn", (_DENSE,)), ("intent_b200_gemm_f16", (_DENSE,)),
    ("intent_b200_bf16_gemm", (_DENSE,)), ("intent_b200_quantized_gemm", (_DENSE,)),
    ("intent_b200_dequant_bf16_fp4", (_DENSE,)),
)


def _status_readers(entry_name: str) -> tuple:
    for prefix, readers in _STATUS_READERS:
        if entry_name.startswith(prefix):
            return readers
    return ()


class NativeProgram:
    """Provider runtime of one program specialisation bound to one device."""

    def __init__(self, *, interface: PublicInterface, entry_name: str, constants: tuple = (),
                 device: int, workspace=None, empty=None, scalar_carriers=None,
                 workspace_status: str | None = None, device_status: tuple = ()) -> None:
        self.interface = interface
        self.entry_name = entry_name
        self.constants = tuple(int(c) for c in constants)
        self.device = device
        self._workspace_spec = workspace     # callable(dimensions) -> workspace bytes (0 = none)
        self._stream_workspaces: dict = {}   # stream handle -> zero-initialised buffer reused by run()
        self._empty = empty                  # callable(dimensions) -> bool
        self._observation: NativeObservation | None = None
        # where this entry's kernels record a bounded wait that gave up: the first word of its workspace
        # (read by the named C function) and / or process-wide status words with a no-argument reader
        self._workspace_status = workspace_status
        self._device_status = tuple(device_status) or _status_readers(entry_name)
        carriers = []
        for parameter in interface.parameters:
            if isinstance(parameter, ViewParameter):
                rank = len(parameter.shape)
                carriers += ["ptr"] + ["i64"] * (2 * rank)
            else:
                carriers.append((scalar_carriers or {}).get(parameter.name) or _scalar_carrier(parameter))
        carriers += ["i32"] * len(self.constants)
        self._carriers_head = tuple(carriers)
        self._function = None
        self._workspace_count = None

    # ---- C entry -----------------------------------------------------------------
    def function(self, workspace_count: int | None = None):
        if workspace_count is None:
            workspace_count = self._workspace_count or 0
        if self._function is None or self._workspace_count != workspace_count:
            carriers = self._carriers_head + ("ptr", "i64") * workspace_count
            self._function = native.entry(self.entry_name, carriers)
            self._workspace_count = workspace_count
        return self._function

    @property
    def observation(self):
        return self._observation

    @property
    def _torch_device(self):
        import torch

        return torch.device("cuda", self.device)

    def check(self, workspace: tuple | None = None) -> None:
        """Read the device-side status of this entry's kernels (synchronises).  ``workspace``: the buffers of
        one prepared call; None = the per-stream buffers that ``run`` reuses."""
        import torch

        library = native.library()
        failures = []
        with torch.cuda.device(self.device):
            stream = torch.cuda.current_stream(self.device).cuda_stream
            if self._workspace_status is not None:
                reader = getattr(library, self._workspace_status)
                reader.restype = ctypes.c_int
                reader.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p]
                buffers = workspace if workspace is not None else tuple(self._stream_workspaces.values())
                for buffer in buffers:
                    if buffer.numel() >= 4:
                        failures.append(int(reader(ctypes.c_void_p(buffer.data_ptr()),
                                                   ctypes.c_int64(buffer.numel() * buffer.element_size()),
                                                   ctypes.c_void_p(stream))))
            for name in self._device_status:
                reader = getattr(library, name)
                reader.restype = ctypes.c_int
                reader.argtypes = []
                failures.append(int(reader()))
        for status in failures:
            native.check(status, self.entry_name, self._observation)

    def is_empty(self, bound: BoundArguments) -> bool:
        return bool(self._empty(bound.dimensions)) if self._empty is not None else False

    def allocate_workspace(self, bound: BoundArguments, *, per_stream: bool = False) -> tuple:
        """Scratch for one binding.  Entries keep their scratch zero-filled across
        launches, so it is zeroed once here.  ``per_stream`` reuses one buffer for
        successive calls on the current stream (what ``run`` does); a prepared
        call owns a private buffer."""
        import torch

        if self._workspace_spec is None:
            return ()
        size = int(self._workspace_spec(bound.dimensions))
        if size <= 0:
            return (torch.empty((0,), dtype=torch.uint8, device=self._torch_device),)
        if not per_stream:
            return (torch.zeros((size,), dtype=torch.uint8, device=self._torch_device),)
        key = torch.cuda.current_stream(self.device).cuda_stream
        cached = self._stream_workspaces.get(key)
        if cached is None or cached.numel() < size:
            cached = torch.zeros((max(size, 1 << 16),), dtype=torch.uint8, device=self._torch_device)
            self._stream_workspaces[key] = cached
        return (cached,)

    def marshal(self, bound: BoundArguments, workspace: tuple) -> tuple:
        slots = []
        for parameter, value, facts in zip(self.interface.parameters, bound.arguments, bound.views):
            if isinstance(parameter, ViewParameter):
                slots.append(ctypes.c_void_p(facts.pointer))
                slots += [ctypes.c_int64(int(e)) for e in facts.shape]
                slots += [ctypes.c_int64(int(s)) for s in facts.strides]
            else:
                slots.append(value)
        slots += [ctypes.c_int32(c) for c in self.constants]
        for buffer in workspace:
            slots.append(ctypes.c_void_p(buffer.data_ptr() if buffer.numel() else None))
            slots.append(ctypes.c_int64(buffer.numel() * buffer.element_size()))
        self.function(len(workspace))
        return tuple(slots)

    # ---- call modes ----------------------------------------------------------------
    def prepare(self, *arguments, outputs: tuple | None = None, explicit_outputs: bool = False) -> PreparedCall:
        if outputs is not None:
            arguments = self.interface.explicit_arguments(tuple(arguments), tuple(outputs))
            explicit_outputs = True
        bound = self.interface.bind(tuple(arguments), device=self._torch_device,
                                    explicit_outputs=explicit_outputs)
        return PreparedCall(self, bound)

    def prepare_call(self, arguments: tuple, *, outputs: tuple | None = None) -> PreparedCall:
        return self.prepare(*arguments, outputs=outputs)

    def run(self, *arguments):
        bound = self.interface.bind(tuple(arguments), device=self._torch_device)
        call = PreparedCall(self, bound, self.allocate_workspace(bound, per_stream=True))
        call.launch()
        return call.result()

    def launch(self, *arguments) -> None:
        self.prepare(*arguments, explicit_outputs=True).launch()

    def infer_outputs(self, arguments: tuple):
        """Shape inference for fake tensors: no pointers, no launch."""
        device = arguments and next((a.device for a in arguments if hasattr(a, "device")), None)
        return self.interface.bind(tuple(arguments), device=device or self._torch_device, abstract=True).result()


def _scalar_carrier(parameter: ScalarParameter) -> str:
    name = parameter.dtype.name
    if name in ("i8", "i16", "i32", "i64", "f32", "f64", "bool"):
        return name
    raise NotImplementedError(f"native scalar carrier for {name}")


@dataclass(slots=True)
class CompiledArtifact:
    source: str
    mlir: str
    device: int
    runtime: Any = field(repr=False)
    device_type: str = field(default="cuda", kw_only=True)
    cache_directory: Path | None = field(default=None, kw_only=True)
    backend_ir: dict = field(default_factory=dict, init=False)

    metadata: dict = field(default_factory=dict, init=False, repr=False)

    def save(self, directory) -> Path:
        """Write ``kernel.source``, ``kernel.mlir`` and ``artifact.json`` into a new directory (the
        reference's artifact layout, python/intent/compiler/artifact.py:105-129).  The device binding
        and native handles are not stored; ``intent_b200.load`` binds the program again."""
        import json
        import tempfile

        from ..errors import CompilationStageError

        path = Path(directory).expanduser().absolute()
        try:
            if path.exists():
                raise FileExistsError(f"generated program destination already exists: {path}")
            if not self.metadata:
                raise ValueError("this artifact was not produced by intent_b200.compile")
            path.parent.mkdir(parents=True, exist_ok=True)
            with tempfile.TemporaryDirectory(prefix=f".{path.name}-", dir=path.parent) as temporary:
                staging = Path(temporary) / "program"
                staging.mkdir()
                (staging / "kernel.source").write_text(self.source, encoding="utf-8")
                (staging / "kernel.mlir").write_text(self.mlir, encoding="utf-8")
                (staging / "artifact.json").write_text(json.dumps(self.metadata, indent=2) + "\n", encoding="utf-8")
                cache = getattr(self.runtime, "cache", None)      # PRELAYOUT artifacts: the tiled weight copies
                if cache is not None:
                    cache.export(staging / "prelayout")
                staging.rename(path)
        except (OSError, UnicodeError, TypeError, ValueError) as error:
            raise CompilationStageError("generated_program_export", str(error),
                                        cache_directory=self.cache_directory) from error
        return path

    @property
    def observation(self):
        """Latest native invocation snapshot, or None before the first launch."""
        return getattr(self.runtime, "observation", None)

    @property
    def entry(self):
        return self.__call__

    @property
    def ir(self) -> dict:
        return {"intent": self.mlir, **self.backend_ir}

    @property
    def interface(self) -> PublicInterface:
        return self.runtime.interface

    def run(self, *arguments: Any):
        """Allocate declared Out buffers and execute with inputs in declaration order."""
        return self._invoke(self.runtime.run, arguments)

    def prepare(self, *arguments: Any, outputs: tuple | None = None) -> PreparedCall:
        """Bind arguments and allocate outputs/workspace without executing."""
        return self._invoke(lambda *args: self.runtime.prepare_call(args, outputs=outputs), arguments)

    def launch(self, *arguments: Any) -> None:
        """Execute with every runtime argument, including explicit Out buffers."""
        self._invoke(self.runtime.launch, arguments)

    __call__ = launch

    def check(self) -> None:
        """Synchronise and raise if a bounded device-side wait gave up in an earlier ``run`` / ``launch`` of
        this artifact (an addition to the reference's surface: its providers have no device-side waits)."""
        self.runtime.check()

    def as_torch_op(self, name: str):
        from .torch_op import register_operator

        return register_operator(self, name)

    def tuning_configurations(self, *arguments: Any):
        raise NotImplementedError("this provider does not export structured tuning configurations")

    def inspect_configurations(self, *arguments: Any, outputs: tuple | None = None):
        return self.prepare(*arguments, outputs=outputs).inspect_configurations()

    def _invoke(self, function, arguments: tuple):
        import torch

        expected = torch.device(self.device_type, self.device)
        for index, argument in enumerate(arguments):
            if isinstance(argument, torch.Tensor) and argument.device != expected:
                raise ValueError(f"compiled artifact is bound to {expected}, but tensor argument "
                                 f"{index} is on {argument.device}")
        if torch.cuda.current_device() == self.device:
            return function(*arguments)
        with torch.cuda.device(self.device):
            return function(*arguments)
