"""intent_b200: sm_100a quantized-contraction programs behind IntentDSL's
artifact call surface (``run`` / ``__call__`` / ``prepare`` / ``as_torch_op``)."""
from . import dtypes, moe, programs, runtime, workloads  # noqa: F401
from .compiler import KernelDefinition, compile, load  # noqa: F401
from .errors import CompilationStageError  # noqa: F401
from .runtime.artifact import CompiledArtifact, NativeObservation, PreparedCall  # noqa: F401
from .runtime.interface import PublicInterface, ScalarParameter, ViewKind, ViewParameter  # noqa: F401
from .targets import B200Target  # noqa: F401

__all__ = ["compile", "load", "programs", "B200Target", "CompilationStageError", "CompiledArtifact",
           "PreparedCall", "KernelDefinition", "PublicInterface", "dtypes", "workloads"]
