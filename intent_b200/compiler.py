"""``compile(definition, target=..., constexprs=...) -> CompiledArtifact``.

Stands where the reference's ``intent.compile`` stands
(python/intent/compiler/pipeline.py:19-34) for the programs this backend
ships.  Nothing is generated or JIT-compiled: "compiling" selects a prebuilt
sm_100a entry point of ``libintent_b200.so`` from the program id and its
compile-time constants, and binds it to one device.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable

from .errors import CompilationStageError
from .runtime.artifact import CompiledArtifact
from .targets import B200Target


@dataclass(frozen=True)
class KernelDefinition:
    """One shipped program: name, compile-time constants with their defaults,
    and the function that lowers a constant assignment to a provider runtime."""

    name: str
    constexprs: dict
    lower: Callable = field(repr=False, compare=False)
    reference: str = ""      # reference kernel body this program implements (file:line)
    summary: str = ""

    def __call__(self, *args, **kwargs):
        raise TypeError(f"{self.name} is a kernel definition; compile it with intent_b200.compile(...)")


def compile(definition: KernelDefinition, *, target: B200Target | None = None,
            constexprs: dict | None = None, resolve_target: bool = True) -> CompiledArtifact:
    """Return the callable artifact of ``definition`` on ``target``.

    ``constexprs`` overrides the definition's compile-time constants; unknown
    names or unsupported values raise ``CompilationStageError('frontend_kir')``
    / ``('provider_native_compilation')``.  ``resolve_target=False`` skips the
    device probe (interface inspection and fake-tensor tracing on machines
    without a GPU); launching such an artifact still requires the device.
    """
    if not isinstance(definition, KernelDefinition):
        raise CompilationStageError(
            "frontend_kir",
            "this backend ships fixed programs; pass one of intent_b200.programs.* "
            f"(got {type(definition).__name__})")
    if target is None:
        import torch

        target = B200Target(torch.cuda.current_device() if torch.cuda.is_available() else 0)
    if resolve_target:
        target.resolve()
    constants = dict(definition.constexprs)
    for name, value in (constexprs or {}).items():
        if name not in constants:
            raise CompilationStageError("frontend_kir", f"{definition.name} has no constexpr {name!r}; "
                                        f"known: {sorted(constants)}")
        constants[name] = value
    program = definition.lower(constants, target.device)
    description = (f"// {definition.name}  [{definition.reference}]\n"
                   f"// provider: b200 (prebuilt sm_100a), entry: {program.entry_name}\n"
                   f"// constexprs: {constants}\n")
    artifact = CompiledArtifact(source=description, mlir=description, device=target.device, runtime=program,
                                device_type=target.device_type)
    artifact.metadata = {"provider": "b200", "program": definition.name, "entry_name": program.entry_name,
                         "constexprs": {k: _plain(v) for k, v in constants.items()},
                         "reference": definition.reference,
                         "parameters": [p.name for p in program.interface.parameters]}
    return artifact


def _plain(value):
    """Compile-time constants as JSON values (enum members by name)."""
    if isinstance(value, (bool, int, float, str)) or value is None:
        return value
    return getattr(value, "name", str(value))


def load(directory, *, target: B200Target | None = None, resolve_target: bool = True) -> CompiledArtifact:
    """Rebuild an artifact from a directory written by ``CompiledArtifact.save``: the stored program
    id and compile-time constants select the prebuilt entry again and bind it to ``target``.  Stands
    where ``GeneratedProgram.load(...).materialize(target=...)`` stands in the reference
    (python/intent/compiler/artifact.py:131-177); no native code is stored in the directory."""
    import json
    from pathlib import Path

    from . import programs

    path = Path(directory).expanduser().absolute()
    try:
        source = (path / "kernel.source").read_text(encoding="utf-8")
        metadata = json.loads((path / "artifact.json").read_text(encoding="utf-8"))
        if not source.strip() or not isinstance(metadata, dict):
            raise ValueError("a saved program needs nonempty source and object metadata")
        if metadata.get("provider") != "b200":
            raise ValueError(f"artifact was written by provider {metadata.get('provider')!r}, not 'b200'")
        definition = programs.ALL[metadata["program"]]
        constants = metadata["constexprs"]
        if not isinstance(constants, dict):
            raise TypeError("constexprs must be an object")
    except (OSError, UnicodeError, ValueError, KeyError, TypeError) as error:
        raise CompilationStageError("generated_program_loading", f"{type(error).__name__}: {error}",
                                    cache_directory=path) from error
    artifact = compile(definition, target=target, constexprs=constants, resolve_target=resolve_target)
    artifact.cache_directory = path
    cache = getattr(artifact.runtime, "cache", None)
    if cache is not None:       # tiled weight copies saved with the artifact are matched to weights by content key
        cache.restore(path / "prelayout")
    return artifact
