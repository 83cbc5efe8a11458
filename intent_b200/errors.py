"""Error taxonomy kept from the reference (python/intent/compiler/toolchain.py:17-26):
one exception class carrying the pipeline stage that failed."""
from __future__ import annotations


class CompilationStageError(RuntimeError):
    """A compile / load / invoke stage failed.

    ``stage`` uses the reference's stage names where a counterpart exists:
    ``frontend_kir`` (unknown program or constexpr), ``target_resolution``,
    ``provider_native_compilation`` (no prebuilt specialisation),
    ``native_loading`` (shared library or symbol missing),
    ``provider_invocation`` (the C entry returned a non-zero status).
    """

    def __init__(self, stage: str, message: str, *, cache_directory=None, candidate=None,
                 observation=None, status: int | None = None) -> None:
        super().__init__(f"[{stage}] {message}")
        self.stage = stage
        self.message = message
        self.cache_directory = cache_directory
        self.candidate = candidate
        self.observation = observation
        self.status = status
