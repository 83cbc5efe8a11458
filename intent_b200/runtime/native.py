"""ctypes binding of ``libintent_b200.so``.

The library is loaded once per process under a lock (the reference does the
same for its CPU providers, python/intent/runtime/native_artifact.py:193-213,
258-276).  There is no fallback: a missing library or symbol raises
``CompilationStageError('native_loading', ...)``.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from threading import Lock

from ..errors import CompilationStageError

_LOCK = Lock()
_LIBRARY: ctypes.CDLL | None = None
_ENTRIES: dict = {}

_CARRIERS = {"ptr": ctypes.c_void_p, "bool": ctypes.c_bool, "i8": ctypes.c_int8, "i16": ctypes.c_int16,
             "i32": ctypes.c_int32, "i64": ctypes.c_int64, "f32": ctypes.c_float, "f64": ctypes.c_double}


def library_path() -> Path:
    override = os.environ.get("INTENT_B200_LIB")
    if override:
        return Path(override)
    return Path(__file__).resolve().parent.parent / "lib" / "libintent_b200.so"


def library() -> ctypes.CDLL:
    global _LIBRARY
    with _LOCK:
        if _LIBRARY is None:
            path = library_path()
            if not path.exists():
                raise CompilationStageError(
                    "native_loading",
                    f"{path} is missing; build it with `python -m intent_b200.build` "
                    "(there is no CPU or eager fallback)")
            try:
                _LIBRARY = ctypes.CDLL(str(path))
            except OSError as error:
                raise CompilationStageError("native_loading", f"cannot load {path}: {error}") from error
            _LIBRARY.intent_b200_version.restype = ctypes.c_char_p
            _LIBRARY.intent_b200_status_string.restype = ctypes.c_char_p
            _LIBRARY.intent_b200_status_string.argtypes = [ctypes.c_int]
            _LIBRARY.intent_b200_launch_count.restype = ctypes.c_int64
        return _LIBRARY


def entry(name: str, carriers: tuple):
    """Bind one exported entry; ``carriers`` names the slot types in order
    (without the trailing stream pointer, which is always appended)."""
    lib = library()
    key = (name, carriers)
    with _LOCK:
        function = _ENTRIES.get(key)
        if function is None:
            try:
                function = getattr(lib, name)
            except AttributeError as error:
                raise CompilationStageError("native_loading", f"{library_path()} does not export {name}") from error
            function.restype = ctypes.c_int
            function.argtypes = [_CARRIERS[c] for c in carriers] + [ctypes.c_void_p]
            _ENTRIES[key] = function
        return function


def status_string(status: int) -> str:
    return library().intent_b200_status_string(int(status)).decode()


def launch_count() -> int:
    return int(library().intent_b200_launch_count())


def version() -> str:
    return library().intent_b200_version().decode()


def check(status: int, entry_name: str, observation=None) -> None:
    if status != 0:
        raise CompilationStageError("provider_invocation",
                                    f"{entry_name} returned status {status}: {status_string(status)}",
                                    observation=observation, status=status)


def set_gemv_launch_overlap(enabled: bool) -> None:
    """Process-wide switch of the bandwidth kernel's programmatic dependent launch: a launch may
    request its packed weights while the previous kernel on the stream is still running.  Only
    valid when the weights are not written by the kernel launched immediately before (static model
    weights in a decode loop)."""
    check(library().intent_b200_w4a16_gemv_overlap(1 if enabled else 0), "intent_b200_w4a16_gemv_overlap")
