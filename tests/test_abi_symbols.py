"""The C-ABI library loads without a GPU and exports every symbol the public
header declares (no compute calls here)."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def library():
    from intent_b200.build import build

    return ctypes.CDLL(str(build()))


def declared_symbols():
    text = (ROOT / "include" / "intent_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"INTENT_B200_API\s+[\w\s\*]+?\b(intent_b200_\w+)\s*\(", text)))


def test_header_declares_entries():
    names = declared_symbols()
    assert "intent_b200_weight_only_int4_matmul_f16" in names
    assert "intent_b200_version" in names


def test_every_declared_symbol_is_exported(library):
    missing = [name for name in declared_symbols() if not hasattr(library, name)]
    assert not missing, f"declared in include/intent_b200.h but not exported: {missing}"


def test_identity_and_status_strings(library):
    library.intent_b200_version.restype = ctypes.c_char_p
    library.intent_b200_status_string.restype = ctypes.c_char_p
    assert b"sm_100a" in library.intent_b200_version()
    assert library.intent_b200_status_string(0) == b"ok"
    assert b"contiguous" in library.intent_b200_status_string(2)
    library.intent_b200_launch_count.restype = ctypes.c_int64
    assert library.intent_b200_launch_count() >= 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import intent_b200.runtime.native as native
    from intent_b200 import CompilationStageError

    monkeypatch.setenv("INTENT_B200_LIB", str(tmp_path / "nope.so"))
    monkeypatch.setattr(native, "_LIBRARY", None)
    with pytest.raises(CompilationStageError) as info:
        native.library()
    assert info.value.stage == "native_loading"
    monkeypatch.setattr(native, "_LIBRARY", None)


def declared_slot_counts():
    """Number of C parameters of every declared entry, with the view macros expanded
    (a view of rank r is a pointer, r extents and r strides)."""
    text = (ROOT / "include" / "intent_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S).replace("\\\n", " ")
    macros = dict(re.findall(r"#define\s+(INTENT_B200_\w+_SLOTS)\s+(.*)", text))
    counts = {}
    for name, arguments in re.findall(r"INTENT_B200_API\s+[\w\s\*]+?\b(intent_b200_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
        for macro, body in macros.items():
            arguments = arguments.replace(macro, body)
        total = 0
        for argument in (a.strip() for a in re.split(r",(?![^()]*\))", arguments)):
            view = re.match(r"INTENT_B200_VIEW(\d)\(", argument)
            total += 1 + 2 * int(view.group(1)) if view else (0 if argument in ("", "void") else 1)
        counts[name] = total
    return counts


def test_programs_marshal_what_the_header_declares():
    """Every shipped program passes exactly the slots its C entry declares: views, compile-time
    constants, the optional workspace pair and the stream."""
    import intent_b200 as ib

    declared = declared_slot_counts()
    assert declared["intent_b200_gemm_i8"] == 5 + 5 + 3 + 5 + 1
    checked = 0
    for definition in ib.programs.ALL.values():
        artifact = ib.compile(definition, resolve_target=False)
        program = artifact.runtime
        slots = len(program._carriers_head) + (2 if program._workspace_spec is not None else 0) + 1
        assert program.entry_name in declared, program.entry_name
        assert declared[program.entry_name] == slots, (definition.name, program.entry_name, declared[program.entry_name], slots)
        checked += 1
    assert checked == len(ib.programs.ALL) >= 29
