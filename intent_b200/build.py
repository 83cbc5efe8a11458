"""In-tree build of ``libintent_b200.so`` (sm_100a only).

``python -m intent_b200.build`` compiles every ``csrc/*.cu`` with nvcc and links
one shared library under ``intent_b200/lib/``.  Nothing is JIT-compiled at run
time: the runtime loads this prebuilt library and fails loudly if it is absent.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = CSRC / "build"
LIB = ROOT / "lib" / "libintent_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(nvcc).exists():
        raise RuntimeError("nvcc not found; the library can only be built with the CUDA toolkit")
    return nvcc


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(source.stat().st_mtime > stamp for source in sources)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + \
        sorted((ROOT.parent / "include").glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    for source in sources:
        obj = OBJ / (source.stem + ".o")
        if force or _stale(obj, [source, *headers]):
            command = [nvcc, *NVCC_FLAGS, "-c", str(source), "-o", str(obj)]
            if verbose:
                command.insert(1, "-Xptxas=-v")
            jobs.append((source, command))

    def run(job):
        source, command = job
        done = subprocess.run(command, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"nvcc failed for {source.name}:\n{done.stdout}\n{done.stderr}")
        # Compiler warnings are never dropped.  One of them is fatal here: without relocatable device code
        # an `extern __device__` declaration silently becomes a private definition (#20044), so a status
        # word "shared" between two files would be two words.
        warnings = [line for line in done.stderr.splitlines() if "warning" in line.lower()]
        if any("20044" in line for line in warnings):
            raise RuntimeError(f"{source.name}: extern device variable without relocatable device code:\n"
                               + done.stderr)
        if verbose:
            sys.stderr.write(done.stderr)
        elif warnings:
            sys.stderr.write(f"[{source.name}]\n" + "\n".join(warnings) + "\n")
        return source

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(run, jobs))

    objects = [OBJ / (source.stem + ".o") for source in sources]
    if force or jobs or _stale(LIB, objects):
        command = [nvcc, "-shared", "-o", str(LIB), *map(str, objects)]
        done = subprocess.run(command, capture_output=True, text=True)
        if done.returncode != 0:
            raise RuntimeError(f"link failed:\n{done.stdout}\n{done.stderr}")
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path, os.path.getsize(path), "bytes")
