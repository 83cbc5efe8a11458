"""Tiled copies of packed int4 weights for the tensor-core kernels, cached and persisted.

The caller-visible weight format stays the reference's ``[K/8, N]`` int32 matrix
(examples/kernels/contraction/weight_only_int4.py:31-39).  A weight that is static model state can be
re-laid once so that each dequantiser thread of the GEMM kernels fetches its four packed words of a k
block with one 16-byte load (``intent_b200/csrc/w4a16_prelayout.cu``).  The reference treats its own
one-off costs the same way: generated programs and native builds are cached on disk and loaded back
(python/intent/compiler/artifact.py:105-157, python/intent/runtime/native_artifact.py:151-190).

    tiled = prelayout.tile(packed)                 # [K/8, N] or [E, K/8, N] int32 on a CUDA device
    tiled.save(path); tiled = TiledInt4Weight.load(path, device)
    artifact = compile(programs.weight_only_int4_matmul, constexprs={..., "WEIGHT_LAYOUT": "tiled"})
    y = artifact.run(x, tiled.tensor, scales)

or, without touching the call sites, ``constexprs={..., "PRELAYOUT": True}``: the artifact keeps a
:class:`PrelayoutCache` and tiles every distinct weight tensor it is given once.
"""
from __future__ import annotations

import ctypes
import json
from dataclasses import dataclass
from pathlib import Path

from .runtime import native


def words(K: int, N: int) -> int:
    query = native.library().intent_b200_w4a16_prelayout_words
    query.restype = ctypes.c_int64
    query.argtypes = [ctypes.c_int64, ctypes.c_int64]
    return int(query(int(K), int(N)))


@dataclass
class TiledInt4Weight:
    """``tensor``: int32 ``[words]`` (one matrix) or ``[E, words]`` (one row per expert); ``K`` / ``N``: the
    logical shape of the packed matrix ``[K/8, N]`` it was made from."""

    tensor: object
    K: int
    N: int

    @property
    def experts(self) -> int | None:
        return int(self.tensor.shape[0]) if self.tensor.dim() == 2 else None

    def save(self, directory) -> Path:
        """``weight.pt`` (the tiled words) and ``weight.json`` (logical shape) in a new directory."""
        import torch

        path = Path(directory).expanduser().absolute()
        path.mkdir(parents=True, exist_ok=False)
        torch.save(self.tensor.cpu(), path / "weight.pt")
        (path / "weight.json").write_text(json.dumps({"format": "intent_b200.tiled_int4.v1", "K": self.K, "N": self.N,
                                                      "experts": self.experts}) + "\n", encoding="utf-8")
        return path

    @classmethod
    def load(cls, directory, device=None) -> "TiledInt4Weight":
        import torch

        path = Path(directory).expanduser().absolute()
        meta = json.loads((path / "weight.json").read_text(encoding="utf-8"))
        if meta.get("format") != "intent_b200.tiled_int4.v1":
            raise ValueError(f"{path} does not hold a tiled int4 weight")
        tensor = torch.load(path / "weight.pt")
        expected = words(meta["K"], meta["N"])
        if tensor.dtype != torch.int32 or tensor.shape[-1] != expected:
            raise ValueError(f"{path}: stored words do not match K={meta['K']} N={meta['N']}")
        return cls(tensor.to(device) if device is not None else tensor, int(meta["K"]), int(meta["N"]))


def tile(packed) -> TiledInt4Weight:
    """Tiled copy of ``packed`` (``[K/8, N]`` or ``[E, K/8, N]`` int32, contiguous, on a CUDA device).  One
    bandwidth-bound kernel on torch's current stream."""
    import torch

    if not isinstance(packed, torch.Tensor) or packed.dtype != torch.int32 or packed.dim() not in (2, 3):
        raise TypeError("packed must be an int32 tensor [K/8, N] or [E, K/8, N]")
    if not packed.is_cuda or not packed.is_contiguous():
        raise ValueError("packed must be a contiguous CUDA tensor")
    K, N = int(packed.shape[-2]) * 8, int(packed.shape[-1])
    count = words(K, N)
    if count <= 0:
        raise ValueError(f"no tiled layout for K={K}, N={N}")
    library = native.library()
    with torch.cuda.device(packed.device):
        stream = ctypes.c_void_p(torch.cuda.current_stream(packed.device).cuda_stream)
        if packed.dim() == 2:
            out = torch.empty((count,), dtype=torch.int32, device=packed.device)
            entry = library.intent_b200_w4a16_prelayout
            entry.restype = ctypes.c_int
            entry.argtypes = [ctypes.c_void_p] + [ctypes.c_int64] * 4 + [ctypes.c_void_p] + [ctypes.c_int64] * 2 + \
                [ctypes.c_void_p]
            status = entry(packed.data_ptr(), *packed.shape, *packed.stride(), out.data_ptr(), count, 1, stream)
        else:
            out = torch.empty((packed.shape[0], count), dtype=torch.int32, device=packed.device)
            entry = library.intent_b200_w4a16_prelayout_grouped
            entry.restype = ctypes.c_int
            entry.argtypes = [ctypes.c_void_p] + [ctypes.c_int64] * 6 + [ctypes.c_void_p] + [ctypes.c_int64] * 4 + \
                [ctypes.c_void_p]
            status = entry(packed.data_ptr(), *packed.shape, *packed.stride(), out.data_ptr(), *out.shape,
                           *out.stride(), stream)
    native.check(status, "intent_b200_w4a16_prelayout")
    return TiledInt4Weight(out, K, N)


def fingerprint(packed) -> str:
    """A short content key of a packed weight: its shape and 256 words sampled at a fixed stride.  Used to
    recognise, after ``load``, a weight whose tiled copy was saved with the artifact (a collision would need two
    weights of one shape that agree on every sampled word)."""
    flat = packed.reshape(-1)
    step = max(1, flat.numel() // 256)
    sample = flat[::step][:256].cpu().tolist()
    digest = 1469598103934665603
    for value in (*packed.shape, *sample):
        digest = ((digest ^ (int(value) & 0xFFFFFFFFFFFFFFFF)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return f"{digest:016x}"


class PrelayoutCache:
    """Tiled copies by weight tensor.  A live tensor is recognised by (address, version counter, shape): a
    weight that is modified through torch gets a new copy, a weight modified behind torch's back does not -
    this cache is for static model weights.  ``export`` / ``restore`` move the copies to and from disk; a
    restored copy is matched to a tensor by :func:`fingerprint` the first time the tensor is seen."""

    def __init__(self, limit: int = 256):
        self._live: dict = {}
        self._restored: dict = {}
        self.limit = limit
        self.repacks = 0

    def get(self, packed) -> TiledInt4Weight:
        key = (packed.data_ptr(), packed._version, tuple(packed.shape), packed.device.index)
        entry = self._live.get(key)
        if entry is not None:
            return entry[0]
        tiled = None
        if self._restored:
            mark = fingerprint(packed)
            stored = self._restored.pop(mark, None)
            if stored is not None and stored.tensor.shape[-1] == words(int(packed.shape[-2]) * 8, int(packed.shape[-1])):
                tiled = TiledInt4Weight(stored.tensor.to(packed.device), stored.K, stored.N)
        if tiled is None:
            tiled = tile(packed)
            self.repacks += 1
        if len(self._live) >= self.limit:
            self._live.pop(next(iter(self._live)))
        self._live[key] = (tiled, packed)      # the packed tensor is kept alive so its address cannot be reused
        return tiled

    def export(self, directory) -> int:
        """Writes every cached copy under ``directory/<fingerprint>/``; returns how many were written."""
        root = Path(directory)
        written = 0
        for tiled, packed in self._live.values():
            target = root / fingerprint(packed)
            if not target.exists():
                tiled.save(target)
                written += 1
        return written

    def restore(self, directory) -> int:
        root = Path(directory)
        if not root.is_dir():
            return 0
        for child in sorted(root.iterdir()):
            if (child / "weight.json").exists():
                self._restored[child.name] = TiledInt4Weight.load(child)
        return len(self._restored)
