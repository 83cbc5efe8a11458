"""Element types of the public interface (names follow the reference's
``intent.language`` dtype names: i8, i32, f16, bf16, f32 ...)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True, slots=True)
class DType:
    name: str
    bits: int
    category: str  # "int" | "uint" | "float" | "bfloat" | "bool"

    def __repr__(self) -> str:
        return self.name

    @property
    def bytes(self) -> int:
        return (self.bits + 7) // 8


i8 = DType("i8", 8, "int")
i16 = DType("i16", 16, "int")
i32 = DType("i32", 32, "int")
i64 = DType("i64", 64, "int")
u8 = DType("u8", 8, "uint")
f16 = DType("f16", 16, "float")
bf16 = DType("bf16", 16, "bfloat")
f32 = DType("f32", 32, "float")
f64 = DType("f64", 64, "float")
boolean = DType("bool", 8, "bool")

_BY_NAME = {d.name: d for d in (i8, i16, i32, i64, u8, f16, bf16, f32, f64, boolean)}
_TORCH_NAMES = {"i8": "int8", "i16": "int16", "i32": "int32", "i64": "int64", "u8": "uint8",
                "f16": "float16", "bf16": "bfloat16", "f32": "float32", "f64": "float64", "bool": "bool"}


def dtype(value) -> DType:
    """Accept a DType, its name, or a torch dtype."""
    if isinstance(value, DType):
        return value
    if isinstance(value, str):
        if value in _BY_NAME:
            return _BY_NAME[value]
        raise ValueError(f"unknown element type {value!r}")
    import torch

    if isinstance(value, torch.dtype):
        for name, torch_name in _TORCH_NAMES.items():
            if getattr(torch, torch_name) is value:
                return _BY_NAME[name]
    raise ValueError(f"unknown element type {value!r}")


def torch_dtype(element: DType):
    import torch

    return getattr(torch, _TORCH_NAMES[element.name])
