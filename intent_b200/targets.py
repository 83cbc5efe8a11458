"""Target description.  The reference resolves a GPU target into device
capabilities through the CUDA driver (python/intent/targets/gpu/target.py:33-50,
targets/gpu/device.py:6-59); this backend has exactly one target."""
from __future__ import annotations

from dataclasses import dataclass

from .errors import CompilationStageError


@dataclass(frozen=True, slots=True)
class ResolvedTarget:
    device: int
    name: str
    compute_capability: tuple[int, int]
    multiprocessors: int
    shared_memory_per_block: int
    l2_bytes: int
    total_memory: int


@dataclass(frozen=True, slots=True)
class B200Target:
    """One Blackwell (sm_100) GPU of this process, by CUDA device ordinal."""

    device: int = 0
    device_type: str = "cuda"

    def resolve(self, *, require_device: bool = True) -> ResolvedTarget | None:
        import torch

        if not torch.cuda.is_available():
            if require_device:
                raise CompilationStageError("target_resolution", "no CUDA device is visible")
            return None
        if not 0 <= self.device < torch.cuda.device_count():
            raise CompilationStageError("target_resolution", f"CUDA device {self.device} does not exist")
        props = torch.cuda.get_device_properties(self.device)
        if props.major != 10:
            raise CompilationStageError(
                "target_resolution",
                f"device {self.device} ({props.name}) has compute capability {props.major}.{props.minor}; "
                "this backend contains sm_100a code only")
        return ResolvedTarget(self.device, props.name, (props.major, props.minor),
                              props.multi_processor_count,
                              getattr(props, "shared_memory_per_block_optin", 0),
                              getattr(props, "L2_cache_size", 0), props.total_memory)
