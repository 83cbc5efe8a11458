"""Typed public interface of a compiled program and the argument binder.

Behavioural mirror of the reference's call-surface contract
(python/intent/runtime/interface.py:99-245, runtime/invocation.py:56-159,
runtime/torch_views.py:23-82, runtime/native_requirements.py:66-91):

  * ``Out`` parameters are omitted from ``run``/``prepare`` and allocated with
    ``torch.empty`` on the artifact's device; ``InOut`` is always supplied.
  * Nothing is coerced.  ``TypeError``: wrong argument count, non-tensor,
    dtype mismatch.  ``ValueError``: wrong device, wrong rank, a violated shape
    relation, pointer alignment.  ``NotImplementedError``: an entry requirement
    (canonical contiguous layout, non-overlapping writable views) is not met,
    or an output extent cannot be derived from the inputs.

The binder here is a plain interpreter over the declaration (the reference
generates Python source per interface); the checks and their order are the same.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import IntEnum

from ..dtypes import DType, torch_dtype


class ViewKind(IntEnum):
    IN = 0
    OUT = 1
    INOUT = 2


@dataclass(frozen=True)
class Derived:
    """An extent computed from other symbolic dimensions (e.g. ``I = WN // 2``).
    Supplied views are checked against it, omitted Out buffers are sized by it."""

    name: str
    function: object

    def __call__(self, dimensions: dict) -> int:
        return int(self.function(dimensions))


@dataclass(frozen=True, slots=True)
class ScalarParameter:
    position: int
    name: str
    dtype: DType


@dataclass(frozen=True, slots=True)
class ViewParameter:
    position: int
    name: str
    dtype: DType
    shape: tuple            # per axis: int (static extent), str (symbolic dimension) or Derived
    access: ViewKind
    alignment: int = 16     # bytes; entry requirement
    layout: str = "contiguous"

    @property
    def writable(self) -> bool:
        return self.access is not ViewKind.IN

    @property
    def output(self) -> bool:
        return self.access is ViewKind.OUT


@dataclass(slots=True)
class ViewFacts:
    """What one binding observed about one tensor (no addresses when abstract)."""

    shape: tuple
    strides: tuple
    pointer: int | None
    begin: int | None
    end: int | None
    dtype: object


@dataclass(slots=True)
class BoundArguments:
    arguments: tuple          # every parameter in declaration order (tensors / scalars)
    outputs: tuple            # declared Out tensors in declaration order
    views: tuple              # ViewFacts | None per parameter
    dimensions: dict          # symbolic dimension -> extent

    def result(self):
        if not self.outputs:
            return None
        return self.outputs[0] if len(self.outputs) == 1 else self.outputs


def byte_spans_overlap(left: tuple[int, int], right: tuple[int, int]) -> bool:
    return left[0] < left[1] and right[0] < right[1] and left[0] < right[1] and right[0] < left[1]


def _byte_span(pointer: int, shape: tuple, strides: tuple, size: int) -> tuple[int, int]:
    if any(extent == 0 for extent in shape):
        return pointer, pointer
    low = high = 0
    for extent, stride in zip(shape, strides):
        displacement = (extent - 1) * stride
        low += min(0, displacement)
        high += max(0, displacement)
    return pointer + low * size, pointer + (high + 1) * size


class PublicInterface:
    """Ordered runtime parameters of one program specialisation."""

    def __init__(self, parameters: tuple, *, dimension_rules=()) -> None:
        names = set()
        for position, parameter in enumerate(parameters):
            if parameter.position != position:
                raise ValueError("parameter positions must follow declaration order")
            if not parameter.name or parameter.name in names:
                raise ValueError("public parameter names must be nonempty and unique")
            names.add(parameter.name)
        self.parameters = tuple(parameters)
        # callables(dimensions: dict) -> None raising ValueError; derived relations such
        # as "packed rows * 8 == K" that tie symbolic dimensions together.
        self.dimension_rules = tuple(dimension_rules)

    # -- views of the declaration ------------------------------------------------
    @property
    def views(self) -> tuple:
        return tuple(p for p in self.parameters if isinstance(p, ViewParameter))

    @property
    def inputs(self) -> tuple:
        return tuple(p for p in self.parameters if not isinstance(p, ViewParameter) or not p.output)

    @property
    def outputs(self) -> tuple:
        return tuple(p for p in self.views if p.output)

    @property
    def mutable_inputs(self) -> tuple:
        return tuple(p for p in self.views if p.access is ViewKind.INOUT)

    def explicit_arguments(self, arguments: tuple, outputs: tuple) -> tuple:
        if len(arguments) != len(self.inputs):
            raise TypeError(f"expected {len(self.inputs)} input arguments, got {len(arguments)}")
        if len(outputs) != len(self.outputs):
            raise TypeError(f"expected {len(self.outputs)} explicit output buffers, got {len(outputs)}")
        supplied, allocated = iter(arguments), iter(outputs)
        return tuple(next(allocated) if isinstance(p, ViewParameter) and p.output else next(supplied)
                     for p in self.parameters)

    def output_allocation_errors(self) -> tuple:
        """Out extents that no supplied parameter determines."""
        known = set()
        for parameter in self.inputs:
            if isinstance(parameter, ViewParameter):
                known.update(e for e in parameter.shape if isinstance(e, str))
        errors = []
        for parameter in self.outputs:
            for axis, extent in enumerate(parameter.shape):
                if isinstance(extent, str) and extent not in known:
                    errors.append(f"{parameter.name}.shape[{axis}] has no extent supplied by inputs "
                                  "or fixed by the public shape declarations")
        return tuple(errors)

    def require_output_allocation(self) -> None:
        errors = self.output_allocation_errors()
        if errors:
            raise NotImplementedError(
                "Cannot allocate the declared outputs: " + "; ".join(errors) +
                ". Provide explicit output buffers with prepare(..., outputs=(...)) or launch(...).")

    # -- binding -----------------------------------------------------------------
    def _observe(self, parameter: ViewParameter, value, device, abstract: bool) -> ViewFacts:
        import torch

        if not isinstance(value, torch.Tensor):
            raise TypeError(f"{parameter.name} must be a torch.Tensor")
        expected = torch_dtype(parameter.dtype)
        if value.dtype != expected:
            raise TypeError(f"{parameter.name} must have dtype {expected}, got {value.dtype}")
        if value.device != device:
            raise ValueError(f"{parameter.name} must be on {device}, got {value.device}")
        shape, strides = tuple(value.shape), tuple(value.stride())
        if len(shape) != len(parameter.shape):
            raise ValueError(f"{parameter.name} must have rank {len(parameter.shape)}, got {len(shape)}")
        if abstract:
            return ViewFacts(shape, strides, None, None, None, value.dtype)
        pointer = value.data_ptr()
        begin, end = _byte_span(pointer, shape, strides, value.element_size())
        return ViewFacts(shape, strides, pointer, begin, end, value.dtype)

    @staticmethod
    def _check_relation(actual, expected, message: str, abstract: bool) -> None:
        if abstract:
            import torch

            torch._check(actual == expected, lambda: message)
        elif actual != expected:
            raise ValueError(message)

    def _check_entry_requirements(self, parameter: ViewParameter, facts: ViewFacts, abstract: bool,
                                  allocated: bool) -> None:
        if parameter.layout == "contiguous":
            expected = 1
            for extent, stride in zip(reversed(facts.shape), reversed(facts.strides)):
                if extent != 1 and stride != expected and not abstract:
                    message = f"{parameter.name}: native entry requires canonical contiguous element strides"
                    if allocated:
                        message += "; provide explicit output buffers with the required layout"
                    raise NotImplementedError(message)
                expected *= extent
        if not abstract and facts.pointer is not None and facts.pointer % parameter.alignment:
            raise ValueError(f"{parameter.name}: native entry requires {parameter.alignment}-byte pointer alignment")

    def bind(self, arguments: tuple, *, device, explicit_outputs: bool = False,
             abstract: bool = False) -> BoundArguments:
        """Validate ``arguments`` against the declaration and allocate omitted
        Out buffers.  ``explicit_outputs``: every parameter is supplied in
        declaration order.  ``abstract``: shape relations only (fake tensors), no
        address facts, no entry-storage checks."""
        import torch

        supplied = self.parameters if explicit_outputs else self.inputs
        if len(arguments) != len(supplied):
            raise TypeError(f"expected {len(supplied)} runtime arguments, got {len(arguments)}")
        if not explicit_outputs:
            self.require_output_allocation()
        values: list = [None] * len(self.parameters)
        facts: list = [None] * len(self.parameters)
        dimensions: dict = {}

        deferred: list = []

        def relate(parameter: ViewParameter, observed: ViewFacts) -> None:
            for axis, extent in enumerate(parameter.shape):
                message = f"{parameter.name}.shape[{axis}] violates the declared interface relation"
                if isinstance(extent, Derived):
                    deferred.append((extent, observed.shape[axis], message))
                elif isinstance(extent, int):
                    self._check_relation(observed.shape[axis], extent, message, abstract)
                elif extent in dimensions:
                    self._check_relation(observed.shape[axis], dimensions[extent], message, abstract)
                else:
                    dimensions[extent] = observed.shape[axis]

        for parameter, value in zip(supplied, arguments):
            values[parameter.position] = value
            if isinstance(parameter, ViewParameter):
                observed = self._observe(parameter, value, device, abstract)
                relate(parameter, observed)
                self._check_entry_requirements(parameter, observed, abstract, allocated=False)
                facts[parameter.position] = observed
            else:
                if isinstance(value, torch.Tensor):
                    raise TypeError(f"{parameter.name} must be a Python scalar")
                if parameter.dtype.category in ("int", "uint") and not isinstance(value, (int, torch.SymInt)):
                    raise TypeError(f"{parameter.name} must be an integer")
        for extent, actual, message in deferred:
            try:
                expected = extent(dimensions)
            except KeyError:
                continue        # depends on a dimension only an omitted output would bind
            self._check_relation(actual, expected, message, abstract)
        if not abstract:
            for rule in self.dimension_rules:
                rule(dimensions)
        if not explicit_outputs:
            for parameter in self.outputs:
                shape = tuple(extent if isinstance(extent, int) else
                              (extent(dimensions) if isinstance(extent, Derived) else dimensions[extent])
                              for extent in parameter.shape)
                value = torch.empty(shape, dtype=torch_dtype(parameter.dtype), device=device)
                observed = self._observe(parameter, value, device, abstract)
                self._check_entry_requirements(parameter, observed, abstract, allocated=True)
                values[parameter.position] = value
                facts[parameter.position] = observed
        if not abstract:
            views = self.views
            for index, left in enumerate(views):
                for right in views[index + 1:]:
                    if not (left.writable or right.writable):
                        continue
                    a, b = facts[left.position], facts[right.position]
                    if byte_spans_overlap((a.begin, a.end), (b.begin, b.end)):
                        raise NotImplementedError(
                            f"{left.name} and {right.name}: native entry requires nonoverlapping accessed byte spans")
        outputs = tuple(values[p.position] for p in self.outputs)
        return BoundArguments(tuple(values), outputs, tuple(facts), dimensions)
