"""``artifact.as_torch_op("ns::name")``: the artifact as a ``torch.library`` custom operator.

Contract taken from the reference (python/intent/runtime/torch.py:27-93): the operator's arguments are
the artifact's public inputs in declaration order; a writable tensor is declared as mutated; declared
``Out`` buffers come back as fresh return values; the fake (meta) implementation infers output shapes
with the same binder and launches nothing; autograd is not registered.

The schema text is assembled from two small tables (scalar category -> schema type, number of outputs ->
return clause); the operator body is one closure that first applies the aliasing rule for mutated
arguments and then forwards to ``run`` (real tensors) or to shape inference (fake tensors).
"""
from __future__ import annotations

from dataclasses import dataclass

from .interface import ScalarParameter, ViewParameter

# schema type of a scalar parameter by dtype category
_SCALAR_SCHEMA = {"bool": "bool", "int": "SymInt", "uint": "SymInt", "float": "float", "bfloat": "float"}


@dataclass(frozen=True)
class _Slot:
    """One operator argument: its schema declaration and what the aliasing rule needs to know."""

    name: str
    declaration: str
    tensor: bool
    mutated: bool
    label: str


def _slots(interface) -> tuple:
    slots = []
    for position, parameter in enumerate(interface.inputs):
        name = f"arg{position}"
        if isinstance(parameter, ViewParameter):
            kind = f"Tensor(a{position}!)" if parameter.writable else "Tensor"
            slots.append(_Slot(name, f"{kind} {name}", True, parameter.writable, parameter.name))
        elif isinstance(parameter, ScalarParameter):
            kind = _SCALAR_SCHEMA.get(parameter.dtype.category)
            if kind is None:
                raise NotImplementedError(f"no operator schema type for scalar {parameter.name}: {parameter.dtype}")
            slots.append(_Slot(name, f"{kind} {name}", False, False, parameter.name))
        else:
            raise NotImplementedError(f"parameter {position} is neither a view nor a scalar")
    return tuple(slots)


def _returns(count: int) -> str:
    if count == 0:
        return "()"
    if count == 1:
        return "Tensor"
    return "(" + ", ".join(["Tensor"] * count) + ")"


def _qualified(name: str) -> None:
    namespace, separator, operator = name.partition("::")
    if not separator or "::" in operator or not namespace.isidentifier() or not operator.isidentifier():
        raise ValueError(f"{name!r} is not an operator name of the form 'namespace::operator'")


def register_operator(artifact, name: str):
    import torch

    if artifact.device_type != "cuda" or not hasattr(artifact.runtime, "infer_outputs"):
        raise NotImplementedError("as_torch_op needs a CUDA artifact whose runtime can infer output shapes")
    interface = artifact.interface
    slots = _slots(interface)
    tensors = [index for index, slot in enumerate(slots) if slot.tensor]
    if not tensors:
        raise NotImplementedError("as_torch_op needs at least one tensor input: the dispatcher picks the "
                                  "device from it")
    interface.require_output_allocation()
    _qualified(name)
    schema = f"({', '.join(slot.declaration for slot in slots)}) -> {_returns(len(interface.outputs))}"
    # a mutated tensor may not share storage with any other tensor argument of the same call
    guarded = [(a, b) for i, a in enumerate(tensors) for b in tensors[i + 1:]
               if slots[a].mutated or slots[b].mutated]
    names = [slot.name for slot in slots]

    def positional(arguments, keywords):
        if len(arguments) > len(names):
            raise TypeError(f"{name} takes {len(names)} arguments, got {len(arguments)}")
        values = list(arguments)
        for slot_name in names[len(arguments):]:
            if slot_name not in keywords:
                raise TypeError(f"{name} is missing argument {slot_name}")
            values.append(keywords[slot_name])
        unknown = set(keywords) - set(names[len(arguments):])
        if unknown:
            raise TypeError(f"{name} got unexpected arguments {sorted(unknown)}")
        return values

    def body(target):
        def call(*arguments, **keywords):
            values = positional(arguments, keywords)
            for a, b in guarded:
                if torch._C._is_alias_of(values[a], values[b]):
                    raise NotImplementedError(
                        f"{name}: {slots[a].label} and {slots[b].label} share storage, and one of them is "
                        "written by the operator; call the artifact directly for such a binding")
            return target(*values)

        return call

    operator = torch.library.custom_op(name, body(artifact.run), schema=schema,
                                       mutates_args=tuple(slot.name for slot in slots if slot.mutated),
                                       device_types=artifact.device_type)
    operator.register_fake(body(lambda *values: artifact.runtime.infer_outputs(values)))
    return operator
