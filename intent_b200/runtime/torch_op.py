"""PyTorch custom-operator registration of an artifact.

Mirrors python/intent/runtime/torch.py:27-93: the schema is built from the
public inputs (``Tensor``, ``Tensor(aN!)`` for writable views, ``SymInt`` /
``float`` / ``bool`` scalars), declared Out buffers become fresh return values,
InOut parameters are declared as mutated, and the fake implementation runs the
same binder without pointers or launches.  Autograd is never inferred.
"""
from __future__ import annotations

from inspect import Parameter, Signature

from .interface import ScalarParameter, ViewParameter


def register_operator(artifact, name: str):
    import torch

    interface = artifact.interface
    if artifact.device_type != "cuda" or not hasattr(artifact.runtime, "infer_outputs"):
        raise NotImplementedError("PyTorch registration requires a CUDA tensor runtime with output inference")
    inputs = interface.inputs
    views = tuple((index, parameter) for index, parameter in enumerate(inputs)
                  if isinstance(parameter, ViewParameter))
    if not views:
        raise NotImplementedError("PyTorch registration requires an input tensor to determine device dispatch")
    interface.require_output_allocation()
    pieces = name.split("::")
    if len(pieces) != 2 or not all(piece.isidentifier() for piece in pieces):
        raise ValueError("operator name must be 'your_namespace::your_operator'")

    mutable_names = tuple(f"arg{index}" for index, parameter in views if parameter.writable)
    alias_pairs = tuple((li, ri, left.name, right.name)
                        for position, (li, left) in enumerate(views)
                        for ri, right in views[position + 1:]
                        if left.writable or right.writable)
    declared = []
    for index, parameter in enumerate(inputs):
        if isinstance(parameter, ViewParameter):
            kind = f"Tensor(a{index}!)" if parameter.writable else "Tensor"
        elif isinstance(parameter, ScalarParameter):
            category = parameter.dtype.category
            if category == "bool":
                kind = "bool"
            elif category in ("int", "uint"):
                kind = "SymInt"
            elif category in ("float", "bfloat"):
                kind = "float"
            else:
                raise NotImplementedError(f"PyTorch scalar schema for {parameter.dtype}")
        declared.append(f"{kind} arg{index}")
    outputs = interface.outputs
    if not outputs:
        returns = "()"
    elif len(outputs) == 1:
        returns = "Tensor"
    else:
        returns = "(" + ", ".join("Tensor" for _ in outputs) + ")"
    schema = f"({', '.join(declared)}) -> {returns}"
    signature = Signature(Parameter(f"arg{index}", Parameter.POSITIONAL_OR_KEYWORD)
                          for index in range(len(declared)))

    def wrap(invoke):
        def operator(*arguments, **keywords):
            arguments = signature.bind(*arguments, **keywords).args
            for left, right, left_name, right_name in alias_pairs:
                if torch._C._is_alias_of(arguments[left], arguments[right]):
                    raise NotImplementedError(
                        "PyTorch mutable calls require independent input storage: "
                        f"{left_name} and {right_name} share storage; use ordinary artifact calls for this binding")
            return invoke(*arguments)

        return operator

    operator = torch.library.custom_op(name, wrap(artifact.run), mutates_args=mutable_names,
                                       device_types=artifact.device_type, schema=schema)
    operator.register_fake(wrap(lambda *arguments: artifact.runtime.infer_outputs(arguments)))
    return operator
