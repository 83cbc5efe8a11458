from .artifact import CompiledArtifact, NativeObservation, NativeProgram, PreparedCall  # noqa: F401
from .interface import (BoundArguments, Derived, PublicInterface, ScalarParameter, ViewKind,  # noqa: F401
                        ViewParameter)
