"""Host-side call surface on CPU: binder checks, output allocation, error types
(the reference raises and never coerces: python/intent/runtime/invocation.py:94-150,
torch_views.py:32-43, native_requirements.py:66-91)."""
import pytest
import torch

import intent_b200 as ib
from intent_b200.runtime.interface import PublicInterface, ViewKind, ViewParameter

CPU = torch.device("cpu")


@pytest.fixture(scope="module")
def artifact():
    return ib.compile(ib.programs.weight_only_int4_matmul, constexprs={"GROUP_SIZE": 128, "ZERO_POINT": 8},
                      resolve_target=False)


def _inputs(M=4, K=256, N=64, dtype=torch.float16):
    return ib.workloads.w4a16_inputs(M, K, N, dtype=dtype)


def test_interface_declaration(artifact):
    interface = artifact.interface
    assert [p.name for p in interface.parameters] == ["activation", "packed_weight", "scales", "output"]
    assert [p.name for p in interface.inputs] == ["activation", "packed_weight", "scales"]
    assert [p.name for p in interface.outputs] == ["output"]
    assert interface.mutable_inputs == ()
    assert "weight_only_int4.py" in artifact.source and artifact.mlir
    assert artifact.device_type == "cuda" and artifact.entry == artifact.__call__


def test_bind_allocates_outputs(artifact):
    x, p, s = _inputs()
    bound = artifact.interface.bind((x, p, s), device=CPU)
    assert bound.result().shape == (4, 64) and bound.result().dtype == torch.float16
    assert bound.dimensions == {"M": 4, "K": 256, "P": 32, "N": 64, "G": 2}


def test_bind_errors(artifact):
    interface = artifact.interface
    x, p, s = _inputs()
    with pytest.raises(TypeError):
        interface.bind((x, p), device=CPU)                       # argument count
    with pytest.raises(TypeError):
        interface.bind((x.numpy(), p, s), device=CPU)             # not a tensor
    with pytest.raises(TypeError):
        interface.bind((x.float(), p, s), device=CPU)             # dtype is never coerced
    with pytest.raises(ValueError):
        interface.bind((x[0], p, s), device=CPU)                  # rank
    with pytest.raises(ValueError):
        interface.bind((x, p, s[:, :32].contiguous()), device=CPU)  # N relation
    with pytest.raises(ValueError):
        interface.bind((x, p[:16].contiguous(), s), device=CPU)     # P * 8 == K
    with pytest.raises(ValueError):
        interface.bind((x, p, torch.cat((s, s))), device=CPU)       # G * group == K
    with pytest.raises(NotImplementedError):
        interface.bind((x.t().contiguous().t(), p, s), device=CPU)  # non-canonical strides
    with pytest.raises(ValueError):
        interface.bind((x, p, s), device=torch.device("meta"))      # device


def test_bind_alignment_and_overlap(artifact):
    interface = artifact.interface
    x, p, s = _inputs()
    storage = torch.zeros(4 * 256 + 8, dtype=torch.float16)
    misaligned = storage[1:1 + 4 * 256].view(4, 256)
    assert misaligned.data_ptr() % 16 != 0
    with pytest.raises(ValueError, match="alignment"):
        interface.bind((misaligned, p, s), device=CPU)
    # explicit output that overlaps an input
    shared = torch.zeros(4 * 256, dtype=torch.float16)
    xin = shared.view(4, 256)
    out = shared[:4 * 64].view(4, 64)
    with pytest.raises(NotImplementedError, match="nonoverlapping"):
        interface.bind((xin, p, s, out), device=CPU, explicit_outputs=True)


def test_explicit_outputs_and_argument_merge(artifact):
    interface = artifact.interface
    x, p, s = _inputs()
    out = torch.empty((4, 64), dtype=torch.float16)
    merged = interface.explicit_arguments((x, p, s), (out,))
    assert merged[3] is out
    bound = interface.bind(merged, device=CPU, explicit_outputs=True)
    assert bound.outputs[0] is out
    with pytest.raises(ValueError):
        interface.bind((x, p, s, torch.empty((4, 32), dtype=torch.float16)), device=CPU, explicit_outputs=True)
    with pytest.raises(TypeError):
        interface.explicit_arguments((x, p, s), ())


def test_unallocatable_output():
    interface = PublicInterface((
        ViewParameter(0, "a", ib.dtypes.f32, ("M",), ViewKind.IN),
        ViewParameter(1, "b", ib.dtypes.f32, ("Q",), ViewKind.OUT),
    ))
    with pytest.raises(NotImplementedError, match="explicit output"):
        interface.bind((torch.zeros(4),), device=CPU)
    bound = interface.bind((torch.zeros(4), torch.zeros(7)), device=CPU, explicit_outputs=True)
    assert bound.dimensions == {"M": 4, "Q": 7}


def test_abstract_binding_has_no_addresses(artifact):
    x, p, s = _inputs()
    bound = artifact.interface.bind((x, p, s), device=CPU, abstract=True)
    assert all(f is None or f.pointer is None for f in bound.views)
    assert bound.result().shape == (4, 64)


def test_compile_errors():
    with pytest.raises(ib.CompilationStageError) as info:
        ib.compile(ib.programs.weight_only_int4_matmul, constexprs={"NOPE": 1}, resolve_target=False)
    assert info.value.stage == "frontend_kir"
    with pytest.raises(ib.CompilationStageError) as info:
        ib.compile(ib.programs.weight_only_int4_matmul, constexprs={"GROUP_SIZE": 48}, resolve_target=False)
    assert info.value.stage == "provider_native_compilation"
    with pytest.raises(ib.CompilationStageError) as info:
        ib.compile(lambda: None, resolve_target=False)
    assert info.value.stage == "frontend_kir"
    if not torch.cuda.is_available():
        with pytest.raises(ib.CompilationStageError) as info:
            ib.compile(ib.programs.weight_only_int4_matmul)
        assert info.value.stage == "target_resolution"


def test_tuning_is_declined(artifact):
    with pytest.raises(NotImplementedError):
        artifact.tuning_configurations()


def test_artifact_rejects_wrong_device(artifact):
    x, p, s = _inputs()
    with pytest.raises(ValueError, match="bound to"):
        artifact.run(x, p, s)          # CPU tensors handed to a CUDA artifact


# ---- dense ragged programs: declaration mirrors the reference's parameter order ------------------
def test_dense_grouped_declarations():
    ragged = ib.compile(ib.programs.ragged_grouped_gemm_bf16, resolve_target=False)
    assert [p.name for p in ragged.interface.parameters] == ["x", "group_offsets", "weight", "y"]
    routed = ib.compile(ib.programs.routed_expert_projection_bf16, constexprs={"TOP_K": 4}, resolve_target=False)
    assert [p.name for p in routed.interface.parameters] == ["x", "expert_offsets", "member_routes", "weight", "output"]
    ffn = ib.compile(ib.programs.moe_expert_ffn, resolve_target=False)
    assert [p.name for p in ffn.interface.parameters] == ["x", "route_offsets", "member_routes", "route_token",
                                                          "route_weights", "w1", "w2", "y"]
    assert [p.name for p in ffn.interface.mutable_inputs] == ["y"] and ffn.interface.outputs == ()

    x = torch.zeros((10, 64), dtype=torch.bfloat16)
    w = torch.zeros((3, 32, 64), dtype=torch.bfloat16)                  # [E, N, K]
    offsets = torch.zeros((4,), dtype=torch.int32)
    members = torch.zeros((40,), dtype=torch.int32)
    bound = routed.interface.bind((x, offsets, members, w), device=CPU)
    assert bound.result().shape == (10, 4, 32)
    with pytest.raises(ValueError):
        routed.interface.bind((x, offsets[:3].contiguous(), members, w), device=CPU)     # E + 1 offsets
    with pytest.raises(ValueError):
        routed.interface.bind((x, offsets, members, torch.zeros((3, 32, 60), dtype=torch.bfloat16)), device=CPU)  # K
    with pytest.raises(TypeError):
        routed.interface.bind((x.half(), offsets, members, w), device=CPU)
    with pytest.raises(TypeError):
        ffn.interface.bind((x.half(),), device=CPU)


# ---- artifact persistence (the reference's save / load / materialize) ------------------------------
def test_artifact_save_and_load(tmp_path):
    artifact = ib.compile(ib.programs.weight_only_int4_matmul, resolve_target=False,
                          constexprs={"GROUP_SIZE": 128, "ZERO_POINT": 8, "ACT_DTYPE": "bf16"})
    path = artifact.save(tmp_path / "w4a16")
    assert sorted(p.name for p in path.iterdir()) == ["artifact.json", "kernel.mlir", "kernel.source"]
    restored = ib.load(path, resolve_target=False)
    assert restored.metadata == artifact.metadata and restored.cache_directory == path
    assert [p.name for p in restored.interface.parameters] == [p.name for p in artifact.interface.parameters]
    assert restored.runtime.entry_name == artifact.runtime.entry_name == "intent_b200_weight_only_int4_matmul_bf16"
    with pytest.raises(ib.CompilationStageError) as error:
        artifact.save(path)                                   # the destination must be new
    assert error.value.stage == "generated_program_export"
    (path / "artifact.json").write_text('{"provider": "other"}')
    with pytest.raises(ib.CompilationStageError) as error:
        ib.load(path, resolve_target=False)
    assert error.value.stage == "generated_program_loading"
    with pytest.raises(ib.CompilationStageError):
        ib.load(tmp_path / "missing", resolve_target=False)


def test_torch_operator_schema_and_fake_inference_without_a_device():
    """as_torch_op: schema from the public inputs, mutated InOut views, fresh Out returns, and shape inference
    under fake tensors - none of which needs a GPU."""
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode

    import intent_b200 as ib

    artifact = ib.compile(ib.programs.weight_only_int4_matmul, target=ib.B200Target(0), resolve_target=False,
                          constexprs={"GROUP_SIZE": 128, "ZERO_POINT": 8})
    operator = artifact.as_torch_op("intent_b200_cpu_test::w4a16")
    assert str(operator._schema) == "(Tensor arg0, Tensor arg1, Tensor arg2) -> Tensor"
    with FakeTensorMode():
        fake = operator(torch.empty((4, 1024), dtype=torch.float16, device="cuda"),
                        torch.empty((128, 256), dtype=torch.int32, device="cuda"),
                        arg2=torch.empty((8, 256), dtype=torch.float16, device="cuda"))
        assert fake.shape == (4, 256) and fake.dtype == torch.float16
    combine = ib.compile(ib.programs.moe_combine, target=ib.B200Target(0), resolve_target=False)
    schema = str(combine.as_torch_op("intent_b200_cpu_test::combine")._schema)
    assert schema == "(Tensor arg0, Tensor arg1, Tensor arg2, Tensor(a3!) arg3) -> ()"
    for bad in ("no_namespace", "a::b::c", "9a::b", "a::"):
        with pytest.raises(ValueError):
            artifact.as_torch_op(bad)
