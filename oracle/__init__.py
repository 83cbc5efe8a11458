"""CPU oracle for the quantized-contraction programs.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: only the test-suite, the smoke check and the bench's CPU-baseline /
reference arm call into it, as the checker or as the timed CPU baseline, never
as a product code path.

Every function restates, in torch-CPU / numpy, the math of one program of the
reference project (IntentDSL).  Each docstring cites the reference kernel body
and the reference's own torch-CPU implementation it follows.

Pinning status: the restatements are checked against outputs of the
reference's torch-CPU implementations (``experiments/cpu/baselines/pytorch/
cpu_runtime.py``) imported unmodified; the vectors are committed under
``tests/golden/`` together with the script that generated them.  The
reference itself ships no golden vectors for this path.
"""
from .contraction import (  # noqa: F401
    gemm,
    quantized_gemm,
    pack_int4,
    unpack_int4,
    dequantize_int4,
    weight_only_int4_matmul,
    weight_only_int4_matmul_rounded,
    gemm_i8,
    gemm_i8_exact_f64,
    w8a8_scaled_gemm,
)
from .routing import (  # noqa: F401
    softmax_f32,
    insertion_top_k,
    moe_route_top2,
    moe_count_routes,
    moe_align_block_size,
    canonical_alignment,
)
from .moe import (  # noqa: F401
    ragged_grouped_gemm,
    routed_expert_projection,
    moe_expert_ffn,
    silu_and_mul,
    moe_w4a16_swiglu_ffn,
    grouped_w4a16_gemm,
)
from .packed import (  # noqa: F401
    bitnet_int2_matmul,
    decode_fp4_bf16,
    dequant_bf16_fp4_matmul,
    unpack_bitnet_int2,
    unpack_w4a8,
    w4a8_packed_matmul,
)
from .quantized import (  # noqa: F401
    q4_k_fields,
    q8_k_quantize,
    quantized_dot,
    quantized_projection,
)
