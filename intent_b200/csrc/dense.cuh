// Internal entry points of the dense tensor-core kernels, for the programs that decode a
// packed operand into a workspace and then contract it.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ib200 {

// out[M,N] (int32, row pitch N) = a[M,K] . b[N,K]^T, both int8 with K contiguous; exact wrapping
// integers.  K and N multiples of 16, pointers 16-byte aligned.  Returns an INTENT_B200 status.
int i8_gemm_nt(const void* a, int64_t M, int64_t K, const void* b, int64_t N, int32_t* out, cudaStream_t stream);

// out[M,N] (bf16) = bf16(a[M,K] . b[N,K]^T), f32 accumulation.  `row_span` points to two device
// int32 {0, M} (the single row group of the ragged kernel).  K and N multiples of 8.
int bf16_gemm_nt(const void* a, int64_t M, int64_t K, const void* b, int64_t N, void* out, const int32_t* row_span,
                 cudaStream_t stream);

}  // namespace ib200
