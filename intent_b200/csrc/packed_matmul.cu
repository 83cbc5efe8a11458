// Packed-weight contractions that sit next to weight_only_int4_matmul in the reference
// (examples/kernels/contraction/weight_only_int4.py:54-175):
//
//   w4a8_packed_matmul        out[N,M] i32 = s4(W)[N,K] . A[M,K]^T      W: u8 [N,K/2], low nibble = even k
//   bitnet_int2_matmul        out[M,N] i32 = A[M,K] . u2(W)[N,K]^T      W: u8 [N,K/4], 16 values per 4-byte word
//   dequant_bf16_fp4_matmul   out[M,N] bf16 = A[M,K] . e2m1(W)[N,K]^T   W: u8 [N,K/2], 4 codes per 16-bit word
//
// Each program decodes the packed operand once into a K-major workspace (a bandwidth-bound
// pass: it reads the packed bytes and writes 2x / 4x / 4x as many) and then runs the dense
// tcgen05 kernel on it (kind::i8 with exact s32 accumulation, or kind::f16 on bf16).  The
// integer programs are bit-exact with wrapping int32 arithmetic.  The int2 program with at most 16
// activation rows (decode) skips both: a dp4a GEMV reads the packed weights once.
#include "common.cuh"
#include "dense.cuh"

namespace ib200 {
namespace {

// (x & 0x0F0F0F0F per byte) -> sign-extended int4 per byte
__device__ __forceinline__ uint32_t sign_extend_nibbles(uint32_t nibbles) {
  return __vsub4(nibbles ^ 0x08080808u, 0x08080808u);
}

// 16 packed bytes (32 nibbles) -> 32 int8, k order: byte b holds k = 2b (low) and 2b + 1 (high)
__global__ void expand_w4_kernel(const uint4* __restrict__ packed, uint4* __restrict__ out, int64_t vectors) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < vectors; i += int64_t(gridDim.x) * blockDim.x) {
    const uint4 v = ldg_stream_v4(packed + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t lo = sign_extend_nibbles(w[j] & 0x0F0F0F0Fu);
      const uint32_t hi = sign_extend_nibbles((w[j] >> 4) & 0x0F0F0F0Fu);
      o[2 * j] = prmt(lo, hi, 0x5140);      // l0 h0 l1 h1
      o[2 * j + 1] = prmt(lo, hi, 0x7362);  // l2 h2 l3 h3
    }
    out[2 * i] = make_uint4(o[0], o[1], o[2], o[3]);
    out[2 * i + 1] = make_uint4(o[4], o[5], o[6], o[7]);
  }
}

// One 4-byte word holds 16 two-bit values: value k sits in byte k % 4 at bit 2 * (k / 4), so
// (word >> 2L) & 0x03030303 is the four values 4L .. 4L+3 in output byte order.
__global__ void expand_int2_kernel(const uint32_t* __restrict__ packed, uint4* __restrict__ out, int64_t words) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < words; i += int64_t(gridDim.x) * blockDim.x) {
    const uint32_t w = __ldg(packed + i);
    out[i] = make_uint4(w & 0x03030303u, (w >> 2) & 0x03030303u, (w >> 4) & 0x03030303u, (w >> 6) & 0x03030303u);
  }
}

__device__ __forceinline__ uint32_t fp4_bits_to_bf16(uint32_t bits) {
  // the code's sign / exponent / mantissa bits already sit at bf16 positions; scaling by 2^126
  // turns the tiny value (subnormal for exponent 0) into 0, 0.5, 1, 1.5, 2, 3, 4 or 6
  const float value = __uint_as_float(bits << 16) * 8.507059173023462e37f;  // 2^126
  return uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(value)));
}

// 4 packed bytes = two big-endian 16-bit words = 8 codes -> 8 bf16 (16 bytes)
__global__ void expand_fp4_kernel(const uint32_t* __restrict__ packed, uint4* __restrict__ out, int64_t words,
                                  int32_t* row_span, int32_t rows) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    row_span[0] = 0;
    row_span[1] = rows;
  }
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < words; i += int64_t(gridDim.x) * blockDim.x) {
    const uint32_t w = __ldg(packed + i);
    uint32_t o[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const uint32_t first = (w >> (16 * h)) & 0xFFu, second = (w >> (16 * h + 8)) & 0xFFu;
      const uint32_t word = (first << 8) | second;
      const uint32_t d0 = word & 0x81C0u;
      const uint32_t d1 = (word << 3) & 0x81C0u;
      const uint32_t d2 = (word << 6) & 0x81C0u;
      const uint32_t d3 = ((word << 1) & 0x8000u) | ((word >> 3) & 0x0180u) | ((word >> 7) & 0x0040u);
      o[2 * h] = fp4_bits_to_bf16(d0) | (fp4_bits_to_bf16(d1) << 16);
      o[2 * h + 1] = fp4_bits_to_bf16(d2) | (fp4_bits_to_bf16(d3) << 16);
    }
    out[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// Few activation rows (decode): no decode pass and no tensor core.  One warp per weight row n walks
// the packed row once; (word >> 2L) & 0x03030303 are the four values 16j + 4L .. + 3 as bytes, which
// meet the four activation bytes of the same k in one dp4a.  Exact int32 arithmetic.
template <int ROWS>
__global__ void int2_gemv_kernel(const int8_t* __restrict__ activation, const uint32_t* __restrict__ packed,
                                 int32_t* __restrict__ out, int M, int N, int K) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int words = K >> 4;  // 16 values per packed word
  for (int n = warp; n < N; n += warps) {
    const uint32_t* row = packed + size_t(n) * words;
    for (int m0 = 0; m0 < M; m0 += ROWS) {
      int acc[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) acc[r] = 0;
      for (int j = lane; j < words; j += 32) {
        const uint32_t w = __ldg(row + j);
        const uint32_t v0 = w & 0x03030303u, v1 = (w >> 2) & 0x03030303u, v2 = (w >> 4) & 0x03030303u,
                       v3 = (w >> 6) & 0x03030303u;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          if (m0 + r < M) {
            const int4 a = __ldg(reinterpret_cast<const int4*>(activation + size_t(m0 + r) * K) + j);
            acc[r] = __dp4a(int(v0), a.x, acc[r]);
            acc[r] = __dp4a(int(v1), a.y, acc[r]);
            acc[r] = __dp4a(int(v2), a.z, acc[r]);
            acc[r] = __dp4a(int(v3), a.w, acc[r]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], d);
        if (lane == 0 && m0 + r < M) out[size_t(m0 + r) * N + n] = acc[r];
      }
    }
  }
}

inline int grid_for(int64_t items, int threads) {
  const int64_t blocks = (items + threads - 1) / threads;
  return int(blocks < 148 * 8 ? (blocks > 0 ? blocks : 1) : 148 * 8);
}

inline int64_t align256(int64_t bytes) { return (bytes + 255) & ~int64_t(255); }

int check_views(const View2& activation, const View2& packed, const View2& output) {
  if (!activation.p || !packed.p || !output.p) return INTENT_B200_ERR_NULL;
  if (!contiguous(activation) || !contiguous(packed) || !contiguous(output) || !aligned16(activation.p) ||
      !aligned16(packed.p) || !aligned16(output.p))
    return INTENT_B200_ERR_LAYOUT;
  return INTENT_B200_OK;
}

}  // namespace
}  // namespace ib200

// a0 activation i8 [M,K], a1 packed_weight u8 [N,K/2] -> a2 output i32 [N,M]
extern "C" int intent_b200_w4a8_packed_matmul(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                              void* workspace, int64_t workspace_bytes, void* stream_) {
  using namespace ib200;
  const int64_t M = a0_d0, K = a0_d1, N = a1_d0, P = a1_d1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (P * 2 != K || a2_d0 != N || a2_d1 != M) return INTENT_B200_ERR_SHAPE;
  if (M == 0 || N == 0) return INTENT_B200_OK;
  int status = check_views(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2));
  if (status != INTENT_B200_OK) return status;
  if (K == 0 || K % 32 != 0 || M % 16 != 0) return INTENT_B200_ERR_UNSUPPORTED;
  if (!workspace || !aligned16(workspace) || workspace_bytes < align256(N * K)) return INTENT_B200_ERR_WORKSPACE;
  const int64_t vectors = N * P / 16;
  expand_w4_kernel<<<grid_for(vectors, 256), 256, 0, stream>>>(static_cast<const uint4*>(a1),
                                                              static_cast<uint4*>(workspace), vectors);
  note_launch();
  status = launch_status();
  if (status != INTENT_B200_OK) return status;
  // rows of the product are the weight rows: out[N,M] = W8[N,K] . A[M,K]^T
  return i8_gemm_nt(workspace, N, K, a0, M, static_cast<int32_t*>(a2), stream);
}

// a0 activation i8 [M,K], a1 packed_weight u8 [N,K/4] -> a2 output i32 [M,N]
extern "C" int intent_b200_bitnet_int2_matmul(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                              void* workspace, int64_t workspace_bytes, void* stream_) {
  using namespace ib200;
  const int64_t M = a0_d0, K = a0_d1, N = a1_d0, P = a1_d1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (P * 4 != K || a2_d0 != M || a2_d1 != N) return INTENT_B200_ERR_SHAPE;
  if (M == 0 || N == 0) return INTENT_B200_OK;
  int status = check_views(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2));
  if (status != INTENT_B200_OK) return status;
  if (K == 0 || K % 16 != 0 || N % 16 != 0) return INTENT_B200_ERR_UNSUPPORTED;
  if (M <= 16) {  // decode: one pass over the packed weights
    const int64_t warps_needed = N;
    const int blocks = int(warps_needed / 8 < 148 * 8 ? (warps_needed + 7) / 8 : 148 * 8);
    if (M <= 4)
      int2_gemv_kernel<4><<<blocks, 256, 0, stream>>>(static_cast<const int8_t*>(a0), static_cast<const uint32_t*>(a1),
                                                     static_cast<int32_t*>(a2), int(M), int(N), int(K));
    else
      int2_gemv_kernel<8><<<blocks, 256, 0, stream>>>(static_cast<const int8_t*>(a0), static_cast<const uint32_t*>(a1),
                                                     static_cast<int32_t*>(a2), int(M), int(N), int(K));
    note_launch();
    return launch_status();
  }
  if (!workspace || !aligned16(workspace) || workspace_bytes < align256(N * K)) return INTENT_B200_ERR_WORKSPACE;
  const int64_t words = N * P / 4;
  expand_int2_kernel<<<grid_for(words, 256), 256, 0, stream>>>(static_cast<const uint32_t*>(a1),
                                                              static_cast<uint4*>(workspace), words);
  note_launch();
  status = launch_status();
  if (status != INTENT_B200_OK) return status;
  return i8_gemm_nt(a0, M, K, workspace, N, static_cast<int32_t*>(a2), stream);
}

// a0 activation bf16 [M,K], a1 packed_weight u8 [N,K/2] -> a2 output bf16 [M,N]
extern "C" int intent_b200_dequant_bf16_fp4_matmul(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                   INTENT_B200_VIEW2(a2), void* workspace, int64_t workspace_bytes,
                                                   void* stream_) {
  using namespace ib200;
  const int64_t M = a0_d0, K = a0_d1, N = a1_d0, P = a1_d1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (P * 2 != K || a2_d0 != M || a2_d1 != N) return INTENT_B200_ERR_SHAPE;
  if (M == 0 || N == 0) return INTENT_B200_OK;
  int status = check_views(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2));
  if (status != INTENT_B200_OK) return status;
  if (K == 0 || K % 8 != 0 || N % 8 != 0) return INTENT_B200_ERR_UNSUPPORTED;
  const int64_t decoded_bytes = align256(N * K * 2);
  if (!workspace || !aligned16(workspace) || workspace_bytes < decoded_bytes + 256) return INTENT_B200_ERR_WORKSPACE;
  int32_t* row_span = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(workspace) + decoded_bytes);
  const int64_t words = N * P / 4;
  expand_fp4_kernel<<<grid_for(words, 256), 256, 0, stream>>>(static_cast<const uint32_t*>(a1),
                                                             static_cast<uint4*>(workspace), words, row_span,
                                                             int32_t(M));
  note_launch();
  status = launch_status();
  if (status != INTENT_B200_OK) return status;
  return bf16_gemm_nt(a0, M, K, workspace, N, a2, row_span, stream);
}
