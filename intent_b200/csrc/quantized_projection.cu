// quantized_projection (examples/kernels/quantization/quantized_projection.py:5-19): a GEMV whose
// weights are Q4_K records (144 bytes per 256 values) and whose f32 activation is quantized to
// Q8_K records (292 bytes per 256 values) inside the call.  Record formats and the order of the
// float roundings follow doc/dsl/quantized-operations.en.md sections 2-4: the integer sums S and T
// of a record are exact, then p = f32(d) * f32(S), n = f32(dmin) * f32(T), v = ds * (p - n), each
// product / difference rounded once (no fused multiply-add), and the records of a row are added
// in increasing order.
//
// Two launches: a one-warp-per-record quantizer (the activation is tiny), then one warp per output
// row streaming the row's records: lane l owns packed word l of the record (four low nibbles of
// sub-block 2*(l/8) and four high nibbles of sub-block 2*(l/8)+1), meets the matching activation
// bytes with dp4a, scales by the sub-block's 6-bit scale and the warp adds the integers.
// HBM-bound: every weight byte is read once.
#include "common.cuh"

namespace ib200 {
namespace {

constexpr int kQ4Bytes = 144, kQ8Bytes = 292, kRecordValues = 256;

// one warp per record; lane l holds values 8l .. 8l+7
__global__ void q8_k_quantize_kernel(const float* __restrict__ activation, int records,
                                     unsigned char* __restrict__ out) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= records) return;
  const float4* src = reinterpret_cast<const float4*>(activation + size_t(warp) * kRecordValues) + 2 * lane;
  const float4 a = src[0], b = src[1];
  const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  float high = v[0], low = v[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) {
    high = fmaxf(high, v[i]);
    low = fminf(low, v[i]);
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) {
    high = fmaxf(high, __shfl_xor_sync(0xffffffffu, high, d));
    low = fminf(low, __shfl_xor_sync(0xffffffffu, low, d));
  }
  const float extreme = fabsf(low) >= fabsf(high) ? low : high;  // the minimum wins ties
  unsigned char* record = out + size_t(warp) * kQ8Bytes;
  int q[8];
  float ds = 0.f;
  if (extreme == 0.f) {
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = 0;
  } else {
    const float inverse = __fdiv_rn(-127.0f, extreme);
    ds = __fdiv_rn(1.0f, inverse);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[i] = max(-128, min(127, __float2int_rn(__fmul_rn(v[i], inverse))));
  }
  if (lane == 0) *reinterpret_cast<float*>(record) = ds;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    lo |= (uint32_t(q[i]) & 0xFFu) << (8 * i);
    hi |= (uint32_t(q[4 + i]) & 0xFFu) << (8 * i);
  }
  uint32_t* qdst = reinterpret_cast<uint32_t*>(record + 4) + 2 * lane;
  qdst[0] = lo;
  qdst[1] = hi;
  int sum = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) sum += q[i];
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);  // 16 values = two lanes
  if ((lane & 1) == 0) *reinterpret_cast<int16_t*>(record + 260 + 2 * (lane >> 1)) = int16_t(sum);
}

// one warp per output row
__global__ void q4_k_projection_kernel(const unsigned char* __restrict__ weights, const unsigned char* __restrict__ xq,
                                       int rows, int records, float* __restrict__ out) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int group = lane >> 3;  // which 64 values of the record this lane's word belongs to
  for (int n = warp; n < rows; n += warps) {
    const unsigned char* row = weights + size_t(n) * records * kQ4Bytes;
    float result = 0.f;
    for (int b = 0; b < records; ++b) {
      const unsigned char* w = row + size_t(b) * kQ4Bytes;
      const unsigned char* x = xq + size_t(b) * kQ8Bytes;
      const uint32_t head = __ldg(reinterpret_cast<const uint32_t*>(w));          // d | dmin (f16 each)
      const uint32_t f0 = __ldg(reinterpret_cast<const uint32_t*>(w + 4));        // scale bytes 4..7
      const uint32_t f1 = __ldg(reinterpret_cast<const uint32_t*>(w + 8));        // bytes 8..11
      const uint32_t f2 = __ldg(reinterpret_cast<const uint32_t*>(w + 12));       // bytes 12..15
      // sub-block s (0..7): sc = field_0[s], m = field_1[s]
      auto field = [&](int r, int s) -> int {
        const uint32_t base = r == 0 ? f0 : f1;
        if (s < 4) return int((base >> (8 * s)) & 63u);
        const int t = s - 4;
        return int(((f2 >> (8 * t + 4 * r)) & 15u) | ((((base >> (8 * t)) & 0xFFu) >> 6) << 4));
      };
      const uint32_t packed = __ldg(reinterpret_cast<const uint32_t*>(w + 16) + lane);
      const int t0 = (lane & 7) * 4;
      const int x_low = int(__ldg(reinterpret_cast<const uint32_t*>(x + 4 + 64 * group + t0)));
      const int x_high = int(__ldg(reinterpret_cast<const uint32_t*>(x + 4 + 64 * group + 32 + t0)));
      int s_sum = field(0, 2 * group) * __dp4a(int(packed & 0x0F0F0F0Fu), x_low, 0) +
                  field(0, 2 * group + 1) * __dp4a(int((packed >> 4) & 0x0F0F0F0Fu), x_high, 0);
      int t_sum = 0;
      if (lane < 8) {
        const uint32_t pair = __ldg(reinterpret_cast<const uint32_t*>(x + 260) + lane);  // bsum[2s], bsum[2s+1]
        t_sum = field(1, lane) * (int(int16_t(pair & 0xFFFFu)) + int(int16_t(pair >> 16)));
      }
#pragma unroll
      for (int d = 16; d >= 1; d >>= 1) {
        s_sum += __shfl_xor_sync(0xffffffffu, s_sum, d);
        t_sum += __shfl_xor_sync(0xffffffffu, t_sum, d);
      }
      const float d = __half2float(__ushort_as_half(uint16_t(head & 0xFFFFu)));
      const float dmin = __half2float(__ushort_as_half(uint16_t(head >> 16)));
      const float ds = __ldg(reinterpret_cast<const float*>(x));
      const float p = __fmul_rn(d, float(s_sum));
      const float m = __fmul_rn(dmin, float(t_sum));
      result = __fadd_rn(result, __fmul_rn(ds, __fsub_rn(p, m)));
    }
    if (lane == 0) out[n] = result;
  }
}

inline int64_t align256(int64_t bytes) { return (bytes + 255) & ~int64_t(255); }

}  // namespace
}  // namespace ib200

// a0 weights u8 [N,G,144] (Q4_K records), a1 activation f32 [G,256] -> a2 output f32 [N]
// workspace: at least G*292 bytes rounded up to 256 (the activation's Q8_K records), not cleared
extern "C" int intent_b200_quantized_projection(INTENT_B200_VIEW3(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW1(a2),
                                                void* workspace, int64_t workspace_bytes, void* stream_) {
  using namespace ib200;
  const int64_t N = a0_d0, G = a0_d1;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a0_d2 != kQ4Bytes || a1_d0 != G || a1_d1 != kRecordValues || a2_d0 != N) return INTENT_B200_ERR_SHAPE;
  if (N == 0) return INTENT_B200_OK;
  if (!a0 || !a2 || (G > 0 && !a1)) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW3_ARG(a0)) || !contiguous(IB200_VIEW2_ARG(a1)) || !contiguous(IB200_VIEW1_ARG(a2)) ||
      !aligned16(a0) || !aligned16(a1))
    return INTENT_B200_ERR_LAYOUT;
  if (N > (1 << 30) || G > (1 << 20)) return INTENT_B200_ERR_UNSUPPORTED;
  if (G > 0 && (!workspace || !aligned16(workspace) || workspace_bytes < align256(G * kQ8Bytes)))
    return INTENT_B200_ERR_WORKSPACE;
  if (G > 0) {
    q8_k_quantize_kernel<<<int((G + 7) / 8), 256, 0, stream>>>(static_cast<const float*>(a1), int(G),
                                                               static_cast<unsigned char*>(workspace));
    note_launch();
    const int status = launch_status();
    if (status != INTENT_B200_OK) return status;
  }
  const int64_t blocks = (N + 7) / 8;
  q4_k_projection_kernel<<<int(blocks < 148 * 8 ? blocks : 148 * 8), 256, 0, stream>>>(
      static_cast<const unsigned char*>(a0), static_cast<const unsigned char*>(workspace), int(N), int(G),
      static_cast<float*>(a2));
  note_launch();
  return launch_status();
}
