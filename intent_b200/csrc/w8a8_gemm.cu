// int8 x int8 -> int32 GEMM on tcgen05 (kind::i8, s32 accumulation in TMEM).
//
// Programs:
//   gemm_i8    C[m,n] = i32(sum_k A[m,k] * B[k,n]) + bias[n]      (reference kernel body
//              examples/kernels/contraction/gemm.py:29-39; exact integer result)
//   w8a8_gemm  Y[m,n] = bf16( f32(acc[m,n]) * sa[m] * sb[n] )      (the benchmark's per-token x
//              per-channel epilogue on the same exact accumulator)
//
// A [M,K] is K-major and B [K,N] is N-major in HBM, exactly as the reference declares them;
// both go to shared memory unchanged through 128B-swizzled TMA boxes (A: 128 rows x 128 k,
// B: two boxes of 128 k rows x 128 columns) and the B operand is described to the tensor core
// as MN-major, so no transposition pass exists anywhere.  One persistent CTA per SM walks
// 128 x 256 tiles: warp 0 issues TMA (4 stages of 48 KiB), one thread of warp 1 issues four
// M128 N256 K32 MMAs per stage, warps 2..5 drain the two TMEM accumulators.
// With B_K_MAJOR the second operand is given as [N,K] (K contiguous, e.g. decoded packed weights)
// and is loaded as one 256-row K-major box.
// Every wait is bounded (see tma.cuh); a wait that gives up records a timeout status.
#include "common.cuh"
#include "dense.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace ib200 {

__device__ int g_w8a8_gemm_status = 0;

namespace {

constexpr int BM = 128, BN = 256, BK = 128;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;       // 16 KiB
constexpr int B_BOX_BYTES = BK * 128;  // one 128-column box, 16 KiB
constexpr int B_BYTES = 2 * B_BOX_BYTES;
constexpr int THREADS = 6 * 32;
constexpr int SMEM_BYTES = 1024 + STAGES * (A_BYTES + B_BYTES) + 256;

struct I8Params {
  void* out;
  const int32_t* bias;      // gemm_i8 (may be null)
  const float* a_scales;    // w8a8
  const float* b_scales;
  int M, N, K;
  int k_blocks, m_tiles, n_tiles;
};

// EPILOGUE 0: bf16(acc * sa[m] * sb[n]);  1: int32 acc + bias[n]
template <int EPILOGUE, bool B_K_MAJOR>
__global__ void __launch_bounds__(THREADS, 1)
i8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const I8Params p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t smem_a = base;
  const uint32_t smem_b = smem_a + STAGES * A_BYTES;
  const uint32_t bars = smem_b + STAGES * B_BYTES;
  const uint32_t full = bars;
  const uint32_t empty = full + 8 * STAGES;
  const uint32_t tmem_full = empty + 8 * STAGES;
  const uint32_t tmem_empty = tmem_full + 16;
  const uint32_t tmem_slot = tmem_empty + 16;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + (tmem_slot - base));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int tiles = p.m_tiles * p.n_tiles;

  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + 8 * s, 1);
      mbar_init(empty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tmem_full + 8 * s, 1);
      mbar_init(tmem_empty + 8 * s, 4);
    }
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          if (!mbar_wait(empty + 8 * s, ((it / STAGES) & 1) ^ 1)) { ok = false; break; }
          const uint32_t bar = full + 8 * s;
          mbar_expect_tx(bar, A_BYTES + B_BYTES);
          tma_load_2d(smem_a + s * A_BYTES, &map_a, kb * BK, m_tile * BM, bar);
          if (B_K_MAJOR) {
            tma_load_2d(smem_b + s * B_BYTES, &map_b, kb * BK, n_tile * BN, bar);
          } else {
            tma_load_2d(smem_b + s * B_BYTES, &map_b, n_tile * BN, kb * BK, bar);
            tma_load_2d(smem_b + s * B_BYTES + B_BOX_BYTES, &map_b, n_tile * BN + 128, kb * BK, bar);
          }
        }
      }
      if (!ok) atomicExch(&g_w8a8_gemm_status, INTENT_B200_ERR_TIMEOUT);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // s32 accumulator, signed 8-bit operands, A K-major, B MN-major (N contiguous)
      constexpr uint32_t idesc = umma_idesc(2, 1, 1, 0, B_K_MAJOR ? 0 : 1, BM, BN);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
        const uint32_t acc = local & 1;
        if (!mbar_wait(tmem_empty + 8 * acc, ((local >> 1) & 1) ^ 1)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          if (!mbar_wait(full + 8 * s, (it / STAGES) & 1)) { ok = false; break; }
          tcgen05_fence_after();
          const uint64_t desc_a = umma_desc_k_major_sw128(smem_a + s * A_BYTES);
          // 128-column spans are one box (16 KiB) apart, 8-row k groups 1 KiB apart
          const uint64_t desc_b = B_K_MAJOR ? umma_desc_k_major_sw128(smem_b + s * B_BYTES)
                                            : umma_desc_mn_major_sw128(smem_b + s * B_BYTES, B_BOX_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 32; ++kk)
            // A: 32 k = 32 bytes along its 128-byte row (2 units); B: 32 k rows of 128 bytes (256 units)
            umma_i8(tmem_d, desc_a + uint64_t(2 * kk), desc_b + uint64_t((B_K_MAJOR ? 2 : 256) * kk), idesc,
                    (kb | kk) != 0);
          umma_commit(empty + 8 * s);
        }
        if (ok) umma_commit(tmem_full + 8 * acc);
      }
      if (!ok) atomicExch(&g_w8a8_gemm_status, INTENT_B200_ERR_TIMEOUT);
    }
  } else {
    const int quadrant = warp & 3;
    uint32_t local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      const int m_tile = tile % p.m_tiles, n_tile = tile / p.m_tiles;
      const uint32_t acc = local & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(tmem_full + 8 * acc, (local >> 1) & 1))) {
        if (lane == 0) atomicExch(&g_w8a8_gemm_status, INTENT_B200_ERR_TIMEOUT);
        break;
      }
      tcgen05_fence_after();
      const int row = m_tile * BM + quadrant * 32 + lane;
      const uint32_t taddr = tmem_base + acc * BN + (uint32_t(quadrant * 32) << 16);
      float row_scale = 0.f;
      if (EPILOGUE == 0 && row < p.M) row_scale = p.a_scales[row];
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_load_32x32(taddr + c * 32, v);
        tmem_load_wait();
        const int col = n_tile * BN + c * 32;
        if (row < p.M) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int n0 = col + q * 8;
            if (n0 < p.N) {  // N is a multiple of 16
              if (EPILOGUE == 0) {
                const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.b_scales + n0));
                const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.b_scales + n0 + 4));
                const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float lo = (float(int32_t(v[8 * q + 2 * j])) * row_scale) * sc[2 * j];
                  const float hi = (float(int32_t(v[8 * q + 2 * j + 1])) * row_scale) * sc[2 * j + 1];
                  o[j] = uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(lo))) |
                         (uint32_t(__bfloat16_as_ushort(__float2bfloat16_rn(hi))) << 16);
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + size_t(row) * p.N + n0) =
                    make_uint4(o[0], o[1], o[2], o[3]);
              } else {
                int32_t* dst = reinterpret_cast<int32_t*>(p.out) + size_t(row) * p.N + n0;
                int4 b0 = make_int4(0, 0, 0, 0), b1 = make_int4(0, 0, 0, 0);
                if (p.bias) {
                  b0 = __ldg(reinterpret_cast<const int4*>(p.bias + n0));
                  b1 = __ldg(reinterpret_cast<const int4*>(p.bias + n0 + 4));
                }
                // integer addition wraps (two's complement), as the reference's numerics require
                *reinterpret_cast<uint4*>(dst) =
                    make_uint4(v[8 * q + 0] + uint32_t(b0.x), v[8 * q + 1] + uint32_t(b0.y),
                               v[8 * q + 2] + uint32_t(b0.z), v[8 * q + 3] + uint32_t(b0.w));
                *reinterpret_cast<uint4*>(dst + 4) =
                    make_uint4(v[8 * q + 4] + uint32_t(b1.x), v[8 * q + 5] + uint32_t(b1.y),
                               v[8 * q + 6] + uint32_t(b1.z), v[8 * q + 7] + uint32_t(b1.w));
              }
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty + 8 * acc);
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

int device_sms() {
  static int sms = [] {
    int device = 0, value = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    return value;
  }();
  return sms;
}

// b is [K,N] (N contiguous), or [N,K] (K contiguous) with B_K_MAJOR
template <int EPILOGUE, bool B_K_MAJOR = false>
int run(View2 a, View2 b, void* out, const int32_t* bias, const float* sa, const float* sb, cudaStream_t stream) {
  const int64_t M = a.d0, K = a.d1, N = B_K_MAJOR ? b.d0 : b.d1;
  if ((B_K_MAJOR ? b.d1 : b.d0) != K) return INTENT_B200_ERR_SHAPE;
  if (M == 0 || N == 0) return INTENT_B200_OK;
  if (!a.p || !b.p || !out) return INTENT_B200_ERR_NULL;
  if (!contiguous(a) || !contiguous(b)) return INTENT_B200_ERR_LAYOUT;
  if (!aligned16(a.p) || !aligned16(b.p) || !aligned16(out)) return INTENT_B200_ERR_LAYOUT;
  if (K == 0 || K % 16 != 0 || N % 16 != 0 || M > (1 << 24) || K > (1 << 24) || N > (1 << 24))
    return INTENT_B200_ERR_UNSUPPORTED;
  const int sms = device_sms();
  if (sms <= 0) return INTENT_B200_ERR_UNSUPPORTED;
  I8Params p{};
  p.out = out;
  p.bias = bias;
  p.a_scales = sa;
  p.b_scales = sb;
  p.M = int(M);
  p.N = int(N);
  p.K = int(K);
  p.k_blocks = int((K + BK - 1) / BK);
  p.m_tiles = int((M + BM - 1) / BM);
  p.n_tiles = int((N + BN - 1) / BN);
  CUtensorMap map_a, map_b;
  if (!make_tensor_map_2d(&map_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.p, uint64_t(M), uint64_t(K), uint64_t(K), BM, BK,
                          CU_TENSOR_MAP_SWIZZLE_128B) ||
      !(B_K_MAJOR ? make_tensor_map_2d(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, b.p, uint64_t(N), uint64_t(K), uint64_t(K),
                                       BN, BK, CU_TENSOR_MAP_SWIZZLE_128B)
                  : make_tensor_map_2d(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, b.p, uint64_t(K), uint64_t(N), uint64_t(N),
                                       BK, 128, CU_TENSOR_MAP_SWIZZLE_128B)))
    return INTENT_B200_ERR_UNSUPPORTED;
  auto kernel = i8_gemm_kernel<EPILOGUE, B_K_MAJOR>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return cuda_status(e);
  const int tiles = p.m_tiles * p.n_tiles;
  if (LaunchFacts* sink = observe_sink())
    return record_launch(sink, reinterpret_cast<const void*>(kernel), "i8_gemm_kernel 128x256 tiles, two accumulators",
                         tiles < sms ? tiles : sms, THREADS, SMEM_BYTES, 1);
  kernel<<<tiles < sms ? tiles : sms, THREADS, SMEM_BYTES, stream>>>(map_a, map_b, p);
  note_launch();
  return launch_status();
}

}  // namespace

int i8_gemm_nt(const void* a, int64_t M, int64_t K, const void* b, int64_t N, int32_t* out, cudaStream_t stream) {
  View2 va{const_cast<void*>(a), M, K, K, 1}, vb{const_cast<void*>(b), N, K, K, 1};
  return run<1, true>(va, vb, out, nullptr, nullptr, nullptr, stream);
}

}  // namespace ib200

extern "C" int intent_b200_gemm_i8(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW1(a2),
                                   INTENT_B200_VIEW2(a3), void* stream) {
  using namespace ib200;
  if (a3_d0 != a0_d0 || a3_d1 != a1_d1 || a2_d0 != a1_d1) return INTENT_B200_ERR_SHAPE;
  if (!contiguous(IB200_VIEW2_ARG(a3)) || !contiguous(IB200_VIEW1_ARG(a2)) || !aligned16(a2)) return INTENT_B200_ERR_LAYOUT;
  return run<1>(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), a3, static_cast<const int32_t*>(a2), nullptr, nullptr,
                static_cast<cudaStream_t>(stream));
}

extern "C" int intent_b200_w8a8_gemm_bf16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW1(a2),
                                          INTENT_B200_VIEW1(a3), INTENT_B200_VIEW2(a4), void* stream) {
  using namespace ib200;
  if (a4_d0 != a0_d0 || a4_d1 != a1_d1 || a2_d0 != a0_d0 || a3_d0 != a1_d1) return INTENT_B200_ERR_SHAPE;
  if (!contiguous(IB200_VIEW2_ARG(a4)) || !contiguous(IB200_VIEW1_ARG(a2)) || !contiguous(IB200_VIEW1_ARG(a3)) ||
      !aligned16(a2) || !aligned16(a3))
    return INTENT_B200_ERR_LAYOUT;
  if (a0_d0 > 0 && a1_d1 > 0 && (!a2 || !a3)) return INTENT_B200_ERR_NULL;
  return run<0>(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), a4, nullptr, static_cast<const float*>(a2),
                static_cast<const float*>(a3), static_cast<cudaStream_t>(stream));
}

extern "C" int intent_b200_i8_gemm_device_status(void) {
  int value = 0, zero = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return ib200::cuda_status(e);
  e = cudaMemcpyFromSymbol(&value, ib200::g_w8a8_gemm_status, sizeof(int));
  if (e != cudaSuccess) return ib200::cuda_status(e);
  if (value != 0) cudaMemcpyToSymbol(ib200::g_w8a8_gemm_status, &zero, sizeof(int));
  return value;
}
