// Ragged grouped GEMM with dense 16-bit weights on tcgen05 (kind::f16, f32 accumulation in TMEM).
//
// Programs (reference kernel bodies):
//   ragged_grouped_gemm[_bf16]      rows offsets[g]:offsets[g+1] of X times W[g]  [G,K,N]
//                                   (examples/kernels/ragged/grouped_gemm.py:11-70)
//   routed_expert_projection_bf16   out[token, slot, :] = x[token] . W[e]^T, W [E,N,K], the rows of an
//                                   expert listed by member_routes (grouped_gemm.py:101-138)
//   moe_expert_ffn                  y[token] += w[route] * (f16(relu(x[token] W1[e])) W2[e])
//                                   (examples/kernels/ragged/moe.py:12-53)
//   gemm / bf16_gemm / quantized_gemm  the dense forms (examples/kernels/contraction/gemm.py:40-106): a single
//                                   group covering every row, optional ReLU, or the int8 epilogue
//                                   i8(clamp((relu(acc + bias[n]) + residual[m,n]) / scale[n]))
//
// One persistent CTA per SM walks 128 x 256 output tiles.  The tile list is ragged: every CTA
// reads the group offsets once, clamps them to the row count and builds the per-group tile
// prefix in shared memory, so no host read of the offsets is needed.  Operands reach shared
// memory unchanged through 128B-swizzled TMA boxes: A rows are K-major; W [G,K,N] is described
// to the tensor core as an MN-major operand (four 64-column boxes per stage), W [E,N,K] as a
// K-major one, so neither layout needs a transposition pass.  A tile that runs past the end of
// its group loads rows of the next group (or zeros past the last row); the epilogue writes
// only rows of its own group.  Programs whose rows are selected through an index list gather
// them once into a workspace in member order; the epilogue scatters through the same list.
// Every wait is bounded; a wait that gives up records a timeout status and the kernel drains.
#include <type_traits>

#include "common.cuh"
#include "dense.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace ib200 {

__device__ int g_grouped16_status = 0;

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_BOX_BYTES = BK * 64 * 2;    // one 64-column box of an MN-major stage, 8 KiB
constexpr int B_BYTES = BK * BN * 2;        // 32 KiB
constexpr int THREADS = 6 * 32;
constexpr int MAX_GROUPS = 1024;
constexpr int TABLE_BYTES = 3 * (MAX_GROUPS + 1) * 4;
constexpr int SMEM_BYTES = 1024 + STAGES * (A_BYTES + B_BYTES) + 256 + TABLE_BYTES;

enum Epilogue { kCast = 0, kReluCast = 1, kWeightedAdd = 2, kQuantize = 3 };

struct Params {
  const int32_t* offsets;      // [groups + 1]; null = one group covering every row
  int groups, rows, N, K;
  int k_blocks, n_tiles;
  void* out;
  int64_t out_rows;
  const int32_t* row_map;      // output row (or route) of member row r; null = r itself
  const int32_t* route_token;  // kWeightedAdd: token of a route
  const float* route_weights;  // kWeightedAdd: weight of a route
  int64_t routes;              // extent of route_token / route_weights
  const float* bias;           // kQuantize: [N]
  const void* residual;        // kQuantize: [rows, N], element type T
  const float* out_scale;      // kQuantize: [N]
};

__device__ __forceinline__ void red_add_v4(float* address, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(address), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

struct TileWalk {
  const int* begin;
  const int* count;
  const int* prefix;
  int groups, group;
  __device__ TileWalk(const int* b, const int* c, const int* p, int n) : begin(b), count(c), prefix(p), groups(n), group(0) {}
  // tiles are visited in increasing order, so the group only moves forward
  __device__ void locate(int tile, int& g, int& m_block, int& n_tile) {
    while (group + 1 < groups && tile >= prefix[group + 1]) ++group;
    const int local = tile - prefix[group];
    const int m_blocks = (count[group] + BM - 1) / BM;
    g = group;
    m_block = local % m_blocks;
    n_tile = local / m_blocks;
  }
};

template <typename T, bool B_K_MAJOR, int EPILOGUE>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const Params p) {
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
  int* s_begin = reinterpret_cast<int*>(base_ptr + (bars - base) + 256);
  int* s_count = s_begin + MAX_GROUPS + 1;
  int* s_prefix = s_count + MAX_GROUPS + 1;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  for (int g = tid; g < p.groups; g += THREADS) {
    const int b = p.offsets ? min(max(p.offsets[g], 0), p.rows) : 0;
    const int e = p.offsets ? min(max(p.offsets[g + 1], 0), p.rows) : p.rows;
    s_begin[g] = b;
    s_count[g] = max(e - b, 0);
  }
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
  __syncthreads();
  if (warp == 0) {
    int running = 0;
    for (int g0 = 0; g0 < p.groups; g0 += 32) {
      const int g = g0 + lane;
      const int mine = g < p.groups ? ((s_count[g] + BM - 1) / BM) * p.n_tiles : 0;
      int inclusive = mine;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inclusive, o);
        if (lane >= o) inclusive += v;
      }
      if (g < p.groups) s_prefix[g] = running + inclusive - mine;
      running += __shfl_sync(0xffffffffu, inclusive, 31);
    }
    if (lane == 0) s_prefix[p.groups] = running;
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  const int tiles = s_prefix[p.groups];

  if (warp == 0) {
    if (lane == 0) {
      TileWalk walk(s_begin, s_count, s_prefix, p.groups);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int g, m_block, n_tile;
        walk.locate(tile, g, m_block, n_tile);
        const int row0 = s_begin[g] + m_block * BM;
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          if (!mbar_wait(empty + 8 * s, ((it / STAGES) & 1) ^ 1)) { ok = false; break; }
          const uint32_t bar = full + 8 * s;
          mbar_expect_tx(bar, A_BYTES + B_BYTES);
          tma_load_2d(smem_a + s * A_BYTES, &map_a, kb * BK, row0, bar);
          if (B_K_MAJOR) {
            tma_load_3d(smem_b + s * B_BYTES, &map_b, kb * BK, n_tile * BN, g, bar);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(smem_b + s * B_BYTES + j * B_BOX_BYTES, &map_b, n_tile * BN + j * 64, kb * BK, g, bar);
          }
        }
      }
      if (!ok) atomicExch(&g_grouped16_status, INTENT_B200_ERR_TIMEOUT);
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t format = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      constexpr uint32_t idesc = umma_idesc(1, format, format, 0, B_K_MAJOR ? 0 : 1, BM, BN);
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
          // MN-major: 64-column spans one box (8 KiB) apart, 8-row k groups 1 KiB apart
          const uint64_t desc_b = B_K_MAJOR ? umma_desc_k_major_sw128(smem_b + s * B_BYTES)
                                            : umma_desc_mn_major_sw128(smem_b + s * B_BYTES, B_BOX_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)
            // 16 k: 32 bytes along a K-major row (2 units); 16 rows of 128 bytes of an MN-major box (128 units)
            umma_f16(tmem_d, desc_a + uint64_t(2 * kk), desc_b + uint64_t((B_K_MAJOR ? 2 : 128) * kk), idesc,
                     (kb | kk) != 0);
          umma_commit(empty + 8 * s);
        }
        if (ok) umma_commit(tmem_full + 8 * acc);
      }
      if (!ok) atomicExch(&g_grouped16_status, INTENT_B200_ERR_TIMEOUT);
    }
  } else {
    const int quadrant = warp & 3;
    TileWalk walk(s_begin, s_count, s_prefix, p.groups);
    uint32_t local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      int g, m_block, n_tile;
      walk.locate(tile, g, m_block, n_tile);
      const uint32_t acc = local & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(tmem_full + 8 * acc, (local >> 1) & 1))) {
        if (lane == 0) atomicExch(&g_grouped16_status, INTENT_B200_ERR_TIMEOUT);
        break;
      }
      tcgen05_fence_after();
      const int in_group = m_block * BM + quadrant * 32 + lane;
      const int member = s_begin[g] + in_group;
      bool valid = in_group < s_count[g];
      int64_t out_row = member;
      float weight = 1.f;
      if (valid && p.row_map) out_row = p.row_map[member];
      if (EPILOGUE == kWeightedAdd) {
        valid = valid && out_row >= 0 && out_row < p.routes;
        if (valid) {
          weight = p.route_weights[out_row];
          out_row = p.route_token[out_row];
        }
      }
      valid = valid && out_row >= 0 && out_row < p.out_rows;
      const uint32_t taddr = tmem_base + acc * BN + (uint32_t(quadrant * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_load_32x32(taddr + c * 32, v);
        tmem_load_wait();
        const int col = n_tile * BN + c * 32;
        if (valid) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int n0 = col + q * 8;
            if (n0 < p.N) {  // N is a multiple of 8
              if (EPILOGUE == kQuantize) {
                // i8(trunc(clamp((relu(acc + bias) + residual) / scale, -128, 127))), all in f32
                const float4 b0 = __ldg(reinterpret_cast<const float4*>(p.bias + n0));
                const float4 b1 = __ldg(reinterpret_cast<const float4*>(p.bias + n0 + 4));
                const float4 s0 = __ldg(reinterpret_cast<const float4*>(p.out_scale + n0));
                const float4 s1 = __ldg(reinterpret_cast<const float4*>(p.out_scale + n0 + 4));
                const uint4 r = __ldg(reinterpret_cast<const uint4*>(
                    reinterpret_cast<const uint16_t*>(p.residual) + size_t(out_row) * p.N + n0));
                const float bias[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
                const float scale[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
                const uint32_t res[4] = {r.x, r.y, r.z, r.w};
                uint32_t packed[2] = {0u, 0u};
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  const float residual = Elem<T>::to_float(uint16_t(res[j >> 1] >> (16 * (j & 1))));
                  float value = fmaxf(__uint_as_float(v[8 * q + j]) + bias[j], 0.f) + residual;
                  value = __fdiv_rn(value, scale[j]);
                  value = fminf(fmaxf(value, -128.f), 127.f);
                  packed[j >> 2] |= (uint32_t(__float2int_rz(value)) & 0xFFu) << (8 * (j & 3));
                }
                *reinterpret_cast<uint2*>(reinterpret_cast<int8_t*>(p.out) + size_t(out_row) * p.N + n0) =
                    make_uint2(packed[0], packed[1]);
              } else if (EPILOGUE == kWeightedAdd) {
                float* dst = reinterpret_cast<float*>(p.out) + size_t(out_row) * p.N + n0;
                red_add_v4(dst, weight * __uint_as_float(v[8 * q + 0]), weight * __uint_as_float(v[8 * q + 1]),
                           weight * __uint_as_float(v[8 * q + 2]), weight * __uint_as_float(v[8 * q + 3]));
                red_add_v4(dst + 4, weight * __uint_as_float(v[8 * q + 4]), weight * __uint_as_float(v[8 * q + 5]),
                           weight * __uint_as_float(v[8 * q + 6]), weight * __uint_as_float(v[8 * q + 7]));
              } else {
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float lo = __uint_as_float(v[8 * q + 2 * j]), hi = __uint_as_float(v[8 * q + 2 * j + 1]);
                  if (EPILOGUE == kReluCast) {
                    lo = fmaxf(lo, 0.f);
                    hi = fmaxf(hi, 0.f);
                  }
                  o[j] = uint32_t(Elem<T>::from_float(lo)) | (uint32_t(Elem<T>::from_float(hi)) << 16);
                }
                *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(p.out) + size_t(out_row) * p.N + n0) =
                    make_uint4(o[0], o[1], o[2], o[3]);
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

// Copies the row of X that each member of the list selects into `out` in member order.
// BY_TABLE: token = route_token[route]; otherwise token = route / top_k.  Members that point
// outside X produce a zero row (the epilogue drops them as well).
template <bool BY_TABLE>
__global__ void gather16_kernel(const uint4* __restrict__ x, int64_t tokens, int row_vectors,
                                const int* __restrict__ members, int count, int top_k,
                                const int* __restrict__ route_token, int64_t routes, uint4* __restrict__ out) {
  for (int m = blockIdx.x; m < count; m += gridDim.x) {
    const int route = members[m];
    int64_t token = -1;
    if (BY_TABLE) {
      if (route >= 0 && route < routes) token = route_token[route];
    } else if (route >= 0) {
      token = route / top_k;
    }
    const bool real = token >= 0 && token < tokens;
    const uint4* src = x + size_t(real ? token : 0) * row_vectors;
    uint4* dst = out + size_t(m) * row_vectors;
    for (int i = threadIdx.x; i < row_vectors; i += blockDim.x) dst[i] = real ? src[i] : make_uint4(0, 0, 0, 0);
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

template <typename T>
constexpr CUtensorMapDataType tensor_map_type() {
  return std::is_same<T, __nv_bfloat16>::value ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

struct Problem {
  const void* a;           // [rows, K] member rows, contiguous
  int64_t rows, K, N, groups;
  const void* weight;      // [groups, K, N] or [groups, N, K]
  const int32_t* offsets;  // [groups + 1]
  void* out;
  int64_t out_rows;
  const int32_t* row_map;
  const int32_t* route_token;
  const float* route_weights;
  int64_t routes;
  const float* bias = nullptr;
  const void* residual = nullptr;
  const float* out_scale = nullptr;
};

template <typename T, bool B_K_MAJOR, int EPILOGUE>
int launch(const Problem& q, cudaStream_t stream) {
  if (q.rows == 0 || q.N == 0 || q.groups == 0) return INTENT_B200_OK;
  if (q.K == 0 || q.K % 8 != 0 || q.N % 8 != 0 || q.groups > MAX_GROUPS || q.rows > (1 << 24) ||
      q.K > (1 << 24) || q.N > (1 << 24))
    return INTENT_B200_ERR_UNSUPPORTED;
  const int sms = device_sms();
  if (sms <= 0) return INTENT_B200_ERR_UNSUPPORTED;
  Params p{};
  p.offsets = q.offsets;
  p.groups = int(q.groups);
  p.rows = int(q.rows);
  p.N = int(q.N);
  p.K = int(q.K);
  p.k_blocks = int((q.K + BK - 1) / BK);
  p.n_tiles = int((q.N + BN - 1) / BN);
  p.out = q.out;
  p.out_rows = q.out_rows;
  p.row_map = q.row_map;
  p.route_token = q.route_token;
  p.route_weights = q.route_weights;
  p.routes = q.routes;
  p.bias = q.bias;
  p.residual = q.residual;
  p.out_scale = q.out_scale;
  // groups may overlap, so the tile count is bounded per group, not by the row count
  if (q.groups * (q.rows / BM + 1) * int64_t(p.n_tiles) >= (int64_t(1) << 31)) return INTENT_B200_ERR_UNSUPPORTED;
  const int64_t tile_bound = (q.rows / BM + q.groups) * int64_t(p.n_tiles);
  CUtensorMap map_a, map_b;
  bool ok = make_tensor_map_2d(&map_a, tensor_map_type<T>(), q.a, uint64_t(q.rows), uint64_t(q.K), uint64_t(q.K) * 2,
                               BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (B_K_MAJOR)
    ok = ok && make_tensor_map_3d(&map_b, tensor_map_type<T>(), q.weight, uint64_t(q.groups), uint64_t(q.N),
                                  uint64_t(q.K), uint64_t(q.K) * 2, uint64_t(q.K) * uint64_t(q.N) * 2, BN, BK,
                                  CU_TENSOR_MAP_SWIZZLE_128B);
  else
    ok = ok && make_tensor_map_3d(&map_b, tensor_map_type<T>(), q.weight, uint64_t(q.groups), uint64_t(q.K),
                                  uint64_t(q.N), uint64_t(q.N) * 2, uint64_t(q.K) * uint64_t(q.N) * 2, BK, 64,
                                  CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return INTENT_B200_ERR_UNSUPPORTED;
  auto kernel = grouped_gemm16_kernel<T, B_K_MAJOR, EPILOGUE>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return cuda_status(e);
  const int grid = int(tile_bound < sms ? (tile_bound > 0 ? tile_bound : 1) : sms);
  if (LaunchFacts* sink = observe_sink())
    return record_launch(sink, reinterpret_cast<const void*>(kernel), "grouped_gemm16_kernel 128x256 tiles", grid,
                         THREADS, SMEM_BYTES, 1);
  kernel<<<grid, THREADS, SMEM_BYTES, stream>>>(map_a, map_b, p);
  note_launch();
  return launch_status();
}

template <bool BY_TABLE>
int gather(const void* x, int64_t tokens, int64_t width, const int32_t* members, int64_t count, int top_k,
           const int32_t* route_token, int64_t routes, void* out, cudaStream_t stream) {
  if (count == 0 || width == 0) return INTENT_B200_OK;
  const int64_t blocks = count < 148 * 16 ? count : 148 * 16;
  if (observe_sink()) return INTENT_B200_OK;      // the contraction behind this gather is what gets observed
  gather16_kernel<BY_TABLE><<<int(blocks), 256, 0, stream>>>(static_cast<const uint4*>(x), tokens, int(width / 8),
                                                            members, int(count), top_k, route_token, routes,
                                                            static_cast<uint4*>(out));
  note_launch();
  return launch_status();
}

inline int64_t align256(int64_t bytes) { return (bytes + 255) & ~int64_t(255); }

// x [R,K], offsets [G+1], weight [G,K,N], y [R,N]
template <typename T>
int ragged_grouped_gemm(View2 x, View1 offsets, View3 w, View2 y, cudaStream_t stream) {
  const int64_t R = x.d0, K = x.d1, G = w.d0, N = w.d2;
  if (w.d1 != K || y.d0 != R || y.d1 != N || offsets.d0 != G + 1) return INTENT_B200_ERR_SHAPE;
  if (R == 0 || N == 0 || G == 0) return INTENT_B200_OK;
  if (!x.p || !offsets.p || !w.p || !y.p) return INTENT_B200_ERR_NULL;
  if (!contiguous(x) || !contiguous(offsets) || !contiguous(w) || !contiguous(y) || !aligned16(x.p) ||
      !aligned16(w.p) || !aligned16(y.p))
    return INTENT_B200_ERR_LAYOUT;
  Problem q{x.p, R, K, N, G, w.p, static_cast<const int32_t*>(offsets.p), y.p, R, nullptr, nullptr, nullptr, 0};
  return launch<T, false, kCast>(q, stream);
}

// x [T,K], expert_offsets [E+1], member_routes [R], weight [E,N,K], output [T,TOP_K,N]
template <typename T>
int routed_expert_projection(View2 x, View1 offsets, View1 members, View3 w, View3 out, int top_k, void* workspace,
                             int64_t workspace_bytes, cudaStream_t stream) {
  const int64_t tokens = x.d0, K = x.d1, E = w.d0, N = w.d1, R = members.d0;
  if (top_k <= 0 || w.d2 != K || out.d0 != tokens || out.d1 != top_k || out.d2 != N || offsets.d0 != E + 1)
    return INTENT_B200_ERR_SHAPE;
  if (R == 0 || N == 0 || E == 0 || tokens == 0) return INTENT_B200_OK;
  if (!x.p || !offsets.p || !members.p || !w.p || !out.p) return INTENT_B200_ERR_NULL;
  if (!contiguous(x) || !contiguous(offsets) || !contiguous(members) || !contiguous(w) || !contiguous(out) ||
      !aligned16(x.p) || !aligned16(w.p) || !aligned16(out.p))
    return INTENT_B200_ERR_LAYOUT;
  if (K % 8 != 0) return INTENT_B200_ERR_UNSUPPORTED;
  if (!workspace || !aligned16(workspace) || workspace_bytes < align256(R * K * 2)) return INTENT_B200_ERR_WORKSPACE;
  int status = gather<false>(x.p, tokens, K, static_cast<const int32_t*>(members.p), R, top_k, nullptr, 0, workspace,
                             stream);
  if (status != INTENT_B200_OK) return status;
  Problem q{workspace, R, K, N, E, w.p, static_cast<const int32_t*>(offsets.p), out.p, tokens * top_k,
            static_cast<const int32_t*>(members.p), nullptr, nullptr, 0};
  return launch<T, true, kCast>(q, stream);
}

// x [T,D], route_offsets [E+1], member_routes [R], route_token [NR], route_weights [NR],
// w1 [E,D,F], w2 [E,F,D], y [T,D] f32 (accumulated into)
template <typename T>
int moe_expert_ffn(View2 x, View1 offsets, View1 members, View1 route_token, View1 route_weights, View3 w1, View3 w2,
                   View2 y, void* workspace, int64_t workspace_bytes, cudaStream_t stream) {
  const int64_t tokens = x.d0, D = x.d1, E = w1.d0, F = w1.d2, R = members.d0, NR = route_token.d0;
  if (w1.d1 != D || w2.d0 != E || w2.d1 != F || w2.d2 != D || y.d0 != tokens || y.d1 != D ||
      route_weights.d0 != NR || offsets.d0 != E + 1)
    return INTENT_B200_ERR_SHAPE;
  if (R == 0 || D == 0 || E == 0 || tokens == 0 || F == 0) return INTENT_B200_OK;
  if (!x.p || !offsets.p || !members.p || !route_token.p || !route_weights.p || !w1.p || !w2.p || !y.p)
    return INTENT_B200_ERR_NULL;
  if (!contiguous(x) || !contiguous(offsets) || !contiguous(members) || !contiguous(route_token) ||
      !contiguous(route_weights) || !contiguous(w1) || !contiguous(w2) || !contiguous(y) || !aligned16(x.p) ||
      !aligned16(w1.p) || !aligned16(w2.p) || !aligned16(y.p))
    return INTENT_B200_ERR_LAYOUT;
  if (D % 8 != 0 || F % 8 != 0) return INTENT_B200_ERR_UNSUPPORTED;
  const int64_t gathered_bytes = align256(R * D * 2), hidden_bytes = align256(R * F * 2);
  if (!workspace || !aligned16(workspace) || workspace_bytes < gathered_bytes + hidden_bytes)
    return INTENT_B200_ERR_WORKSPACE;
  void* gathered = workspace;
  void* hidden = static_cast<unsigned char*>(workspace) + gathered_bytes;
  const int32_t* member_ptr = static_cast<const int32_t*>(members.p);
  const int32_t* token_ptr = static_cast<const int32_t*>(route_token.p);
  int status = gather<true>(x.p, tokens, D, member_ptr, R, 1, token_ptr, NR, gathered, stream);
  if (status != INTENT_B200_OK) return status;
  Problem up{gathered, R, D, F, E, w1.p, static_cast<const int32_t*>(offsets.p), hidden, R, nullptr, nullptr, nullptr, 0};
  status = launch<T, false, kReluCast>(up, stream);
  if (status != INTENT_B200_OK) return status;
  Problem down{hidden, R, F, D, E, w2.p, static_cast<const int32_t*>(offsets.p), y.p, tokens, member_ptr, token_ptr,
               static_cast<const float*>(route_weights.p), NR};
  return launch<T, false, kWeightedAdd>(down, stream);
}

}  // namespace

// a [M,K], b [K,N] -> c [M,N]; one row group, no offsets array
template <typename T, int EPILOGUE>
int dense_gemm(View2 a, View2 b, View2 c, const float* bias, const void* residual, const float* out_scale,
               cudaStream_t stream) {
  const int64_t M = a.d0, K = a.d1, N = b.d1;
  if (b.d0 != K || c.d0 != M || c.d1 != N) return INTENT_B200_ERR_SHAPE;
  if (M == 0 || N == 0) return INTENT_B200_OK;
  if (!a.p || !b.p || !c.p) return INTENT_B200_ERR_NULL;
  if (!contiguous(a) || !contiguous(b) || !contiguous(c) || !aligned16(a.p) || !aligned16(b.p) || !aligned16(c.p))
    return INTENT_B200_ERR_LAYOUT;
  Problem q{a.p, M, K, N, 1, b.p, nullptr, c.p, M, nullptr, nullptr, nullptr, 0};
  q.bias = bias;
  q.residual = residual;
  q.out_scale = out_scale;
  return launch<T, false, EPILOGUE>(q, stream);
}

int bf16_gemm_nt(const void* a, int64_t M, int64_t K, const void* b, int64_t N, void* out, const int32_t* row_span,
                 cudaStream_t stream) {
  Problem q{a, M, K, N, 1, b, row_span, out, M, nullptr, nullptr, nullptr, 0};
  return launch<__nv_bfloat16, true, kCast>(q, stream);
}

}  // namespace ib200

#define IB200_RAGGED_ENTRY(name, T)                                                                            \
  extern "C" int name(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW3(a2), INTENT_B200_VIEW2(a3), \
                      void* stream) {                                                                          \
    return ib200::ragged_grouped_gemm<T>(IB200_VIEW2_ARG(a0), IB200_VIEW1_ARG(a1), IB200_VIEW3_ARG(a2),        \
                                         IB200_VIEW2_ARG(a3), static_cast<cudaStream_t>(stream));              \
  }
IB200_RAGGED_ENTRY(intent_b200_ragged_grouped_gemm_f16, __half)
IB200_RAGGED_ENTRY(intent_b200_ragged_grouped_gemm_bf16, __nv_bfloat16)

#define IB200_ROUTED_ENTRY(name, T)                                                                             \
  extern "C" int name(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW3(a3), \
                      INTENT_B200_VIEW3(a4), int32_t top_k, void* workspace, int64_t workspace_bytes,           \
                      void* stream) {                                                                           \
    return ib200::routed_expert_projection<T>(IB200_VIEW2_ARG(a0), IB200_VIEW1_ARG(a1), IB200_VIEW1_ARG(a2),    \
                                              IB200_VIEW3_ARG(a3), IB200_VIEW3_ARG(a4), top_k, workspace,       \
                                              workspace_bytes, static_cast<cudaStream_t>(stream));              \
  }
IB200_ROUTED_ENTRY(intent_b200_routed_expert_projection_bf16, __nv_bfloat16)
IB200_ROUTED_ENTRY(intent_b200_routed_expert_projection_f16, __half)

#define IB200_MOE_FFN_ENTRY(name, T)                                                                            \
  extern "C" int name(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW1(a3), \
                      INTENT_B200_VIEW1(a4), INTENT_B200_VIEW3(a5), INTENT_B200_VIEW3(a6), INTENT_B200_VIEW2(a7), \
                      void* workspace, int64_t workspace_bytes, void* stream) {                                 \
    return ib200::moe_expert_ffn<T>(IB200_VIEW2_ARG(a0), IB200_VIEW1_ARG(a1), IB200_VIEW1_ARG(a2),              \
                                    IB200_VIEW1_ARG(a3), IB200_VIEW1_ARG(a4), IB200_VIEW3_ARG(a5),              \
                                    IB200_VIEW3_ARG(a6), IB200_VIEW2_ARG(a7), workspace, workspace_bytes,       \
                                    static_cast<cudaStream_t>(stream));                                         \
  }
IB200_MOE_FFN_ENTRY(intent_b200_moe_expert_ffn_f16, __half)
IB200_MOE_FFN_ENTRY(intent_b200_moe_expert_ffn_bf16, __nv_bfloat16)

extern "C" int intent_b200_grouped_gemm16_device_status(void) {
  int value = 0, zero = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return ib200::cuda_status(e);
  e = cudaMemcpyFromSymbol(&value, ib200::g_grouped16_status, sizeof(int));
  if (e != cudaSuccess) return ib200::cuda_status(e);
  if (value != 0) cudaMemcpyToSymbol(ib200::g_grouped16_status, &zero, sizeof(int));
  return value;
}

// gemm (examples/kernels/contraction/gemm.py:40-61): f16, activation 0 = none, 1 = ReLU
extern "C" int intent_b200_gemm_f16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                    int32_t activation, void* stream) {
  using namespace ib200;
  if (activation != 0 && activation != 1) return INTENT_B200_ERR_UNSUPPORTED;
  return activation ? dense_gemm<__half, kReluCast>(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2),
                                                    nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream))
                    : dense_gemm<__half, kCast>(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2),
                                                nullptr, nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

// bf16_gemm (gemm.py:64-80)
extern "C" int intent_b200_bf16_gemm(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                     void* stream) {
  using namespace ib200;
  return dense_gemm<__nv_bfloat16, kCast>(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2), nullptr,
                                          nullptr, nullptr, static_cast<cudaStream_t>(stream));
}

// quantized_gemm (gemm.py:83-106): a0 a [M,K] f16, a1 b [K,N] f16, a2 bias [N] f32, a3 residual [M,N] f16,
// a4 output_scale [N] f32 -> a5 output [M,N] i8
extern "C" int intent_b200_quantized_gemm_f16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW1(a2),
                                              INTENT_B200_VIEW2(a3), INTENT_B200_VIEW1(a4), INTENT_B200_VIEW2(a5),
                                              void* stream) {
  using namespace ib200;
  if (a2_d0 != a1_d1 || a4_d0 != a1_d1 || a3_d0 != a0_d0 || a3_d1 != a1_d1) return INTENT_B200_ERR_SHAPE;
  if (a0_d0 > 0 && a1_d1 > 0 && (!a2 || !a3 || !a4)) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW1_ARG(a2)) || !contiguous(IB200_VIEW2_ARG(a3)) || !contiguous(IB200_VIEW1_ARG(a4)) ||
      !aligned16(a2) || !aligned16(a3) || !aligned16(a4))
    return INTENT_B200_ERR_LAYOUT;
  return dense_gemm<__half, kQuantize>(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a5),
                                       static_cast<const float*>(a2), a3, static_cast<const float*>(a4),
                                       static_cast<cudaStream_t>(stream));
}
