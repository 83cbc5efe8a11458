// W4A16 skinny contraction (decode GEMV and small-M GEMM): a bandwidth kernel.
//
//   Y[m, n] = T( sum_k f32(X[m, k]) * (q[k, n] - 8) * f32(S[k / G, n]) ),   M <= 32
//
// Program: weight_only_int4_matmul (reference kernel body
// examples/kernels/contraction/weight_only_int4.py:18-51).  The reference has
// no decode-specific lowering; this kernel is the B200 one.
//
// Data movement.  The packed weight is [K/8, N] int32 with N contiguous, so a
// 128-bit load fetches 4 adjacent columns x 8 consecutive k.  A warp reads four
// 128-byte row segments per load instruction: lane = 4*g + t loads row
// (r + t), columns 4g..4g+3 (g = 0..7 covers 32 columns).  Every weight byte is
// read exactly once with streaming (no-allocate) loads.
//
// Arithmetic.  The nibbles are expanded in registers with the magic-number
// trick: (w >> 4j) & 0x000F000F | magic gives the pair (k = j, k = j + 4) of one
// column as two exact 16-bit floats, one subtraction removes magic + 8.  The
// pairs feed mma.sync.m16n8k16 directly as the A fragment (rows of the MMA =
// weight columns, the k slots of quad lane t = the 8 k of the row that lane
// loaded), the activations are the B fragment, so all M <= 8 rows of X cost
// one instruction and accumulate in f32.  Activations are staged once per CTA
// in shared memory, already permuted to the (0,4)(1,5)(2,6)(3,7) pair order.
// Scales are applied once per quantisation group to the f32 group sum.
//
// Reduction over K: inside the MMA across the quad, across warps of the CTA
// through shared memory, across the CTAs of a thread-block cluster (split-K)
// through distributed shared memory.  No global scratch, no atomics, the
// summation order is fixed => bitwise reproducible.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace ib200 {
namespace {

struct SkinnyParams {
  const void* x;
  const uint32_t* packed;
  const void* scales;
  void* y;
  int M, K, N, G;
  uint32_t xor_mask;      // 0x88888888 turns a two's-complement nibble into nibble-minus-8 form
  int groups;             // K / G
  int groups_per_slice;   // quantisation groups handled by one CTA of the cluster
};

// One packed word -> four registers holding the pairs (0,4) (1,5) (2,6) (3,7) as q - 8.
template <typename T>
__device__ __forceinline__ void expand(uint32_t w, uint32_t (&pair)[4]) {
  pair[0] = Elem<T>::sub2(lop3_and_or(w, 0x000F000Fu, Elem<T>::kMagic2), Elem<T>::kBias2);
  pair[1] = Elem<T>::sub2(lop3_and_or(w >> 4, 0x000F000Fu, Elem<T>::kMagic2), Elem<T>::kBias2);
  pair[2] = Elem<T>::sub2(lop3_and_or(w >> 8, 0x000F000Fu, Elem<T>::kMagic2), Elem<T>::kBias2);
  pair[3] = Elem<T>::sub2(lop3_and_or(w >> 12, 0x000F000Fu, Elem<T>::kMagic2), Elem<T>::kBias2);
}

// MB = number of 8-row activation blocks (M <= 8*MB); WN/WK = warps along N / K.
// STEPS = G / 32 = 128-bit loads per lane and group.
template <typename T, int MB, int WN, int WK, int STEPS>
__global__ void __launch_bounds__(WN* WK * 32)
w4a16_skinny_kernel(const SkinnyParams p) {
  constexpr int TILE_N = 32 * WN;
  extern __shared__ __align__(16) unsigned char smem[];

  cg::cluster_group cluster = cg::this_cluster();
  const int slice = static_cast<int>(cluster.block_rank());
  const int slices = static_cast<int>(cluster.num_blocks());

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int wn = warp % WN;
  const int wk = warp / WN;
  const int g = lane >> 2;
  const int t = lane & 3;

  const int group_begin = slice * p.groups_per_slice;
  const int group_end = min(p.groups, group_begin + p.groups_per_slice);
  const int rows_per_group = p.G >> 3;
  const int slice_row0 = group_begin * rows_per_group;
  const int slice_rows = max(0, group_end - group_begin) * rows_per_group;

  uint4* xs = reinterpret_cast<uint4*>(smem);                                // [slice_rows][M]
  float* red = reinterpret_cast<float*>(smem + size_t(p.groups_per_slice) * rows_per_group * p.M * 16);
  // red: [WK][8*MB][TILE_N]

  // ---- stage the activations of this K slice, permuted to pair order ----------
  {
    const uint4* xg = reinterpret_cast<const uint4*>(p.x);
    const int k8 = p.K >> 3;
    for (int i = tid; i < slice_rows * p.M; i += WN * WK * 32) {
      const int m = i / slice_rows;
      const int r = i - m * slice_rows;
      const uint4 v = xg[size_t(m) * k8 + slice_row0 + r];
      uint4 o;
      o.x = prmt(v.x, v.z, 0x5410);  // (k0, k4)
      o.y = prmt(v.x, v.z, 0x7632);  // (k1, k5)
      o.z = prmt(v.y, v.w, 0x5410);  // (k2, k6)
      o.w = prmt(v.y, v.w, 0x7632);  // (k3, k7)
      xs[r * p.M + m] = o;
    }
  }
  __syncthreads();

  const int col = blockIdx.x * TILE_N + wn * 32 + 4 * g;  // first of this lane's 4 columns
  const bool col_ok = col < p.N;

  float facc[MB][8];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int i = 0; i < 8; ++i) facc[mb][i] = 0.f;

  const uint32_t* wbase = p.packed + col;
  const uint16_t* sbase = reinterpret_cast<const uint16_t*>(p.scales) + col;

  auto load_group = [&](int grp, uint4 (&w)[STEPS], uint2& s) {
    const int row = grp * rows_per_group + t;
#pragma unroll
    for (int i = 0; i < STEPS; ++i) w[i] = ldg_stream_v4(wbase + size_t(row + 4 * i) * p.N);
    s = ldg_stream_v2(sbase + size_t(grp) * p.N);
  };

  int grp = group_begin + wk;
  uint4 wcur[STEPS];
  uint2 scur = make_uint2(0, 0);
#pragma unroll
  for (int i = 0; i < STEPS; ++i) wcur[i] = make_uint4(0, 0, 0, 0);
  if (col_ok && grp < group_end) load_group(grp, wcur, scur);

  for (; grp < group_end; grp += WK) {
    uint4 wnext[STEPS];
    uint2 snext = make_uint2(0, 0);
#pragma unroll
    for (int i = 0; i < STEPS; ++i) wnext[i] = make_uint4(0, 0, 0, 0);
    if (col_ok && grp + WK < group_end) load_group(grp + WK, wnext, snext);

    float gacc[MB][8];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < 8; ++i) gacc[mb][i] = 0.f;

    const int local_row = grp * rows_per_group - slice_row0 + t;
#pragma unroll
    for (int i = 0; i < STEPS; ++i) {
      uint32_t c0[4], c1[4], c2[4], c3[4];
      expand<T>(wcur[i].x ^ p.xor_mask, c0);
      expand<T>(wcur[i].y ^ p.xor_mask, c1);
      expand<T>(wcur[i].z ^ p.xor_mask, c2);
      expand<T>(wcur[i].w ^ p.xor_mask, c3);
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        uint4 b = make_uint4(0, 0, 0, 0);
        const int m = mb * 8 + g;
        if (m < p.M) b = xs[(local_row + 4 * i) * p.M + m];
        float(&a01)[4] = *reinterpret_cast<float(*)[4]>(&gacc[mb][0]);  // columns +0, +1
        float(&a23)[4] = *reinterpret_cast<float(*)[4]>(&gacc[mb][4]);  // columns +2, +3
        Elem<T>::mma16816(a01, c0[0], c1[0], c0[1], c1[1], b.x, b.y);
        Elem<T>::mma16816(a01, c0[2], c1[2], c0[3], c1[3], b.z, b.w);
        Elem<T>::mma16816(a23, c2[0], c3[0], c2[1], c3[1], b.x, b.y);
        Elem<T>::mma16816(a23, c2[2], c3[2], c2[3], c3[3], b.z, b.w);
      }
    }
    const float s0 = Elem<T>::to_float(uint16_t(scur.x & 0xFFFF));
    const float s1 = Elem<T>::to_float(uint16_t(scur.x >> 16));
    const float s2 = Elem<T>::to_float(uint16_t(scur.y & 0xFFFF));
    const float s3 = Elem<T>::to_float(uint16_t(scur.y >> 16));
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      facc[mb][0] = fmaf(gacc[mb][0], s0, facc[mb][0]);
      facc[mb][1] = fmaf(gacc[mb][1], s0, facc[mb][1]);
      facc[mb][2] = fmaf(gacc[mb][2], s1, facc[mb][2]);
      facc[mb][3] = fmaf(gacc[mb][3], s1, facc[mb][3]);
      facc[mb][4] = fmaf(gacc[mb][4], s2, facc[mb][4]);
      facc[mb][5] = fmaf(gacc[mb][5], s2, facc[mb][5]);
      facc[mb][6] = fmaf(gacc[mb][6], s3, facc[mb][6]);
      facc[mb][7] = fmaf(gacc[mb][7], s3, facc[mb][7]);
    }
#pragma unroll
    for (int i = 0; i < STEPS; ++i) wcur[i] = wnext[i];
    scur = snext;
  }

  // ---- reduce over the K warps of the CTA -----------------------------------
  // Accumulator element (mb, j): row m = 8*mb + 2t + (j & 1), column 4g + (j >> 1) for j < 4
  // (first MMA pair) and 4g + 2 + ((j - 4) >> 1) for j >= 4.
#pragma unroll
  for (int mb = 0; mb < MB; ++mb) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int m = mb * 8 + 2 * t + h;
      float4 v = make_float4(facc[mb][0 + h], facc[mb][2 + h], facc[mb][4 + h], facc[mb][6 + h]);
      *reinterpret_cast<float4*>(&red[(size_t(wk) * 8 * MB + m) * TILE_N + wn * 32 + 4 * g]) = v;
    }
  }
  __syncthreads();
  constexpr int OUT = 8 * MB * TILE_N;
  for (int i = tid; i < OUT; i += WN * WK * 32) {
    float sum = red[i];
#pragma unroll
    for (int w = 1; w < WK; ++w) sum += red[size_t(w) * OUT + i];
    red[i] = sum;  // partial of this CTA (only this thread touches index i)
  }

  // ---- reduce over the K slices of the cluster, write the result -------------
  if (slices > 1) cluster.sync(); else __syncthreads();
  if (slice == 0) {
    uint16_t* y = reinterpret_cast<uint16_t*>(p.y);
    for (int i = tid; i < OUT; i += WN * WK * 32) {
      const int m = i / TILE_N;
      const int c = blockIdx.x * TILE_N + (i - m * TILE_N);
      float sum = red[i];
      for (int s = 1; s < slices; ++s) sum += cluster.map_shared_rank(red, s)[i];
      if (m < p.M && c < p.N) y[size_t(m) * p.N + c] = Elem<T>::from_float(sum);
    }
  }
  if (slices > 1) cluster.sync();  // keep the other CTAs' shared memory alive until read
}

int g_cfg_warps_n = 0, g_cfg_warps_k = 0, g_cfg_split_k = 0;

template <typename T, int MB, int WN, int WK, int STEPS>
int launch(const SkinnyParams& p, int split_k, size_t smem_bytes, cudaStream_t stream) {
  auto kernel = w4a16_skinny_kernel<T, MB, WN, WK, STEPS>;
  if (smem_bytes > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem_bytes));
    if (e != cudaSuccess) return cuda_status(e);
  }
  cudaLaunchConfig_t config = {};
  const int tiles = (p.N + 32 * WN - 1) / (32 * WN);
  config.gridDim = dim3(tiles, split_k, 1);
  config.blockDim = dim3(WN * WK * 32, 1, 1);
  config.dynamicSmemBytes = smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 1;
  attribute[0].val.clusterDim.y = split_k;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, p);
  if (e != cudaSuccess) return cuda_status(e);
  note_launch();
  return launch_status();
}

template <typename T, int MB, int STEPS>
int dispatch_shape(const SkinnyParams& p, int wn, int wk, int split_k, size_t smem, cudaStream_t stream) {
#define IB200_SKINNY_CASE(WN_, WK_) \
  if (wn == WN_ && wk == WK_) return launch<T, MB, WN_, WK_, STEPS>(p, split_k, smem, stream);
  IB200_SKINNY_CASE(1, 4)
  IB200_SKINNY_CASE(1, 8)
  IB200_SKINNY_CASE(2, 2)
  IB200_SKINNY_CASE(2, 4)
  IB200_SKINNY_CASE(4, 1)
  IB200_SKINNY_CASE(4, 2)
#undef IB200_SKINNY_CASE
  return INTENT_B200_ERR_UNSUPPORTED;
}

template <typename T>
int run(View2 x, View2 w, View2 s, View2 y, int group_size, int zero_point, cudaStream_t stream) {
  if (!x.p || !w.p || !s.p || !y.p) return (x.d0 == 0 || y.d1 == 0) ? INTENT_B200_OK : INTENT_B200_ERR_NULL;
  const int64_t M = x.d0, K = x.d1, N = w.d1;
  if (group_size <= 0 || group_size % 32 != 0 || (group_size != 32 && group_size != 64 && group_size != 128))
    return INTENT_B200_ERR_UNSUPPORTED;
  if (zero_point != -1 && zero_point != 8) return INTENT_B200_ERR_UNSUPPORTED;
  if (K % group_size != 0 || w.d0 * 8 != K || s.d0 * group_size != K || s.d1 != N || y.d0 != M || y.d1 != N)
    return INTENT_B200_ERR_SHAPE;
  if (!contiguous(x) || !contiguous(w) || !contiguous(s) || !contiguous(y)) return INTENT_B200_ERR_LAYOUT;
  if (!aligned16(x.p) || !aligned16(w.p) || !aligned16(s.p) || !aligned16(y.p)) return INTENT_B200_ERR_LAYOUT;
  if (M == 0 || N == 0) return INTENT_B200_OK;
  if (K == 0) return INTENT_B200_ERR_UNSUPPORTED;
  if (N % 4 != 0 || M > 32 || K > (1 << 24) || N > (1 << 24)) return INTENT_B200_ERR_UNSUPPORTED;

  SkinnyParams p;
  p.x = x.p;
  p.packed = static_cast<const uint32_t*>(w.p);
  p.scales = s.p;
  p.y = y.p;
  p.M = int(M);
  p.K = int(K);
  p.N = int(N);
  p.G = group_size;
  p.xor_mask = zero_point == -1 ? 0x88888888u : 0u;
  p.groups = int(K / group_size);

  const int mb = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  // Launch shape: 64-column tiles, 4 K-warps; split K over a cluster until the grid
  // has a few CTAs per SM and the staged activations fit in shared memory.
  int wn = g_cfg_warps_n ? g_cfg_warps_n : 2;
  int wk = g_cfg_warps_k ? g_cfg_warps_k : 4;
  const int tiles = int((N + 32 * wn - 1) / (32 * wn));
  int split_k = 1;
  if (g_cfg_split_k) {
    split_k = g_cfg_split_k;
  } else {
    while (split_k < 8 && (tiles * split_k < 3 * 148) && (p.groups / (split_k * 2) >= wk)) split_k *= 2;
  }
  size_t smem = 0;
  for (;; split_k *= 2) {
    if (split_k > 8) return INTENT_B200_ERR_UNSUPPORTED;
    p.groups_per_slice = (p.groups + split_k - 1) / split_k;
    smem = size_t(p.groups_per_slice) * (group_size / 8) * M * 16 + size_t(wk) * 8 * mb * 32 * wn * 4;
    if (smem <= 160 * 1024) break;
  }
  const int steps = group_size / 32;
#define IB200_SKINNY_MB(MB_)                                                                   \
  if (mb == MB_) {                                                                             \
    if (steps == 4) return dispatch_shape<T, MB_, 4>(p, wn, wk, split_k, smem, stream);        \
    if (steps == 2) return dispatch_shape<T, MB_, 2>(p, wn, wk, split_k, smem, stream);        \
    return dispatch_shape<T, MB_, 1>(p, wn, wk, split_k, smem, stream);                        \
  }
  IB200_SKINNY_MB(1)
  IB200_SKINNY_MB(2)
  IB200_SKINNY_MB(4)
#undef IB200_SKINNY_MB
  return INTENT_B200_ERR_UNSUPPORTED;
}

}  // namespace

int w4a16_skinny_f16(View2 x, View2 w, View2 s, View2 y, int g, int zp, cudaStream_t stream) {
  return run<__half>(x, w, s, y, g, zp, stream);
}
int w4a16_skinny_bf16(View2 x, View2 w, View2 s, View2 y, int g, int zp, cudaStream_t stream) {
  return run<__nv_bfloat16>(x, w, s, y, g, zp, stream);
}

}  // namespace ib200

extern "C" int intent_b200_w4a16_gemv_f16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                          INTENT_B200_VIEW2(a3), int32_t group_size, int32_t zero_point,
                                          void* stream) {
  return ib200::w4a16_skinny_f16(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2),
                                 IB200_VIEW2_ARG(a3), group_size, zero_point, static_cast<cudaStream_t>(stream));
}

extern "C" int intent_b200_w4a16_gemv_bf16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                           INTENT_B200_VIEW2(a3), int32_t group_size, int32_t zero_point,
                                           void* stream) {
  return ib200::w4a16_skinny_bf16(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2),
                                  IB200_VIEW2_ARG(a3), group_size, zero_point, static_cast<cudaStream_t>(stream));
}

extern "C" int intent_b200_w4a16_gemv_configure(int32_t warps_n, int32_t warps_k, int32_t split_k) {
  if (warps_n != 0 && warps_n != 1 && warps_n != 2 && warps_n != 4) return INTENT_B200_ERR_UNSUPPORTED;
  if (warps_k < 0 || warps_k > 8) return INTENT_B200_ERR_UNSUPPORTED;
  if (split_k != 0 && split_k != 1 && split_k != 2 && split_k != 4 && split_k != 8) return INTENT_B200_ERR_UNSUPPORTED;
  ib200::g_cfg_warps_n = warps_n;
  ib200::g_cfg_warps_k = warps_k;
  ib200::g_cfg_split_k = split_k;
  return INTENT_B200_OK;
}
