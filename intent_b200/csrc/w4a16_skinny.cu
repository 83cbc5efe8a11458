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
// trick: one lop3 ((w & mask) ^ magic) turns the nibble pair (k = j, k = j + 4)
// of one column into two exact 16-bit floats "bias + q".  The pairs feed
// mma.sync.m16n8k16 directly as the A fragment (rows of the MMA = weight
// columns, the k slots of quad lane t = the 8 k of the row that lane loaded),
// the activations are the B fragment, so all M <= 8 rows of X cost one
// instruction and accumulate in f32.  The bias and the zero point are removed
// once per quantisation group: sum_k x_k (bias_k + q_k) - sum_k x_k (bias_k + 8),
// the second sum being computed when the activations are staged.  For f16 the
// odd pairs are taken in place at bit 4 (value 1024 + 16 q) and meet
// activations pre-scaled by 1/16, which saves their shift.  Activations are
// staged once per CTA in shared memory, already permuted to the
// (0,4)(1,5)(2,6)(3,7) pair order.  Scales are applied once per group to the
// f32 group sum.
//
// Latency.  Each warp issues the weight loads of its first two groups before
// anything else; with programmatic dependent launch enabled the kernel only
// then waits for the preceding kernel (griddepcontrol.wait) and stages the
// activations, so the weight stream of one GEMV overlaps the tail of the
// previous kernel.  The weights must therefore not be produced by the kernel
// immediately before this one when that option is on.
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
  int twos_complement;    // 1: nibbles are two's-complement int4; 0: unsigned nibble minus 8
  int overlap;            // 1: launched with programmatic stream serialisation
  int groups;             // K / G
  int groups_per_slice;   // quantisation groups handled by one CTA of the cluster
};

__device__ __forceinline__ uint32_t lop3_and_xor(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(d) : "r"(a), "r"(b), "r"(c));  // (a & b) ^ c
  return d;
}

// Per element type: how one packed word becomes four pair registers
// (k0,k4) (k1,k5) (k2,k6) (k3,k7) holding "bias + (q or q^8)", how the staged
// activations are pre-scaled, and the per-k coefficient of the correction sum.
template <typename T>
struct Expand;

template <>
struct Expand<__half> {
  // even pairs: 0x6400 | q        = 1024 + q     (activation as is,   correction 1032 * x)
  // odd pairs : 0x6400 | (q << 4) = 1024 + 16 q  (activation x / 16,  correction 1152 * x/16)
  __device__ static __forceinline__ void magic(bool twos, uint32_t& a, uint32_t& b) {
    a = 0x64006400u ^ (twos ? 0x00080008u : 0u);
    b = 0x64006400u ^ (twos ? 0x00800080u : 0u);
  }
  __device__ static __forceinline__ void word(uint32_t w, uint32_t ma, uint32_t mb, uint32_t (&pair)[4]) {
    const uint32_t hi = w >> 8;
    pair[0] = lop3_and_xor(w, 0x000F000Fu, ma);
    pair[1] = lop3_and_xor(w, 0x00F000F0u, mb);
    pair[2] = lop3_and_xor(hi, 0x000F000Fu, ma);
    pair[3] = lop3_and_xor(hi, 0x00F000F0u, mb);
  }
  __device__ static __forceinline__ uint32_t scale_odd(uint32_t pair) {
    return Elem<__half>::mul2(pair, 0x2C002C00u);  // * 1/16 (exact unless subnormal)
  }
  static constexpr float kEven = 1032.f, kOdd = 1152.f;
};

template <>
struct Expand<__nv_bfloat16> {
  // 0x4300 | q = 128 + q for every pair (7 mantissa bits leave no room for the in-place form)
  __device__ static __forceinline__ void magic(bool twos, uint32_t& a, uint32_t& b) {
    a = b = 0x43004300u ^ (twos ? 0x00080008u : 0u);
  }
  __device__ static __forceinline__ void word(uint32_t w, uint32_t ma, uint32_t, uint32_t (&pair)[4]) {
    pair[0] = lop3_and_xor(w, 0x000F000Fu, ma);
    pair[1] = lop3_and_xor(w >> 4, 0x000F000Fu, ma);
    pair[2] = lop3_and_xor(w >> 8, 0x000F000Fu, ma);
    pair[3] = lop3_and_xor(w >> 12, 0x000F000Fu, ma);
  }
  __device__ static __forceinline__ uint32_t scale_odd(uint32_t pair) { return pair; }
  static constexpr float kEven = 136.f, kOdd = 136.f;
};

template <typename T>
__device__ __forceinline__ float pair_sum(uint32_t pair) {
  return Elem<T>::to_float(uint16_t(pair & 0xFFFF)) + Elem<T>::to_float(uint16_t(pair >> 16));
}

// MB = number of 8-row activation blocks (M <= 8*MB); WN/WK = warps along N / K.
// STEPS = G / 32 = 128-bit loads per lane and group.
template <typename T, int MB, int WN, int WK, int STEPS>
__global__ void __launch_bounds__(WN* WK * 32)
w4a16_skinny_kernel(const SkinnyParams p) {
  constexpr int TILE_N = 32 * WN;
  constexpr int THREADS = WN * WK * 32;
  constexpr int ROWS_PER_GROUP = STEPS * 4;  // packed rows (8 k each) per quantisation group
  constexpr int CP = 8 * MB;                 // row pitch of the correction table
  extern __shared__ __align__(16) unsigned char smem[];

  if (p.overlap) asm volatile("griddepcontrol.launch_dependents;");

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
  const int slice_row0 = group_begin * ROWS_PER_GROUP;
  const int slice_rows = max(0, group_end - group_begin) * ROWS_PER_GROUP;

  uint4* xs = reinterpret_cast<uint4*>(smem);  // [slice rows][M], pair order
  float* corr = reinterpret_cast<float*>(smem + size_t(p.groups_per_slice) * ROWS_PER_GROUP * p.M * 16);
  float* red = corr + size_t(p.groups_per_slice) * CP;  // [WK][8*MB][TILE_N]

  const int col = blockIdx.x * TILE_N + wn * 32 + 4 * g;  // first of this lane's 4 columns
  const bool col_ok = col < p.N;
  const uint32_t* wbase = p.packed + col;
  const uint16_t* sbase = reinterpret_cast<const uint16_t*>(p.scales) + col;

  auto load_group = [&](int grp, uint4 (&w)[STEPS], uint2& s) {
    const int row = grp * ROWS_PER_GROUP + t;
#pragma unroll
    for (int i = 0; i < STEPS; ++i) w[i] = ldg_stream_v4(wbase + size_t(row + 4 * i) * p.N);
    s = ldg_stream_v2(sbase + size_t(grp) * p.N);
  };

  // ---- the weight stream starts first: two groups per lane in flight ----------
  const int g0 = group_begin + wk;
  uint4 w0[STEPS], w1[STEPS];
  uint2 s0 = make_uint2(0, 0), s1 = make_uint2(0, 0);
#pragma unroll
  for (int i = 0; i < STEPS; ++i) w0[i] = w1[i] = make_uint4(0, 0, 0, 0);
  if (col_ok && g0 < group_end) load_group(g0, w0, s0);
  if (col_ok && g0 + WK < group_end) load_group(g0 + WK, w1, s1);

  // ---- stage the activations of this K slice ---------------------------------
  if (p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
  {
    const uint4* xg = reinterpret_cast<const uint4*>(p.x);
    const int k8 = p.K >> 3;
    const int total = slice_rows * p.M;
    for (int base = 0; base < total; base += THREADS) {
      const int i = base + tid;
      const bool active = i < total;
      float partial = 0.f;
      int m = 0, r = 0;
      if (active) {
        m = i / slice_rows;
        r = i - m * slice_rows;
        const uint4 v = xg[size_t(m) * k8 + slice_row0 + r];
        uint4 o;
        o.x = prmt(v.x, v.z, 0x5410);                          // (k0, k4)
        o.y = Expand<T>::scale_odd(prmt(v.x, v.z, 0x7632));    // (k1, k5)
        o.z = prmt(v.y, v.w, 0x5410);                          // (k2, k6)
        o.w = Expand<T>::scale_odd(prmt(v.y, v.w, 0x7632));    // (k3, k7)
        xs[r * p.M + m] = o;
        partial = Expand<T>::kEven * (pair_sum<T>(o.x) + pair_sum<T>(o.z)) +
                  Expand<T>::kOdd * (pair_sum<T>(o.y) + pair_sum<T>(o.w));
      }
      // rows of one group sit in ROWS_PER_GROUP adjacent lanes: fixed-order butterfly
#pragma unroll
      for (int d = ROWS_PER_GROUP / 2; d >= 1; d >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, d);
      if (active && (r % ROWS_PER_GROUP) == 0) corr[(r / ROWS_PER_GROUP) * CP + m] = partial;
    }
  }
  __syncthreads();

  uint32_t magic_a, magic_b;
  Expand<T>::magic(p.twos_complement != 0, magic_a, magic_b);

  float facc[MB][8];
#pragma unroll
  for (int mb = 0; mb < MB; ++mb)
#pragma unroll
    for (int i = 0; i < 8; ++i) facc[mb][i] = 0.f;

  auto consume = [&](int grp, const uint4 (&w)[STEPS], const uint2 s) {
    float gacc[MB][8];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < 8; ++i) gacc[mb][i] = 0.f;
    const int local_group = grp - group_begin;
    const int local_row = local_group * ROWS_PER_GROUP + t;
#pragma unroll
    for (int i = 0; i < STEPS; ++i) {
      uint32_t c0[4], c1[4], c2[4], c3[4];
      Expand<T>::word(w[i].x, magic_a, magic_b, c0);
      Expand<T>::word(w[i].y, magic_a, magic_b, c1);
      Expand<T>::word(w[i].z, magic_a, magic_b, c2);
      Expand<T>::word(w[i].w, magic_a, magic_b, c3);
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
    const float sc0 = Elem<T>::to_float(uint16_t(s.x & 0xFFFF));
    const float sc1 = Elem<T>::to_float(uint16_t(s.x >> 16));
    const float sc2 = Elem<T>::to_float(uint16_t(s.y & 0xFFFF));
    const float sc3 = Elem<T>::to_float(uint16_t(s.y >> 16));
#pragma unroll
    for (int mb = 0; mb < MB; ++mb) {
      // rows m = 8*mb + 2t and + 1; entries of rows >= M are never written out
      const float2 c = *reinterpret_cast<const float2*>(&corr[local_group * CP + mb * 8 + 2 * t]);
      facc[mb][0] = fmaf(gacc[mb][0] - c.x, sc0, facc[mb][0]);
      facc[mb][1] = fmaf(gacc[mb][1] - c.y, sc0, facc[mb][1]);
      facc[mb][2] = fmaf(gacc[mb][2] - c.x, sc1, facc[mb][2]);
      facc[mb][3] = fmaf(gacc[mb][3] - c.y, sc1, facc[mb][3]);
      facc[mb][4] = fmaf(gacc[mb][4] - c.x, sc2, facc[mb][4]);
      facc[mb][5] = fmaf(gacc[mb][5] - c.y, sc2, facc[mb][5]);
      facc[mb][6] = fmaf(gacc[mb][6] - c.x, sc3, facc[mb][6]);
      facc[mb][7] = fmaf(gacc[mb][7] - c.y, sc3, facc[mb][7]);
    }
  };

  for (int grp = g0; grp < group_end; grp += 2 * WK) {
    consume(grp, w0, s0);
    if (col_ok && grp + 2 * WK < group_end) load_group(grp + 2 * WK, w0, s0);
    if (grp + WK < group_end) {
      consume(grp + WK, w1, s1);
      if (col_ok && grp + 3 * WK < group_end) load_group(grp + 3 * WK, w1, s1);
    }
  }

  // ---- reduce over the K warps of the CTA -----------------------------------
  // Accumulator element (mb, j): row m = 8*mb + 2t + (j & 1), column 4g + (j >> 1).
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
  for (int i = tid; i < OUT; i += THREADS) {
    float sum = red[i];
#pragma unroll
    for (int w = 1; w < WK; ++w) sum += red[size_t(w) * OUT + i];
    red[i] = sum;  // partial of this CTA (only this thread touches index i)
  }

  // ---- reduce over the K slices of the cluster, write the result -------------
  if (slices > 1) cluster.sync(); else __syncthreads();
  if (slice == 0) {
    uint16_t* y = reinterpret_cast<uint16_t*>(p.y);
    for (int i = tid; i < OUT; i += THREADS) {
      const int m = i / TILE_N;
      const int c = blockIdx.x * TILE_N + (i - m * TILE_N);
      float sum = red[i];
      for (int s = 1; s < slices; ++s) sum += cluster.map_shared_rank(red, s)[i];
      if (m < p.M && c < p.N) y[size_t(m) * p.N + c] = Elem<T>::from_float(sum);
    }
  }
  if (slices > 1) cluster.sync();  // keep the other CTAs' shared memory alive until read
}

int g_cfg_warps_n = 0, g_cfg_warps_k = 0, g_cfg_split_k = 0, g_cfg_overlap = 0;

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
  cudaLaunchAttribute attribute[2];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = 1;
  attribute[0].val.clusterDim.y = split_k;
  attribute[0].val.clusterDim.z = 1;
  attribute[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[1].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = p.overlap ? 2 : 1;
  cudaError_t e = cudaLaunchKernelEx(&config, kernel, p);
  if (e != cudaSuccess) return cuda_status(e);
  note_launch();
  return launch_status();
}

template <typename T, int MB, int STEPS>
int dispatch_shape(const SkinnyParams& p, int wn, int wk, int split_k, size_t smem, cudaStream_t stream) {
#define IB200_SKINNY_CASE(WN_, WK_) \
  if (wn == WN_ && wk == WK_) return launch<T, MB, WN_, WK_, STEPS>(p, split_k, smem, stream);
  IB200_SKINNY_CASE(1, 8)
  IB200_SKINNY_CASE(1, 16)
  IB200_SKINNY_CASE(2, 4)
  IB200_SKINNY_CASE(2, 8)
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
  p.twos_complement = zero_point == -1 ? 1 : 0;
  p.overlap = g_cfg_overlap;
  p.groups = int(K / group_size);

  const int mb = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
  // Launch shape: 64-column tiles, 4 K-warps; split K over a cluster until the grid
  // has a few CTAs per SM and the staged activations fit in shared memory.
  int wn = g_cfg_warps_n ? g_cfg_warps_n : 1;
  int wk = g_cfg_warps_k ? g_cfg_warps_k : 8;
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
    smem = size_t(p.groups_per_slice) * (group_size / 8) * M * 16 + size_t(p.groups_per_slice) * 8 * mb * 4 +
           size_t(wk) * 8 * mb * 32 * wn * 4;
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
  if (warps_k < 0 || warps_k > 16) return INTENT_B200_ERR_UNSUPPORTED;
  if (split_k != 0 && split_k != 1 && split_k != 2 && split_k != 4 && split_k != 8) return INTENT_B200_ERR_UNSUPPORTED;
  ib200::g_cfg_warps_n = warps_n;
  ib200::g_cfg_warps_k = warps_k;
  ib200::g_cfg_split_k = split_k;
  return INTENT_B200_OK;
}

extern "C" int intent_b200_w4a16_gemv_overlap(int32_t enable) {
  ib200::g_cfg_overlap = enable ? 1 : 0;
  return INTENT_B200_OK;
}
