// W4A16 decode GEMV / small-M GEMM as a persistent, TMA-fed bandwidth kernel.
//
//   Y[m, n] = T( sum_k f32(X[m, k]) * (q[k, n] - 8) * f32(S[k / G, n]) ),   M <= 16
//
// Program: weight_only_int4_matmul (reference kernel body
// examples/kernels/contraction/weight_only_int4.py:18-51).  The reference has no
// decode-specific lowering; this is the B200 one.
//
// Work decomposition.  The packed weight [K/8, N] is cut into units of 64
// columns x 32 packed rows (256 k) = 8 KiB.  Units are numbered tile-major
// (all K chunks of a column tile are consecutive) and the range is split evenly
// over one CTA per SM, so every SM streams the same number of bytes (+-1 unit).
// Inside a CTA, warp w owns local units w, w+8, ...; each unit lands in a
// warp-private shared-memory slot through two 128B-swizzled TMA boxes
// (32 columns x 32 rows each) plus one box with the matching 256 activations of
// every row of X, all on one mbarrier.  The slots cover the CTA's whole share
// whenever it fits (it does for the decode shapes), so all of a CTA's weight
// bytes are requested in the first microsecond and arrive at HBM speed without
// any register staging; a slot is refilled by its own warp when the share is
// larger than shared memory.
//
// Arithmetic: as in w4a16_expand.cuh - one lop3 per nibble pair, pairs feed
// mma.sync.m16n8k16 as the A fragment (MMA rows = weight columns), activations
// are the B fragment, f32 accumulation per quantisation group, the magic bias
// and the zero point are removed per group with a correction sum computed once
// per CTA while the first TMA loads are in flight.
//
// Reduction over K: in the MMA, then per warp in registers across its units of
// one column tile, across the warps of the CTA in shared memory, and - only for
// column tiles that straddle CTAs - through a global scratch buffer: every
// contributor stores its partial, the last one to arrive (atomic ticket) adds
// the partials in slot order and writes Y.  No spin waits between CTAs; the
// summation order is fixed, so results are bitwise reproducible.
#include <type_traits>

#include "common.cuh"
#include "tma.cuh"
#include "w4a16_expand.cuh"

namespace ib200 {
namespace {

constexpr int kUnitCols = 64;
constexpr int kUnitRows = 32;                       // packed rows (8 k each)
constexpr int kUnitWeightBytes = kUnitCols * kUnitRows * 4;
constexpr int kSmemLimit = 227 * 1024;

struct StreamParams {
  const void* scales;
  const void* x;
  void* y;
  int M, K, N;
  int groups;           // K / G
  int chunks;           // ceil(K / 256)
  int tiles;            // ceil(N / 64)
  int units;            // tiles * chunks
  int slots_per_warp;
  int slot_bytes;       // weight unit + activation box, multiple of 1024
  int tiles_local_max;  // column tiles one CTA can touch
  int max_contributors; // scratch slots per column tile
  int twos_complement;
  int overlap;
  int* status;
  int* counters;
  float* scratch;
};

template <typename T, int MB, int STEPS, int kWarps>
__global__ void __launch_bounds__(kWarps * 32, 1)
w4a16_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const StreamParams p) {
  constexpr int kThreads = kWarps * 32;
  constexpr int RPG = 4 * STEPS;        // packed rows per quantisation group
  constexpr int GPC = kUnitRows / RPG;  // groups per unit
  constexpr int CP = 8 * MB;            // row pitch of the correction table
  extern __shared__ unsigned char smem_raw[];

  if (p.overlap) asm volatile("griddepcontrol.launch_dependents;");

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g = lane >> 2;
  const int t = lane & 3;

  // ---- shared memory carve-up -------------------------------------------------
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const int total_slots = kWarps * p.slots_per_warp;
  const uint32_t slots = base;
  const uint32_t bars = slots + uint32_t(total_slots) * p.slot_bytes;
  float* corr = reinterpret_cast<float*>(base_ptr + size_t(total_slots) * p.slot_bytes + size_t(total_slots) * 8);
  float* part = corr + size_t(p.groups) * CP;  // [warp][tile_local][M][64]
  const int part_tile = p.M * kUnitCols;
  __shared__ int s_last;

  // ---- this CTA's unit range -----------------------------------------------------
  const long long grid = gridDim.x;
  const int u0 = int((long long)blockIdx.x * p.units / grid);
  const int u1 = int((long long)(blockIdx.x + 1) * p.units / grid);
  const int n_units = u1 - u0;
  const int my_units = n_units > warp ? (n_units - warp + kWarps - 1) / kWarps : 0;
  const int tile0 = u0 / p.chunks;
  const uint32_t x_bytes = uint32_t(p.M) * 512u;

  auto slot_addr = [&](int n) { return slots + uint32_t(warp * p.slots_per_warp + n % p.slots_per_warp) * p.slot_bytes; };
  auto bar_addr = [&](int n) { return bars + uint32_t(warp * p.slots_per_warp + n % p.slots_per_warp) * 8u; };
  auto issue_weights = [&](int n) {
    const int u = u0 + warp + kWarps * n;
    const int tile = u / p.chunks, chunk = u - tile * p.chunks;
    mbar_expect_tx(bar_addr(n), kUnitWeightBytes + x_bytes);
    tma_load_2d(slot_addr(n), &map_w, tile * kUnitCols, chunk * kUnitRows, bar_addr(n));
    tma_load_2d(slot_addr(n) + 4096, &map_w, tile * kUnitCols + 32, chunk * kUnitRows, bar_addr(n));
  };
  auto issue_activations = [&](int n) {
    const int u = u0 + warp + kWarps * n;
    const int chunk = u % p.chunks;
    tma_load_2d(slot_addr(n) + kUnitWeightBytes, &map_x, chunk * 256, 0, bar_addr(n));
  };

  // ---- start the weight stream before anything else ----------------------------
  const int first_wave = min(my_units, p.slots_per_warp);
  if (lane == 0) {
    for (int s = 0; s < p.slots_per_warp; ++s) mbar_init(bar_addr(s), 1);
    fence_mbar_init();
    for (int n = 0; n < first_wave; ++n) issue_weights(n);
  }
  if (p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (lane == 0)
    for (int n = 0; n < first_wave; ++n) issue_activations(n);

  // ---- while the loads fly: zero the partial table, build the correction table ----
  const int tiles_local = n_units > 0 ? (u1 - 1) / p.chunks - tile0 + 1 : 0;
  for (int i = tid; i < kWarps * p.tiles_local_max * part_tile; i += kThreads) part[i] = 0.f;
  {
    // corr[group][m] = sum over the group's k of x[m,k] * (bias_k + 8), for the chunks this CTA touches
    const uint4* xg = reinterpret_cast<const uint4*>(p.x);
    const int k8 = p.K >> 3;
    const int touched = min(p.chunks, n_units);
    const int rows = touched * kUnitRows;
    const int total = rows * p.M;
    for (int start = 0; start < total; start += kThreads) {
      const int i = start + tid;
      float partial = 0.f;
      int m = 0, row = 0;
      bool active = i < total;
      if (active) {
        m = i / rows;
        const int lr = i - m * rows;
        const int chunk = (u0 + lr / kUnitRows) % p.chunks;
        row = chunk * kUnitRows + (lr % kUnitRows);
        active = row < k8;
        if (active) {
          const uint4 v = xg[size_t(m) * k8 + row];
          const uint32_t p04 = prmt(v.x, v.z, 0x5410), p15 = Expand<T>::scale_odd(prmt(v.x, v.z, 0x7632));
          const uint32_t p26 = prmt(v.y, v.w, 0x5410), p37 = Expand<T>::scale_odd(prmt(v.y, v.w, 0x7632));
          partial = Expand<T>::kEven * (pair_sum<T>(p04) + pair_sum<T>(p26)) +
                    Expand<T>::kOdd * (pair_sum<T>(p15) + pair_sum<T>(p37));
        }
      }
#pragma unroll
      for (int d = RPG / 2; d >= 1; d >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, d);
      if (active && (row % RPG) == 0) corr[(row / RPG) * CP + m] = partial;
    }
  }
  __syncthreads();

  uint32_t magic_a, magic_b;
  Expand<T>::magic(p.twos_complement != 0, magic_a, magic_b);
  const uint16_t* sg = reinterpret_cast<const uint16_t*>(p.scales);

  float facc[2][MB][8];
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < 8; ++i) facc[h][mb][i] = 0.f;

  // accumulator element (h, mb, j): row m = 8*mb + 2t + (j & 1), column 32h + 4g + (j >> 1)
  auto flush = [&](int tile) {
    float* dst = part + size_t(warp * p.tiles_local_max + (tile - tile0)) * part_tile;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int m = mb * 8 + 2 * t + hh;
          if (m < p.M) {
            float4* q = reinterpret_cast<float4*>(dst + m * kUnitCols + h * 32 + 4 * g);
            float4 v = *q;
            v.x += facc[h][mb][0 + hh];
            v.y += facc[h][mb][2 + hh];
            v.z += facc[h][mb][4 + hh];
            v.w += facc[h][mb][6 + hh];
            *q = v;
          }
          facc[h][mb][0 + hh] = facc[h][mb][2 + hh] = facc[h][mb][4 + hh] = facc[h][mb][6 + hh] = 0.f;
        }
  };

  int current_tile = -1;
  bool failed = false;
  for (int n = 0; n < my_units && !failed; ++n) {
    const int u = u0 + warp + kWarps * n;
    const int tile = u / p.chunks, chunk = u - tile * p.chunks;
    if (tile != current_tile) {
      if (current_tile >= 0) flush(current_tile);
      current_tile = tile;
    }
    uint2 sc[2][GPC];
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int gi = 0; gi < GPC; ++gi) {
        const int col = tile * kUnitCols + h * 32 + 4 * g;
        const int group = chunk * GPC + gi;
        sc[h][gi] = (col < p.N && group < p.groups) ? ldg_stream_v2(sg + size_t(group) * p.N + col) : make_uint2(0, 0);
      }
    if (!__all_sync(0xffffffffu, mbar_wait(bar_addr(n), (n / p.slots_per_warp) & 1))) {
      failed = true;  // warp-uniform: the loads of this unit never completed
      if (lane == 0) atomicExch(p.status, INTENT_B200_ERR_TIMEOUT);
      break;
    }
    const uint32_t wslot = slot_addr(n);
    const uint32_t xslot = wslot + kUnitWeightBytes;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int gi = 0; gi < GPC; ++gi) {
        float gacc[MB][8];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb)
#pragma unroll
          for (int i = 0; i < 8; ++i) gacc[mb][i] = 0.f;
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
          // rows 2t + parity keep the eight lanes of a quarter-warp on distinct swizzled bank groups
          const int row = gi * RPG + (STEPS >= 2 ? 8 * (i >> 1) + 2 * t + (i & 1) : t);
          const uint4 w = lds128(wslot + h * 4096 + row * 128 + ((g ^ (row & 7)) << 4));
          uint32_t c0[4], c1[4], c2[4], c3[4];
          Expand<T>::word(w.x, magic_a, magic_b, c0);
          Expand<T>::word(w.y, magic_a, magic_b, c1);
          Expand<T>::word(w.z, magic_a, magic_b, c2);
          Expand<T>::word(w.w, magic_a, magic_b, c3);
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) {
            uint4 b = make_uint4(0, 0, 0, 0);
            const int m = mb * 8 + g;
            if (m < p.M) {
              const uint4 v = lds128(xslot + m * 512 + row * 16);
              b.x = prmt(v.x, v.z, 0x5410);
              b.y = Expand<T>::scale_odd(prmt(v.x, v.z, 0x7632));
              b.z = prmt(v.y, v.w, 0x5410);
              b.w = Expand<T>::scale_odd(prmt(v.y, v.w, 0x7632));
            }
            float(&a01)[4] = *reinterpret_cast<float(*)[4]>(&gacc[mb][0]);
            float(&a23)[4] = *reinterpret_cast<float(*)[4]>(&gacc[mb][4]);
            Elem<T>::mma16816(a01, c0[0], c1[0], c0[1], c1[1], b.x, b.y);
            Elem<T>::mma16816(a01, c0[2], c1[2], c0[3], c1[3], b.z, b.w);
            Elem<T>::mma16816(a23, c2[0], c3[0], c2[1], c3[1], b.x, b.y);
            Elem<T>::mma16816(a23, c2[2], c3[2], c2[3], c3[3], b.z, b.w);
          }
        }
        const int group = chunk * GPC + gi;
        const uint2 s = sc[h][gi];
        const float s0 = Elem<T>::to_float(uint16_t(s.x & 0xFFFF)), s1 = Elem<T>::to_float(uint16_t(s.x >> 16));
        const float s2 = Elem<T>::to_float(uint16_t(s.y & 0xFFFF)), s3 = Elem<T>::to_float(uint16_t(s.y >> 16));
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          float2 c = make_float2(0.f, 0.f);
          if (group < p.groups) c = *reinterpret_cast<const float2*>(&corr[group * CP + mb * 8 + 2 * t]);
          facc[h][mb][0] = fmaf(gacc[mb][0] - c.x, s0, facc[h][mb][0]);
          facc[h][mb][1] = fmaf(gacc[mb][1] - c.y, s0, facc[h][mb][1]);
          facc[h][mb][2] = fmaf(gacc[mb][2] - c.x, s1, facc[h][mb][2]);
          facc[h][mb][3] = fmaf(gacc[mb][3] - c.y, s1, facc[h][mb][3]);
          facc[h][mb][4] = fmaf(gacc[mb][4] - c.x, s2, facc[h][mb][4]);
          facc[h][mb][5] = fmaf(gacc[mb][5] - c.y, s2, facc[h][mb][5]);
          facc[h][mb][6] = fmaf(gacc[mb][6] - c.x, s3, facc[h][mb][6]);
          facc[h][mb][7] = fmaf(gacc[mb][7] - c.y, s3, facc[h][mb][7]);
        }
      }
    }
    if (n + p.slots_per_warp < my_units) {  // refill this slot with the warp's next unit
      __syncwarp();
      fence_proxy_async();
      if (lane == 0) {
        issue_weights(n + p.slots_per_warp);
        issue_activations(n + p.slots_per_warp);
      }
    }
  }
  if (current_tile >= 0 && !failed) flush(current_tile);
  __syncthreads();

  // ---- per column tile: add the warps' partials, then write Y or go through scratch ----
  uint16_t* y = reinterpret_cast<uint16_t*>(p.y);
  for (int tl = 0; tl < tiles_local; ++tl) {
    const int tile = tile0 + tl;
    const int first_u = tile * p.chunks, last_u = first_u + p.chunks - 1;
    const bool whole = u0 <= first_u && last_u < u1;
    const int c_first = int(((long long)(first_u + 1) * grid - 1) / p.units);
    const int c_last = int(((long long)(last_u + 1) * grid - 1) / p.units);
    const int contributors = c_last - c_first + 1;
    float* mine = p.scratch + (size_t(tile) * p.max_contributors + (blockIdx.x - c_first)) * part_tile;
    for (int i = tid; i < part_tile; i += kThreads) {
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) sum += part[size_t(w * p.tiles_local_max + tl) * part_tile + i];
      if (whole) {
        const int m = i / kUnitCols, col = tile * kUnitCols + (i - m * kUnitCols);
        if (col < p.N) y[size_t(m) * p.N + col] = Elem<T>::from_float(sum);
      } else {
        mine[i] = sum;
      }
    }
    if (!whole) {
      __threadfence();
      __syncthreads();
      if (tid == 0) s_last = (atomicAdd(&p.counters[tile], 1) == contributors - 1) ? 1 : 0;
      __syncthreads();
      if (s_last) {
        __threadfence();
        const float* all = p.scratch + size_t(tile) * p.max_contributors * part_tile;
        for (int i = tid; i < part_tile; i += kThreads) {
          float sum = 0.f;
          for (int s = 0; s < contributors; ++s) sum += __ldcg(all + size_t(s) * part_tile + i);
          const int m = i / kUnitCols, col = tile * kUnitCols + (i - m * kUnitCols);
          if (col < p.N) y[size_t(m) * p.N + col] = Elem<T>::from_float(sum);
        }
        if (tid == 0) p.counters[tile] = 0;  // leave the ticket counter ready for the next launch
      }
      __syncthreads();
    }
  }
}


struct Plan {
  int grid, slots_per_warp, slot_bytes, tiles_local_max, max_contributors;
  size_t smem_bytes, counters_offset, scratch_offset, workspace_bytes;
  int tiles, chunks, units;
};

// Launch geometry and workspace layout for one problem size (pure arithmetic).
bool make_plan(int M, int K, int N, int mb, int sms, int kWarps, Plan* plan) {
  Plan q{};
  q.tiles = (N + kUnitCols - 1) / kUnitCols;
  q.chunks = (K / 8 + kUnitRows - 1) / kUnitRows;
  q.units = q.tiles * q.chunks;
  q.grid = q.units < sms ? q.units : sms;
  const int per_cta_max = (q.units + q.grid - 1) / q.grid;
  const int per_cta_min = q.units / q.grid;
  const int per_warp_max = (per_cta_max + kWarps - 1) / kWarps;
  q.slot_bytes = kUnitWeightBytes + ((M * 512 + 1023) / 1024) * 1024;
  q.tiles_local_max = (per_cta_max + q.chunks - 2) / q.chunks + 1;
  q.max_contributors = (q.chunks - 1) / per_cta_min + 2;
  if (q.max_contributors > q.grid) q.max_contributors = q.grid;
  const size_t fixed = 1024 + size_t((K + 31) / 32) * 8 * mb * 4  // corr: at most K/32 groups
                       + size_t(kWarps) * q.tiles_local_max * M * kUnitCols * 4;
  int spw = per_warp_max;
  while (spw > 0 && fixed + size_t(kWarps) * spw * (q.slot_bytes + 8) > size_t(kSmemLimit)) --spw;
  if (spw < 1) return false;
  q.slots_per_warp = spw;
  q.smem_bytes = fixed + size_t(kWarps) * spw * (q.slot_bytes + 8);
  q.counters_offset = 256;
  q.scratch_offset = ((q.counters_offset + size_t(q.tiles) * 4 + 255) / 256) * 256;
  q.workspace_bytes = q.scratch_offset + size_t(q.tiles) * q.max_contributors * M * kUnitCols * 4;
  *plan = q;
  return true;
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

int g_overlap = 0;
int g_grid_override = 0;
int g_warps = 8;

template <typename T, int MB, int STEPS, int kWarps>
int launch_warps(const CUtensorMap& map_w, const CUtensorMap& map_x, const StreamParams& p, const Plan& plan,
                 cudaStream_t stream) {
  constexpr int kThreads = kWarps * 32;
  auto kernel = w4a16_stream_kernel<T, MB, STEPS, kWarps>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(plan.smem_bytes));
  if (e != cudaSuccess) return cuda_status(e);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(plan.grid, 1, 1);
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = plan.smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = p.overlap ? 1 : 0;
  e = cudaLaunchKernelEx(&config, kernel, map_w, map_x, p);
  if (e != cudaSuccess) return cuda_status(e);
  note_launch();
  return launch_status();
}

template <typename T, int MB, int STEPS>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const StreamParams& p, const Plan& plan,
           cudaStream_t stream) {
  if (g_warps == 16) return launch_warps<T, MB, STEPS, 16>(map_w, map_x, p, plan, stream);
  return launch_warps<T, MB, STEPS, 8>(map_w, map_x, p, plan, stream);
}

template <typename T>
int run(View2 x, View2 w, View2 s, View2 y, int group_size, int zero_point, void* workspace,
        int64_t workspace_bytes, cudaStream_t stream) {
  const int64_t M = x.d0, K = x.d1, N = w.d1;
  if (group_size != 32 && group_size != 64 && group_size != 128) return INTENT_B200_ERR_UNSUPPORTED;
  if (zero_point != -1 && zero_point != 8) return INTENT_B200_ERR_UNSUPPORTED;
  if (K % group_size != 0 || w.d0 * 8 != K || s.d0 * group_size != K || s.d1 != N || y.d0 != M || y.d1 != N)
    return INTENT_B200_ERR_SHAPE;
  if (M == 0 || N == 0) return INTENT_B200_OK;
  if (!x.p || !w.p || !s.p || !y.p) return INTENT_B200_ERR_NULL;
  if (!contiguous(x) || !contiguous(w) || !contiguous(s) || !contiguous(y)) return INTENT_B200_ERR_LAYOUT;
  if (!aligned16(x.p) || !aligned16(w.p) || !aligned16(s.p) || !aligned16(y.p)) return INTENT_B200_ERR_LAYOUT;
  if (K == 0 || N % 4 != 0 || M > 16 || K > (1 << 24) || N > (1 << 24)) return INTENT_B200_ERR_UNSUPPORTED;
  const int mb = M <= 8 ? 1 : 2;
  const int sms = g_grid_override > 0 ? g_grid_override : device_sms();
  if (sms <= 0) return INTENT_B200_ERR_UNSUPPORTED;
  Plan plan;
  if (!make_plan(int(M), int(K), int(N), mb, sms, g_warps, &plan)) return INTENT_B200_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < int64_t(plan.workspace_bytes) || !aligned16(workspace))
    return INTENT_B200_ERR_WORKSPACE;

  CUtensorMap map_w, map_x;
  if (!make_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_INT32, w.p, uint64_t(K / 8), uint64_t(N), uint64_t(N) * 4,
                          kUnitRows, 32, CU_TENSOR_MAP_SWIZZLE_128B))
    return INTENT_B200_ERR_UNSUPPORTED;
  const CUtensorMapDataType xt = sizeof(T) == 2 && std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                                  : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  if (!make_tensor_map_2d(&map_x, xt, x.p, uint64_t(M), uint64_t(K), uint64_t(K) * 2, uint32_t(M), 256,
                          CU_TENSOR_MAP_SWIZZLE_NONE))
    return INTENT_B200_ERR_UNSUPPORTED;

  StreamParams p{};
  p.scales = s.p;
  p.x = x.p;
  p.y = y.p;
  p.M = int(M);
  p.K = int(K);
  p.N = int(N);
  p.groups = int(K / group_size);
  p.chunks = plan.chunks;
  p.tiles = plan.tiles;
  p.units = plan.units;
  p.slots_per_warp = plan.slots_per_warp;
  p.slot_bytes = plan.slot_bytes;
  p.tiles_local_max = plan.tiles_local_max;
  p.max_contributors = plan.max_contributors;
  p.twos_complement = zero_point == -1 ? 1 : 0;
  p.overlap = g_overlap;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  p.status = reinterpret_cast<int*>(ws);
  p.counters = reinterpret_cast<int*>(ws + plan.counters_offset);
  p.scratch = reinterpret_cast<float*>(ws + plan.scratch_offset);

  const int steps = group_size / 32;
#define IB200_STREAM_MB(MB_)                                                            \
  if (mb == MB_) {                                                                      \
    if (steps == 4) return launch<T, MB_, 4>(map_w, map_x, p, plan, stream);            \
    if (steps == 2) return launch<T, MB_, 2>(map_w, map_x, p, plan, stream);            \
    return launch<T, MB_, 1>(map_w, map_x, p, plan, stream);                            \
  }
  IB200_STREAM_MB(1)
  IB200_STREAM_MB(2)
#undef IB200_STREAM_MB
  return INTENT_B200_ERR_UNSUPPORTED;
}

}  // namespace
}  // namespace ib200

namespace ib200 {
int w4a16_stream_f16(View2 x, View2 w, View2 s, View2 y, int g, int zp, void* ws, int64_t ws_bytes,
                     cudaStream_t stream) {
  return run<__half>(x, w, s, y, g, zp, ws, ws_bytes, stream);
}
int w4a16_stream_bf16(View2 x, View2 w, View2 s, View2 y, int g, int zp, void* ws, int64_t ws_bytes,
                      cudaStream_t stream) {
  return run<__nv_bfloat16>(x, w, s, y, g, zp, ws, ws_bytes, stream);
}
int64_t w4a16_stream_workspace_bytes(int64_t M, int64_t K, int64_t N) {
  if (M <= 0 || N <= 0 || K <= 0 || M > 16 || K > (1 << 24) || N > (1 << 24)) return 0;
  const int mb = M <= 8 ? 1 : 2;
  const int sms = g_grid_override > 0 ? g_grid_override : device_sms();
  Plan plan;
  // without a visible device the size is computed for the largest grid this library targets
  if (!make_plan(int(M), int(K), int(N), mb, sms > 0 ? sms : 148, g_warps, &plan)) return 0;
  return int64_t(plan.workspace_bytes);
}
}  // namespace ib200

extern "C" int64_t intent_b200_w4a16_gemv_workspace_bytes(int64_t M, int64_t K, int64_t N) {
  return ib200::w4a16_stream_workspace_bytes(M, K, N);
}

extern "C" int intent_b200_w4a16_gemv_overlap(int32_t enable) {
  ib200::g_overlap = enable ? 1 : 0;
  return INTENT_B200_OK;
}

extern "C" int intent_b200_w4a16_gemv_grid(int32_t ctas) {
  if (ctas < 0) return INTENT_B200_ERR_UNSUPPORTED;
  ib200::g_grid_override = ctas;
  return INTENT_B200_OK;
}

extern "C" int intent_b200_w4a16_gemv_warps(int32_t warps) {
  if (warps != 8 && warps != 16) return INTENT_B200_ERR_UNSUPPORTED;
  ib200::g_warps = warps;
  return INTENT_B200_OK;
}
