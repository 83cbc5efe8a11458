// MoE routing, route alignment and row permutation kernels (integer results are bit-exact).
//
// Reference programs:
//   insertion top-k   examples/kernels/sampling/top_k.py:10-33 (strict '>' : the lower index wins ties)
//   softmax           examples/kernels/normalization/softmax.py:23-37
//   moe_count_routes / moe_prefix_routes / moe_scatter_routes / moe_mark_expert_blocks
//                     examples/kernels/routing/moe_align.py:14-86, host composition
//                     examples/programs/composition.py:98-174
// The reference scatters with an atomic cursor, so the order inside an expert span depends on
// the race; here the scatter is a stable partition (ascending route id inside a span), which is
// what the reference's torch implementation produces (stable argsort) and needs no
// canonicalisation before comparing.
#include "common.cuh"

namespace ib200 {
namespace {

// ---- router: top-2 experts by logit (ties -> lower id) and their softmax probabilities ----
struct Top2 {
  float v0, v1;
  int i0, i1;
};

__device__ __forceinline__ bool better(float va, int ia, float vb, int ib) {
  return va > vb || (va == vb && ia < ib);
}

__device__ __forceinline__ void top2_insert(Top2& t, float v, int i) {
  if (better(v, i, t.v0, t.i0)) {
    t.v1 = t.v0; t.i1 = t.i0; t.v0 = v; t.i0 = i;
  } else if (better(v, i, t.v1, t.i1)) {
    t.v1 = v; t.i1 = i;
  }
}

__global__ void moe_route_top2_kernel(const float* __restrict__ logits, int tokens, int experts,
                                      int* __restrict__ ids, float* __restrict__ weights) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= tokens) return;
  const float* row = logits + size_t(warp) * experts;
  Top2 t{-INFINITY, -INFINITY, 0x7fffffff, 0x7fffffff};
  float vmax = -INFINITY;
  for (int e = lane; e < experts; e += 32) {
    const float v = row[e];
    vmax = fmaxf(vmax, v);
    top2_insert(t, v, e);
  }
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) {
    vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, d));
    const float ov0 = __shfl_xor_sync(0xffffffffu, t.v0, d), ov1 = __shfl_xor_sync(0xffffffffu, t.v1, d);
    const int oi0 = __shfl_xor_sync(0xffffffffu, t.i0, d), oi1 = __shfl_xor_sync(0xffffffffu, t.i1, d);
    top2_insert(t, ov0, oi0);
    top2_insert(t, ov1, oi1);
  }
  float sum = 0.f;
  for (int e = lane; e < experts; e += 32) sum += expf(row[e] - vmax);
#pragma unroll
  for (int d = 16; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  if (lane == 0) {
    ids[2 * warp] = t.i0;
    ids[2 * warp + 1] = t.i1;
    weights[2 * warp] = expf(t.v0 - vmax) / sum;
    weights[2 * warp + 1] = expf(t.v1 - vmax) / sum;
  }
}

// ---- count: counts[e] += number of routes to e (integer atomics: order-free and exact) ----
__global__ void moe_count_kernel(const int* __restrict__ ids, int routes, int experts, int* __restrict__ counts,
                                 int* __restrict__ error) {
  extern __shared__ int local[];
  for (int e = threadIdx.x; e < experts; e += blockDim.x) local[e] = 0;
  __syncthreads();
  for (int r = blockIdx.x * blockDim.x + threadIdx.x; r < routes; r += gridDim.x * blockDim.x) {
    const int e = ids[r];
    if (e >= 0 && e < experts) atomicAdd(&local[e], 1);
    else if (error) atomicExch(error, INTENT_B200_ERR_SHAPE);   // out-of-range expert id: skipped, reported
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x)
    if (local[e]) atomicAdd(&counts[e], local[e]);
}

// ---- prefix: padded exclusive offsets and the padded total ----
__global__ void moe_prefix_kernel(const int* __restrict__ counts, int experts, int block, int* __restrict__ offsets,
                                  int* __restrict__ total) {
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    int running = 0;
    offsets[0] = 0;
    for (int e = 0; e < experts; ++e) {
      running += (counts[e] + block - 1) / block * block;
      offsets[e + 1] = running;
    }
    total[0] = running;
  }
}

// ---- scatter: CTA e compacts, in ascending route order, the routes that chose expert e ----
// Warp w of the CTA owns the contiguous slice w of the routes.  Pass 1: every warp counts its matches;
// one barrier; pass 2: every warp walks its slice again and writes each match at (span start + matches in
// earlier slices + matches earlier in its own slice).  Slices are contiguous and in order, so the partition
// is stable; the two passes read the ids from L2 and need no barrier per step.
__global__ void __launch_bounds__(1024)
moe_scatter_kernel(const int* __restrict__ ids, int routes, const int* __restrict__ offsets,
                   int* __restrict__ cursors, int* __restrict__ sorted, int sorted_capacity) {
  __shared__ int warp_count[32];
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int begin = offsets[e], end = offsets[e + 1];
  const int slice = ((routes + 31) / 32 + 31) / 32 * 32;          // per warp, a multiple of the warp size
  const int first = min(routes, warp * slice), last = min(routes, first + slice);
  int count = 0;
  for (int base = first; base < last; base += 32) {
    const int r = base + lane;
    count += __popc(__ballot_sync(0xffffffffu, r < last && ids[r] == e));
  }
  if (lane == 0) warp_count[warp] = count;
  __syncthreads();
  int before = 0, total = 0;
  for (int w = 0; w < 32; ++w) {
    if (w < warp) before += warp_count[w];
    total += warp_count[w];
  }
  int position = begin + before;
  for (int base = first; base < last; base += 32) {
    const int r = base + lane;
    const bool mine = r < last && ids[r] == e;
    const unsigned ballot = __ballot_sync(0xffffffffu, mine);
    if (mine) {
      const int at = position + __popc(ballot & ((1u << lane) - 1u));
      if (at < end && at < sorted_capacity) sorted[at] = r;
    }
    position += __popc(ballot);
  }
  // the padding of the span holds the sentinel `routes`
  for (int at = begin + total + threadIdx.x; at < end && at < sorted_capacity; at += 1024) sorted[at] = routes;
  if (threadIdx.x == 0 && cursors) cursors[e] += total;  // final value of the reference's atomic cursor
}

// ---- mark: expert owning every block of the padded layout ----
__global__ void moe_mark_kernel(const int* __restrict__ offsets, int experts, int block, int* __restrict__ blocks,
                                int blocks_capacity) {
  const int e = blockIdx.x;
  if (e >= experts) return;
  const int first = offsets[e] / block, last = offsets[e + 1] / block;
  for (int b = first + threadIdx.x; b < last && b < blocks_capacity; b += blockDim.x) blocks[b] = e;
}

// ---- positions: inverse of the alignment, position[route] = slot in the sorted layout ----
__global__ void moe_positions_kernel(const int* __restrict__ sorted, const int* __restrict__ total, int capacity,
                                     int routes, int* __restrict__ position) {
  const int limit = min(capacity, *total);
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < limit; p += gridDim.x * blockDim.x) {
    const int r = sorted[p];
    if (r >= 0 && r < routes) position[r] = p;
  }
}

// ---- gather: xs[p, :] = x[sorted[p] / top_k, :], zero rows for the padding ----
__global__ void moe_gather_rows_kernel(const uint4* __restrict__ x, const int* __restrict__ sorted,
                                       const int* __restrict__ total, int capacity, int routes, int top_k,
                                       int row_vectors, uint4* __restrict__ out) {
  const int limit = min(capacity, *total);
  for (int p = blockIdx.x; p < limit; p += gridDim.x) {
    const int r = sorted[p];
    const bool real = r >= 0 && r < routes;
    const uint4* src = x + size_t(real ? r / top_k : 0) * row_vectors;
    uint4* dst = out + size_t(p) * row_vectors;
    for (int i = threadIdx.x; i < row_vectors; i += blockDim.x) dst[i] = real ? src[i] : make_uint4(0, 0, 0, 0);
  }
}

// ---- combine: y[t, :] += sum over the token's choices, in choice order, of weight * rows[position] ----
__global__ void moe_combine_kernel(const float4* __restrict__ rows, const int* __restrict__ position,
                                   const float* __restrict__ weights, int tokens, int top_k, int row_vectors,
                                   bool accumulate, float4* __restrict__ y) {
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    for (int i = threadIdx.x; i < row_vectors; i += blockDim.x) {
      float4 acc = accumulate ? y[size_t(t) * row_vectors + i] : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c = 0; c < top_k; ++c) {
        const float w = weights[t * top_k + c];
        const float4 v = rows[size_t(position[t * top_k + c]) * row_vectors + i];
        // product and sum are rounded separately (no fused multiply-add), so that this ordered combine and the
        // atomic one in the down projection's epilogue give the same bits for two choices on a zeroed row
        acc.x = __fadd_rn(acc.x, __fmul_rn(w, v.x)); acc.y = __fadd_rn(acc.y, __fmul_rn(w, v.y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(w, v.z)); acc.w = __fadd_rn(acc.w, __fmul_rn(w, v.w));
      }
      y[size_t(t) * row_vectors + i] = acc;
    }
  }
}

int grid_for(int64_t items, int threads, int cap = 148 * 8) {
  int64_t blocks = (items + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  return int(blocks < cap ? blocks : cap);
}

}  // namespace
}  // namespace ib200

using namespace ib200;

// logits [T,E] f32 -> ids [T,2] i32, weights [T,2] f32
extern "C" int intent_b200_moe_route_top2(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                          void* stream) {
  if (a1_d0 != a0_d0 || a2_d0 != a0_d0 || a1_d1 != 2 || a2_d1 != 2) return INTENT_B200_ERR_SHAPE;
  if (a0_d0 == 0) return INTENT_B200_OK;
  if (a0_d1 < 2) return INTENT_B200_ERR_UNSUPPORTED;
  if (!a0 || !a1 || !a2) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW2_ARG(a0)) || !contiguous(IB200_VIEW2_ARG(a1)) || !contiguous(IB200_VIEW2_ARG(a2)))
    return INTENT_B200_ERR_LAYOUT;
  const int tokens = int(a0_d0);
  moe_route_top2_kernel<<<(tokens + 7) / 8, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(a0), tokens, int(a0_d1), static_cast<int*>(a1), static_cast<float*>(a2));
  note_launch();
  return launch_status();
}

// topk_ids [T,K] i32, expert_counts [E] i32 (InOut, accumulated)
extern "C" int intent_b200_moe_count_routes(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), void* stream) {
  if (a0_d0 * a0_d1 == 0 || a1_d0 == 0) return INTENT_B200_OK;
  if (!a0 || !a1) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW2_ARG(a0)) || !contiguous(IB200_VIEW1_ARG(a1))) return INTENT_B200_ERR_LAYOUT;
  if (a1_d0 > 8192) return INTENT_B200_ERR_UNSUPPORTED;
  const int routes = int(a0_d0 * a0_d1);
  moe_count_kernel<<<grid_for(routes, 256, 148), 256, size_t(a1_d0) * 4, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(a0), routes, int(a1_d0), static_cast<int*>(a1), nullptr);
  note_launch();
  return launch_status();
}

// expert_counts [E] -> expert_offsets [E+1], total_padded [1]
extern "C" int intent_b200_moe_prefix_routes(INTENT_B200_VIEW1(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                             int32_t block_size, void* stream) {
  if (a1_d0 != a0_d0 + 1 || a2_d0 != 1 || block_size <= 0) return INTENT_B200_ERR_SHAPE;
  if (!a0 || !a1 || !a2) return INTENT_B200_ERR_NULL;
  moe_prefix_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const int*>(a0), int(a0_d0),
                                                                    block_size, static_cast<int*>(a1),
                                                                    static_cast<int*>(a2));
  note_launch();
  return launch_status();
}

// topk_ids [T,K], expert_offsets [E+1], expert_cursors [E] (InOut), sorted_route_ids [capacity] (InOut)
extern "C" int intent_b200_moe_scatter_routes(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                              INTENT_B200_VIEW1(a3), void* stream) {
  if (a1_d0 != a2_d0 + 1) return INTENT_B200_ERR_SHAPE;
  if (a2_d0 == 0) return INTENT_B200_OK;
  if (!a0 || !a1 || !a2 || !a3) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW2_ARG(a0))) return INTENT_B200_ERR_LAYOUT;
  moe_scatter_kernel<<<int(a2_d0), 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(a0), int(a0_d0 * a0_d1), static_cast<const int*>(a1), static_cast<int*>(a2),
      static_cast<int*>(a3), int(a3_d0));
  note_launch();
  return launch_status();
}

// expert_offsets [E+1] -> expert_blocks [B]
extern "C" int intent_b200_moe_mark_expert_blocks(INTENT_B200_VIEW1(a0), INTENT_B200_VIEW1(a1), int32_t block_size,
                                                  void* stream) {
  if (a0_d0 < 1 || block_size <= 0) return INTENT_B200_ERR_SHAPE;
  if (a0_d0 == 1 || a1_d0 == 0) return INTENT_B200_OK;
  if (!a0 || !a1) return INTENT_B200_ERR_NULL;
  moe_mark_kernel<<<int(a0_d0 - 1), 64, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(a0), int(a0_d0 - 1), block_size, static_cast<int*>(a1), int(a1_d0));
  note_launch();
  return launch_status();
}

// sorted_route_ids [capacity], total_padded [1] -> route_positions [R]
extern "C" int intent_b200_moe_route_positions(INTENT_B200_VIEW1(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                               void* stream) {
  if (a1_d0 != 1) return INTENT_B200_ERR_SHAPE;
  if (a0_d0 == 0 || a2_d0 == 0) return INTENT_B200_OK;
  if (!a0 || !a1 || !a2) return INTENT_B200_ERR_NULL;
  moe_positions_kernel<<<grid_for(a0_d0, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(a0), static_cast<const int*>(a1), int(a0_d0), int(a2_d0), static_cast<int*>(a2));
  note_launch();
  return launch_status();
}

// x [T,H] (16-bit), sorted_route_ids [capacity], total_padded [1] -> rows [capacity, H]; top_k scalar
extern "C" int intent_b200_moe_gather_rows(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                           INTENT_B200_VIEW2(a3), int32_t top_k, void* stream) {
  if (a3_d1 != a0_d1 || a3_d0 != a1_d0 || a2_d0 != 1 || top_k <= 0) return INTENT_B200_ERR_SHAPE;
  if (a1_d0 == 0 || a0_d1 == 0) return INTENT_B200_OK;
  if (!a0 || !a1 || !a2 || !a3) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW2_ARG(a0)) || !contiguous(IB200_VIEW2_ARG(a3)) || !aligned16(a0) || !aligned16(a3))
    return INTENT_B200_ERR_LAYOUT;
  if (a0_d1 % 8 != 0) return INTENT_B200_ERR_UNSUPPORTED;
  moe_gather_rows_kernel<<<grid_for(a1_d0, 1, 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(a0), static_cast<const int*>(a1), static_cast<const int*>(a2), int(a1_d0),
      int(a0_d0 * top_k), top_k, int(a0_d1 / 8), static_cast<uint4*>(a3));
  note_launch();
  return launch_status();
}

// rows [P,H] f32, route_positions [T*K] i32, route_weights [T,K] f32, y [T,H] f32 (InOut; with
// accumulate = 0 the sum starts from zero and the old contents of y are not read)
extern "C" int intent_b200_moe_combine(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW2(a2),
                                       INTENT_B200_VIEW2(a3), int32_t accumulate, void* stream) {
  if (a3_d1 != a0_d1 || a2_d0 != a3_d0 || a1_d0 != a2_d0 * a2_d1) return INTENT_B200_ERR_SHAPE;
  if (a3_d0 == 0 || a3_d1 == 0) return INTENT_B200_OK;
  if (!a0 || !a1 || !a2 || !a3) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW2_ARG(a0)) || !contiguous(IB200_VIEW2_ARG(a2)) || !contiguous(IB200_VIEW2_ARG(a3)) ||
      !aligned16(a0) || !aligned16(a3))
    return INTENT_B200_ERR_LAYOUT;
  if (a3_d1 % 4 != 0) return INTENT_B200_ERR_UNSUPPORTED;
  moe_combine_kernel<<<grid_for(a3_d0, 1, 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float4*>(a0), static_cast<const int*>(a1), static_cast<const float*>(a2), int(a3_d0),
      int(a2_d1), int(a3_d1 / 4), accumulate != 0, static_cast<float4*>(a3));
  note_launch();
  return launch_status();
}
