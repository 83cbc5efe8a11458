// Expert-parallel MoE exchange over peer memory (NVLink / NVSwitch), without a collective on the
// data path: every rank writes its token rows straight into the expert-sorted row buffer of the
// rank that owns the expert, and reads the finished f32 rows straight out of the owners'
// result buffers while it combines them.  Only real rows cross the links (no padded spans, no
// staging copy).  Between the phases the ranks meet at sync points: either stream-ordered
// collectives issued by the host, or the post / wait kernels at the end of this file (flag writes and
// bounded flag waits over peer memory).  The data kernels themselves never wait on another GPU.
//
// The reference's programs behind these kernels: route grouping examples/kernels/routing/moe_align.py:14-86,
// row gather and weighted scatter_reduce examples/kernels/ragged/moe.py:34-53.
//
// Layout of an owner's row buffer: experts in local order, each span padded to `block_rows`; inside
// a span the rows of source rank 0 come first, then rank 1, ...; rows of one source keep their
// route order.  With tokens split contiguously over the ranks this is exactly the order of the
// single-GPU stable alignment over all tokens, so results are bit-identical to one GPU.
#include "common.cuh"

namespace ib200 {
namespace {

// counts [W, E]: routes of every source rank to every global expert (E = W * experts_per_rank).
// dest_base[e]     first row, inside the owner's buffer, of this rank's routes to expert e
// local_offsets[l] first row of local expert l in this rank's own buffer; [EL] = padded total
// expert_blocks[b] local expert of the b-th block_rows-row block of this rank's buffer (blocks past the
//                  padded total are not written)
__global__ void moe_peer_layout_kernel(const int* __restrict__ counts, int world, int experts, int experts_per_rank,
                                       int rank, int block_rows, int* __restrict__ dest_base,
                                       int* __restrict__ local_offsets, int* __restrict__ total_padded,
                                       int* __restrict__ expert_blocks, int block_capacity) {
  extern __shared__ int padded[];  // [experts] padded span of every global expert
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int total = 0;
    for (int s = 0; s < world; ++s) total += counts[s * experts + e];
    padded[e] = (total + block_rows - 1) / block_rows * block_rows;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    const int owner_first = e / experts_per_rank * experts_per_rank;
    int offset = 0;
    for (int f = owner_first; f < e; ++f) offset += padded[f];
    int before = 0;
    for (int s = 0; s < rank; ++s) before += counts[s * experts + e];
    dest_base[e] = offset + before;
    if (owner_first == rank * experts_per_rank) {
      local_offsets[e - owner_first] = offset;
      for (int b = offset / block_rows; b < (offset + padded[e]) / block_rows && b < block_capacity; ++b)
        expert_blocks[b] = e - owner_first;
      if (e - owner_first == experts_per_rank - 1) {
        local_offsets[experts_per_rank] = offset + padded[e];
        total_padded[0] = offset + padded[e];
      }
    }
  }
}

// One CTA per route in expert-sorted order: copies the token row into the owner's buffer.
__global__ void moe_peer_dispatch_kernel(const uint4* __restrict__ x, int row_vectors, int tokens, int top_k,
                                         const int* __restrict__ sorted_routes, int routes,
                                         const int* __restrict__ send_offsets, int experts, int experts_per_rank,
                                         const int* __restrict__ dest_base, const long long* __restrict__ peer_rows,
                                         long long capacity_rows, int* __restrict__ route_dest) {
  extern __shared__ int offsets[];  // [experts + 1]
  for (int e = threadIdx.x; e <= experts; e += blockDim.x) offsets[e] = send_offsets[e];
  __syncthreads();
  for (int i = blockIdx.x; i < routes; i += gridDim.x) {
    // expert of sorted position i: the last e with offsets[e] <= i
    int lo = 0, hi = experts;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (offsets[mid] <= i) lo = mid; else hi = mid;
    }
    const int route = sorted_routes[i];
    const int owner = lo / experts_per_rank;
    const long long position = (long long)dest_base[lo] + (i - offsets[lo]);
    const bool ok = route >= 0 && route < routes && route / top_k < tokens && position >= 0 && position < capacity_rows;
    if (threadIdx.x == 0 && route >= 0 && route < routes) {
      route_dest[2 * route] = ok ? owner : -1;
      route_dest[2 * route + 1] = ok ? int(position) : 0;
    }
    if (!ok) continue;
    const uint4* src = x + size_t(route / top_k) * row_vectors;
    uint4* dst = reinterpret_cast<uint4*>(peer_rows[owner]) + size_t(position) * row_vectors;
    for (int v = threadIdx.x; v < row_vectors; v += blockDim.x) dst[v] = src[v];
  }
}

// y[t,:] += sum over choices c, in order, of weights[t,c] * owner(t,c)'s result row
__global__ void moe_peer_combine_kernel(const long long* __restrict__ peer_out, int world,
                                        const int* __restrict__ route_dest, const float* __restrict__ weights,
                                        int tokens, int top_k, int row_vectors, long long capacity_rows,
                                        bool accumulate, float4* __restrict__ y) {
  for (int t = blockIdx.x; t < tokens; t += gridDim.x) {
    for (int i = threadIdx.x; i < row_vectors; i += blockDim.x) {
      float4 acc = accumulate ? y[size_t(t) * row_vectors + i] : make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c = 0; c < top_k; ++c) {
        const int owner = route_dest[2 * (t * top_k + c)];
        const int position = route_dest[2 * (t * top_k + c) + 1];
        if (owner < 0 || owner >= world || position < 0 || position >= capacity_rows) continue;
        const float w = weights[t * top_k + c];
        const float4 v = reinterpret_cast<const float4*>(peer_out[owner])[size_t(position) * row_vectors + i];
        // product and sum are rounded separately (no fused multiply-add), so that this ordered combine and the
        // atomic one in the down projection's epilogue give the same bits for two choices on a zeroed row
        acc.x = __fadd_rn(acc.x, __fmul_rn(w, v.x)); acc.y = __fadd_rn(acc.y, __fmul_rn(w, v.y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(w, v.z)); acc.w = __fadd_rn(acc.w, __fmul_rn(w, v.w));
      }
      y[size_t(t) * row_vectors + i] = acc;
    }
  }
}

// ---- cross-rank signalling over peer memory ---------------------------------------------------
// Every rank owns a flag array [channels][W] in memory all ranks can address.  To pass a sync
// point a rank first POSTS: it bumps its private sequence number of the channel, optionally copies a
// small payload (its per-expert counts) into every rank's table, fences, and stores the sequence
// number into slot [channel][rank] of every rank's flag array.  It then WAITS until every slot of
// its own array [channel][*] has reached the same number.  Sequence numbers only grow, so a rank
// that runs ahead never confuses a slower one.  The wait is bounded: after `max_polls` polls (about a
// microsecond apart) it
// records INTENT_B200_ERR_TIMEOUT in `status` and returns, so a missing rank cannot hang the GPU.
__global__ void moe_peer_post_kernel(const long long* __restrict__ peer_flags, int world, int rank, int channel,
                                     int* __restrict__ sequence, const long long* __restrict__ peer_tables,
                                     const int* __restrict__ payload, int payload_count) {
  __shared__ int seq;
  if (threadIdx.x == 0) seq = ++sequence[2 * channel];   // launches of one stream are ordered: no race
  if (peer_tables != nullptr)
    for (int i = threadIdx.x; i < world * payload_count; i += blockDim.x) {
      const int dst = i / payload_count, e = i - dst * payload_count;
      reinterpret_cast<int*>(peer_tables[dst])[rank * payload_count + e] = payload[e];
    }
  __threadfence_system();
  __syncthreads();
  for (int dst = threadIdx.x; dst < world; dst += blockDim.x) {
    int* flag = reinterpret_cast<int*>(peer_flags[dst]) + channel * world + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(seq) : "memory");
  }
}

__global__ void moe_peer_wait_kernel(const int* __restrict__ my_flags, int world, int channel,
                                     int* __restrict__ sequence, int max_polls, int* __restrict__ status) {
  __shared__ int seq;
  __shared__ int broken;
  if (threadIdx.x == 0) {
    seq = ++sequence[2 * channel + 1];
    broken = *status;   // an earlier wait already gave up: later ones return at once, so that the work
  }                     // queued behind a lost rank drains in one bound, not one bound per wait
  __syncthreads();
  if (broken != 0) return;
  for (int src = threadIdx.x; src < world; src += blockDim.x) {
    const int* flag = my_flags + channel * world + src;
    bool seen = false;
    for (int poll = 0; poll < max_polls; ++poll) {
      int value;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(value) : "l"(flag) : "memory");
      if (value - seq >= 0) { seen = true; break; }
      __nanosleep(1000);
    }
    if (!seen) atomicExch(status, INTENT_B200_ERR_TIMEOUT);
  }
  __threadfence_system();
}

}  // namespace
}  // namespace ib200

// a0 peer_flags [W] i64 (device addresses of every rank's flag array [channels, W] i32), a1 sequence [2*channels] i32
// (private to this rank; a post counter and a wait counter per channel), a2 peer_tables [W] i64 and a3 payload [C] i32:
// optional payload copied into row `rank` of every rank's table [W, C] (pass a2 with extent 0 for none)
extern "C" int intent_b200_moe_peer_post(INTENT_B200_VIEW1(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                         INTENT_B200_VIEW1(a3), int32_t rank, int32_t channel, void* stream) {
  using namespace ib200;
  const int64_t world = a0_d0;
  if (world <= 0 || rank < 0 || rank >= world || channel < 0 || a1_d0 < 2 * (channel + 1) ||
      (a2_d0 != 0 && a2_d0 != world))
    return INTENT_B200_ERR_SHAPE;
  if (!a0 || !a1 || (a2_d0 != 0 && (!a2 || !a3))) return INTENT_B200_ERR_NULL;
  if (world > 1024 || a3_d0 > 8192) return INTENT_B200_ERR_UNSUPPORTED;
  moe_peer_post_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(a0), int(world), rank, channel, static_cast<int*>(a1),
      a2_d0 != 0 ? static_cast<const long long*>(a2) : nullptr, static_cast<const int*>(a3), int(a3_d0));
  note_launch();
  return launch_status();
}

// a0 my_flags [channels, W] i32 (this rank's own flag array), a1 sequence [2*channels] i32, a2 status [1] i32
// (set to INTENT_B200_ERR_TIMEOUT when a slot did not reach the sequence number within max_polls polls)
extern "C" int intent_b200_moe_peer_wait(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                         int32_t channel, int32_t max_polls, void* stream) {
  using namespace ib200;
  const int64_t world = a0_d1;
  if (world <= 0 || channel < 0 || channel >= a0_d0 || a1_d0 < 2 * (channel + 1) || a2_d0 < 1 || max_polls <= 0)
    return INTENT_B200_ERR_SHAPE;
  if (!a0 || !a1 || !a2) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW2_ARG(a0))) return INTENT_B200_ERR_LAYOUT;
  if (world > 1024) return INTENT_B200_ERR_UNSUPPORTED;
  moe_peer_wait_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(a0), int(world), channel, static_cast<int*>(a1), max_polls, static_cast<int*>(a2));
  note_launch();
  return launch_status();
}

// a0 counts [W,E] i32 -> a1 dest_base [E], a2 local_offsets [E/W + 1], a3 total_padded [1], a4 expert_blocks [B]
extern "C" int intent_b200_moe_peer_layout(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                           INTENT_B200_VIEW1(a3), INTENT_B200_VIEW1(a4), int32_t rank,
                                           int32_t block_rows, void* stream) {
  using namespace ib200;
  const int64_t world = a0_d0, experts = a0_d1;
  if (world <= 0 || experts <= 0 || experts % world != 0 || a1_d0 != experts || a2_d0 != experts / world + 1 ||
      a3_d0 != 1 || rank < 0 || rank >= world || block_rows <= 0)
    return INTENT_B200_ERR_SHAPE;
  if (!a0 || !a1 || !a2 || !a3 || !a4) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW2_ARG(a0))) return INTENT_B200_ERR_LAYOUT;
  if (experts > 8192 || world > 1024 || a4_d0 > (1 << 30)) return INTENT_B200_ERR_UNSUPPORTED;
  moe_peer_layout_kernel<<<1, 256, size_t(experts) * 4, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(a0), int(world), int(experts), int(experts / world), rank, block_rows,
      static_cast<int*>(a1), static_cast<int*>(a2), static_cast<int*>(a3), static_cast<int*>(a4), int(a4_d0));
  note_launch();
  return launch_status();
}

// a0 x [T,H] 16-bit, a1 sorted_routes [R] (by expert, no padding), a2 send_offsets [E+1], a3 dest_base [E],
// a4 peer_rows [W] i64 (device addresses of every rank's row buffer [capacity_rows, H]) -> a5 route_dest [R,2]
extern "C" int intent_b200_moe_peer_dispatch(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2),
                                             INTENT_B200_VIEW1(a3), INTENT_B200_VIEW1(a4), INTENT_B200_VIEW2(a5),
                                             int32_t top_k, int32_t capacity_rows, void* stream) {
  using namespace ib200;
  const int64_t tokens = a0_d0, width = a0_d1, routes = a1_d0, experts = a3_d0, world = a4_d0;
  if (top_k <= 0 || routes != tokens * top_k || a2_d0 != experts + 1 || world <= 0 || experts % world != 0 ||
      a5_d0 != routes || a5_d1 != 2 || capacity_rows < 0)
    return INTENT_B200_ERR_SHAPE;
  if (routes == 0 || width == 0) return INTENT_B200_OK;
  if (!a0 || !a1 || !a2 || !a3 || !a4 || !a5) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW2_ARG(a0)) || !contiguous(IB200_VIEW2_ARG(a5)) || !aligned16(a0))
    return INTENT_B200_ERR_LAYOUT;
  if (width % 8 != 0 || experts > 8192 || routes > (1 << 30)) return INTENT_B200_ERR_UNSUPPORTED;
  const int grid = int(routes < 148 * 16 ? routes : 148 * 16);
  moe_peer_dispatch_kernel<<<grid, 256, size_t(experts + 1) * 4, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(a0), int(width / 8), int(tokens), top_k, static_cast<const int*>(a1), int(routes),
      static_cast<const int*>(a2), int(experts), int(experts / world), static_cast<const int*>(a3),
      static_cast<const long long*>(a4), capacity_rows, static_cast<int*>(a5));
  note_launch();
  return launch_status();
}

// a0 peer_out [W] i64 (device addresses of every rank's f32 result rows [capacity_rows, H]), a1 route_dest [R,2],
// a2 weights [T,K] f32, a3 y [T,H] f32 (InOut; with accumulate = 0 the old contents are not read)
extern "C" int intent_b200_moe_peer_combine(INTENT_B200_VIEW1(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),
                                            INTENT_B200_VIEW2(a3), int32_t capacity_rows, int32_t accumulate,
                                            void* stream) {
  using namespace ib200;
  const int64_t world = a0_d0, tokens = a3_d0, width = a3_d1, top_k = a2_d1;
  if (world <= 0 || a2_d0 != tokens || a1_d0 != tokens * top_k || a1_d1 != 2 || capacity_rows < 0)
    return INTENT_B200_ERR_SHAPE;
  if (tokens == 0 || width == 0) return INTENT_B200_OK;
  if (!a0 || !a1 || !a2 || !a3) return INTENT_B200_ERR_NULL;
  if (!contiguous(IB200_VIEW2_ARG(a1)) || !contiguous(IB200_VIEW2_ARG(a2)) || !contiguous(IB200_VIEW2_ARG(a3)) ||
      !aligned16(a3))
    return INTENT_B200_ERR_LAYOUT;
  if (width % 4 != 0) return INTENT_B200_ERR_UNSUPPORTED;
  const int grid = int(tokens < 148 * 16 ? tokens : 148 * 16);
  moe_peer_combine_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const long long*>(a0), int(world), static_cast<const int*>(a1), static_cast<const float*>(a2),
      int(tokens), int(top_k), int(width / 4), capacity_rows, accumulate != 0, static_cast<float4*>(a3));
  note_launch();
  return launch_status();
}
