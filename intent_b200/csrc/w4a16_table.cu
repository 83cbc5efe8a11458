// W4A16 decode GEMV over a TABLE of independent problems in one persistent launch.
//
//   for every problem p of the table:  Y_p[m, n] = T( sum_k f32(X_p[m, k]) * (q_p[k, n] - 8) * f32(S_p[k / G, n]) )
//
// Program: weight_only_int4_matmul (reference kernel body
// examples/kernels/contraction/weight_only_int4.py:18-51), M <= 16 per problem.  The reference has no
// decode-specific lowering and launches one kernel per contraction; a single 30 MB GEMV per launch
// spends as long ramping up and draining as it spends streaming, so here the projections of a decode
// step (or of several layers) share one launch and the weight stream never stops at a problem boundary.
//
// One CTA per SM.  Every problem's packed weight [K/8, N] is cut into units of 32 columns x 32 packed
// rows (256 k, 4 KiB) and the units of a problem are split evenly over the CTAs (+-1).  A CTA owns a
// ring of S shared-memory slots (S is chosen per launch); unit number g of the CTA's sequence - the
// concatenation of its shares of all problems - lands in slot g % S through one 128B-swizzled TMA box
// (plus a box of its scales) on the slot's mbarrier, and the warp that consumed it requests unit g + S
// into the same slot, whichever problem that belongs to.
//
// Two kernels share this frame.
//
// w4a16_ride_kernel (problems of at most eight rows; described in full above its definition): every
// unit's TMA transaction also brings the 256 activations per row it needs, so nothing is staged and
// there is no CTA-wide barrier after start-up; the unit-to-problem bookkeeping is a schedule in shared
// memory built once; ring warps take units by ticket; a span's K range is one piece ("chunk block").
//
// w4a16_table_kernel (more rows, or every problem when the ride-along kernel is switched off): K is
// cut into chunk blocks of `cb` chunks (cb = all chunks when the activations of the whole K range fit
// in shared memory, smaller for larger M); units are numbered block-major, then column tile, then
// chunk.  A CTA's share is therefore a run of whole "spans" (one column tile x one chunk block) plus a
// partial span at either end, and the activations it needs are those of at most a few neighbouring
// chunk blocks: they are staged once per problem, permuted to the nibble-pair order
// (w4a16_expand.cuh), together with the per-group correction sums, between two CTA-wide barriers.
// Its reduction over K, fixed order (bitwise reproducible):
//   1. units of one span inside one CTA: per-unit partials [M x 32] f32 in shared memory, a shared
//      ticket per span, the warp with the last ticket adds them in chunk order;
//   2. a span shared by neighbouring CTAs: each publishes ONE partial to global scratch and takes a
//      ticket on the span's global counter; the last one adds the partials in CTA order;
//   3. several chunk blocks: the block sums of a column tile meet the same way on the tile's counter
//      and are added in block order.
//
// No memory fence at GPU scope anywhere: such a fence makes the SM wait for all its loads in flight
// (measured on a bare ring, ring_probe.cu: two per 48 units cost a quarter of the stream).  Partial
// sums published for another CTA carry their own validity instead (publish / take_published), and
// tickets are relaxed atomics.  Counters and scratch are left at zero for the next launch.  Partial
// spans at the ends of a CTA's share are processed first.
//
// Every wait is bounded; a wait that gives up records INTENT_B200_ERR_TIMEOUT in the workspace's
// status word, the CTA skips its remaining units (still meeting its barriers) and exits.
#include <type_traits>

#include "common.cuh"
#include "tma.cuh"
#include "w4a16_expand.cuh"

namespace ib200 {
namespace {

constexpr int kCols = 32;            // columns of a unit
constexpr int kRows = 32;            // packed rows of a unit (8 k each)
constexpr int kWeightBytes = kCols * kRows * 4;
constexpr int kMinSlots = 32;        // slots of the ring every plan is made for; a launch takes as many as fit
constexpr int kMaxSlots = 64;
constexpr int kMaxProblems = 8;
constexpr int kMaxSpans = 64;        // spans a CTA may touch in one problem
constexpr int kMailEntries = 4;      // ride-along form: spans waiting for the reducer warp
constexpr int kSmemLimit = 227 * 1024 - 5120;   // dynamic shared memory (the kernels' static part is below 5 KB)

struct TableProblem {
  const void* x;
  void* y;
  int M, K, N;
  int groups;          // K / G
  int chunks, tiles;   // ceil(K / 256), ceil(N / 32)
  int cb, nblocks;     // chunks per chunk block, number of chunk blocks
  int units;           // tiles * chunks
  int each, extra;     // units per CTA: the first `extra` CTAs get each + 1
  int maxp;            // partial slots per span in scratch1
  uint32_t magic_full, magic_cb, magic_last;   // ceil(2^32 / d) for d = tiles * cb, cb, chunks of the last block
  int* counters1;      // [nblocks * tiles] span tickets
  int* counters2;      // [tiles] tile tickets (nblocks > 1)
  float* scratch1;     // [nblocks * tiles][maxp][M][32]
  float* scratch2;     // [tiles][nblocks][M][32]
};

struct TableParams {
  TableProblem problem[kMaxProblems];
  int count;
  int twos_complement;
  int overlap;
  int* status;
  // shared-memory layout behind the slot ring (byte offsets from the 1 KiB-aligned base), sized for the launch:
  //   corr   correction sums (staged kernel: per staged group; ride-along kernel: per warp, of the unit in hand)
  //   xs     staged kernel: the staged activations
  //   span   staged kernel: span tickets; ride-along kernel: the chains' turn counters, then the sets' `done`
  //   part   staged kernel: per-unit partial sums; ride-along kernel: the chains' accumulators
  //   uses   per slot: how many refills have been requested (read when a slot is not tied to one warp)
  //   xbox   ride-along kernel: per slot, the unit's activations ([rows][256] per 32 packed rows)
  //   sched  ride-along kernel: the CTA's schedule, 16 bytes per unit of its whole sequence
  int corr_offset, xs_offset, span_offset, part_offset, uses_offset, xbox_offset, sched_offset;
  int xbox_bytes;            // bytes of one slot's activations
  int part_stride;           // floats between partial areas (staged) / between chain accumulators (ride-along)
  int slots;                 // slots of the ring
  uint32_t magic_slots;      // ceil(2^32 / slots)
  int chains, chain_shift;   // ride-along kernel: chains per segment (a power of two) and its logarithm
  int acc_ring_shift;        // ride-along kernel: log2 of the number of segments whose chains exist at a time
  int probe;                 // measurement only (intent_b200_w4a16_gemv_table_tune): parts of the work skipped
};

struct TableMaps {
  CUtensorMap w[kMaxProblems];
  CUtensorMap s[kMaxProblems];
  CUtensorMap x[kMaxProblems];   // ride-along form only
};

// What a CTA knows about its share of one problem (kept in shared memory).
struct Share {
  int u0, u1;        // unit range
  int head, tail;    // partial spans at the ends: units u0 .. u0+head-1 and u1-tail .. u1-1
  int first;         // position of the share's first unit in the CTA's whole sequence
  int row0;          // first staged packed row (start of the first chunk block touched)
  int rows;          // staged packed rows
  int span0;         // span index (block * tiles + tile) of unit u0
  int reads;         // ride-along form: 1 if the share ends a span that began in another CTA (the reducer adds it up)
};

struct Unit {
  int block, tile, chunk;
  int span_first, span_len;   // first unit and length of the span (tile x chunk block)
};

// Cross-CTA hand-over of a partial sum without memory fences.  Scratch words are zero while empty; a value is
// stored as the complement of its bits, which is never zero (the one pattern that would be, the NaN 0xFFFFFFFF,
// is stored as the canonical NaN).  The reader polls each word until it is non-zero, then clears it for the
// next launch.  Every vector is written once and read once per launch.
__device__ __forceinline__ uint32_t published_word(float v) {
  const uint32_t bits = __float_as_uint(v);
  return ~(bits == 0xFFFFFFFFu ? 0x7FFFFFFFu : bits);
}

__device__ __forceinline__ void publish(float4* dst, float4 v) {
  asm volatile("st.global.cg.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(published_word(v.x)), "r"(published_word(v.y)),
               "r"(published_word(v.z)), "r"(published_word(v.w))
               : "memory");
}

// false if the vector did not arrive within the bound (about a second)
__device__ __forceinline__ bool take_published(const float4* src, float4* out) {
  for (int spin = 0; spin < (1 << 22); ++spin) {
    uint32_t a, b, c, d;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "l"(src) : "memory");
    if (a != 0u && b != 0u && c != 0u && d != 0u) {
      *out = make_float4(__uint_as_float(~a), __uint_as_float(~b), __uint_as_float(~c), __uint_as_float(~d));
      asm volatile("st.global.cg.v4.u32 [%0], {%1,%1,%1,%1};" ::"l"(src), "r"(0u) : "memory");
      return true;
    }
    if (spin > 16) __nanosleep(128);
  }
  *out = make_float4(0.f, 0.f, 0.f, 0.f);
  return false;
}

// u / d for 0 <= u < 2^31 with magic = ceil(2^32 / d): the product can overestimate by one, never underestimate
__device__ __forceinline__ int fast_div(int u, int d, uint32_t magic) {
  if (d == 1) return u;                                  // 2^32 does not fit the magic word
  const int q = int(__umulhi(uint32_t(u), magic));
  return q - (u - q * d < 0 ? 1 : 0);
}

__device__ __forceinline__ Unit decode_unit(const TableProblem& q, int u) {
  Unit r;
  if (q.nblocks == 1) {                                  // one chunk block: a span is a whole column tile
    r.block = 0;
    r.span_len = q.chunks;
    r.tile = fast_div(u, q.chunks, q.magic_cb);
    r.chunk = u - r.tile * q.chunks;
    r.span_first = u - r.chunk;
    return r;
  }
  const int full = q.tiles * q.cb;                       // units of a full chunk block
  r.block = min(fast_div(u, full, q.magic_full), q.nblocks - 1);
  const int rest = u - r.block * full;
  const bool last = r.block == q.nblocks - 1;            // only the last block can be shorter
  r.span_len = last ? q.chunks - r.block * q.cb : q.cb;
  r.tile = fast_div(rest, r.span_len, last ? q.magic_last : q.magic_cb);
  r.chunk = r.block * q.cb + (rest - r.tile * r.span_len);
  r.span_first = r.block * full + r.tile * r.span_len;
  return r;
}

__device__ __forceinline__ int cta_of(const TableProblem& q, int u) {
  const int boundary = q.extra * (q.each + 1);
  return u < boundary ? u / (q.each + 1) : q.extra + (u - boundary) / q.each;   // each > 0 past the boundary
}

// j-th unit of a share in processing order: the partial span at the end, the one at the start, the rest
__device__ __forceinline__ int unit_at(const Share& s, int j) {
  if (j < s.tail) return s.u1 - s.tail + j;
  if (j < s.tail + s.head) return s.u0 + (j - s.tail);
  return s.u0 + s.head + (j - s.tail - s.head);
}

template <typename T, int MB, int STEPS, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1)
w4a16_table_kernel(const __grid_constant__ TableMaps maps, const __grid_constant__ TableParams p) {
  constexpr int THREADS = WARPS * 32;
  constexpr int RPG = 4 * STEPS;        // packed rows per quantisation group
  constexpr int GPC = kRows / RPG;      // groups per unit
  constexpr int CP = 8 * MB;            // row pitch of the correction table
  extern __shared__ unsigned char smem_raw[];
  __shared__ Share shares[kMaxProblems];
  __shared__ int total_units;
  __shared__ int abort_flag;

  if (p.overlap) asm volatile("griddepcontrol.launch_dependents;");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int cta = int(blockIdx.x);

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  constexpr int kScaleBytes = GPC * 64;   // a unit's scales: GPC groups x 32 columns x 16 bit
  const int S = p.slots;
  const uint32_t scale_base = base + uint32_t(S) * kWeightBytes;
  const uint32_t bars = scale_base + uint32_t(S) * kScaleBytes;
  volatile int* uses = reinterpret_cast<volatile int*>(base_ptr + p.uses_offset);
  // With slots % WARPS == 0 a slot is always consumed by the same warp, in order.  Otherwise the warp that
  // takes a slot's k-th unit first makes sure the (k-1)-th was consumed and the k-th requested: a parity wait
  // on a barrier that is still a whole phase behind would return at once.
  const bool shared_slots = (S % WARPS) != 0;
  float* corr = reinterpret_cast<float*>(base_ptr + p.corr_offset);
  uint4* xs = reinterpret_cast<uint4*>(base_ptr + p.xs_offset);
  const uint32_t xs_addr = base + uint32_t(p.xs_offset);
  int* span_count = reinterpret_cast<int*>(base_ptr + p.span_offset);   // tickets of the spans this CTA touches
  float* part = reinterpret_cast<float*>(base_ptr + p.part_offset);      // per-unit partial sums of the problem in hand

  // ---- this CTA's share of every problem ---------------------------------------------------
  if (tid < p.count) {
    const TableProblem& q = p.problem[tid];
    Share s;
    s.u0 = cta * q.each + min(cta, q.extra);
    s.u1 = s.u0 + q.each + (cta < q.extra ? 1 : 0);
    s.head = s.tail = 0;
    s.row0 = s.rows = s.span0 = s.reads = 0;
    if (s.u1 > s.u0) {
      const Unit a = decode_unit(q, s.u0), b = decode_unit(q, s.u1 - 1);
      if (a.span_first < s.u0) s.head = min(s.u1, a.span_first + a.span_len) - s.u0;
      if (b.span_first + b.span_len > s.u1 && b.span_first >= s.u0 + s.head) s.tail = s.u1 - max(b.span_first, s.u0);
      if (s.head == s.u1 - s.u0) s.tail = 0;
      s.row0 = a.block * q.cb * kRows;
      s.rows = min(q.chunks, (b.block + 1) * q.cb) * kRows - s.row0;
      s.span0 = a.block * q.tiles + a.tile;
    }
    shares[tid] = s;
  }
  if (tid == 0) abort_flag = 0;
  __syncthreads();
  if (tid == 0) {
    int first = 0;
    for (int i = 0; i < p.count; ++i) {
      shares[i].first = first;
      first += shares[i].u1 - shares[i].u0;
    }
    total_units = first;
  }
  for (int i = tid; i < S; i += THREADS) {
    mbar_init(bars + uint32_t(i) * 8u, 1);
    uses[i] = 0;
  }
  if (tid == 0) fence_mbar_init();
  __syncthreads();
  const int total = total_units;

  // Requests unit number `seq` of the CTA's sequence into its slot (one lane calls this).
  auto issue = [&](int seq, int hint) {
    int i = hint;                        // the sequence only moves forward: start at the caller's problem
    while (i + 1 < p.count && seq >= shares[i + 1].first) ++i;
    const TableProblem& q = p.problem[i];
    const Unit u = decode_unit(q, unit_at(shares[i], seq - shares[i].first));
    const uint32_t slot = uint32_t(seq - fast_div(seq, S, p.magic_slots) * S);
    const uint32_t bar = bars + slot * 8u;
    if (p.probe >= 3) {   // measurement: the packed weights alone
      mbar_expect_tx(bar, kWeightBytes);
      tma_load_2d(base + slot * kWeightBytes, &maps.w[i], u.tile * kCols, u.chunk * kRows, bar);
      return;
    }
    mbar_expect_tx(bar, kWeightBytes + GPC * 64);
    tma_load_2d(base + slot * kWeightBytes, &maps.w[i], u.tile * kCols, u.chunk * kRows, bar);
    tma_load_2d(scale_base + slot * kScaleBytes, &maps.s[i], u.tile * kCols, u.chunk * GPC, bar);
  };
  // First wave: slot s is owned by warp s % WARPS.  With launch overlap the packed weights (static) are requested
  // before the wait for the kernel ahead of this one; activations, which that kernel may have produced, after it.
  if (lane == 0)
    for (int seq = warp; seq < min(total, S); seq += WARPS) issue(seq, 0);
  if (p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");

  uint32_t magic_a, magic_b;
  Expand<T>::magic(p.twos_complement != 0, magic_a, magic_b);
  int row_of[STEPS];
  uint32_t off_of[STEPS];
#pragma unroll
  for (int i = 0; i < STEPS; ++i) {
    row_of[i] = STEPS >= 2 ? 8 * (i >> 1) + 2 * t + (i & 1) : t;
    off_of[i] = uint32_t(row_of[i]) * 128u + (uint32_t(g ^ (row_of[i] & 7)) << 4);
  }
  const int q4 = lane >> 3, v8 = lane & 7;   // reduction lanes: quarter q4 takes partials q4, q4+4, ...; columns 4*v8..+3

  for (int pi = 0; pi < p.count; ++pi) {
    const TableProblem& q = p.problem[pi];
    const Share sh = shares[pi];
    const int n_units = sh.u1 - sh.u0;
    const int M = q.M;
    const int part_floats = M * kCols;

    // ---- stage this problem's activations and correction sums -------------------------------
    // corr[group][m] = - sum over the group's k of x[m,k] * (bias_k + 8); rows of one group sit in RPG
    // adjacent lanes and are added by a fixed-order butterfly.
    const uint4* xg = reinterpret_cast<const uint4*>(q.x);
    const int k8 = q.K >> 3;
    const int items = sh.rows * M;
    constexpr int BATCH = 4;
    for (int start = 0; start < items; start += THREADS * BATCH) {
      uint4 val[BATCH];
      int ms[BATCH], lr[BATCH];
      bool in_range[BATCH], real[BATCH];
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        const int i = start + b * THREADS + tid;
        in_range[b] = i < items;
        ms[b] = in_range[b] ? i / sh.rows : 0;
        lr[b] = in_range[b] ? i - ms[b] * sh.rows : 0;
        real[b] = in_range[b] && sh.row0 + lr[b] < k8;
        val[b] = real[b] ? xg[size_t(ms[b]) * k8 + sh.row0 + lr[b]] : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        float partial = 0.f;
        uint4 o = make_uint4(0, 0, 0, 0);   // rows past K/8 (last chunk) are staged as zeros
        if (real[b]) {
          o.x = prmt(val[b].x, val[b].z, 0x5410);                        // (k0, k4)
          o.y = Expand<T>::scale_odd(prmt(val[b].x, val[b].z, 0x7632));  // (k1, k5)
          o.z = prmt(val[b].y, val[b].w, 0x5410);                        // (k2, k6)
          o.w = Expand<T>::scale_odd(prmt(val[b].y, val[b].w, 0x7632));  // (k3, k7)
          partial = Expand<T>::kEven * (pair_sum<T>(o.x) + pair_sum<T>(o.z)) +
                    Expand<T>::kOdd * (pair_sum<T>(o.y) + pair_sum<T>(o.w));
        }
        if (in_range[b]) xs[lr[b] * M + ms[b]] = o;
#pragma unroll
        for (int d = RPG / 2; d >= 1; d >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, d);
        if (in_range[b] && (lr[b] % RPG) == 0) corr[(lr[b] / RPG) * CP + ms[b]] = real[b] ? -partial : 0.f;
      }
    }
    for (int i = tid; i < kMaxSpans; i += THREADS) span_count[i] = 0;
    __syncthreads();   // staged data visible; nobody still reads the previous problem's (barrier below)

    uint16_t* y = reinterpret_cast<uint16_t*>(q.y);
    const int group0 = sh.row0 / RPG;   // first staged group

    // this warp's units of the problem: sequence numbers congruent to the warp modulo WARPS
    int j = ((warp - sh.first) % WARPS + WARPS) % WARPS;
    for (; j < n_units; j += WARPS) {
      if (*reinterpret_cast<volatile int*>(&abort_flag)) break;
      const int seq = sh.first + j;
      const int unit = unit_at(sh, j);
      const Unit u = decode_unit(q, unit);
      const int use = fast_div(seq, S, p.magic_slots);
      const uint32_t slot = uint32_t(seq - use * S);
      const uint32_t bar = bars + slot * 8u;
      bool requested = true;
      if (shared_slots && use > 0) {
        requested = false;
        for (int spin = 0; spin < (1 << 20); ++spin) {
          if (uses[slot] >= use) { requested = true; break; }
          if (*reinterpret_cast<volatile int*>(&abort_flag)) break;
          __nanosleep(64);
        }
        __threadfence_block();
      }
      if (!__all_sync(0xffffffffu, requested && mbar_wait(bar, uint32_t(use) & 1u))) {
        if (lane == 0) {
          atomicExch(p.status, INTENT_B200_ERR_TIMEOUT);   // this unit's loads never completed
          *reinterpret_cast<volatile int*>(&abort_flag) = 1;
        }
        break;
      }
      const uint32_t wslot = base + slot * kWeightBytes;
      const uint32_t sslot = scale_base + slot * kScaleBytes;
      auto refill = [&]() {
        if (seq + S < total) {
          __syncwarp();
          fence_proxy_async();
          if (lane == 0) {
            issue(seq + S, pi);
            if (shared_slots) {
              __threadfence_block();
              uses[slot] = use + 1;
            }
          }
        }
      };
      const bool skip_math = p.probe >= 1 && p.probe <= 5;
      float facc[MB][8];
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int i = 0; i < 8; ++i) facc[mb][i] = 0.f;

      const int staged_row = u.chunk * kRows - sh.row0;   // first staged row of this unit
      // Rows of X beyond M: the lanes that would hold them read row M - 1 instead.  An MMA output column depends
      // only on its own column of the activation fragment, and output columns >= M are never stored.
      const int m_lane = min(g, M - 1);
#pragma unroll
      for (int gi = 0; gi < (skip_math ? 0 : GPC); ++gi) {
        const int group = u.chunk * GPC + gi;
        float gacc[MB][8];
#pragma unroll
        for (int mb = 0; mb < MB; ++mb) {
          // (entries of rows >= M hold stale values: they only reach accumulator rows that are never stored)
          float2 c = make_float2(0.f, 0.f);
          if (group < q.groups) c = *reinterpret_cast<const float2*>(&corr[(group - group0) * CP + mb * 8 + 2 * t]);
#pragma unroll
          for (int i = 0; i < 8; ++i) gacc[mb][i] = (i & 1) ? c.y : c.x;
        }
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
          const int row = gi * RPG + row_of[i];
          const uint32_t off = STEPS >= 2 ? off_of[i] + uint32_t(gi * RPG * 128)
                                          : uint32_t(row) * 128u + (uint32_t(g ^ (row & 7)) << 4);
          const uint4 w = lds128(wslot + off);
          uint32_t c0[4], c1[4], c2[4], c3[4];
          Expand<T>::word(w.x, magic_a, magic_b, c0);
          Expand<T>::word(w.y, magic_a, magic_b, c1);
          Expand<T>::word(w.z, magic_a, magic_b, c2);
          Expand<T>::word(w.w, magic_a, magic_b, c3);
#pragma unroll
          for (int mb = 0; mb < MB; ++mb) {
            const int m = MB == 1 ? m_lane : min(mb * 8 + g, M - 1);
            const uint4 b = lds128(xs_addr + uint32_t((staged_row + row) * M + m) * 16u);
            float(&a01)[4] = *reinterpret_cast<float(*)[4]>(&gacc[mb][0]);
            float(&a23)[4] = *reinterpret_cast<float(*)[4]>(&gacc[mb][4]);
            Elem<T>::mma16816(a01, c0[0], c1[0], c0[1], c1[1], b.x, b.y);
            Elem<T>::mma16816(a23, c2[0], c3[0], c2[1], c3[1], b.x, b.y);
            Elem<T>::mma16816(a01, c0[2], c1[2], c0[3], c1[3], b.z, b.w);
            Elem<T>::mma16816(a23, c2[2], c3[2], c2[3], c3[3], b.z, b.w);
          }
        }
        uint2 s;  // this lane's four column scales of the group (zero outside the matrix)
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(s.x), "=r"(s.y) : "r"(sslot + gi * 64 + g * 8));
        const float s0 = Elem<T>::to_float(uint16_t(s.x & 0xFFFF)), s1 = Elem<T>::to_float(uint16_t(s.x >> 16));
        const float s2 = Elem<T>::to_float(uint16_t(s.y & 0xFFFF)), s3 = Elem<T>::to_float(uint16_t(s.y >> 16));
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
      }
      // the slot is free: request the unit that maps to it next, whichever problem that is
      refill();

      if (p.probe == 2 || p.probe == 3) continue;   // measurement: no reduction either
      // ---- level 1: the unit's partial joins its span's partials in shared memory --------------
      // accumulator element (mb, i): row m = 8*mb + 2t + (i & 1), column 4g + (i >> 1)
      const int seg_begin = max(u.span_first, sh.u0), seg_end = min(u.span_first + u.span_len, sh.u1);
      const int seg_len = seg_end - seg_begin;
      const int span = u.block * q.tiles + u.tile;
      const int seg = span - sh.span0;           // < kMaxSpans, checked on the host
      float* mine = part + size_t(unit - sh.u0) * part_floats;
#pragma unroll
      for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          const int m = mb * 8 + 2 * t + hh;
          if (m < M)
            *reinterpret_cast<float4*>(mine + m * kCols + 4 * g) =
                make_float4(facc[mb][0 + hh], facc[mb][2 + hh], facc[mb][4 + hh], facc[mb][6 + hh]);
        }
      __syncwarp();
      int last = 0;
      if (lane == 0) {
        __threadfence_block();
        last = atomicAdd(span_count + seg, 1) == seg_len - 1;
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (!last || p.probe == 4) continue;
      __threadfence_block();

      // sum of `count` partials spaced `stride` floats apart, for row m: quarter q4 adds partials q4, q4+4, ...
      // (four loads in flight), then the quarters are added in a fixed order
      auto sum_partials = [&](const float* first, int count, int stride, bool global, int m) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c = q4; c < count; c += 16) {
          float4 a[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int cc = c + 4 * k;
            a[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (cc < count) {
              const float4* src = reinterpret_cast<const float4*>(first + size_t(cc) * stride + m * kCols + 4 * v8);
              if (!global) {
                a[k] = *src;
              } else if (!take_published(src, &a[k])) {
                atomicExch(p.status, INTENT_B200_ERR_TIMEOUT);   // a neighbour's partial never arrived
                *reinterpret_cast<volatile int*>(&abort_flag) = 1;
              }
            }
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            sum.x += a[k].x; sum.y += a[k].y; sum.z += a[k].z; sum.w += a[k].w;
          }
        }
#pragma unroll
        for (int d = 16; d >= 8; d >>= 1) {
          sum.x += __shfl_xor_sync(0xffffffffu, sum.x, d);
          sum.y += __shfl_xor_sync(0xffffffffu, sum.y, d);
          sum.z += __shfl_xor_sync(0xffffffffu, sum.z, d);
          sum.w += __shfl_xor_sync(0xffffffffu, sum.w, d);
        }
        return sum;
      };
      auto write_y = [&](int m, float4 sum) {
        const int n = u.tile * kCols + 4 * v8;
        if (q4 == 0 && n < q.N) {  // N is a multiple of 8, so the four columns are inside together
          uint2 out;
          out.x = uint32_t(Elem<T>::from_float(sum.x)) | (uint32_t(Elem<T>::from_float(sum.y)) << 16);
          out.y = uint32_t(Elem<T>::from_float(sum.z)) | (uint32_t(Elem<T>::from_float(sum.w)) << 16);
          *reinterpret_cast<uint2*>(y + size_t(m) * q.N + n) = out;
        }
      };
      auto store_rows = [&](float* dst, float4 sum, int m) {   // to global scratch, for another CTA's warp
        if (q4 == 0) publish(reinterpret_cast<float4*>(dst + m * kCols + 4 * v8), sum);
      };
      // No fence on either side of the ticket: a release or acquire at GPU scope makes the SM wait for all of
      // its loads in flight (measured: two per 48 units cost a quarter of the stream).  The partials carry their
      // own validity instead (publish / take_published), and the ticket only elects the warp that adds them.
      auto take_ticket = [&](int* counter, int arrivals) {   // true for the last of `arrivals`
        __syncwarp();
        int final_one = 0;
        if (lane == 0) final_one = atomicAdd(counter, 1) == arrivals - 1;
        return __shfl_sync(0xffffffffu, final_one, 0) != 0;
      };

      const float* seg_first = part + size_t(seg_begin - sh.u0) * part_floats;
      const bool whole = seg_len == u.span_len || p.probe == 5;     // the whole span was added here: this is the block sum
      float* block_dst = q.nblocks > 1 ? q.scratch2 + (size_t(u.tile) * q.nblocks + u.block) * part_floats : nullptr;
      if (whole) {
        for (int m = 0; m < M; ++m) {
          const float4 sum = sum_partials(seg_first, seg_len, part_floats, false, m);
          if (block_dst) store_rows(block_dst, sum, m); else write_y(m, sum);
        }
      } else {
        // ---- level 2: a span shared with neighbouring CTAs ------------------------------------
        const int first_cta = cta_of(q, u.span_first), last_cta = cta_of(q, u.span_first + u.span_len - 1);
        float* span_scratch = q.scratch1 + size_t(span) * q.maxp * part_floats;
        float* slot_dst = span_scratch + size_t(cta - first_cta) * part_floats;
        for (int m = 0; m < M; ++m) store_rows(slot_dst, sum_partials(seg_first, seg_len, part_floats, false, m), m);
        if (!take_ticket(q.counters1 + span, last_cta - first_cta + 1)) continue;
        for (int m = 0; m < M; ++m) {
          const float4 sum = sum_partials(span_scratch, last_cta - first_cta + 1, part_floats, true, m);
          if (block_dst) store_rows(block_dst, sum, m); else write_y(m, sum);
        }
        if (lane == 0) q.counters1[span] = 0;   // ready for the next launch
      }
      if (block_dst) {
        // ---- level 3: the chunk blocks of a column tile -----------------------------------------
        if (!take_ticket(q.counters2 + u.tile, q.nblocks)) continue;
        const float* tile_first = q.scratch2 + size_t(u.tile) * q.nblocks * part_floats;
        for (int m = 0; m < M; ++m) write_y(m, sum_partials(tile_first, q.nblocks, part_floats, true, m));
        if (lane == 0) q.counters2[u.tile] = 0;
      }
    }
    // everybody is done with this problem's staged activations and partials before the next problem
    // overwrites them (the weight ring keeps streaming meanwhile)
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------
// The ride-along form as a kernel of its own (problems of at most eight rows: one MMA row block).
//
// What bounds this kernel is the number of instructions it issues (about as many as the SM can take
// while the stream runs), so the bookkeeping is kept out of the loop:
//   * at start-up every thread works out ONE unit of the CTA's whole sequence - problem, column tile, chunk,
//     its place in its segment (the part of a span inside this CTA), what happens when the segment is
//     complete - and leaves it as a 16-byte entry in a schedule in shared memory;
//   * units are taken in sequence order by whichever ring warp is free (a ticket per unit): the warps' cycles
//     vary by tens of percent, and with a fixed unit-to-warp map the CTA would end with its unluckiest warp;
//   * a segment's units are dealt round-robin to a few chains, each with an accumulator in shared memory: the
//     warp that finishes a chain's k-th unit waits until the first k have been added, adds its own, and passes
//     the turn on; the warp with the segment's last unit adds the chains (fixed order throughout: bitwise
//     reproducible) and writes Y, publishes the sum for the CTA that holds the span's end, or hands it to the
//     reducer.  Every accumulator is used once per launch, so nothing is reused and no warp waits for a buffer.
// Unit number u lives in slot u % S; the warp that takes it first makes sure that the slot's previous unit
// was consumed and this one requested (almost always so: units arrive in order), because a parity wait on a
// barrier that is still a whole phase behind would return at once.
// ---------------------------------------------------------------------------------------------
constexpr int kRideRows = 8;

// UR = packed rows of a unit: 32 (a unit is 4 KiB of weights, as in the other kernels) or 64 (8 KiB: the
// bookkeeping of a unit is paid once per 8 KiB; measured slower, only reachable through the tune entry).
// CORR_MMA (problems of three rows and more): the per-group correction sums come from two extra MMAs per step
// whose weight operand is the constant bias, instead of being added up row by row from the activations (which
// costs as many instructions per row as the whole permutation).
template <typename T, int STEPS, int UR, bool CORR_MMA>
__global__ void __launch_bounds__(1024, 1)
w4a16_ride_kernel(const __grid_constant__ TableMaps maps, const __grid_constant__ TableParams p) {
  constexpr int THREADS = 1024, RING = 31;
  constexpr int RPG = 4 * STEPS;        // packed rows per quantisation group
  constexpr int GPC = UR / RPG;         // groups per unit
  constexpr int CP = 8;                 // row pitch of the correction table
  constexpr int kScaleBytes = GPC * 64;
  constexpr int kUnitBytes = UR * kCols * 4;   // packed weights of a unit
  constexpr int kHalves = UR / 32;             // activation boxes per unit (a TMA box is at most 256 elements wide)
  extern __shared__ unsigned char smem_raw[];
  __shared__ Share shares[kMaxProblems];
  __shared__ int acc_first[kMaxProblems];      // index of the problem's first segment accumulator
  __shared__ int total_units, total_segments;
  __shared__ int abort_flag;
  __shared__ __align__(16) float mail_data[kMailEntries][kRideRows][kCols];
  __shared__ int mail_ctx[kMailEntries][4];    // problem, column tile, partials published by other CTAs
  __shared__ int mail_ready[kMailEntries];     // ticket + 1 once the entry is complete
  __shared__ int mail_tail, mail_head;         // tickets given out / entries consumed
  __shared__ int next_unit;                    // the next unit of the CTA's sequence nobody has taken yet

  if (p.probe == 7) return;   // measurement: what the bare launch of this kernel costs
  if (p.overlap) asm volatile("griddepcontrol.launch_dependents;");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int cta = int(blockIdx.x);

  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const int S = p.slots;
  const uint32_t scale_base = base + uint32_t(S) * kUnitBytes;
  const uint32_t bars = scale_base + uint32_t(S) * kScaleBytes;
  volatile int* uses = reinterpret_cast<volatile int*>(base_ptr + p.uses_offset);   // refills requested so far, per slot
  float* corr = reinterpret_cast<float*>(base_ptr + p.corr_offset);
  volatile int* turn = reinterpret_cast<volatile int*>(base_ptr + p.span_offset);   // per chain: units added so far
  float* accs = reinterpret_cast<float*>(base_ptr + p.part_offset);                 // per chain: [rows][32] sums
  const uint32_t xbox_base = base + uint32_t(p.xbox_offset);
  uint4* sched = reinterpret_cast<uint4*>(base_ptr + p.sched_offset);

  // Schedule entry: x = tile | problem << 24 | whole span << 28 | ends the span << 29
  //                 y = chunk | (M - 1) << 20
  //                 z = units of the segment | CTAs that hold earlier parts of the span << 20
  //                 w = place of the unit in its segment | number of the segment in the CTA's sequence << 16
  auto issue = [&](uint4 ent, uint32_t slot, int what) {
    const int tile = int(ent.x & 0xFFFFFFu), i = int((ent.x >> 24) & 15u), chunk = int(ent.y & 0xFFFFFu);
    const uint32_t rows = 1u + ((ent.y >> 20) & 7u);
    const uint32_t bar = bars + slot * 8u;
    if (p.probe >= 3) {   // measurement: the packed weights alone
      if (what & 1) {
        mbar_expect_tx(bar, kUnitBytes);
        tma_load_2d(base + slot * kUnitBytes, &maps.w[i], tile * kCols, chunk * UR, bar);
      }
      return;
    }
    if (what & 1) {
      mbar_expect_tx(bar, kUnitBytes + GPC * 64 + rows * (512u * kHalves));
      tma_load_2d(base + slot * kUnitBytes, &maps.w[i], tile * kCols, chunk * UR, bar);
      tma_load_2d(scale_base + slot * kScaleBytes, &maps.s[i], tile * kCols, chunk * GPC, bar);
    }
    if (what & 2) {
      // the unit's activations: per half of the unit a box [rows][256 values]
#pragma unroll
      for (int h = 0; h < kHalves; ++h)
        tma_load_2d(xbox_base + slot * uint32_t(p.xbox_bytes) + uint32_t(h) * rows * 512u, &maps.x[i],
                    (chunk * kHalves + h) * 256, 0, bar);
    }
  };
  // this CTA's share of problem q (everything but its place in the sequence)
  auto share_of = [&](const TableProblem& q) {
    Share s;
    s.u0 = cta * q.each + min(cta, q.extra);
    s.u1 = s.u0 + q.each + (cta < q.extra ? 1 : 0);
    s.head = s.tail = 0;
    s.first = s.row0 = s.rows = s.span0 = s.reads = 0;
    if (s.u1 > s.u0) {
      const Unit a = decode_unit(q, s.u0), b = decode_unit(q, s.u1 - 1);
      if (a.span_first < s.u0) s.head = min(s.u1, a.span_first + a.span_len) - s.u0;
      if (b.span_first + b.span_len > s.u1 && b.span_first >= s.u0 + s.head) s.tail = s.u1 - max(b.span_first, s.u0);
      if (s.head == s.u1 - s.u0) s.tail = 0;
      s.span0 = a.tile;
      s.rows = b.tile - a.tile + 1;   // segments of the share (one per column tile touched)
      s.reads = s.head > 0 && a.span_first + a.span_len <= s.u1 ? 1 : 0;
    }
    return s;
  };

  // ---- start-up ---------------------------------------------------------------------------------------
  // The first units are requested before anything else is set up: lane L of warp 1 initialises the barrier of
  // slot L, works out unit L of the CTA's sequence by itself and requests its packed weights and scales (static
  // data: with launch overlap this happens before the wait for the kernel ahead; the activations follow after it).
  const int early = min(S, 32);
  uint4 early_ent = make_uint4(0, 0, 0, 0);
  bool early_unit = false;
  if (warp == 1 && lane < early) {
    mbar_init(bars + uint32_t(lane) * 8u, 1);
    fence_mbar_init();
    fence_proxy_async();
    int first = 0;
    for (int i = 0; i < p.count && !early_unit; ++i) {
      const TableProblem& q = p.problem[i];
      const int n = q.each + (cta < q.extra ? 1 : 0);
      if (lane < first + n) {
        const Share sh = share_of(q);
        const Unit u = decode_unit(q, unit_at(sh, lane - first));
        early_ent.x = uint32_t(u.tile) | (uint32_t(i) << 24);
        early_ent.y = uint32_t(u.chunk) | (uint32_t(q.M - 1) << 20);
        early_unit = true;
      }
      first += n;
    }
    if (early_unit) issue(early_ent, uint32_t(lane), 1);
  }
  if (warp == 0) {
    // lane i: the share of problem i; its place in the sequence and its first segment by a scan over the lanes
    Share sh;
    sh.u0 = sh.u1 = sh.head = sh.tail = sh.first = sh.row0 = sh.rows = sh.span0 = sh.reads = 0;
    if (lane < p.count) sh = share_of(p.problem[lane]);
    int units_before = sh.u1 - sh.u0, segments_before = sh.rows;   // inclusive scans
#pragma unroll
    for (int d = 1; d < kMaxProblems; d <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, units_before, d), b = __shfl_up_sync(0xffffffffu, segments_before, d);
      if (lane >= d) {
        units_before += a;
        segments_before += b;
      }
    }
    if (lane < p.count) {
      sh.first = units_before - (sh.u1 - sh.u0);
      shares[lane] = sh;
      acc_first[lane] = segments_before - sh.rows;
    }
    if (lane == p.count - 1) {
      total_units = units_before;
      total_segments = segments_before;
    }
  }
  if (tid == 0) abort_flag = 0;
  if (tid == 0) mail_tail = mail_head = 0;
  if (tid == 0) next_unit = 0;
  if (tid < kMailEntries) mail_ready[tid] = 0;
  for (int i = tid; i < S; i += THREADS) {
    if (i >= early) mbar_init(bars + uint32_t(i) * 8u, 1);
    uses[i] = 0;
  }
  for (int i = tid; i < ((1 << p.acc_ring_shift) << p.chain_shift) + (1 << p.acc_ring_shift); i += THREADS) turn[i] = 0;
  if (tid == 0) fence_mbar_init();
  __syncthreads();
  const int total = total_units;

  // One schedule entry per thread; the threads of the first S entries that were not requested above do so now.
  uint4 mine_ent = make_uint4(0, 0, 0, 0);
  for (int e = tid; e < total; e += THREADS) {
    int i = 0;
    while (i + 1 < p.count && e >= shares[i + 1].first) ++i;
    const TableProblem& q = p.problem[i];
    const Share& sh = shares[i];
    const int unit = unit_at(sh, e - sh.first);
    const Unit u = decode_unit(q, unit);
    const int seg_begin = max(u.span_first, sh.u0), seg_end = min(u.span_first + u.span_len, sh.u1);
    const int seg_len = seg_end - seg_begin;
    const bool whole = seg_len == u.span_len;
    const bool ends = seg_end == u.span_first + u.span_len;
    const int earlier = whole ? 0 : cta - cta_of(q, u.span_first);
    uint4 ent;
    ent.x = uint32_t(u.tile) | (uint32_t(i) << 24) | (whole ? 1u << 28 : 0u) | (ends ? 1u << 29 : 0u);
    ent.y = uint32_t(u.chunk) | (uint32_t(q.M - 1) << 20);
    ent.z = uint32_t(seg_len) | (uint32_t(earlier) << 20);
    ent.w = uint32_t(unit - seg_begin) | (uint32_t(acc_first[i] + u.tile - sh.span0) << 16);
    sched[e] = ent;
    if (e == tid) mine_ent = ent;
  }
  if (tid >= early && tid < min(total, S)) issue(mine_ent, uint32_t(tid), 1);
  if (p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (early_unit) issue(early_ent, uint32_t(lane), 2);
  if (tid >= early && tid < min(total, S)) issue(mine_ent, uint32_t(tid), 2);
  __syncthreads();   // the schedule is complete

  if (warp == RING) {
    // ---- the reducer warp ------------------------------------------------------------------------
    // A span cut by a CTA boundary: every CTA but the one holding its end publishes its segment's sum to global
    // scratch and moves on; the warp that completes the LAST segment leaves that sum here.  This warp then waits
    // for the published sums (round trips behind a deep queue of bulk loads: microseconds), adds them in CTA
    // order, its own last, and writes Y.  The warps that serve the ring never wait for global memory.
    int expected = 0;
    for (int i = 0; i < p.count; ++i) expected += shares[i].reads;
    if (p.probe >= 2 && p.probe <= 5) expected = 0;   // measurement modes that skip the hand-over
    const int v8r = lane & 7;
    for (int n = 0; n < expected; ++n) {
      const int e = n % kMailEntries;
      bool ok = false;
      for (int spin = 0; spin < (1 << 22); ++spin) {
        if (*reinterpret_cast<volatile int*>(&mail_ready[e]) == n + 1) { ok = true; break; }
        if (*reinterpret_cast<volatile int*>(&abort_flag)) break;
        __nanosleep(512);
      }
      if (!ok) {
        if (lane == 0 && !*reinterpret_cast<volatile int*>(&abort_flag)) {
          atomicExch(p.status, INTENT_B200_ERR_TIMEOUT);
          *reinterpret_cast<volatile int*>(&abort_flag) = 1;
        }
        return;
      }
      __threadfence_block();
      const TableProblem& q = p.problem[mail_ctx[e][0]];
      const int tile = mail_ctx[e][1], published = mail_ctx[e][2];
      const int part_floats = q.M * kCols;
      const float* span_scratch = q.scratch1 + size_t(tile) * q.maxp * part_floats;   // one chunk block: span = tile
      uint16_t* y = reinterpret_cast<uint16_t*>(q.y);
      for (int m = lane >> 3; m < q.M; m += 4) {
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int c = 0; c < published; ++c) {
          float4 a;
          if (!take_published(reinterpret_cast<const float4*>(span_scratch + size_t(c) * part_floats + m * kCols + 4 * v8r), &a)) {
            atomicExch(p.status, INTENT_B200_ERR_TIMEOUT);   // a neighbour's sum never arrived
            *reinterpret_cast<volatile int*>(&abort_flag) = 1;
          }
          sum.x += a.x; sum.y += a.y; sum.z += a.z; sum.w += a.w;
        }
        const float4 own = *reinterpret_cast<const float4*>(&mail_data[e][m][4 * v8r]);
        sum.x += own.x; sum.y += own.y; sum.z += own.z; sum.w += own.w;
        const int col = tile * kCols + 4 * v8r;
        if (col < q.N) {
          uint2 out;
          out.x = uint32_t(Elem<T>::from_float(sum.x)) | (uint32_t(Elem<T>::from_float(sum.y)) << 16);
          out.y = uint32_t(Elem<T>::from_float(sum.z)) | (uint32_t(Elem<T>::from_float(sum.w)) << 16);
          *reinterpret_cast<uint2*>(y + size_t(m) * q.N + col) = out;
        }
      }
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&mail_head) = n + 1;   // the entry may be reused
      }
    }
    return;
  }

  // ---- the ring warps ------------------------------------------------------------------------------
  uint32_t magic_a, magic_b;
  Expand<T>::magic(p.twos_complement != 0, magic_a, magic_b);
  int row_of[STEPS];
  uint32_t off_of[STEPS];
#pragma unroll
  for (int i = 0; i < STEPS; ++i) {
    row_of[i] = STEPS >= 2 ? 8 * (i >> 1) + 2 * t + (i & 1) : t;
    off_of[i] = uint32_t(row_of[i]) * 128u + (uint32_t(g ^ (row_of[i] & 7)) << 4);
  }
  float* my_corr = corr + warp * (GPC * CP);  // this warp's correction sums of the unit in hand
  const bool skip_math = p.probe >= 1 && p.probe <= 5;
  // the bias of an expanded nibble as a weight operand: even pairs (k0,k4), (k2,k6) and odd pairs (k1,k5), (k3,k7)
  const uint32_t bias_even = uint32_t(Elem<T>::from_float(Expand<T>::kEven)) * 0x00010001u;
  const uint32_t bias_odd = uint32_t(Elem<T>::from_float(Expand<T>::kOdd)) * 0x00010001u;

  for (;;) {
    if (*reinterpret_cast<volatile int*>(&abort_flag)) break;
    int seq = 0;
    if (lane == 0) seq = atomicAdd(&next_unit, 1);
    seq = __shfl_sync(0xffffffffu, seq, 0);
    if (seq >= total) break;
    const uint4 now = sched[seq];
    const int use = fast_div(seq, S, p.magic_slots);
    const uint32_t slot = uint32_t(seq - use * S);
    const int M = int((now.y >> 20) & 7u) + 1;
    const uint32_t bar = bars + slot * 8u;
    bool requested = true;
    if (use > 0 && uses[slot] < use) {
      requested = false;
      for (int spin = 0; spin < (1 << 20); ++spin) {
        if (uses[slot] >= use) { requested = true; break; }
        if (*reinterpret_cast<volatile int*>(&abort_flag)) break;
        __nanosleep(64);
      }
    }
    __threadfence_block();
    if (!__all_sync(0xffffffffu, requested && mbar_wait(bar, uint32_t(use) & 1u))) {
      if (lane == 0) {
        atomicExch(p.status, INTENT_B200_ERR_TIMEOUT);   // this unit's loads never completed
        *reinterpret_cast<volatile int*>(&abort_flag) = 1;
      }
      break;
    }
    const uint32_t wslot = base + slot * kUnitBytes;
    const uint32_t sslot = scale_base + slot * kScaleBytes;
    const uint32_t xslot = xbox_base + slot * uint32_t(p.xbox_bytes);
    const uint32_t xhalf = uint32_t(M) * 512u;   // bytes of one activation box
    float facc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) facc[i] = 0.f;

    if (!skip_math) {
      // lane L takes packed row L of the unit's activations (8 values of one row of X), puts it back in the
      // nibble-pair order the MMA fragments are read in, and the rows of a group (RPG adjacent lanes) add
      // their share of the correction sum  - sum_k x[m,k] * (bias_k + 8)  with a fixed-order butterfly
      for (int mh = 0; mh < M * kHalves; ++mh) {
        const int m = kHalves == 1 ? mh : mh >> 1, h = kHalves == 1 ? 0 : mh & 1;
        const uint32_t addr = xslot + uint32_t(h) * xhalf + uint32_t(m) * 512u + uint32_t(lane) * 16u;
        const uint4 val = lds128(addr);
        uint4 o;
        o.x = prmt(val.x, val.z, 0x5410);                        // (k0, k4)
        o.y = Expand<T>::scale_odd(prmt(val.x, val.z, 0x7632));  // (k1, k5)
        o.z = prmt(val.y, val.w, 0x5410);                        // (k2, k6)
        o.w = Expand<T>::scale_odd(prmt(val.y, val.w, 0x7632));  // (k3, k7)
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(o.x), "r"(o.y), "r"(o.z), "r"(o.w)
                     : "memory");
        if (!CORR_MMA) {
          float partial = Expand<T>::kEven * (pair_sum<T>(o.x) + pair_sum<T>(o.z)) +
                          Expand<T>::kOdd * (pair_sum<T>(o.y) + pair_sum<T>(o.w));
#pragma unroll
          for (int d = RPG / 2; d >= 1; d >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, d);
          if ((lane % RPG) == 0) my_corr[((h * 32 + lane) / RPG) * CP + m] = -partial;
        }
      }
      __syncwarp();
      // Rows of X beyond M: the lanes that would hold them read row M - 1 instead.  An MMA output column depends
      // only on its own column of the activation fragment, and output columns >= M are never stored.
      const uint32_t xrow = xslot + uint32_t(min(g, M - 1)) * 512u;
#pragma unroll
      for (int gi = 0; gi < GPC; ++gi) {
        float gacc[8];
        float cacc[4] = {0.f, 0.f, 0.f, 0.f};   // CORR_MMA: sum over the group of bias_k * x[m, k] (every row the same)
        if (CORR_MMA) {
#pragma unroll
          for (int i = 0; i < 8; ++i) gacc[i] = 0.f;
        } else {
          // (entries of rows >= M hold stale values: they only reach accumulator rows that are never stored)
          const float2 c = *reinterpret_cast<const float2*>(&my_corr[gi * CP + 2 * t]);
#pragma unroll
          for (int i = 0; i < 8; ++i) gacc[i] = (i & 1) ? c.y : c.x;
        }
#pragma unroll
        for (int i = 0; i < STEPS; ++i) {
          const int row = gi * RPG + row_of[i];
          const uint32_t off = STEPS >= 2 ? off_of[i] + uint32_t(gi * RPG * 128)
                                          : uint32_t(row) * 128u + (uint32_t(g ^ (row & 7)) << 4);
          const uint4 w = lds128(wslot + off);
          const uint4 b = lds128(xrow + uint32_t(row >> 5) * xhalf + uint32_t(row & 31) * 16u);
          uint32_t c0[4], c1[4], c2[4], c3[4];
          Expand<T>::word(w.x, magic_a, magic_b, c0);
          Expand<T>::word(w.y, magic_a, magic_b, c1);
          Expand<T>::word(w.z, magic_a, magic_b, c2);
          Expand<T>::word(w.w, magic_a, magic_b, c3);
          float(&a01)[4] = *reinterpret_cast<float(*)[4]>(&gacc[0]);
          float(&a23)[4] = *reinterpret_cast<float(*)[4]>(&gacc[4]);
          Elem<T>::mma16816(a01, c0[0], c1[0], c0[1], c1[1], b.x, b.y);
          Elem<T>::mma16816(a23, c2[0], c3[0], c2[1], c3[1], b.x, b.y);
          Elem<T>::mma16816(a01, c0[2], c1[2], c0[3], c1[3], b.z, b.w);
          Elem<T>::mma16816(a23, c2[2], c3[2], c2[3], c3[3], b.z, b.w);
          if (CORR_MMA) {
            Elem<T>::mma16816(cacc, bias_even, bias_even, bias_odd, bias_odd, b.x, b.y);
            Elem<T>::mma16816(cacc, bias_even, bias_even, bias_odd, bias_odd, b.z, b.w);
          }
        }
        if (CORR_MMA) {
#pragma unroll
          for (int i = 0; i < 8; ++i) gacc[i] -= cacc[i & 1];
        }
        uint2 s;  // this lane's four column scales of the group (zero outside the matrix)
        asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(s.x), "=r"(s.y) : "r"(sslot + gi * 64 + g * 8));
        const float s0 = Elem<T>::to_float(uint16_t(s.x & 0xFFFF)), s1 = Elem<T>::to_float(uint16_t(s.x >> 16));
        const float s2 = Elem<T>::to_float(uint16_t(s.y & 0xFFFF)), s3 = Elem<T>::to_float(uint16_t(s.y >> 16));
        facc[0] = fmaf(gacc[0], s0, facc[0]);
        facc[1] = fmaf(gacc[1], s0, facc[1]);
        facc[2] = fmaf(gacc[2], s1, facc[2]);
        facc[3] = fmaf(gacc[3], s1, facc[3]);
        facc[4] = fmaf(gacc[4], s2, facc[4]);
        facc[5] = fmaf(gacc[5], s2, facc[5]);
        facc[6] = fmaf(gacc[6], s3, facc[6]);
        facc[7] = fmaf(gacc[7], s3, facc[7]);
      }
    }

    // the slot is free: the unit S places further on goes into it
    if (seq + S < total) {
      __syncwarp();
      fence_proxy_async();
      if (lane == 0) {
        issue(sched[seq + S], slot, 3);
        __threadfence_block();
        uses[slot] = use + 1;
      }
    }
    if (p.probe == 2 || p.probe == 3) continue;   // measurement: no reduction either

    // ---- the unit joins its segment's sum --------------------------------------------------------------
    // A segment's units are dealt round-robin to C chains, each with an accumulator [rows][32] in shared memory
    // and a turn counter: the warp with the chain's k-th unit waits until the first k have been added, adds its
    // own and passes the turn on.  One chain could not keep up (a hand-over through shared memory takes longer
    // than the stream needs per unit), C of them can, and the order of every addition stays fixed.
    // accumulator element i of a lane: row m = 2t + (i & 1), columns 4g + (i >> 1)
    // The CTA's segments take the chain sets of a small ring in turn (set = segment number modulo the ring,
    // generation = segment number / ring): the units in flight belong to a handful of segments at most.  Turn
    // counters carry the generation in their upper half, and a set is handed to its next segment by `done`.
    const int place = int(now.w & 0xFFFFu), seg_len = int(now.z & 0xFFFFFu);
    const int set = int(now.w >> 16) & ((1 << p.acc_ring_shift) - 1), generation = int(now.w >> 16) >> p.acc_ring_shift;
    const int chain0 = set << p.chain_shift;                     // the set's first chain
    const int chain = chain0 + (place & (p.chains - 1)), position = place >> p.chain_shift;
    const int turn0 = generation << 16;
    volatile int* done = turn + ((1 << p.acc_ring_shift) << p.chain_shift);   // per set: generations finished
    float* acc = accs + size_t(chain) * p.part_stride + 4 * g;
    auto await = [&](volatile int* counter, int count) {   // true once the counter has reached `count`
      for (int spin = 0; spin < (1 << 22); ++spin) {
        if (*counter >= count) return true;
        if (*reinterpret_cast<volatile int*>(&abort_flag)) return false;
        if (spin > 8) __nanosleep(32);
      }
      if (lane == 0) {
        atomicExch(p.status, INTENT_B200_ERR_TIMEOUT);
        *reinterpret_cast<volatile int*>(&abort_flag) = 1;
      }
      return false;
    };
    if (position == 0) {
      if (generation > 0 && !await(done + set, generation)) break;   // the set's previous segment has been read out
    } else {
      if (!await(turn + chain, turn0 + position)) break;
      __threadfence_block();
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
        if (2 * t + hh < M) {
          const float4 v = *reinterpret_cast<const float4*>(acc + (2 * t + hh) * kCols);
          facc[0 + hh] += v.x; facc[2 + hh] += v.y; facc[4 + hh] += v.z; facc[6 + hh] += v.w;
        }
    }
#pragma unroll
    for (int hh = 0; hh < 2; ++hh)
      if (2 * t + hh < M)
        *reinterpret_cast<float4*>(acc + (2 * t + hh) * kCols) = make_float4(facc[0 + hh], facc[2 + hh], facc[4 + hh], facc[6 + hh]);
    __syncwarp();
    if (lane == 0) {
      __threadfence_block();
      turn[chain] = turn0 + position + 1;
    }
    if (place + 1 < seg_len || p.probe == 4) continue;

    // ---- the segment's last unit: add the chains in order ----------------------------------------------
    {
      bool complete = true;
      const int used = min(p.chains, seg_len);
      for (int c = 0; c < used && complete; ++c)
        complete = await(turn + chain0 + c, turn0 + ((seg_len - c + p.chains - 1) >> p.chain_shift));
      if (!complete) break;
      __threadfence_block();
#pragma unroll
      for (int i = 0; i < 8; ++i) facc[i] = 0.f;
      for (int c = 0; c < used; ++c) {
        const float* from = accs + size_t(chain0 + c) * p.part_stride + 4 * g;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
          if (2 * t + hh < M) {
            const float4 v = *reinterpret_cast<const float4*>(from + (2 * t + hh) * kCols);
            facc[0 + hh] += v.x; facc[2 + hh] += v.y; facc[4 + hh] += v.z; facc[6 + hh] += v.w;
          }
      }
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        done[set] = generation + 1;
      }
    }

    // ---- the segment is complete: this warp holds its sum ----------------------------------------------
    const int pi = int((now.x >> 24) & 15u);
    const int tile = int(now.x & 0xFFFFFFu);
    const TableProblem& q = p.problem[pi];
    const bool whole = ((now.x >> 28) & 1u) != 0 || p.probe == 5;
    const int col = tile * kCols + 4 * g;
    if (whole) {
      uint16_t* y = reinterpret_cast<uint16_t*>(q.y);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int m = 2 * t + hh;
        if (m < M && col < q.N) {   // N is a multiple of 8, so the four columns are inside together
          uint2 out;
          out.x = uint32_t(Elem<T>::from_float(facc[0 + hh])) | (uint32_t(Elem<T>::from_float(facc[2 + hh])) << 16);
          out.y = uint32_t(Elem<T>::from_float(facc[4 + hh])) | (uint32_t(Elem<T>::from_float(facc[6 + hh])) << 16);
          *reinterpret_cast<uint2*>(y + size_t(m) * q.N + col) = out;
        }
      }
    } else if (((now.x >> 29) & 1u) == 0) {
      // the span goes on in the next CTA: publish this segment's sum and move on
      float* dst = q.scratch1 + (size_t(tile) * q.maxp + (now.z >> 20)) * (M * kCols);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int m = 2 * t + hh;
        if (m < M)
          publish(reinterpret_cast<float4*>(dst + m * kCols + 4 * g),
                  make_float4(facc[0 + hh], facc[2 + hh], facc[4 + hh], facc[6 + hh]));
      }
    } else {
      // the span ends here: its sum goes to the reducer warp
      int ticket = 0;
      if (lane == 0) ticket = atomicAdd(&mail_tail, 1);
      ticket = __shfl_sync(0xffffffffu, ticket, 0);
      bool room = false;
      for (int spin = 0; spin < (1 << 22); ++spin) {
        if (ticket - *reinterpret_cast<volatile int*>(&mail_head) < kMailEntries) { room = true; break; }
        if (*reinterpret_cast<volatile int*>(&abort_flag)) break;
        __nanosleep(256);
      }
      if (!room) {
        if (lane == 0 && !*reinterpret_cast<volatile int*>(&abort_flag)) {
          atomicExch(p.status, INTENT_B200_ERR_TIMEOUT);
          *reinterpret_cast<volatile int*>(&abort_flag) = 1;
        }
        break;
      }
      __threadfence_block();
      const int e = ticket % kMailEntries;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int m = 2 * t + hh;
        if (m < M)
          *reinterpret_cast<float4*>(&mail_data[e][m][4 * g]) = make_float4(facc[0 + hh], facc[2 + hh], facc[4 + hh], facc[6 + hh]);
      }
      __syncwarp();
      if (lane == 0) {
        mail_ctx[e][0] = pi;
        mail_ctx[e][1] = tile;
        mail_ctx[e][2] = int(now.z >> 20);
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&mail_ready[e]) = ticket + 1;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
struct HostProblem {
  const void* x;
  const void* w;
  const void* s;
  void* y;
  int64_t M, K, N;
};

struct ProblemPlan {
  int chunks, tiles, cb, nblocks, units, each, extra, maxp;
  bool ride;                                     // the ride-along form (no staging, no CTA barriers)
  int segments, sequence;                        // ride-along form: segment accumulators and schedule entries (worst CTA)
  int unit_rows;                                 // packed rows of a unit: 32, or 64 in the ride-along form for few rows
  size_t xs_bytes, corr_bytes, part_bytes;       // shared memory this problem needs (worst CTA)
  size_t counters1, counters2, scratch1, scratch2, bytes;   // workspace layout (offsets) and size
};

// One slot of the ring: the packed weights, the unit's scales, the mbarrier and the use count.
size_t slot_bytes(int group_size, int unit_rows = kRows) {
  return size_t(unit_rows) * kCols * 4 + size_t(unit_rows * 8 / group_size) * 64 + 8 + 4;
}
// alignment slack + smallest ring + span tickets (one row per problem) + finished counters + rounding of the regions
size_t fixed_bytes(int group_size) {
  return 1024 + size_t(kMinSlots) * slot_bytes(group_size) + 256 + kMaxProblems * kMaxSpans * 4 + 64 + 128;
}
// ride-along form: per-warp correction sums of the unit in hand (32 warps x groups of a unit x 8 rows)
size_t ride_corr_bytes(int group_size, int unit_rows) { return size_t(32) * (unit_rows * 8 / group_size) * 8 * 4; }
int g_table_unit_rows = 0;   // 64 = the ride-along form uses 64-row units for problems of up to four rows; for measurement
// the ride-along form is planned only if this many slots fit (about 80 KB of packed weights in flight per SM)
int min_ride_slots(int unit_rows) { return unit_rows == 64 ? 12 : 20; }
// ride-along form: what a launch needs in shared memory besides its slots
int ride_chains(int rows) { return rows <= 2 ? 8 : 4; }        // chains per segment
int ride_ring_shift(int rows) { return rows <= 4 ? 4 : 3; }     // log2 of the chain sets that exist at a time
size_t ride_other_bytes(size_t sequence, int rows, size_t corr_bytes) {
  const size_t sets = size_t(1) << ride_ring_shift(rows);
  return 1024 + 512 + corr_bytes + sets * (ride_chains(rows) * (size_t(rows) * kCols * 4 + 4) + 4) + sequence * 16;
}

// Spans a CTA may touch and rows it must stage, worst case over CTAs, for a chunk-block size.
void share_bounds(int tiles, int chunks, int cb, int n_max, int* blocks_touched, int* spans_touched) {
  const long long block_units = (long long)tiles * cb;
  const int nblocks = (chunks + cb - 1) / cb;
  long long touched = n_max <= 0 ? 0 : (n_max + block_units - 2) / block_units + 1;
  if (touched > nblocks) touched = nblocks;
  *blocks_touched = int(touched);
  const int shortest = chunks - (nblocks - 1) * cb;      // the last block's spans may be shorter
  *spans_touched = n_max <= 0 ? 0 : (n_max - 1) / (shortest < cb ? shortest : cb) + 2;
}

bool plan_problem(int M, int K, int N, int group_size, int grid, bool allow_ride, ProblemPlan* out) {
  ProblemPlan q{};
  const size_t smem_budget = size_t(kSmemLimit) - fixed_bytes(group_size);
  int n_max = 0;
  const auto geometry = [&](int unit_rows) {
    q.unit_rows = unit_rows;
    q.tiles = (N + kCols - 1) / kCols;
    q.chunks = (K / 8 + unit_rows - 1) / unit_rows;
    if ((long long)q.tiles * q.chunks > (1ll << 30)) return false;   // unit numbers are 32-bit
    q.units = q.tiles * q.chunks;
    q.each = q.units / grid;
    q.extra = q.units % grid;
    n_max = q.each + (q.extra ? 1 : 0);
    return true;
  };
  // ride-along form: the activations travel with every unit, the whole K range is one chunk block.  Units of
  // 64 packed rows (the bookkeeping of a unit paid once per 8 KiB) are built but not chosen: measured slower
  // (M = 1: 6.6 against 6.5 us per projection in a long table, 10.7 against 9.6 with one launch per step;
  // M = 4: 9.1 against 7.7) - fewer slots than ring warps, and a longer wait for the first unit of a launch.
  q.ride = false;
  for (int unit_rows : {64, 32}) {
    if (!allow_ride || M > kRideRows || q.ride) break;
    if (unit_rows == 64 && (M > 4 || g_table_unit_rows != 64)) continue;
    if (!geometry(unit_rows)) return false;
    int blocks, spans;
    share_bounds(q.tiles, q.chunks, q.chunks, n_max, &blocks, &spans);
    q.segments = spans;
    q.sequence = n_max;
    q.ride = n_max < 65536 && size_t(min_ride_slots(unit_rows)) * (slot_bytes(group_size, unit_rows) + size_t(M) * unit_rows * 16) +
                                      ride_other_bytes(n_max, M, ride_corr_bytes(group_size, unit_rows)) <=
                                  size_t(kSmemLimit);
  }
  if (!q.ride && !geometry(kRows)) return false;
  q.part_bytes = size_t(n_max) * M * kCols * 4;
  const int rpg = group_size / 8;
  int cb = q.chunks;
  if (q.ride) {
    q.xs_bytes = 0;
    q.corr_bytes = ride_corr_bytes(group_size, q.unit_rows);
    q.part_bytes = 0;
  } else {
    // the largest chunk block whose staged activations (all blocks a CTA can touch) fit beside the rest
    for (;;) {
      int blocks, spans;
      share_bounds(q.tiles, q.chunks, cb, n_max, &blocks, &spans);
      const size_t rows = size_t(blocks) * cb * kRows;
      q.xs_bytes = rows * M * 16;
      q.corr_bytes = (rows / rpg + 1) * 16 * 4;   // sized for the wider correction pitch (M > 8 in the same launch)
      if (spans <= kMaxSpans && q.xs_bytes + q.corr_bytes + q.part_bytes <= smem_budget) break;
      if (cb == 1) return false;
      cb = (cb + 1) / 2;
    }
  }
  q.cb = cb;
  q.nblocks = (q.chunks + cb - 1) / cb;
  q.maxp = q.each == 0 ? cb : ((cb + q.each - 2) / q.each + 1 < cb ? (cb + q.each - 2) / q.each + 1 : cb);
  if (q.maxp < 1) q.maxp = 1;
  const size_t spans = size_t(q.nblocks) * q.tiles;
  size_t offset = 0;
  q.counters1 = offset;
  offset += (spans * 4 + 255) / 256 * 256;
  q.counters2 = offset;
  offset += (size_t(q.tiles) * 4 + 255) / 256 * 256;
  q.scratch1 = offset;
  offset += (spans * q.maxp * M * kCols * 4 + 255) / 256 * 256;
  q.scratch2 = offset;
  if (q.nblocks > 1) offset += (size_t(q.tiles) * q.nblocks * M * kCols * 4 + 255) / 256 * 256;
  q.bytes = offset;
  *out = q;
  return true;
}

int table_sms() {
  static int sms = [] {
    int device = 0, value = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    return value;
  }();
  return sms;
}

int g_table_overlap = 0;
int g_table_ride = 1;     // 0 forces the staged form (measurement and tests)

int validate(const HostProblem& h, int group_size) {
  if (h.M < 0 || h.K < 0 || h.N < 0) return INTENT_B200_ERR_SHAPE;
  if (h.M == 0 || h.N == 0) return INTENT_B200_OK;
  if (!h.x || !h.w || !h.s || !h.y) return INTENT_B200_ERR_NULL;
  if (!aligned16(h.x) || !aligned16(h.w) || !aligned16(h.s) || !aligned16(h.y)) return INTENT_B200_ERR_LAYOUT;
  if (h.K == 0 || h.K % group_size != 0 || h.N % 8 != 0 || h.M > 16 || h.K > (1 << 24) || h.N > (1 << 24))
    return INTENT_B200_ERR_UNSUPPORTED;
  return INTENT_B200_OK;
}

int g_table_probe = 0;
int g_table_corr_mma = -1;   // ride-along kernel: correction sums by MMA (1), from the activations (0), built-in choice (-1)
int g_table_slots = 0;     // upper limit on the ring's slots (0 = the built-in choice); for measurement

template <typename T, int MB, int STEPS>
int launch_table(const TableMaps& maps, const TableParams& p, int grid, size_t smem, cudaStream_t stream) {
  constexpr int WARPS = MB == 1 ? 32 : 16;
  auto kernel = w4a16_table_kernel<T, MB, STEPS, WARPS>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (e != cudaSuccess) return cuda_status(e);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid, 1, 1);
  config.blockDim = dim3(WARPS * 32, 1, 1);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = p.overlap ? 1 : 0;
  if (LaunchFacts* sink = observe_sink())
    return record_launch(sink, reinterpret_cast<const void*>(kernel), "w4a16_table_kernel staged activations", grid,
                         WARPS * 32, int(smem), 1);
  e = cudaLaunchKernelEx(&config, kernel, maps, p);
  if (e != cudaSuccess) return cuda_status(e);
  note_launch();
  return launch_status();
}

template <typename T, int STEPS, int UR, bool CORR_MMA>
int launch_ride(const TableMaps& maps, const TableParams& p, int grid, size_t smem, cudaStream_t stream) {
  auto kernel = w4a16_ride_kernel<T, STEPS, UR, CORR_MMA>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  if (e != cudaSuccess) return cuda_status(e);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid, 1, 1);
  config.blockDim = dim3(1024, 1, 1);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = p.overlap ? 1 : 0;
  if (LaunchFacts* sink = observe_sink())
    return record_launch(sink, reinterpret_cast<const void*>(kernel), "w4a16_ride_kernel activations ride with the units",
                         grid, 1024, int(smem), 1);
  e = cudaLaunchKernelEx(&config, kernel, maps, p);
  if (e != cudaSuccess) return cuda_status(e);
  note_launch();
  return launch_status();
}

// Lays out the workspace of a whole table: a 256-byte header (status word), then every problem's part.
int64_t table_workspace(const HostProblem* problems, int count, int group_size, int grid, ProblemPlan* plans,
                        size_t* offsets) {
  size_t offset = 256;
  for (int begin = 0; begin < count; begin += kMaxProblems) {
    const int n = count - begin < kMaxProblems ? count - begin : kMaxProblems;
    // the problems of one launch share the space behind the ring: every one must fit next to the others' maximum,
    // which the per-problem budget below guarantees without a second pass
    for (int i = begin; i < begin + n; ++i) {
      const HostProblem& h = problems[i];
      if (h.M <= 0 || h.N <= 0) {
        plans[i] = ProblemPlan{};
        offsets[i] = offset;
        continue;
      }
      if (!plan_problem(int(h.M), int(h.K), int(h.N), group_size, grid, g_table_ride != 0, &plans[i])) return -1;
      offsets[i] = offset;
      offset += plans[i].bytes;
    }
  }
  return int64_t(offset);
}

template <typename T>
int run_table(const HostProblem* problems, int count, int group_size, int zero_point, void* workspace,
              int64_t workspace_bytes, cudaStream_t stream) {
  if (count < 0) return INTENT_B200_ERR_SHAPE;
  if (count == 0) return INTENT_B200_OK;
  if (!problems) return INTENT_B200_ERR_NULL;
  if (count > 4096) return INTENT_B200_ERR_UNSUPPORTED;
  if (group_size != 32 && group_size != 64 && group_size != 128) return INTENT_B200_ERR_UNSUPPORTED;
  if (zero_point != -1 && zero_point != 8) return INTENT_B200_ERR_UNSUPPORTED;
  for (int i = 0; i < count; ++i) {
    const int status = validate(problems[i], group_size);
    if (status != INTENT_B200_OK) return status;
  }
  const int grid = table_sms();
  if (grid <= 0) return INTENT_B200_ERR_UNSUPPORTED;
  ProblemPlan* plans = new ProblemPlan[count];
  size_t* offsets = new size_t[count];
  struct Cleanup {
    ProblemPlan* a;
    size_t* b;
    ~Cleanup() { delete[] a; delete[] b; }
  } cleanup{plans, offsets};
  const int64_t need = table_workspace(problems, count, group_size, grid, plans, offsets);
  if (need < 0) return INTENT_B200_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < need || !aligned16(workspace)) return INTENT_B200_ERR_WORKSPACE;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  const CUtensorMapDataType xt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int steps = group_size / 32;

  // Problems that share a launch share the space behind the slot ring, each region sized for the largest of
  // them: a launch takes as many problems (at most kMaxProblems) of one form as fit together.  The problems are
  // independent, so they may run in any order: the ride-along ones first, then the staged ones.
  const size_t behind_ring = size_t(kSmemLimit) - fixed_bytes(group_size);
  int* order = new int[count];
  struct OrderCleanup {
    int* a;
    ~OrderCleanup() { delete[] a; }
  } order_cleanup{order};
  {
    int k = 0;
    for (int pass = 0; pass < 2; ++pass)
      for (int i = 0; i < count; ++i)
        if ((pass == 0) == plans[i].ride) order[k++] = i;
  }
  for (int begin = 0; begin < count;) {
    TableMaps maps;
    TableParams p{};
    size_t xs_max = 0, corr_max = 0, part_max = 0, sequence = 0, segments = 0;
    int n = 0, mb = 1, i = begin, rows_max = 0;
    bool ride = false;
    int unit_rows = kRows;
    for (; i < count && n < kMaxProblems; ++i) {
      const int index = order[i];
      const HostProblem& h = problems[index];
      if (h.M <= 0 || h.N <= 0) continue;   // nothing to compute
      const ProblemPlan& q = plans[index];
      if (n == 0) {
        ride = q.ride;
        unit_rows = q.unit_rows;
      }
      if (q.ride != ride || q.unit_rows != unit_rows) break;   // a launch is one form of the kernel
      {
        const size_t xs = q.xs_bytes > xs_max ? q.xs_bytes : xs_max;
        const size_t corr_b = q.corr_bytes > corr_max ? q.corr_bytes : corr_max;
        const size_t part_b = q.part_bytes > part_max ? q.part_bytes : part_max;
        const int rows = int(h.M) > rows_max ? int(h.M) : rows_max;
        if (ride) {
          if (n > 0 && size_t(min_ride_slots(unit_rows)) * (slot_bytes(group_size, unit_rows) + size_t(rows) * unit_rows * 16) +
                               ride_other_bytes(sequence + q.sequence, rows, q.corr_bytes) >
                           size_t(kSmemLimit))
            break;
        } else if (n > 0 && xs + corr_b + part_b > behind_ring) {
          break;
        }
      }
      TableProblem& d = p.problem[n];
      d.x = h.x;
      d.y = h.y;
      d.M = int(h.M);
      d.K = int(h.K);
      d.N = int(h.N);
      d.groups = int(h.K / group_size);
      d.chunks = q.chunks;
      d.tiles = q.tiles;
      d.cb = q.cb;
      d.nblocks = q.nblocks;
      d.units = q.units;
      d.each = q.each;
      d.extra = q.extra;
      d.maxp = q.maxp;
      {
        auto magic = [](long long divisor) { return uint32_t(((1ll << 32) + divisor - 1) / divisor); };
        const int last_len = q.chunks - (q.nblocks - 1) * q.cb;
        d.magic_full = magic((long long)q.tiles * q.cb);
        d.magic_cb = magic(q.cb);
        d.magic_last = magic(last_len);
      }
      d.counters1 = reinterpret_cast<int*>(ws + offsets[index] + q.counters1);
      d.counters2 = reinterpret_cast<int*>(ws + offsets[index] + q.counters2);
      d.scratch1 = reinterpret_cast<float*>(ws + offsets[index] + q.scratch1);
      d.scratch2 = reinterpret_cast<float*>(ws + offsets[index] + q.scratch2);
      if (!make_tensor_map_2d(&maps.w[n], CU_TENSOR_MAP_DATA_TYPE_INT32, h.w, uint64_t(h.K / 8), uint64_t(h.N),
                              uint64_t(h.N) * 4, uint32_t(unit_rows), kCols, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B) ||
          !make_tensor_map_2d(&maps.s[n], xt, h.s, uint64_t(h.K / group_size), uint64_t(h.N), uint64_t(h.N) * 2,
                              uint32_t(unit_rows * 8 / group_size), kCols, CU_TENSOR_MAP_SWIZZLE_NONE))
        return INTENT_B200_ERR_UNSUPPORTED;
      if (ride && !make_tensor_map_2d(&maps.x[n], xt, h.x, uint64_t(h.M), uint64_t(h.K), uint64_t(h.K) * 2,
                                      uint32_t(h.M), 256, CU_TENSOR_MAP_SWIZZLE_NONE))
        return INTENT_B200_ERR_UNSUPPORTED;
      if (int(h.M) > rows_max) rows_max = int(h.M);
      sequence += size_t(q.sequence);
      segments += size_t(q.segments);
      xs_max = q.xs_bytes > xs_max ? q.xs_bytes : xs_max;
      corr_max = q.corr_bytes > corr_max ? q.corr_bytes : corr_max;
      part_max = q.part_bytes > part_max ? q.part_bytes : part_max;
      if (h.M > 8) mb = 2;
      ++n;
    }
    begin = i;
    if (n == 0) continue;
    for (int k = 0; k < kMaxProblems; ++k) {   // unused descriptors must still be valid objects
      if (k >= n) {
        maps.w[k] = maps.w[0];
        maps.s[k] = maps.s[0];
      }
      if (k >= n || !ride) maps.x[k] = maps.w[0];
    }
    p.count = n;
    p.twos_complement = zero_point == -1 ? 1 : 0;
    p.overlap = g_table_overlap;
    p.status = reinterpret_cast<int*>(ws);
    // As many slots as fit beside this launch's other regions, up to the built-in choice.
    const auto round16 = [](size_t v) { return (v + 15) & ~size_t(15); };
    p.xbox_bytes = ride ? rows_max * unit_rows * 16 : 0;
    {
      const size_t others = ride ? ride_other_bytes(sequence, rows_max, corr_max)
                                 : 1024 + 256 + size_t(kMaxSpans) * 4 + 64 + 128 + round16(corr_max) + round16(xs_max) +
                                       round16(part_max);
      if (others >= size_t(kSmemLimit)) return INTENT_B200_ERR_UNSUPPORTED;
      size_t slots = (size_t(kSmemLimit) - others) / (slot_bytes(group_size, unit_rows) + p.xbox_bytes);
      // Staged form: a whole number of slots per warp (every slot then always belongs to the same warp, and no
      // warp has to check who used a slot before it).  Ride-along form: one slot per ring warp; measured on
      // M = 1, a deeper ring (40 slots) does not stream faster and a shallower one (24) hardly slower.
      const size_t choice = ride ? 31 : size_t(mb == 1 ? 32 : 16);
      if (g_table_slots > 0) {
        if (slots > size_t(g_table_slots)) slots = g_table_slots;
      } else if (slots >= choice) {
        slots = ride ? choice : slots / choice * choice;
      }
      if (slots > size_t(kMaxSlots)) slots = kMaxSlots;
      if (slots < 8) return INTENT_B200_ERR_UNSUPPORTED;   // cannot happen: every problem was planned with more
      p.slots = int(slots);
      p.magic_slots = uint32_t(((1ll << 32) + p.slots - 1) / p.slots);
    }
    size_t offset = size_t(p.slots) * (slot_bytes(group_size, unit_rows) - 4);
    offset = (offset + 15) & ~size_t(15);
    p.uses_offset = int(offset);
    offset += size_t(p.slots) * 4;
    offset = (offset + 127) & ~size_t(127);
    p.xbox_offset = int(offset);
    offset += size_t(p.slots) * p.xbox_bytes;
    p.chains = ride ? ride_chains(rows_max) : 1;
    p.chain_shift = p.chains == 8 ? 3 : p.chains == 4 ? 2 : 0;
    p.acc_ring_shift = ride_ring_shift(rows_max);
    const size_t sets = size_t(1) << p.acc_ring_shift;
    p.span_offset = int(offset);    // staged: span tickets; ride-along: the chains' turn counters, then the sets' `done`
    offset += round16(ride ? sets * (p.chains + 1) * 4 : size_t(kMaxSpans) * 4);
    p.corr_offset = int(offset);
    offset += round16(corr_max);
    p.xs_offset = int(offset);
    offset += round16(xs_max);
    p.part_offset = int(offset);    // staged: per-unit partials; ride-along: the chains' accumulators
    p.part_stride = ride ? rows_max * kCols : int(round16(part_max) / 4);      // in floats
    p.probe = g_table_probe;
    offset += ride ? sets * p.chains * size_t(rows_max) * kCols * 4 : round16(part_max);
    p.sched_offset = int(offset);
    if (ride) offset += sequence * 16;
    const size_t smem = 1024 + offset;
    if (smem > size_t(kSmemLimit)) return INTENT_B200_ERR_UNSUPPORTED;   // cannot happen: every problem was planned to fit
    int status;
#define IB200_TABLE_STEPS(MB_)                                                           \
  status = steps == 4   ? launch_table<T, MB_, 4>(maps, p, grid, smem, stream)           \
           : steps == 2 ? launch_table<T, MB_, 2>(maps, p, grid, smem, stream)           \
                        : launch_table<T, MB_, 1>(maps, p, grid, smem, stream);
    if (ride) {
      const bool corr_mma = g_table_corr_mma < 0 ? rows_max >= 3 : g_table_corr_mma != 0;
      if (unit_rows == 64)
        status = steps == 4   ? launch_ride<T, 4, 64, false>(maps, p, grid, smem, stream)
                 : steps == 2 ? launch_ride<T, 2, 64, false>(maps, p, grid, smem, stream)
                              : launch_ride<T, 1, 64, false>(maps, p, grid, smem, stream);
      else if (corr_mma)
        status = steps == 4   ? launch_ride<T, 4, 32, true>(maps, p, grid, smem, stream)
                 : steps == 2 ? launch_ride<T, 2, 32, true>(maps, p, grid, smem, stream)
                              : launch_ride<T, 1, 32, true>(maps, p, grid, smem, stream);
      else
        status = steps == 4   ? launch_ride<T, 4, 32, false>(maps, p, grid, smem, stream)
                 : steps == 2 ? launch_ride<T, 2, 32, false>(maps, p, grid, smem, stream)
                              : launch_ride<T, 1, 32, false>(maps, p, grid, smem, stream);
    } else if (mb == 1) {
      IB200_TABLE_STEPS(1)
    } else {
      IB200_TABLE_STEPS(2)
    }
#undef IB200_TABLE_STEPS
    if (status != INTENT_B200_OK) return status;
  }
  return INTENT_B200_OK;
}

int g_single_through_table = 1;   // a single small problem runs as a table of one (0 = never; for measurement)

bool plain_matrix(const View2& v) { return v.p != nullptr && v.s1 == 1 && v.s0 == v.d1; }

}  // namespace

// A single contraction of at most eight rows as a table of one problem, for the entries that take one problem
// and a workspace: w4a16_ride_kernel handles M = 3 .. 8 far better than the single-problem bandwidth kernel.
// Returns kTableDeclined when the call is not of that kind (the caller then uses its own kernel, which also
// produces the proper error for invalid arguments).
int64_t w4a16_table_single_workspace_bytes(int64_t M, int64_t K, int64_t N) {
  if (M <= 0 || M > kRideRows || K <= 0 || N <= 0 || K > (1 << 24) || N > (1 << 24)) return 0;
  const int sms = table_sms();
  int64_t most = 0;
  for (int group : {32, 64, 128}) {
    if (K % group) continue;
    HostProblem h{nullptr, nullptr, nullptr, nullptr, M, K, N};
    ProblemPlan plan;
    size_t offset;
    const int64_t need = table_workspace(&h, 1, group, sms > 0 ? sms : 148, &plan, &offset);
    if (need > most && plan.ride) most = need;
  }
  return most;
}

template <typename T>
int table_single(View2 x, View2 w, View2 s, View2 y, int group_size, int zero_point, void* workspace,
                 int64_t workspace_bytes, cudaStream_t stream) {
  if (!g_single_through_table || !g_table_ride) return kTableDeclined;
  if (!plain_matrix(x) || !plain_matrix(w) || !plain_matrix(s) || !plain_matrix(y)) return kTableDeclined;
  if (group_size != 32 && group_size != 64 && group_size != 128) return kTableDeclined;
  const int64_t M = x.d0, K = x.d1, N = w.d1;
  if (M < 1 || M > kRideRows || K <= 0 || K % group_size || w.d0 * 8 != K || s.d0 * group_size != K || s.d1 != N ||
      y.d0 != M || y.d1 != N || N % 8)
    return kTableDeclined;
  HostProblem h{x.p, w.p, s.p, y.p, M, K, N};
  if (validate(h, group_size) != INTENT_B200_OK) return kTableDeclined;
  const int grid = table_sms();
  if (grid <= 0) return kTableDeclined;
  ProblemPlan plan;
  size_t offset;
  const int64_t need = table_workspace(&h, 1, group_size, grid, &plan, &offset);
  if (need < 0 || !plan.ride || !workspace || workspace_bytes < need) return kTableDeclined;
  return run_table<T>(&h, 1, group_size, zero_point, workspace, workspace_bytes, stream);
}

int w4a16_table_single_f16(View2 x, View2 w, View2 s, View2 y, int g, int zp, void* ws, int64_t bytes, cudaStream_t stream) {
  return table_single<__half>(x, w, s, y, g, zp, ws, bytes, stream);
}
int w4a16_table_single_bf16(View2 x, View2 w, View2 s, View2 y, int g, int zp, void* ws, int64_t bytes, cudaStream_t stream) {
  return table_single<__nv_bfloat16>(x, w, s, y, g, zp, ws, bytes, stream);
}
}  // namespace ib200

static_assert(sizeof(intent_b200_w4a16_problem) == sizeof(ib200::HostProblem), "table entry layout");

extern "C" int64_t intent_b200_w4a16_gemv_table_workspace_bytes(const intent_b200_w4a16_problem* problems,
                                                                int32_t count, int32_t group_size) {
  using namespace ib200;
  if (!problems || count <= 0 || count > 4096) return 0;
  if (group_size != 32 && group_size != 64 && group_size != 128) return 0;
  for (int i = 0; i < count; ++i)
    if (problems[i].M > 16 || problems[i].M < 0 || problems[i].K <= 0 || problems[i].N < 0 ||
        problems[i].K > (1 << 24) || problems[i].N > (1 << 24))
      return 0;
  const int sms = table_sms();
  ProblemPlan* plans = new ProblemPlan[count];
  size_t* offsets = new size_t[count];
  // without a visible device the size is computed for the 148-SM part this library targets
  const int64_t need = table_workspace(reinterpret_cast<const HostProblem*>(problems), count, group_size,
                                       sms > 0 ? sms : 148, plans, offsets);
  delete[] plans;
  delete[] offsets;
  return need < 0 ? 0 : need;
}

extern "C" int intent_b200_w4a16_gemv_table_f16(const intent_b200_w4a16_problem* problems, int32_t count,
                                                int32_t group_size, int32_t zero_point, void* workspace,
                                                int64_t workspace_bytes, void* stream) {
  return ib200::run_table<__half>(reinterpret_cast<const ib200::HostProblem*>(problems), count, group_size, zero_point,
                                  workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int intent_b200_w4a16_gemv_table_bf16(const intent_b200_w4a16_problem* problems, int32_t count,
                                                 int32_t group_size, int32_t zero_point, void* workspace,
                                                 int64_t workspace_bytes, void* stream) {
  return ib200::run_table<__nv_bfloat16>(reinterpret_cast<const ib200::HostProblem*>(problems), count, group_size,
                                         zero_point, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" int intent_b200_w4a16_gemv_table_overlap(int32_t enable) {
  ib200::g_table_overlap = enable ? 1 : 0;
  return INTENT_B200_OK;
}

// Measurement knobs (process-global): "single" 0 = the single-problem entries never run as a table of one;
// "slots" = upper limit on the ring's slots (0 = the built-in choice); "unit_rows" 64 = the ride-along kernel
// uses units of 64 packed rows for problems of up to four rows (0 = built-in choice: 32; set it before querying
// the workspace size); "corr_mma" 1 / 0 = the ride-along kernel takes the correction sums from extra MMAs / adds
// them up from the activations, -1 = built-in choice (MMAs for three rows and more);
// "probe" 1 = every unit's arithmetic is skipped, 2 = the reduction too, 3 = only the packed weights are loaded,
// 4 / 5 = arithmetic skipped and the reduction stops after the segment sums / before the cross-CTA hand-over,
// 7 = the ride-along kernel returns at once (what its bare launch costs)
// (the results are WRONG by design for every value but 0: these launches only show where the time goes).
extern "C" int intent_b200_w4a16_gemv_table_tune(const char* knob, int32_t value) {
  if (!knob) return INTENT_B200_ERR_NULL;
  const auto is = [&](const char* name) {
    int i = 0;
    for (; name[i] && knob[i] == name[i]; ++i) {}
    return name[i] == 0 && knob[i] == 0;
  };
  if (is("single") && (value == 0 || value == 1)) {
    ib200::g_single_through_table = value;
    return INTENT_B200_OK;
  }
  if (is("unit_rows") && (value == 0 || value == 64)) {
    ib200::g_table_unit_rows = value;
    return INTENT_B200_OK;
  }
  if (is("corr_mma") && value >= -1 && value <= 1) {
    ib200::g_table_corr_mma = value;
    return INTENT_B200_OK;
  }
  if (is("slots") && (value == 0 || (value >= 8 && value <= 64))) {
    ib200::g_table_slots = value;
    return INTENT_B200_OK;
  }
  if (is("probe") && ((value >= 0 && value <= 5) || value == 7)) {
    ib200::g_table_probe = value;
    return INTENT_B200_OK;
  }
  return INTENT_B200_ERR_UNSUPPORTED;
}

extern "C" int intent_b200_w4a16_gemv_table_ride(int32_t enable) {
  ib200::g_table_ride = enable ? 1 : 0;
  return INTENT_B200_OK;
}
