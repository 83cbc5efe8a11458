// W4A16 decode GEMV / small-M GEMM as a persistent, TMA-fed bandwidth kernel.
//
//   Y[m, n] = T( sum_k f32(X[m, k]) * (q[k, n] - 8) * f32(S[k / G, n]) ),   M <= 16
//
// Program: weight_only_int4_matmul (reference kernel body
// examples/kernels/contraction/weight_only_int4.py:18-51).  The reference has no
// decode-specific lowering; this is the B200 one.
//
// Work decomposition.  The packed weight [K/8, N] is cut into units of 32
// columns x 32 packed rows (256 k) = 4 KiB, numbered tile-major (the K chunks of
// a column tile are consecutive), and the unit range is split evenly over one
// CTA per SM, so every SM streams the same number of bytes (+-1 unit).  Local
// unit j of a CTA belongs to warp j % WARPS and lands in shared-memory slot
// j % SLOTS through one 128B-swizzled TMA box on its own mbarrier.  For the
// decode shapes SLOTS covers the CTA's whole share, so every weight byte of the
// launch is requested in the first microsecond and arrives at HBM speed with no
// register staging; for larger problems a slot is refilled by the warp that owns
// it.
//
// Activations.  When M*K*2 bytes fit, the CTA stages all of X once in shared
// memory, already permuted to the nibble-pair order and pre-scaled (see
// w4a16_expand.cuh), together with the per-group correction sums.  Otherwise
// each unit carries a TMA box with its own 256 activations per row of X.
//
// Arithmetic: one lop3 per nibble pair, pairs feed mma.sync.m16n8k16 as the A
// fragment (MMA rows = weight columns), activations are the B fragment, f32
// accumulation per quantisation group starting from minus the correction sum
// (which removes the magic bias and the zero point), one FMA with the group
// scale per accumulator and group.
//
// Reduction over K: inside the MMA and the warp's registers for one unit.  Across
// units: column tiles a CTA owns whole are summed in its shared memory (per-unit
// partials [M x 32] f32, a shared ticket counter, the warp with the last ticket adds
// them in chunk order and writes Y).  A tile that is split over K between CTAs is
// first summed per CTA in shared memory the same way; each CTA then publishes ONE
// partial of the tile to global scratch, fences and takes a ticket on the tile's
// global counter, and the warp that takes the last ticket adds those two or three
// partials in CTA order and writes Y.  No CTA-wide barrier after start-up, no spin
// waits between CTAs, a fixed summation order => bitwise reproducible.
#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "tma.cuh"
#include "w4a16_expand.cuh"

namespace ib200 {
namespace {

constexpr int kUnitCols = 32;
constexpr int kUnitRows = 32;  // packed rows (8 k each)
constexpr int kUnitWeightBytes = kUnitCols * kUnitRows * 4;
constexpr int kUnitScaleBytes = 512;  // room for up to 8 groups x 32 columns of 16-bit scales
constexpr int kUnitActOffset = kUnitWeightBytes + kUnitScaleBytes;
constexpr int kSmemLimit = 227 * 1024;

struct StreamParams {
  const void* scales;
  const void* x;
  void* y;
  int M, K, N;
  int groups;      // K / G
  int chunks;      // ceil(K / 256)
  int tiles;       // ceil(N / 32)
  int units;       // tiles * chunks
  int slots;       // shared-memory slots per CTA
  int slot_bytes;  // weight unit (+ activation box), multiple of 1024
  int own_tiles;   // column tiles every CTA owns whole (reduced in shared memory); the rest is split over K
  int left_local;  // K-split tiles: a CTA first adds its own consecutive chunks of a tile in shared memory and
                   // publishes one partial per (CTA, tile); 0 = one global partial per unit
  int left_max;    // most K-split units any CTA gets (size of the shared-memory partial area)
  int left_each, left_extra;  // K-split units per CTA: the first left_extra CTAs get left_each + 1, the rest left_each
  int twos_complement;
  int overlap;
  int* status;
  int* counters;   // one ticket counter per column tile, zero between launches
  float* scratch;  // [tile][chunk][M][32] partial sums
};

// RING: 0 = every unit of the CTA has its own slot; 1 = fewer slots than units, a multiple of WARPS, each slot is
// refilled by the warp that owns it; 2 = any slot count, a refill is announced through a per-slot counter
template <typename T, int MB, int STEPS, int WARPS, bool XSTAGED, int RING>
__global__ void __launch_bounds__(WARPS * 32, 1)
w4a16_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_s,
                    const __grid_constant__ CUtensorMap map_x, const StreamParams p) {
  constexpr int THREADS = WARPS * 32;
  constexpr int RPG = 4 * STEPS;        // packed rows per quantisation group
  constexpr int GPC = kUnitRows / RPG;  // groups per unit
  constexpr int CP = 8 * MB;            // row pitch of the correction table
  extern __shared__ unsigned char smem_raw[];

  if (p.overlap) asm volatile("griddepcontrol.launch_dependents;");
  if (threadIdx.x == 0) {   // the descriptors are needed by the very first instructions that matter
    prefetch_tensormap(&map_w);
    prefetch_tensormap(&map_s);
  }

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g = lane >> 2;
  const int t = lane & 3;

  // ---- shared memory carve-up: slots | barriers | correction table | staged X ----
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t bars = base + uint32_t(p.slots) * p.slot_bytes;
  // after the barriers: one counter per slot, the number of loads issued into it so far
  const size_t corr_offset = size_t(p.slots) * p.slot_bytes + ((size_t(p.slots) * (RING == 2 ? 12 : 8) + 15) & ~size_t(15));
  volatile int* issued = reinterpret_cast<volatile int*>(base_ptr + size_t(p.slots) * p.slot_bytes + size_t(p.slots) * 8);
  float* corr = reinterpret_cast<float*>(base_ptr + corr_offset);
  uint4* xs = reinterpret_cast<uint4*>(base_ptr + corr_offset + size_t(p.groups) * CP * 4);  // [chunks*32][M]
  const uint32_t xs_addr = base + uint32_t(corr_offset) + uint32_t(p.groups) * CP * 4;
  // partial sums and ticket counters of the column tiles this CTA owns whole
  const size_t own_offset = corr_offset + size_t(p.groups) * CP * 4 + (XSTAGED ? size_t(p.chunks) * kUnitRows * p.M * 16 : 0);
  int* own_count = reinterpret_cast<int*>(base_ptr + own_offset);
  float* own_part = reinterpret_cast<float*>(base_ptr + own_offset + 256);
  // K-split units of this CTA: per-unit partials and one ticket per tile segment
  const size_t left_offset = own_offset + 256 + size_t(p.own_tiles) * p.chunks * p.M * kUnitCols * 4;
  int* left_count = reinterpret_cast<int*>(base_ptr + left_offset);
  float* left_part = reinterpret_cast<float*>(base_ptr + left_offset + 256);

  // ---- this CTA's unit range -----------------------------------------------------
  // Units of this CTA: first its share of the K-split ("left-over") column tiles, whose partial sums
  // meet in global scratch - their store/ticket round trips then overlap the rest of the stream - and
  // then every K chunk of the column tiles it owns whole, which are reduced in shared memory.
  const int grid = int(gridDim.x);
  const int left_base = p.own_tiles * int(grid) * p.chunks;   // first unit of the K-split tiles
  // quotient and remainder come from the host: no division on the way to the first load
  const int l0 = int(blockIdx.x) * p.left_each + min(int(blockIdx.x), p.left_extra);
  const int l1 = l0 + p.left_each + (int(blockIdx.x) < p.left_extra ? 1 : 0);
  const int n_left = l1 - l0;
  const int n_units = n_left + p.own_tiles * p.chunks;
  // first K-split unit of this CTA as (tile, chunk): the one division of the prologue
  const int left_first_tile = (left_base + l0) / p.chunks;
  const int left_first_chunk = (left_base + l0) - left_first_tile * p.chunks;
  auto unit_of = [&](int j, int& tile, int& chunk) {   // returns true for a unit of an owned tile
    // a CTA's units are few and consecutive: counting up replaces the divisions
    if (j < n_left) {
      tile = left_first_tile;
      chunk = left_first_chunk + j;
      while (chunk >= p.chunks) {
        chunk -= p.chunks;
        ++tile;
      }
      return false;
    }
    tile = int(blockIdx.x) * p.own_tiles;
    chunk = j - n_left;
    while (chunk >= p.chunks) {
      chunk -= p.chunks;
      ++tile;
    }
    return true;
  };
  const uint32_t x_bytes = XSTAGED ? 0u : uint32_t(p.M) * 512u;

  // without a ring every unit has its own slot: no modulo, phase 0
  auto slot_of = [&](int j) { return RING == 0 ? j : j % p.slots; };
  auto slot_addr = [&](int j) { return base + uint32_t(slot_of(j)) * p.slot_bytes; };
  auto bar_addr = [&](int j) { return bars + uint32_t(slot_of(j)) * 8u; };
  auto issue_weights = [&](int j) {
    int tile, chunk;
    unit_of(j, tile, chunk);
    mbar_expect_tx(bar_addr(j), kUnitWeightBytes + GPC * 64 + x_bytes);
    tma_load_2d(slot_addr(j), &map_w, tile * kUnitCols, chunk * kUnitRows, bar_addr(j));
    tma_load_2d(slot_addr(j) + kUnitWeightBytes, &map_s, tile * kUnitCols, chunk * GPC, bar_addr(j));
  };
  auto issue_activations = [&](int j) {
    if (!XSTAGED) {
      int tile, chunk;
      unit_of(j, tile, chunk);
      tma_load_2d(slot_addr(j) + kUnitActOffset, &map_x, chunk * 256, 0, bar_addr(j));
    }
  };

  // ---- start the weight stream before anything else ----------------------------
  // Warp w consumes local units w, w + WARPS, ...; unit j lives in slot j % slots.  The warp that
  // consumed unit j refills the slot with unit j + slots and bumps the slot's issue counter; the
  // consumer of that unit (any warp) looks at the counter before it waits on the barrier, so a
  // barrier is never polled two phases ahead and the slot count need not be a multiple of WARPS.
  const int first_wave = min(n_units, p.slots);
  if (lane == 0) {
    for (int s = warp; s < p.slots; s += WARPS) {
      mbar_init(bars + uint32_t(s) * 8u, 1);
      if (RING == 2) issued[s] = 1;
    }
    fence_mbar_init();
    for (int j = warp; j < first_wave; j += WARPS) issue_weights(j);
  }
  if (p.overlap) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (lane == 0)
    for (int j = warp; j < first_wave; j += WARPS) issue_activations(j);

  // ---- while the loads fly: correction sums (and the staged activations) -----------
  {
    // corr[group][m] = - sum over the group's k of x[m,k] * (bias_k + 8); rows of one group sit
    // in RPG adjacent lanes and are added by a fixed-order butterfly.
    const uint4* xg = reinterpret_cast<const uint4*>(p.x);
    const int k8 = p.K >> 3;
    const bool all_chunks = XSTAGED || p.own_tiles > 0 || p.left_local != 0;
    const int touched = all_chunks ? p.chunks : min(p.chunks, n_left);
    const int rows = touched * kUnitRows;
    const int total = rows * p.M;
    // four items per thread and pass: their loads are issued together, so the passes (M times as many
    // as for one activation row) do not each pay a full memory latency
    constexpr int BATCH = 4;
    for (int start = 0; start < total; start += THREADS * BATCH) {
      uint4 v[BATCH];
      int ms[BATCH], row_of_item[BATCH];
      bool in_range[BATCH], active[BATCH];
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        const int i = start + b * THREADS + tid;
        in_range[b] = i < total;
        ms[b] = 0;
        row_of_item[b] = 0;
        if (in_range[b]) {
          ms[b] = i / rows;
          const int lr = i - ms[b] * rows;
          const int chunk = all_chunks ? lr / kUnitRows : (left_base + l0 + lr / kUnitRows) % p.chunks;
          row_of_item[b] = chunk * kUnitRows + (lr % kUnitRows);
        }
        active[b] = in_range[b] && row_of_item[b] < k8;
        v[b] = active[b] ? xg[size_t(ms[b]) * k8 + row_of_item[b]] : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int b = 0; b < BATCH; ++b) {
        const int m = ms[b], row = row_of_item[b];
        float partial = 0.f;
        uint4 o = make_uint4(0, 0, 0, 0);  // rows past K/8 (last chunk) are staged as zeros
        if (active[b]) {
          o.x = prmt(v[b].x, v[b].z, 0x5410);                        // (k0, k4)
          o.y = Expand<T>::scale_odd(prmt(v[b].x, v[b].z, 0x7632));  // (k1, k5)
          o.z = prmt(v[b].y, v[b].w, 0x5410);                        // (k2, k6)
          o.w = Expand<T>::scale_odd(prmt(v[b].y, v[b].w, 0x7632));  // (k3, k7)
          partial = Expand<T>::kEven * (pair_sum<T>(o.x) + pair_sum<T>(o.z)) +
                    Expand<T>::kOdd * (pair_sum<T>(o.y) + pair_sum<T>(o.w));
        }
        if (XSTAGED && in_range[b]) xs[row * p.M + m] = o;
#pragma unroll
        for (int d = RPG / 2; d >= 1; d >>= 1) partial += __shfl_xor_sync(0xffffffffu, partial, d);
        if (active[b] && (row % RPG) == 0) corr[(row / RPG) * CP + m] = -partial;
      }
    }
  }
  for (int i = tid; i < p.own_tiles; i += THREADS) own_count[i] = 0;
  if (p.left_local && tid < 64) left_count[tid] = 0;
  __syncthreads();

  uint32_t magic_a, magic_b;
  Expand<T>::magic(p.twos_complement != 0, magic_a, magic_b);
  uint16_t* y = reinterpret_cast<uint16_t*>(p.y);
  const int part = p.M * kUnitCols;  // floats per unit partial

  // byte offset of this lane's 16-byte word inside a unit, per load step: rows 2t + parity keep
  // the eight lanes of a quarter-warp on distinct swizzled bank groups
  int row_of[STEPS];
  uint32_t off_of[STEPS];
#pragma unroll
  for (int i = 0; i < STEPS; ++i) {
    row_of[i] = STEPS >= 2 ? 8 * (i >> 1) + 2 * t + (i & 1) : t;
    off_of[i] = uint32_t(row_of[i]) * 128u + (uint32_t(g ^ (row_of[i] & 7)) << 4);
  }

  for (int j = warp; j < n_units; j += WARPS) {
    int tile, chunk;
    const bool owned = unit_of(j, tile, chunk);
    if (RING == 2 && j >= p.slots) {  // a refilled slot: wait (bounded) until the refill has been issued
      const int need = j / p.slots + 1;
      for (int spin = 0; spin < (1 << 22) && issued[j % p.slots] < need; ++spin) __nanosleep(20);
      __threadfence_block();
    }
    if (!__all_sync(0xffffffffu, mbar_wait(bar_addr(j), RING == 0 ? 0 : (j / p.slots) & 1))) {
      if (lane == 0) atomicExch(p.status, INTENT_B200_ERR_TIMEOUT);  // this unit's loads never completed
      break;
    }
    const uint32_t wslot = slot_addr(j);
    float facc[MB][8];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int i = 0; i < 8; ++i) facc[mb][i] = 0.f;

#pragma unroll
    for (int gi = 0; gi < GPC; ++gi) {
      const int group = chunk * GPC + gi;
      float gacc[MB][8];
#pragma unroll
      for (int mb = 0; mb < MB; ++mb) {
        // rows m = 8*mb + 2t and + 1 start from minus their correction sum
        float2 c = make_float2(0.f, 0.f);
        if (group < p.groups) c = *reinterpret_cast<const float2*>(&corr[group * CP + mb * 8 + 2 * t]);
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
          uint4 b = make_uint4(0, 0, 0, 0);
          const int m = mb * 8 + g;
          if (m < p.M) {
            if (XSTAGED) {
              b = lds128(xs_addr + uint32_t((chunk * kUnitRows + row) * p.M + m) * 16u);
            } else {
              const uint4 v = lds128(wslot + kUnitActOffset + m * 512 + row * 16);
              b.x = prmt(v.x, v.z, 0x5410);
              b.y = Expand<T>::scale_odd(prmt(v.x, v.z, 0x7632));
              b.z = prmt(v.y, v.w, 0x5410);
              b.w = Expand<T>::scale_odd(prmt(v.y, v.w, 0x7632));
            }
          }
          float(&a01)[4] = *reinterpret_cast<float(*)[4]>(&gacc[mb][0]);
          float(&a23)[4] = *reinterpret_cast<float(*)[4]>(&gacc[mb][4]);
          Elem<T>::mma16816(a01, c0[0], c1[0], c0[1], c1[1], b.x, b.y);
          Elem<T>::mma16816(a23, c2[0], c3[0], c2[1], c3[1], b.x, b.y);
          Elem<T>::mma16816(a01, c0[2], c1[2], c0[3], c1[3], b.z, b.w);
          Elem<T>::mma16816(a23, c2[2], c3[2], c2[3], c3[3], b.z, b.w);
        }
      }
      uint2 s;  // this lane's four column scales of the group (zero outside the matrix)
      asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(s.x), "=r"(s.y) : "r"(wslot + kUnitWeightBytes + gi * 64 + g * 8));
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
    if (RING != 0 && j + p.slots < n_units) {  // refill this slot with the unit that maps to it next
      __syncwarp();
      fence_proxy_async();
      if (lane == 0) {
        issue_weights(j + p.slots);
        issue_activations(j + p.slots);
        if (RING == 2) {
          __threadfence_block();
          issued[j % p.slots] = (j + p.slots) / p.slots + 1;
        }
      }
    }

    // ---- the unit's partial is stored; the last ticket of its group of partials finishes the group ----
    // accumulator element (mb, i): row m = 8*mb + 2t + (i & 1), column 4g + (i >> 1)
    // Three kinds of group: an owned tile (all chunks in this CTA, shared memory), a segment (this CTA's
    // consecutive chunks of a K-split tile, shared memory; its sum becomes ONE global partial of the tile),
    // and, without left_local, the K-split tile itself with one global partial per unit.
    const int tile_local = tile - int(blockIdx.x) * p.own_tiles;
    const bool segment = !owned && p.left_local != 0;
    int seg = 0, seg_first = 0, seg_len = p.chunks;     // segment: index in this CTA, first local unit, units
    if (segment) {
      const int first_tile = (left_base + l0) / p.chunks;
      seg = tile - first_tile;
      const int begin = max(tile * p.chunks, left_base + l0), end = min((tile + 1) * p.chunks, left_base + l1);
      seg_first = begin - (left_base + l0);
      seg_len = end - begin;
    }
    float* mine = owned     ? own_part + (size_t(tile_local) * p.chunks + chunk) * part
                  : segment ? left_part + size_t(j) * part
                            : p.scratch + (size_t(tile) * p.chunks + chunk) * part;
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int m = mb * 8 + 2 * t + hh;
        if (m < p.M)
          *reinterpret_cast<float4*>(mine + m * kUnitCols + 4 * g) =
              make_float4(facc[mb][0 + hh], facc[mb][2 + hh], facc[mb][4 + hh], facc[mb][6 + hh]);
      }
    // One ticket per unit.  Shared-memory groups: block-scope fences around a shared counter.  Global
    // partials: one acq_rel atomic (the warp barrier orders every lane's stores before lane 0's release;
    // the acquire side covers the reads of the last arriver).
    __syncwarp();
    int last = 0;
    if (lane == 0) {
      int old;
      if (owned || segment) {
        __threadfence_block();
        old = atomicAdd(owned ? own_count + tile_local : left_count + seg, 1);
        last = old == seg_len - 1;
      } else {
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + tile) : "memory");
        last = old == p.chunks - 1;
      }
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) continue;
    if (owned || segment) __threadfence_block();

    // lane = 8*q + v: quarter q adds partials q, q+4, ... for columns 4v..4v+3 (four loads in flight at
    // a time), then the four quarters are added in a fixed order: bitwise reproducible
    const int q = lane >> 3, v = lane & 7;
    auto sum_partials = [&](const float* first, int count, bool global, int m) {
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c = q; c < count; c += 16) {
        float4 a[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int cc = c + 4 * u;
          a[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (cc < count) {
            const float4* src = reinterpret_cast<const float4*>(first + size_t(cc) * part + m * kUnitCols + 4 * v);
            a[u] = global ? __ldcg(src) : *src;
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          sum.x += a[u].x; sum.y += a[u].y; sum.z += a[u].z; sum.w += a[u].w;
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
    auto write_row = [&](int m, float4 sum) {
      const int n = tile * kUnitCols + 4 * v;
      if (q == 0 && n < p.N) {  // N is a multiple of 8, so the four columns are inside together
        uint2 out;
        out.x = uint32_t(Elem<T>::from_float(sum.x)) | (uint32_t(Elem<T>::from_float(sum.y)) << 16);
        out.y = uint32_t(Elem<T>::from_float(sum.z)) | (uint32_t(Elem<T>::from_float(sum.w)) << 16);
        *reinterpret_cast<uint2*>(y + size_t(m) * p.N + n) = out;
      }
    };

    if (owned || (segment && seg_len == p.chunks)) {
      // every chunk of the tile was added here: the sum is the result
      const float* first = owned ? own_part + size_t(tile_local) * p.chunks * part : left_part + size_t(seg_first) * part;
      for (int m = 0; m < p.M; ++m) write_row(m, sum_partials(first, p.chunks, false, m));
    } else if (segment) {
      // publish the segment's sum as partial number (this CTA - first CTA of the tile) of the tile, then
      // take the tile's global ticket; the CTA that takes the last one adds the tile's few partials
      auto cta_of = [&](int left_unit) {   // the CTA whose K-split range holds this unit
        const int boundary = p.left_extra * (p.left_each + 1);
        return left_unit < boundary ? left_unit / (p.left_each + 1)
                                    : p.left_extra + (left_unit - boundary) / p.left_each;   // left_each > 0 here
      };
      const int tile_begin = tile * p.chunks - left_base;
      const int first_cta = cta_of(tile_begin), last_cta = cta_of(tile_begin + p.chunks - 1);
      float* slot = p.scratch + (size_t(tile) * p.chunks + (int(blockIdx.x) - first_cta)) * part;
      for (int m = 0; m < p.M; ++m) {
        const float4 sum = sum_partials(left_part + size_t(seg_first) * part, seg_len, false, m);
        if (q == 0) *reinterpret_cast<float4*>(slot + m * kUnitCols + 4 * v) = sum;
      }
      __syncwarp();
      int final_one = 0;
      if (lane == 0) {
        int old;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(p.counters + tile) : "memory");
        final_one = old == last_cta - first_cta;
      }
      final_one = __shfl_sync(0xffffffffu, final_one, 0);
      if (final_one) {
        const float* first = p.scratch + size_t(tile) * p.chunks * part;
        for (int m = 0; m < p.M; ++m) write_row(m, sum_partials(first, last_cta - first_cta + 1, true, m));
        if (lane == 0) p.counters[tile] = 0;  // ready for the next launch
      }
    } else {
      const float* first = p.scratch + size_t(tile) * p.chunks * part;
      for (int m = 0; m < p.M; ++m) write_row(m, sum_partials(first, p.chunks, true, m));
      if (lane == 0) p.counters[tile] = 0;  // ready for the next launch
    }
  }
}

struct Plan {
  int grid, slots, slot_bytes, warps, tiles, chunks, units, own_tiles, left_max;
  bool staged, left_local;
  int ring;   // 0 none, 1 slots refilled by their owner warp, 2 refills announced per slot
  size_t smem_bytes, counters_offset, scratch_offset, workspace_bytes;
};

// Launch geometry and workspace layout for one problem size (pure arithmetic).
bool make_plan(int M, int K, int N, int mb, int sms, int warps_override, Plan* plan) {
  Plan q{};
  q.tiles = (N + kUnitCols - 1) / kUnitCols;
  q.chunks = (K / 8 + kUnitRows - 1) / kUnitRows;
  q.units = q.tiles * q.chunks;
  q.grid = q.units < sms ? q.units : sms;
  q.warps = warps_override ? warps_override : (mb == 1 ? 32 : 16);
  // Candidate layouts: activations staged whole in shared memory or riding with every unit; column tiles
  // owned whole by a CTA or every tile split over K.  The layout that keeps the largest share of a CTA's
  // units in flight wins, with a bonus for staged activations and for owned tiles.
  const size_t x_bytes = size_t(M) * q.chunks * kUnitRows * 16;  // staged rows are padded to whole chunks
  int own_candidate = q.tiles / q.grid;
  if (own_candidate > 64 || size_t(own_candidate) * q.chunks * M * kUnitCols * 4 > 32 * 1024) own_candidate = 0;
  const int wanted_warps = q.warps;
  double best_score = -1.0;
  size_t fixed = 0;
  Plan best{};
  for (int staged = 1; staged >= 0; --staged) {
    if (staged && x_bytes > 96 * 1024) continue;
    for (int pass = 0; pass < 2; ++pass) {
      if (pass == 1 && own_candidate == 0) break;
      Plan c = q;
      c.staged = staged != 0;
      c.own_tiles = pass == 0 ? own_candidate : 0;
      c.warps = wanted_warps;
      const int left_units = c.units - c.own_tiles * c.grid * c.chunks;
      c.left_max = (left_units + c.grid - 1) / c.grid;
      const int per_cta_max = c.own_tiles * c.chunks + c.left_max;
      // K-split tiles: a CTA adds its own chunks of a tile in shared memory first (only when every CTA gets
      // at least one K-split unit - the CTAs that share a tile are then consecutive -, at most 64 tile
      // segments per CTA, and the per-unit partials must stay small next to the weight slots)
      const size_t left_bytes = 256 + size_t(c.left_max) * M * kUnitCols * 4;
      c.left_local = left_units >= c.grid && (c.left_max + c.chunks - 1) / c.chunks + 1 <= 64 && left_bytes <= 56 * 1024;
      c.slot_bytes = ((kUnitActOffset + (c.staged ? 0 : M * 512) + 1023) / 1024) * 1024;
      const size_t f = 1024 + 32 + size_t((K + 31) / 32) * 8 * mb * 4 + (c.staged ? x_bytes : 0) + 256 + 16 +
                       size_t(c.own_tiles) * c.chunks * M * kUnitCols * 4 + (c.left_local ? left_bytes : 0);
      if (size_t(kSmemLimit) <= f) continue;
      const long long capacity = (long long)(size_t(kSmemLimit) - f) / (c.slot_bytes + 12);
      if (capacity >= per_cta_max) {
        c.ring = 0;
        c.slots = per_cta_max;
      } else {
        if (capacity < c.warps && c.warps == 32) c.warps = 16;
        if (capacity < c.warps) continue;
        // at least one and a half slots per warp: keep them all and announce refills per slot; otherwise
        // whole rounds of the warps, every slot refilled by its owner
        c.ring = capacity * 2 >= c.warps * 3 && capacity % c.warps != 0 ? 2 : 1;
        c.slots = int(c.ring == 2 ? capacity : capacity / c.warps * c.warps);
      }
      // staged activations save a shuffle and a multiply per load in the inner loop: worth a quarter of the
      // CTA's units in flight; owned tiles skip the global ticket chain
      const double score = double(c.slots) / double(per_cta_max) + (c.staged ? 0.25 : 0.0) + (c.own_tiles > 0 ? 0.05 : 0.0);
      if (score > best_score) {
        best_score = score;
        best = c;
        fixed = f;
      }
    }
  }
  if (best_score < 0.0) return false;
  q = best;
  q.smem_bytes = fixed + size_t(q.slots) * (q.slot_bytes + 12);
  q.counters_offset = 256;
  q.scratch_offset = ((q.counters_offset + size_t(q.tiles) * 4 + 255) / 256) * 256;
  q.workspace_bytes = q.scratch_offset + size_t(q.units) * M * kUnitCols * 4;
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
int g_warps_override = 0;

template <typename T, int MB, int STEPS, int WARPS, bool XSTAGED, int RING>
int launch_kernel(const CUtensorMap& map_w, const CUtensorMap& map_s, const CUtensorMap& map_x, const StreamParams& p, const Plan& plan,
                  cudaStream_t stream) {
  auto kernel = w4a16_stream_kernel<T, MB, STEPS, WARPS, XSTAGED, RING>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(plan.smem_bytes));
  if (e != cudaSuccess) return cuda_status(e);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(plan.grid, 1, 1);
  config.blockDim = dim3(WARPS * 32, 1, 1);
  config.dynamicSmemBytes = plan.smem_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = p.overlap ? 1 : 0;
  if (LaunchFacts* sink = observe_sink())
    return record_launch(sink, reinterpret_cast<const void*>(kernel),
                         XSTAGED ? (RING ? "w4a16_stream_kernel staged activations, slot ring" : "w4a16_stream_kernel staged activations")
                                 : (RING ? "w4a16_stream_kernel activations per unit, slot ring" : "w4a16_stream_kernel activations per unit"),
                         plan.grid, WARPS * 32, int(plan.smem_bytes), 1);
  e = cudaLaunchKernelEx(&config, kernel, map_w, map_s, map_x, p);
  if (e != cudaSuccess) return cuda_status(e);
  note_launch();
  return launch_status();
}

template <typename T, int MB, int STEPS, int WARPS, bool XSTAGED>
int launch_ring(const CUtensorMap& map_w, const CUtensorMap& map_s, const CUtensorMap& map_x, const StreamParams& p,
                const Plan& plan, cudaStream_t stream) {
  if (plan.ring == 0) return launch_kernel<T, MB, STEPS, WARPS, XSTAGED, 0>(map_w, map_s, map_x, p, plan, stream);
  if (plan.ring == 1) return launch_kernel<T, MB, STEPS, WARPS, XSTAGED, 1>(map_w, map_s, map_x, p, plan, stream);
  return launch_kernel<T, MB, STEPS, WARPS, XSTAGED, 2>(map_w, map_s, map_x, p, plan, stream);
}

template <typename T, int MB, int STEPS, int WARPS>
int launch_warps(const CUtensorMap& map_w, const CUtensorMap& map_s, const CUtensorMap& map_x, const StreamParams& p,
                 const Plan& plan, cudaStream_t stream) {
  if (plan.staged) return launch_ring<T, MB, STEPS, WARPS, true>(map_w, map_s, map_x, p, plan, stream);
  return launch_ring<T, MB, STEPS, WARPS, false>(map_w, map_s, map_x, p, plan, stream);
}

template <typename T, int MB, int STEPS>
int launch(const CUtensorMap& map_w, const CUtensorMap& map_s, const CUtensorMap& map_x, const StreamParams& p, const Plan& plan,
           cudaStream_t stream) {
  if (MB == 1 && plan.warps == 32) return launch_warps<T, 1, STEPS, 32>(map_w, map_s, map_x, p, plan, stream);
  return launch_warps<T, MB, STEPS, 16>(map_w, map_s, map_x, p, plan, stream);
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
  if (K == 0 || N % 8 != 0 || M > 16 || K > (1 << 24) || N > (1 << 24)) return INTENT_B200_ERR_UNSUPPORTED;
  const int mb = M <= 8 ? 1 : 2;
  const int sms = g_grid_override > 0 ? g_grid_override : device_sms();
  if (sms <= 0) return INTENT_B200_ERR_UNSUPPORTED;
  Plan plan;
  if (!make_plan(int(M), int(K), int(N), mb, sms, mb == 1 ? g_warps_override : 0, &plan))
    return INTENT_B200_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < int64_t(plan.workspace_bytes) || !aligned16(workspace))
    return INTENT_B200_ERR_WORKSPACE;

  CUtensorMap map_w, map_x;
  if (!make_tensor_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_INT32, w.p, uint64_t(K / 8), uint64_t(N), uint64_t(N) * 4,
                          kUnitRows, kUnitCols, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B))
    return INTENT_B200_ERR_UNSUPPORTED;
  const CUtensorMapDataType xt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  CUtensorMap map_s;
  if (!make_tensor_map_2d(&map_s, xt, s.p, uint64_t(K / group_size), uint64_t(N), uint64_t(N) * 2,
                          uint32_t(256 / group_size), kUnitCols, CU_TENSOR_MAP_SWIZZLE_NONE))
    return INTENT_B200_ERR_UNSUPPORTED;
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
  p.slots = plan.slots;
  p.slot_bytes = plan.slot_bytes;
  p.own_tiles = plan.own_tiles;
  p.left_local = plan.left_local ? 1 : 0;
  p.left_max = plan.left_max;
  {
    const int left_units = plan.units - plan.own_tiles * plan.grid * plan.chunks;
    p.left_each = left_units / plan.grid;
    p.left_extra = left_units % plan.grid;
  }
  p.twos_complement = zero_point == -1 ? 1 : 0;
  p.overlap = g_overlap;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  p.status = reinterpret_cast<int*>(ws);
  p.counters = reinterpret_cast<int*>(ws + plan.counters_offset);
  p.scratch = reinterpret_cast<float*>(ws + plan.scratch_offset);

  const int steps = group_size / 32;
#define IB200_STREAM_MB(MB_)                                                 \
  if (mb == MB_) {                                                           \
    if (steps == 4) return launch<T, MB_, 4>(map_w, map_s, map_x, p, plan, stream); \
    if (steps == 2) return launch<T, MB_, 2>(map_w, map_s, map_x, p, plan, stream); \
    return launch<T, MB_, 1>(map_w, map_s, map_x, p, plan, stream);                 \
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
  // without a visible device the size is computed for the 148-SM part this library targets
  if (!make_plan(int(M), int(K), int(N), mb, sms > 0 ? sms : 148, mb == 1 ? g_warps_override : 0, &plan)) return 0;
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
  if (warps != 0 && warps != 16 && warps != 32) return INTENT_B200_ERR_UNSUPPORTED;
  ib200::g_warps_override = warps;
  return INTENT_B200_OK;
}

// Reads the status word at the head of a bandwidth-kernel workspace after synchronising `stream`.  When a
// launch gave up on a bounded wait its warps stopped early: tickets were left untaken and parts of Y
// unwritten, so the workspace is no longer zero-filled.  In that case the whole workspace is cleared
// again (and the stream synchronised once more) before the code is returned, so the next launch starts
// from a clean one.
static int take_workspace_status(void* workspace, int64_t bytes, cudaStream_t stream) {
  if (!workspace || bytes < 4) return INTENT_B200_ERR_WORKSPACE;
  cudaError_t e = cudaStreamSynchronize(stream);
  if (e != cudaSuccess) return ib200::cuda_status(e);
  int value = 0;
  e = cudaMemcpy(&value, workspace, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return ib200::cuda_status(e);
  if (value != 0) {
    e = cudaMemsetAsync(workspace, 0, size_t(bytes), stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return ib200::cuda_status(e);
  }
  return value;
}

extern "C" int intent_b200_w4a16_gemv_workspace_status(void* workspace, int64_t workspace_bytes, void* stream) {
  return take_workspace_status(workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------------------------
// Entry point that performs no allocation at all.
//
// Some hosts cannot hand this library a workspace: a serving loop that has frozen its
// memory pool, a plugin interface that passes only the operator's inputs and outputs, or
// code that runs between cudaStreamBeginCapture and EndCapture, where cudaMalloc is not
// permitted.  For them the scratch of the bandwidth kernel lives in the library image
// itself: a fixed device array that every GPU loading the library holds until the
// process exits.
// ---------------------------------------------------------------------------------
namespace ib200 {

constexpr size_t kBuiltinScratchBytes = size_t(8) << 20;  // 8 MiB: the decode shapes up to M = 8
static __device__ __align__(256) unsigned char g_builtin_scratch[kBuiltinScratchBytes];

// In host code `g_builtin_scratch` is only a handle for the symbol, not an address a kernel
// could use; the device address is looked up once per device (with that device current).
static int builtin_scratch_address(void** address) {
  static std::mutex lock;
  static void* per_device[64] = {};
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return cuda_status(e);
  if (device < 0 || device >= 64) return INTENT_B200_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> guard(lock);
  if (!per_device[device]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_builtin_scratch);
    if (e != cudaSuccess) return cuda_status(e);
    if (!p) return INTENT_B200_ERR_NULL;
    per_device[device] = p;
  }
  *address = per_device[device];
  return INTENT_B200_OK;
}

}  // namespace ib200

// Status of the latest call of the no-allocation entry on the current device (see the header): must be read
// before the next call of that entry, which clears the word.
extern "C" int intent_b200_w4a16_gemv_builtin_scratch_status(void* stream) {
  void* scratch = nullptr;
  const int status = ib200::builtin_scratch_address(&scratch);
  if (status != INTENT_B200_OK) return status;
  return take_workspace_status(scratch, int64_t(ib200::kBuiltinScratchBytes), static_cast<cudaStream_t>(stream));
}

extern "C" int intent_b200_w4a16_gemv_f16_builtin_scratch(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                          INTENT_B200_VIEW2(a2), INTENT_B200_VIEW2(a3),
                                                          int32_t group_size, int32_t zero_point, void* stream) {
  using namespace ib200;
  const int64_t M = a0_d0, K = a0_d1, N = a1_d1;
  if (M == 0 || N == 0) return INTENT_B200_OK;
  if (M < 0 || M > 16 || K <= 0 || N < 0 || K > (1 << 24) || N > (1 << 24)) return INTENT_B200_ERR_UNSUPPORTED;
  const int sms = g_grid_override > 0 ? g_grid_override : device_sms();
  Plan plan;
  if (sms <= 0 || !make_plan(int(M), int(K), int(N), M <= 8 ? 1 : 2, sms, M <= 8 ? g_warps_override : 0, &plan))
    return INTENT_B200_ERR_UNSUPPORTED;
  if (plan.workspace_bytes > kBuiltinScratchBytes) return INTENT_B200_ERR_SCRATCH_LIMIT;
  void* scratch = nullptr;
  int status = builtin_scratch_address(&scratch);
  if (status != INTENT_B200_OK) return status;
  // The array keeps whatever the previous call left: the status word and the ticket counters
  // must start at zero, the partial sums behind them are overwritten before they are read.
  cudaError_t e = cudaMemsetAsync(scratch, 0, plan.scratch_offset, static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return cuda_status(e);
  return w4a16_stream_f16(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2), IB200_VIEW2_ARG(a3),
                          group_size, zero_point, scratch, int64_t(kBuiltinScratchBytes),
                          static_cast<cudaStream_t>(stream));
}
