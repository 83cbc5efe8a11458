// W4A16 prefill GEMM on CTA pairs (tcgen05 cta_group::2): the large-M form of w4a16_gemm.cu.
//
//   Y[m, n] = T( sum_k f32(X[m, k]) * f32( T( (q[k, n] - 8) * S[k / G, n] ) ) )
//
// Program: weight_only_int4_matmul, reference kernel body
// examples/kernels/contraction/weight_only_int4.py:18-51.
//
// Two CTAs on neighbouring SMs (a cluster of 2) compute one 512 x 256 output tile.  Each CTA
// owns 256 rows of it (two 128-row blocks, accumulated in its own TMEM: 2 x 256 columns) and
// dequantises HALF of the tile's weight columns (128 of 256) into its shared memory; every
// tcgen05.mma (M 256 across the pair, N 256, K 16) reads the A rows and the B columns of both
// CTAs.  Per flop each CTA therefore expands a quarter of the int4 weights that a lone
// 128 x 256 CTA would, which is what bounded the single-CTA kernel.
//
// Roles per CTA (22 warps): warp 0 TMA producer (its own rows of X; the transaction bytes of
// both CTAs complete on the leader's mbarrier), warps 6..21 dequantisers (thread = weight column
// x half of the k block; packed words straight from global memory, three k blocks ahead), warps
// 2..5 epilogue (own TMEM lanes).  Only the leader CTA (cluster rank 0) issues MMAs (one thread
// of warp 1); its commits arrive on the stage barriers of both CTAs.
// No TMA load here is a multicast load.  Every wait is bounded (tma.cuh).
#include <type_traits>

#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace ib200 {

// Status word of this translation unit's kernel (device variables are private to the file they are
// defined in unless the library is built with relocatable device code, which it is not); read and
// cleared by w4a16_gemm_pair_take_status below.
__device__ int g_w4a16_pair_status = 0;

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int MT = 2;                       // 128-row blocks per CTA
constexpr int PAIR_ROWS = 2 * MT * BM;      // 512
constexpr int A_BYTES = BM * BK * 2;        // one 128-row box of X
constexpr int B_HALF_BYTES = (BN / 2) * BK * 2;  // this CTA's half of the operand tile, 16 KiB
constexpr int A_STAGES = 3, B_STAGES = 4;
constexpr int DEQUANT_WARPS = 16;
constexpr int DQ_PARTS = DEQUANT_WARPS * 32 / (BN / 2);  // threads per weight column (4)
constexpr int DQ_ROWS = (BK / 8) / DQ_PARTS;             // packed words per thread and k block (2)
constexpr int THREADS = (6 + DEQUANT_WARPS) * 32;
constexpr int SMEM_BYTES = 1024 + A_STAGES * MT * A_BYTES + B_STAGES * B_HALF_BYTES + 256;
constexpr int BAND_TILES = 4;               // 512-row tiles per band of the tile walk

struct PairParams {
  void* y;
  const uint32_t* packed;
  const uint16_t* scales;
  int M, K, N;
  int k_blocks, m_tiles, n_tiles;
  int group_size, twos_complement;
  int prelaid;      // packed points at the tiled copy (w4a16_prelayout.cu) instead of the [K/8, N] matrix
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  return remote;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// plain (non-multicast) 2-D tiled load of a CTA pair: data to this CTA, bytes complete on `cluster_bar`
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int c0, int c1,
                                                 uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(cluster_bar)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                              bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u, zero = 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc), "r"(zero)
      : "memory");
}
// arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued
// so far have completed
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask)
               : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(columns)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t tmem_base, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(columns) : "memory");
}

__device__ __forceinline__ void pair_tile_coords(int tile, int m_tiles, int n_tiles, int& m_tile, int& n_tile) {
  const int band_size = BAND_TILES * n_tiles;
  const int band = tile / band_size;
  const int in_band = tile - band * band_size;
  const int rows_in_band = min(BAND_TILES, m_tiles - band * BAND_TILES);
  n_tile = in_band / rows_in_band;
  m_tile = band * BAND_TILES + (in_band - n_tile * rows_in_band);
}

template <typename T>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
w4a16_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const PairParams p) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t smem_a = base;
  const uint32_t smem_b = smem_a + A_STAGES * MT * A_BYTES;
  const uint32_t bars = smem_b + B_STAGES * B_HALF_BYTES;
  const uint32_t full_a = bars;                        // leader: X of both CTAs landed
  const uint32_t empty_a = full_a + 8 * A_STAGES;      // each CTA: MMAs done with the stage
  const uint32_t full_b = empty_a + 8 * A_STAGES;      // leader: both halves of the operand tile written
  const uint32_t empty_b = full_b + 8 * B_STAGES;      // each CTA: MMAs done with it
  const uint32_t tmem_full = empty_b + 8 * B_STAGES;   // each CTA: accumulators complete
  const uint32_t tmem_empty = tmem_full + 8;           // leader: accumulators of both CTAs drained
  const uint32_t tmem_slot = tmem_empty + 8;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + (tmem_slot - base));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t rank = cluster_rank();
  const int pair = int(blockIdx.x) >> 1, pairs = int(gridDim.x) >> 1;
  const int tiles = p.m_tiles * p.n_tiles;

  if (tid == 0) {
    for (int s = 0; s < A_STAGES; ++s) {
      mbar_init(full_a + 8 * s, 1);
      mbar_init(empty_a + 8 * s, 1);
    }
    for (int s = 0; s < B_STAGES; ++s) {
      // leader: its own dequantiser warps + one relayed arrival for the peer's; peer: its own warps
      mbar_init(full_b + 8 * s, rank == 0 ? DEQUANT_WARPS + 1 : DEQUANT_WARPS);
      mbar_init(empty_b + 8 * s, 1);
    }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, 8);
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, 512);
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync();   // barriers of both CTAs are initialised before anything arrives remotely
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs) {
        int m_tile, n_tile;
        pair_tile_coords(tile, p.m_tiles, p.n_tiles, m_tile, n_tile);
        const int row0 = m_tile * PAIR_ROWS + int(rank) * (MT * BM);
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % A_STAGES;
          if (!mbar_wait(empty_a + 8 * s, ((it / A_STAGES) & 1) ^ 1)) { ok = false; break; }
          if (rank == 0) mbar_expect_tx(full_a + 8 * s, 2 * MT * A_BYTES);
          const uint32_t leader_bar = map_to_rank(full_a + 8 * s, 0);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            tma_load_2d_pair(smem_a + (s * MT + mt) * A_BYTES, &map_x, kb * BK, row0 + mt * BM, leader_bar);
        }
      }
      if (!ok) atomicExch(&g_w4a16_pair_status, INTENT_B200_ERR_TIMEOUT);
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer (leader CTA only) --------------------------
    if (lane == 0 && rank != 0) {
      // Peer CTA: relay "my half of operand tile t is written" to the leader with one cluster-scope
      // arrival per k block (the dequantiser warps themselves only synchronise inside their CTA).
      const int my_tiles = tiles > pair ? (tiles - pair + pairs - 1) / pairs : 0;
      const uint32_t total = uint32_t(my_tiles) * uint32_t(p.k_blocks);
      const uint32_t leader_full_b = map_to_rank(full_b, 0);
      bool ok = true;
      for (uint32_t it = 0; it < total; ++it) {
        const uint32_t t = it % B_STAGES;
        if (!mbar_wait(full_b + 8 * t, (it / B_STAGES) & 1)) { ok = false; break; }
        mbar_arrive_cluster(leader_full_b + 8 * t);
      }
      if (!ok) atomicExch(&g_w4a16_pair_status, INTENT_B200_ERR_TIMEOUT);
    }
    if (lane == 0 && rank == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc = umma_idesc(1, fmt, fmt, 0, 0, 2 * BM, BN);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = pair; tile < tiles && ok; tile += pairs, ++local) {
        if (!mbar_wait(tmem_empty, (local & 1) ^ 1)) { ok = false; break; }
        tcgen05_fence_after();
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % A_STAGES, t = it % B_STAGES;
          if (!mbar_wait(full_a + 8 * s, (it / A_STAGES) & 1) ||
              !mbar_wait(full_b + 8 * t, (it / B_STAGES) & 1)) { ok = false; break; }
          tcgen05_fence_after();
          const uint64_t desc_b = umma_desc_k_major_sw128(smem_b + t * B_HALF_BYTES);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint64_t desc_a = umma_desc_k_major_sw128(smem_a + (s * MT + mt) * A_BYTES);
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
              umma_f16_pair(tmem_base + mt * BN, desc_a + uint64_t(2 * kk), desc_b + uint64_t(2 * kk), idesc,
                            (kb | kk) != 0);
          }
          umma_commit_pair(empty_a + 8 * s);
          umma_commit_pair(empty_b + 8 * t);
        }
        if (ok) umma_commit_pair(tmem_full);
      }
      if (!ok) atomicExch(&g_w4a16_pair_status, INTENT_B200_ERR_TIMEOUT);
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue (both CTAs, own TMEM) -------------------------
    const int quadrant = warp & 3;
    uint16_t* y = reinterpret_cast<uint16_t*>(p.y);
    const uint32_t leader_empty = map_to_rank(tmem_empty, 0);
    uint32_t local = 0;
    for (int tile = pair; tile < tiles; tile += pairs, ++local) {
      int m_tile, n_tile;
      pair_tile_coords(tile, p.m_tiles, p.n_tiles, m_tile, n_tile);
      if (!__all_sync(0xffffffffu, mbar_wait(tmem_full, local & 1))) {
        if (lane == 0) atomicExch(&g_w4a16_pair_status, INTENT_B200_ERR_TIMEOUT);
        break;
      }
      tcgen05_fence_after();
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int row = m_tile * PAIR_ROWS + int(rank) * (MT * BM) + mt * BM + quadrant * 32 + lane;
        const uint32_t taddr = tmem_base + mt * BN + (uint32_t(quadrant * 32) << 16);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t v[32];
          tmem_load_32x32(taddr + c * 32, v);
          tmem_load_wait();
          const int col = n_tile * BN + c * 32;
          if (row < p.M) {
            uint16_t* dst = y + size_t(row) * p.N + col;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              if (col + q * 8 < p.N) {
                uint4 o;
                o.x = uint32_t(Elem<T>::from_float(__uint_as_float(v[8 * q + 0]))) |
                      (uint32_t(Elem<T>::from_float(__uint_as_float(v[8 * q + 1]))) << 16);
                o.y = uint32_t(Elem<T>::from_float(__uint_as_float(v[8 * q + 2]))) |
                      (uint32_t(Elem<T>::from_float(__uint_as_float(v[8 * q + 3]))) << 16);
                o.z = uint32_t(Elem<T>::from_float(__uint_as_float(v[8 * q + 4]))) |
                      (uint32_t(Elem<T>::from_float(__uint_as_float(v[8 * q + 5]))) << 16);
                o.w = uint32_t(Elem<T>::from_float(__uint_as_float(v[8 * q + 6]))) |
                      (uint32_t(Elem<T>::from_float(__uint_as_float(v[8 * q + 7]))) << 16);
                *reinterpret_cast<uint4*>(dst + q * 8) = o;
              }
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader_empty);
    }
  } else {
    // ------------------------------ dequantisers (both CTAs, own half of the columns) -------
    const int dq = tid - 6 * 32;
    const int n = dq & (BN / 2 - 1);        // row of this CTA's operand tile = weight column of its half
    const int part = dq / (BN / 2);         // which DQ_ROWS packed rows of every k block
    const uint32_t magic = Elem<T>::kMagic2 ^ (p.twos_complement ? 0x00080008u : 0u);
    const uint32_t row_off = uint32_t(n) * 128u;
    const uint32_t swz = uint32_t(n & 7);
    const int packed_rows = p.K >> 3, scale_rows = p.K / p.group_size;
    const int my_tiles = tiles > pair ? (tiles - pair + pairs - 1) / pairs : 0;
    const int total = my_tiles * p.k_blocks;
    const int group_shift = 31 - __clz(p.group_size);

    struct Block {
      uint32_t w[DQ_ROWS];
      uint32_t s_lo, s_hi;
    };
    int f_tile = pair, f_kb = 0, f_left = total;
    bool f_col_ok = false;
    const uint32_t* f_w = p.packed;
    const uint16_t* f_s = p.scales;
    auto fetch = [&](Block& b) {
      if (f_left <= 0) return;
      --f_left;
      if (f_kb == 0) {
        int m_tile, n_tile;
        pair_tile_coords(f_tile, p.m_tiles, p.n_tiles, m_tile, n_tile);
        const int col = n_tile * BN + int(rank) * (BN / 2) + n;
        f_col_ok = col < p.N;
        f_w = p.packed + (f_col_ok ? col : 0);
        f_s = p.scales + (f_col_ok ? col : 0);
        // tiled copy: [column block of 128][k block][half of the k block][column][4 words].  This kernel puts four
        // threads on a column (DQ_ROWS = 2 words each): thread `part` takes words 2 * (part & 1) .. + 1 of half
        // part >> 1.  A column past N reads word 0 of the buffer, unused.
        if (p.prelaid)
          f_w = f_col_ok ? p.packed + ((size_t(col >> 7) * p.k_blocks * 2 + (part >> 1)) * 128 + (col & 127)) * 4 +
                               (part & 1) * 2
                         : p.packed;
      }
      const int rows_left = packed_rows - f_kb * (BK / 8) - part * DQ_ROWS;
      if (p.prelaid) {
        // tiled copy: this thread's words of the k block are adjacent (rows past K are stored as zeros)
        static_assert(DQ_ROWS == 2, "the tiled fetch below reads this thread's two words as one 8-byte load");
        const uint2 v = __ldg(reinterpret_cast<const uint2*>(f_w));
        b.w[0] = f_col_ok ? v.x : 0u;
        b.w[1] = f_col_ok ? v.y : 0u;
      } else if (f_col_ok && rows_left >= DQ_ROWS) {
        const uint32_t* q = f_w + size_t(part * DQ_ROWS) * p.N;
#pragma unroll
        for (int r = 0; r < DQ_ROWS; ++r, q += p.N) b.w[r] = __ldg(q);
      } else {
#pragma unroll
        for (int r = 0; r < DQ_ROWS; ++r)
          b.w[r] = (f_col_ok && r < rows_left) ? __ldg(f_w + size_t(part * DQ_ROWS + r) * p.N) : 0u;
      }
      const int g0 = (f_kb * BK) >> group_shift;
      const int g1 = p.group_size < BK ? g0 + 1 : g0;
      const uint32_t a = (f_col_ok && g0 < scale_rows) ? __ldg(f_s + size_t(g0) * p.N) : 0u;
      const uint32_t c = g1 == g0 ? a : ((f_col_ok && g1 < scale_rows) ? __ldg(f_s + size_t(g1) * p.N) : 0u);
      b.s_lo = a | (a << 16);
      b.s_hi = c | (c << 16);
      f_w += p.prelaid ? (f_col_ok ? size_t(2) * 128 * 4 : 0) : size_t(BK / 8) * p.N;
      if (++f_kb == p.k_blocks) {
        f_kb = 0;
        f_tile += pairs;
      }
    };
    bool ok = true;
    auto consume = [&](int i, const Block& b) {
      if (i >= total || !ok) return;
      const uint32_t t = uint32_t(i) % B_STAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(empty_b + 8 * t, ((uint32_t(i) / B_STAGES) & 1) ^ 1));
      if (!ok) return;
      const uint32_t dst = smem_b + t * B_HALF_BYTES + row_off;
#pragma unroll
      for (int j = 0; j < DQ_ROWS; ++j) {
        const int r = part * DQ_ROWS + j;
        const uint32_t w = b.w[j], w4 = w >> 4;
        const uint32_t scale2 = r < 4 ? b.s_lo : b.s_hi;
        uint4 o;
        o.x = lop3_and_xor_u32(prmt(w, w4, 0x0400), 0x000F000Fu, magic);
        o.y = lop3_and_xor_u32(prmt(w, w4, 0x0501), 0x000F000Fu, magic);
        o.z = lop3_and_xor_u32(prmt(w, w4, 0x0602), 0x000F000Fu, magic);
        o.w = lop3_and_xor_u32(prmt(w, w4, 0x0703), 0x000F000Fu, magic);
        o.x = Elem<T>::mul2(Elem<T>::sub2(o.x, Elem<T>::kBias2), scale2);
        o.y = Elem<T>::mul2(Elem<T>::sub2(o.y, Elem<T>::kBias2), scale2);
        o.z = Elem<T>::mul2(Elem<T>::sub2(o.z, Elem<T>::kBias2), scale2);
        o.w = Elem<T>::mul2(Elem<T>::sub2(o.w, Elem<T>::kBias2), scale2);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + ((uint32_t(r) ^ swz) << 4)), "r"(o.x),
                     "r"(o.y), "r"(o.z), "r"(o.w)
                     : "memory");
      }
      fence_proxy_async();  // the tensor cores read this tile through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(full_b + 8 * t);  // CTA-local; the peer's arrivals are relayed by its warp 1
    };
    Block b0, b1, b2;
    fetch(b0);
    fetch(b1);
    fetch(b2);
    for (int i = 0; i < total && ok; i += 3) {
      consume(i, b0);
      fetch(b0);
      consume(i + 1, b1);
      fetch(b1);
      consume(i + 2, b2);
      fetch(b2);
    }
    if (!ok && lane == 0) atomicExch(&g_w4a16_pair_status, INTENT_B200_ERR_TIMEOUT);
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_sync();   // the peer's shared memory and TMEM stay alive until both CTAs are done
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

int g_pair_enabled = 1;

}  // namespace

// Dense W4A16 on CTA pairs; returns INTENT_B200_ERR_UNSUPPORTED when the shape should use the
// single-CTA kernel instead.  Arguments are already validated by the caller.
template <typename T>
int w4a16_gemm_pair(const void* x, int64_t M, int64_t K, const void* w, const void* s, int64_t N, void* y,
                    int group_size, int zero_point, cudaStream_t stream, bool prelaid) {
  if (!g_pair_enabled || M < PAIR_ROWS) return INTENT_B200_ERR_UNSUPPORTED;
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms < 2)
    return INTENT_B200_ERR_UNSUPPORTED;
  const CUtensorMapDataType type =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  PairParams p{};
  p.y = y;
  p.packed = static_cast<const uint32_t*>(w);
  p.scales = static_cast<const uint16_t*>(s);
  p.M = int(M);
  p.K = int(K);
  p.N = int(N);
  p.k_blocks = int((K + BK - 1) / BK);
  p.m_tiles = int((M + PAIR_ROWS - 1) / PAIR_ROWS);
  p.n_tiles = int((N + BN - 1) / BN);
  p.group_size = group_size;
  p.twos_complement = zero_point == -1 ? 1 : 0;
  p.prelaid = prelaid ? 1 : 0;
  CUtensorMap map_x;
  if (!make_tensor_map_2d(&map_x, type, x, uint64_t(M), uint64_t(K), uint64_t(K) * 2, BM, BK,
                          CU_TENSOR_MAP_SWIZZLE_128B))
    return INTENT_B200_ERR_UNSUPPORTED;
  auto kernel = w4a16_gemm_pair_kernel<T>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
  if (e != cudaSuccess) return cuda_status(e);
  const int tiles = p.m_tiles * p.n_tiles;
  int pairs = sms / 2;
  if (pairs > tiles) pairs = tiles;
  if (LaunchFacts* sink = observe_sink())
    return record_launch(sink, reinterpret_cast<const void*>(kernel), "w4a16_gemm_pair_kernel CTA pairs, 512x256 tiles",
                         2 * pairs, THREADS, SMEM_BYTES, 2);
  kernel<<<2 * pairs, THREADS, SMEM_BYTES, stream>>>(map_x, p);
  note_launch();
  return launch_status();
}

// Reads the pair kernel's status word into *value and clears it when it was set (the caller has
// synchronised the device).
int w4a16_gemm_pair_take_status(int* value) {
  const int zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(value, g_w4a16_pair_status, sizeof(int));
  if (e != cudaSuccess) return cuda_status(e);
  if (*value != 0) {
    e = cudaMemcpyToSymbol(g_w4a16_pair_status, &zero, sizeof(int));
    if (e != cudaSuccess) return cuda_status(e);
  }
  return INTENT_B200_OK;
}

template int w4a16_gemm_pair<__half>(const void*, int64_t, int64_t, const void*, const void*, int64_t, void*, int, int,
                                     cudaStream_t, bool);
template int w4a16_gemm_pair<__nv_bfloat16>(const void*, int64_t, int64_t, const void*, const void*, int64_t, void*,
                                            int, int, cudaStream_t, bool);

}  // namespace ib200

extern "C" int intent_b200_w4a16_gemm_pairs(int32_t enable) {
  ib200::g_pair_enabled = enable ? 1 : 0;
  return INTENT_B200_OK;
}
