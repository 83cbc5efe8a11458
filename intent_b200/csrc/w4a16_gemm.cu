// W4A16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM).
//
//   Y[m, n] = T( sum_k f32(X[m, k]) * f32( T( (q[k, n] - 8) * S[k / G, n] ) ) )
//
// Program: weight_only_int4_matmul, reference kernel body
// examples/kernels/contraction/weight_only_int4.py:18-51 (the dequantised weight is
// rounded to the activation type before the f32-accumulated product, as at :42-47).
//
// One persistent CTA per SM walks output tiles of (MT * 128) rows x 256 columns; 22 warps in
// four roles:
//   warp 0        TMA producer: per 64-wide k block MT 128B-swizzled boxes of X (128 rows x 64 k).
//   warps 6..21   dequantisers: two threads per weight column of the tile, each expanding half of
//                 the k block (four packed words).  A thread reads its packed words straight from
//                 global memory (a warp reads 128 contiguous bytes per packed row; three k blocks
//                 are kept in flight in registers), expands them to values of T with the
//                 magic-number trick (prmt + lop3, exact subtract, one rounding multiply by the
//                 scale) and writes them into the 128-byte row n of the K-major, 128B-swizzled B
//                 operand tile.  Shared memory therefore carries each weight once (the operand
//                 tile), not twice.
//   warp 1        MMA issuer: one thread issues, per k block, four tcgen05.mma (M128 N256 K16,
//                 kind::f16, f32 accumulation in TMEM) for each of the MT row blocks - the row
//                 blocks share the dequantised B tile - and commits to the mbarriers that free
//                 the stages.
//   warps 2..5    epilogue: tcgen05.ld the accumulators (each warp its 32-lane TMEM quadrant),
//                 convert, store.  With MT = 1 two accumulators alternate so the epilogue of a
//                 tile overlaps the next tile's MMAs; with MT = 2 the two row blocks fill TMEM.
// Shared-memory bandwidth is what bounds this kernel (operand reads by the tensor core, operand
// tile writes, TMA writes); MT = 2 halves the B traffic per flop.  Tiles are walked in bands of
// rows so that the band of X and all of W stay in L2.
// Every wait is bounded; a wait that gives up records INTENT_B200_ERR_TIMEOUT and the CTA drains
// and frees its TMEM.
//
// The same kernel serves the MoE grouped contractions (reference programs
// examples/kernels/ragged/grouped_gemm.py:11-70 and examples/kernels/ragged/moe.py:12-53 with
// int4 expert weights): rows are sorted by expert and padded to 128 per expert, so a 128-row
// block belongs to one expert, read from the block -> expert table of the route alignment; the
// number of row blocks is read from device memory (no host round trip).
//   MODE 1  up|gate projection: the N tile is 128 gate columns + the matching 128 up columns,
//           the epilogue writes T( silu(gate) * up ).
//   MODE 2  down projection with f32 output rows (combined per token by a later kernel).
//   MODE 3  down projection whose epilogue does the weighted combine itself: row r of the expert-sorted
//           buffer belongs to route sorted_routes[r]; y[route / TOP_K, :] += weight[route] * row with
//           red.global.add.v4.f32 (the reference's GPU lowering of scatter_reduce(add) is the same relaxed
//           atomic, lib/Target/Triton/Transforms/Access/Scatter.cpp:43-60).  On a zeroed y with TOP_K <= 2
//           the result does not depend on the order of the two additions: (0 + a) + b == (0 + b) + a.
#include <type_traits>

#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

namespace ib200 {

__device__ int g_w4a16_gemm_status = 0;

template <typename T>
int w4a16_gemm_pair(const void* x, int64_t M, int64_t K, const void* w, const void* s, int64_t N, void* y,
                    int group_size, int zero_point, cudaStream_t stream, bool prelaid);
int w4a16_gemm_pair_take_status(int* value);
int64_t w4a16_prelayout_words(int64_t K, int64_t N);

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int A_BYTES = BM * BK * 2;  // one 128-row box of X, 16 KiB
constexpr int B_BYTES = BN * BK * 2;  // dequantised operand tile, 32 KiB
constexpr int DEQUANT_WARPS = 16;          // two threads per weight column, each expands half a k block
constexpr int DQ_PARTS = DEQUANT_WARPS / 8;  // threads per column
constexpr int DQ_ROWS = (BK / 8) / DQ_PARTS; // packed words per thread and k block
constexpr int THREADS = (6 + DEQUANT_WARPS) * 32;
constexpr int BAND_TILES = 8;         // row tiles per band of the tile walk

constexpr int PAIR_LIST_BLOCKS = 8192;  // most 128-row blocks the in-kernel block pairing handles

template <int MT>
struct Stages {
  static constexpr int A = MT == 1 ? 5 : 3;   // stages of X
  static constexpr int B = 3;                 // stages of the dequantised tile
  static constexpr int SMEM = 1024 + A * MT * A_BYTES + B * B_BYTES + 256;
  // grouped modes with two row blocks per tile keep the list of block pairs behind the barriers
  static constexpr int SMEM_PAIRED = SMEM + PAIR_LIST_BLOCKS * 2 + 16;
};

struct GemmParams {
  void* y;
  const uint32_t* packed;    // [E, K/8, WN]
  const uint16_t* scales;    // [E, K/G, WN]
  int M, K;
  int WN;                    // columns of the weight matrix
  int k_blocks;              // ceil(K / 64)
  int m_tiles, n_tiles;      // tiles of (MT*128) rows, tiles of 256 accumulator columns
  int group_size;
  int twos_complement;
  int second_half_offset;    // weight-column distance of accumulator columns 128..255 (128, or I for up|gate)
  int out_cols;              // columns of the output matrix
  const int* total_rows;     // grouped modes: device pointer to the padded row count (multiple of MT*128)
  const int* tile_expert;    // grouped modes: expert of each (MT*128)-row block; of each 128-row block with pair_blocks
  int pair_blocks;           // grouped modes, MT = 2: rows are padded to 128 per expert and the kernel pairs
                             // neighbouring blocks of one expert itself (an odd last block runs as half a tile)
  int experts;               // grouped modes: E; a block whose expert id is outside [0, E) is computed with zero
                             // weights and recorded as INTENT_B200_ERR_INDEX
  int prelaid;               // packed points at the tiled copy (w4a16_prelayout.cu); per expert in the grouped modes
  const int* row_route;      // MODE 3: route id of every expert-sorted row (>= routes: a padding row)
  const float* route_weight; // MODE 3: [routes]
  int routes, top_k;         // MODE 3
};

constexpr int MODE_DENSE = 0, MODE_UPGATE_SILU = 1, MODE_GROUPED_F32 = 2, MODE_DOWN_SCATTER = 3;

__device__ __forceinline__ void red_add_v4(float* address, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(address), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Tile walk: bands of BAND_TILES row tiles; inside a band the row tile varies fastest.
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int& m_tile, int& n_tile) {
  const int band_size = BAND_TILES * n_tiles;
  const int band = tile / band_size;
  const int in_band = tile - band * band_size;
  const int rows_in_band = min(BAND_TILES, m_tiles - band * BAND_TILES);
  n_tile = in_band / rows_in_band;
  m_tile = band * BAND_TILES + (in_band - n_tile * rows_in_band);
}

template <typename T, int MODE, int MT>
__global__ void __launch_bounds__(THREADS, 1)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const GemmParams p) {
  constexpr int A_STAGES = Stages<MT>::A, B_STAGES = Stages<MT>::B;
  constexpr int ACC_BUFFERS = 2 / MT;       // accumulator sets that alternate between tiles
  extern __shared__ unsigned char smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t smem_a = base;
  const uint32_t smem_b = smem_a + A_STAGES * MT * A_BYTES;
  const uint32_t bars = smem_b + B_STAGES * B_BYTES;
  const uint32_t full_a = bars;                        // [A_STAGES] TMA bytes landed
  const uint32_t empty_a = full_a + 8 * A_STAGES;      // [A_STAGES] MMA done with the stage
  const uint32_t full_b = empty_a + 8 * A_STAGES;      // [B_STAGES] dequantised tile written
  const uint32_t empty_b = full_b + 8 * B_STAGES;      // [B_STAGES] MMA done with it
  const uint32_t tmem_full = empty_b + 8 * B_STAGES;   // [2] accumulators complete
  const uint32_t tmem_empty = tmem_full + 16;          // [2] accumulators drained
  const uint32_t tmem_slot = tmem_empty + 16;          // TMEM base address written by tcgen05.alloc
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(base_ptr + (tmem_slot - base));

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  constexpr bool CAN_PAIR = MODE != MODE_DENSE && MT == 2;
  const bool paired = CAN_PAIR && p.pair_blocks != 0;
  // tile list of the paired form: low 15 bits = first 128-row block, bit 15 = the next block belongs to it too
  uint16_t* pair_list = reinterpret_cast<uint16_t*>(base_ptr + (tmem_slot - base) + 16);
  volatile int* pair_count = reinterpret_cast<volatile int*>(base_ptr + (tmem_slot - base) + 8);

  if (tid == 0) {
    for (int s = 0; s < A_STAGES; ++s) {
      mbar_init(full_a + 8 * s, 1);
      mbar_init(empty_a + 8 * s, 1);
    }
    for (int s = 0; s < B_STAGES; ++s) {
      mbar_init(full_b + 8 * s, DEQUANT_WARPS);
      mbar_init(empty_b + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(tmem_full + 8 * s, 1);
      mbar_init(tmem_empty + 8 * s, 4);
    }
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, 512);
  if (CAN_PAIR && paired && warp == 0) {
    // Pair neighbouring 128-row blocks of one expert: a block whose position inside its expert's run
    // is even starts a tile; the tile has a second half when the next block has the same expert.
    const int blocks = min(min(2 * p.m_tiles, PAIR_LIST_BLOCKS), (*p.total_rows + BM - 1) / BM);
    int count = 0, carry_expert = -1, carry_start = 0;
    for (int b0 = 0; b0 < blocks; b0 += 32) {
      const int b = b0 + lane;
      const int e = b < blocks ? __ldg(p.tile_expert + b) : -1;
      int previous = __shfl_up_sync(0xffffffffu, e, 1);
      if (lane == 0) previous = carry_expert;
      int next = __shfl_down_sync(0xffffffffu, e, 1);
      if (lane == 31) next = b + 1 < blocks ? __ldg(p.tile_expert + b + 1) : -1;
      int start = (b < blocks && (b == 0 || e != previous)) ? b : -1;  // first block of its expert's run
      if (lane == 0 && start < 0) start = carry_start;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {  // running maximum: the latest run start at or before this block
        const int v = __shfl_up_sync(0xffffffffu, start, o);
        if (lane >= o) start = max(start, v);
      }
      const bool first = b < blocks && ((b - start) & 1) == 0;
      const uint32_t ballot = __ballot_sync(0xffffffffu, first);
      if (first) {
        const int t = count + __popc(ballot & ((1u << lane) - 1u));
        pair_list[t] = uint16_t(b | ((b + 1 < blocks && next == e) ? 0x8000 : 0));
      }
      count += __popc(ballot);
      carry_expert = __shfl_sync(0xffffffffu, e, 31);
      carry_start = __shfl_sync(0xffffffffu, start, 31);
    }
    if (lane == 0) *pair_count = count;
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // grouped modes: row blocks actually in use, read from device memory
  const int m_tiles = MODE == MODE_DENSE ? p.m_tiles
                      : paired           ? *pair_count
                                         : min(p.m_tiles, (*p.total_rows + MT * BM - 1) / (MT * BM));
  const int tiles = m_tiles * p.n_tiles;
  // first 128-row block of a row tile and whether its second block is present
  auto tile_blocks = [&](int m_tile, int& first_block, int& halves) {
    if (CAN_PAIR && paired) {
      const uint32_t entry = pair_list[m_tile];
      first_block = int(entry & 0x7FFFu);
      halves = (entry & 0x8000u) ? 2 : 1;
    } else {
      first_block = m_tile * MT;
      halves = MT;
    }
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        int m_tile, n_tile;
        tile_coords(tile, m_tiles, p.n_tiles, m_tile, n_tile);
        int first_block, halves;
        tile_blocks(m_tile, first_block, halves);
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % A_STAGES;
          if (!mbar_wait(empty_a + 8 * s, ((it / A_STAGES) & 1) ^ 1)) { ok = false; break; }
          const uint32_t bar = full_a + 8 * s;
          mbar_expect_tx(bar, halves * A_BYTES);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            if (mt < halves)
              tma_load_2d(smem_a + (s * MT + mt) * A_BYTES, &map_x, kb * BK, (first_block + mt) * BM, bar);
        }
      }
      if (!ok) atomicExch(&g_w4a16_gemm_status, INTENT_B200_ERR_TIMEOUT);
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer --------------------------------
    if (lane == 0) {
      constexpr uint32_t fmt = std::is_same<T, __half>::value ? 0u : 1u;
      constexpr uint32_t idesc = umma_idesc(1, fmt, fmt, 0, 0, BM, BN);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++local) {
        int first_block = 0, halves = MT;
        if (CAN_PAIR && paired) {
          int m_tile, n_tile;
          tile_coords(tile, m_tiles, p.n_tiles, m_tile, n_tile);
          tile_blocks(m_tile, first_block, halves);
        }
        const uint32_t acc = local % ACC_BUFFERS;
        if (!mbar_wait(tmem_empty + 8 * acc, ((local / ACC_BUFFERS) & 1) ^ 1)) { ok = false; break; }
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * (MT * BN);
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const uint32_t s = it % A_STAGES, t = it % B_STAGES;
          if (!mbar_wait(full_a + 8 * s, (it / A_STAGES) & 1) ||
              !mbar_wait(full_b + 8 * t, (it / B_STAGES) & 1)) { ok = false; break; }
          tcgen05_fence_after();
          const uint64_t desc_b = umma_desc_k_major_sw128(smem_b + t * B_BYTES);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            if (mt >= halves) break;
            const uint64_t desc_a = umma_desc_k_major_sw128(smem_a + (s * MT + mt) * A_BYTES);
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)  // 16 elements of 2 bytes = 32 bytes = 2 descriptor units
              umma_f16(tmem_d + mt * BN, desc_a + uint64_t(2 * kk), desc_b + uint64_t(2 * kk), idesc, (kb | kk) != 0);
          }
          umma_commit(empty_a + 8 * s);
          umma_commit(empty_b + 8 * t);
        }
        if (ok) umma_commit(tmem_full + 8 * acc);
      }
      if (!ok) atomicExch(&g_w4a16_gemm_status, INTENT_B200_ERR_TIMEOUT);
    }
  } else if (warp < 6) {
    // ------------------------------ epilogue -----------------------------------
    const int quadrant = warp & 3;  // TMEM lanes 32*quadrant .. +31 are the ones this warp may read
    uint16_t* y = reinterpret_cast<uint16_t*>(p.y);
    uint32_t local = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
      int m_tile, n_tile;
      tile_coords(tile, m_tiles, p.n_tiles, m_tile, n_tile);
      int first_block, halves;
      tile_blocks(m_tile, first_block, halves);
      const uint32_t acc = local % ACC_BUFFERS;
      if (!__all_sync(0xffffffffu, mbar_wait(tmem_full + 8 * acc, (local / ACC_BUFFERS) & 1))) {
        if (lane == 0) atomicExch(&g_w4a16_gemm_status, INTENT_B200_ERR_TIMEOUT);
        break;
      }
      tcgen05_fence_after();
#pragma unroll 1
      for (int mt = 0; mt < halves; ++mt) {
        const int row = (first_block + mt) * BM + quadrant * 32 + lane;
        const uint32_t taddr = tmem_base + acc * (MT * BN) + mt * BN + (uint32_t(quadrant * 32) << 16);
        if (MODE == MODE_UPGATE_SILU) {
          // accumulator columns 0..127 = gate, 128..255 = the matching up columns
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t gate[32], up[32];
            tmem_load_32x32(taddr + c * 32, gate);
            tmem_load_32x32(taddr + 128 + c * 32, up);
            tmem_load_wait();
            const int col = n_tile * 128 + c * 32;
            if (row < p.M) {
              uint16_t* dst = y + size_t(row) * p.out_cols + col;
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint32_t o[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float h[2];
#pragma unroll
                  for (int e = 0; e < 2; ++e) {
                    const float gv = __uint_as_float(gate[8 * q + 2 * j + e]);
                    const float uv = __uint_as_float(up[8 * q + 2 * j + e]);
                    h[e] = gv * (1.0f / (1.0f + __expf(-gv))) * uv;  // silu(gate) * up in f32, one rounding
                  }
                  o[j] = uint32_t(Elem<T>::from_float(h[0])) | (uint32_t(Elem<T>::from_float(h[1])) << 16);
                }
                if (col + q * 8 < p.out_cols)
                  *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        } else {
          // MODE 3: where this lane's row goes and with what weight (padding rows go nowhere)
          float route_w = 0.f;
          float* token_row = nullptr;
          if (MODE == MODE_DOWN_SCATTER && row < p.M) {
            const int route = p.row_route[row];
            if (route >= 0 && route < p.routes) {
              route_w = p.route_weight[route];
              token_row = reinterpret_cast<float*>(p.y) + size_t(route / p.top_k) * p.out_cols;
            }
          }
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t v[32];
            tmem_load_32x32(taddr + c * 32, v);
            tmem_load_wait();
            const int col = n_tile * BN + c * 32;
            if (MODE == MODE_DOWN_SCATTER) {
              if (token_row != nullptr) {
#pragma unroll
                for (int q = 0; q < 8; ++q)
                  if (col + q * 4 < p.out_cols)
                    red_add_v4(token_row + col + q * 4, __fmul_rn(route_w, __uint_as_float(v[4 * q])),
                               __fmul_rn(route_w, __uint_as_float(v[4 * q + 1])),
                               __fmul_rn(route_w, __uint_as_float(v[4 * q + 2])),
                               __fmul_rn(route_w, __uint_as_float(v[4 * q + 3])));
              }
            } else if (row < p.M) {
              if (MODE == MODE_GROUPED_F32) {
                float* dst = reinterpret_cast<float*>(p.y) + size_t(row) * p.out_cols + col;
#pragma unroll
                for (int q = 0; q < 8; ++q)
                  if (col + q * 4 < p.out_cols)
                    *reinterpret_cast<uint4*>(dst + q * 4) =
                        make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
              } else {
                uint16_t* dst = y + size_t(row) * p.out_cols + col;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                  if (col + q * 8 < p.out_cols) {  // the column count is a multiple of 8
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
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tmem_empty + 8 * acc);
    }
  } else {
    // ------------------------------ dequantisers --------------------------------
    const int n = (tid - 6 * 32) & 255;   // accumulator column of the tile owned by this thread, 0..255
    const int part = (tid - 6 * 32) >> 8; // which DQ_ROWS packed rows of every k block it expands
    const uint32_t magic = Elem<T>::kMagic2 ^ (p.twos_complement ? 0x00080008u : 0u);
    const uint32_t row_off = uint32_t(n) * 128u;
    const uint32_t swz = uint32_t(n & 7);
    const int packed_rows = p.K >> 3, scale_rows = p.K / p.group_size;
    const int my_tiles = tiles > int(blockIdx.x) ? (tiles - int(blockIdx.x) + int(gridDim.x) - 1) / int(gridDim.x) : 0;
    const int total = my_tiles * p.k_blocks;

    struct Block {
      uint32_t w[DQ_ROWS];
      uint32_t s_lo, s_hi;  // scale of k 0..31 and of k 32..63 of the block, duplicated into both halves
    };
    // Fetch state: walks this CTA's (tile, k block) sequence in order, three blocks ahead of the
    // consumer; everything that depends only on the tile is recomputed when the tile changes.
    const int group_shift = 31 - __clz(p.group_size);  // the group size is a power of two
    int f_tile = int(blockIdx.x), f_kb = 0, f_left = total;
    bool f_col_ok = false;
    const uint32_t* f_w = p.packed;
    const uint16_t* f_s = p.scales;
    auto fetch = [&](Block& b) {
      if (f_left <= 0) return;
      --f_left;
      if (f_kb == 0) {
        int m_tile, n_tile;
        tile_coords(f_tile, m_tiles, p.n_tiles, m_tile, n_tile);
        int first_block, halves;
        tile_blocks(m_tile, first_block, halves);
        int expert = MODE == MODE_DENSE ? 0 : p.tile_expert[(CAN_PAIR && paired) ? first_block : m_tile];
        const int col = (MODE == MODE_UPGATE_SILU ? n_tile * 128 : n_tile * BN) +
                        (n < 128 ? n : p.second_half_offset + (n - 128));
        f_col_ok = col < p.WN;
        if (MODE != MODE_DENSE && unsigned(expert) >= unsigned(p.experts)) {
          // an id that names no expert (a stale or sentinel table entry): never used as an index
          if (lane == 0) atomicExch(&g_w4a16_gemm_status, INTENT_B200_ERR_INDEX);
          f_col_ok = false;
          expert = 0;
        }
        f_w = p.packed + size_t(expert) * packed_rows * p.WN + (f_col_ok ? col : 0);
        f_s = p.scales + size_t(expert) * scale_rows * p.WN + (f_col_ok ? col : 0);
        if (p.prelaid) {   // per expert: [column block of 128][k block][part][column][4 words]
          const size_t column_blocks = size_t(p.WN + 127) >> 7;
          const size_t expert_words = column_blocks * p.k_blocks * DQ_PARTS * 128 * 4;
          f_w = p.packed + size_t(expert) * expert_words +
                ((size_t(col >> 7) * p.k_blocks * DQ_PARTS + part) * 128 + (col & 127)) * 4;
          if (!f_col_ok) f_w = p.packed;   // a column past WN: any valid address, the words are not used
        }
      }
      const int rows_left = packed_rows - f_kb * (BK / 8) - part * DQ_ROWS;
      if (p.prelaid) {
        // tiled copy: this thread's four words of the k block are one 16-byte load (rows past K are zeros)
        static_assert(DQ_ROWS == 4 && DQ_PARTS == 2, "the tiled layout is two halves of four words per column");
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(f_w));
        const bool use = f_col_ok;
        b.w[0] = use ? v.x : 0u; b.w[1] = use ? v.y : 0u; b.w[2] = use ? v.z : 0u; b.w[3] = use ? v.w : 0u;
      } else if (f_col_ok && rows_left >= DQ_ROWS) {
        const uint32_t* q = f_w + size_t(part * DQ_ROWS) * p.WN;
#pragma unroll
        for (int r = 0; r < DQ_ROWS; ++r, q += p.WN) b.w[r] = __ldg(q);
      } else {
#pragma unroll
        for (int r = 0; r < DQ_ROWS; ++r)
          b.w[r] = (f_col_ok && r < rows_left) ? __ldg(f_w + size_t(part * DQ_ROWS + r) * p.WN) : 0u;
      }
      const int g0 = (f_kb * BK) >> group_shift;
      const int g1 = p.group_size < BK ? g0 + 1 : g0;
      const uint32_t a = (f_col_ok && g0 < scale_rows) ? __ldg(f_s + size_t(g0) * p.WN) : 0u;
      const uint32_t c = g1 == g0 ? a : ((f_col_ok && g1 < scale_rows) ? __ldg(f_s + size_t(g1) * p.WN) : 0u);
      b.s_lo = a | (a << 16);
      b.s_hi = c | (c << 16);
      f_w += p.prelaid ? (f_col_ok ? size_t(DQ_PARTS) * 128 * 4 : 0) : size_t(BK / 8) * p.WN;
      if (++f_kb == p.k_blocks) {
        f_kb = 0;
        f_tile += int(gridDim.x);
      }
    };
    bool ok = true;
    auto consume = [&](int i, const Block& b) {
      if (i >= total || !ok) return;
      const uint32_t t = uint32_t(i) % B_STAGES;
      ok = __all_sync(0xffffffffu, mbar_wait(empty_b + 8 * t, ((uint32_t(i) / B_STAGES) & 1) ^ 1));
      if (!ok) return;
      const uint32_t dst = smem_b + t * B_BYTES + row_off;
#pragma unroll
      for (int j = 0; j < DQ_ROWS; ++j) {
        const int r = part * DQ_ROWS + j;   // packed row (16-byte chunk) of the k block
        const uint32_t w = b.w[j], w4 = w >> 4;
        const uint32_t scale2 = r < 4 ? b.s_lo : b.s_hi;
        uint4 o;
        o.x = lop3_and_xor_u32(prmt(w, w4, 0x0400), 0x000F000Fu, magic);  // (k0, k1)
        o.y = lop3_and_xor_u32(prmt(w, w4, 0x0501), 0x000F000Fu, magic);  // (k2, k3)
        o.z = lop3_and_xor_u32(prmt(w, w4, 0x0602), 0x000F000Fu, magic);  // (k4, k5)
        o.w = lop3_and_xor_u32(prmt(w, w4, 0x0703), 0x000F000Fu, magic);  // (k6, k7)
        o.x = Elem<T>::mul2(Elem<T>::sub2(o.x, Elem<T>::kBias2), scale2);
        o.y = Elem<T>::mul2(Elem<T>::sub2(o.y, Elem<T>::kBias2), scale2);
        o.z = Elem<T>::mul2(Elem<T>::sub2(o.z, Elem<T>::kBias2), scale2);
        o.w = Elem<T>::mul2(Elem<T>::sub2(o.w, Elem<T>::kBias2), scale2);
        asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(dst + ((uint32_t(r) ^ swz) << 4)), "r"(o.x),
                     "r"(o.y), "r"(o.z), "r"(o.w)
                     : "memory");
      }
      fence_proxy_async();  // the tensor core reads this tile through the async proxy
      __syncwarp();
      if (lane == 0) mbar_arrive(full_b + 8 * t);
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
    if (!ok && lane == 0) atomicExch(&g_w4a16_gemm_status, INTENT_B200_ERR_TIMEOUT);
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

// x: [rows, K] activations; w: [E, K/8, WN] packed; s: [E, K/G, WN] scales; out: [rows, out_cols].
template <typename T, int MODE, int MT>
int launch_gemm(const void* x, int64_t rows, int64_t K, const void* w, const void* s, int64_t WN, void* out,
                int64_t out_cols, int group_size, int zero_point, const int* total_rows, const int* tile_expert,
                cudaStream_t stream, bool pair_blocks = false, int64_t experts = 1, const int* row_route = nullptr,
                const float* route_weight = nullptr, int64_t routes = 0, int top_k = 1, bool prelaid = false) {
  const int sms = device_sms();
  if (sms <= 0) return INTENT_B200_ERR_UNSUPPORTED;
  const CUtensorMapDataType type =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  GemmParams p{};
  p.y = out;
  p.packed = static_cast<const uint32_t*>(w);
  p.scales = static_cast<const uint16_t*>(s);
  p.M = int(rows);
  p.K = int(K);
  p.WN = int(WN);
  p.k_blocks = int((K + BK - 1) / BK);
  p.m_tiles = int((rows + MT * BM - 1) / (MT * BM));
  p.n_tiles = MODE == MODE_UPGATE_SILU ? int(out_cols / 128) : int((out_cols + BN - 1) / BN);
  p.group_size = group_size;
  p.twos_complement = zero_point == -1 ? 1 : 0;
  p.second_half_offset = MODE == MODE_UPGATE_SILU ? int(out_cols) : 128;
  p.out_cols = int(out_cols);
  p.total_rows = total_rows;
  p.tile_expert = tile_expert;
  p.pair_blocks = pair_blocks ? 1 : 0;
  p.experts = int(experts);
  p.prelaid = prelaid ? 1 : 0;
  p.row_route = row_route;
  p.route_weight = route_weight;
  p.routes = int(routes);
  p.top_k = top_k;

  CUtensorMap map_x;
  if (!make_tensor_map_2d(&map_x, type, x, uint64_t(rows), uint64_t(K), uint64_t(K) * 2, BM, BK,
                          CU_TENSOR_MAP_SWIZZLE_128B))
    return INTENT_B200_ERR_UNSUPPORTED;

  auto kernel = w4a16_gemm_kernel<T, MODE, MT>;
  constexpr int smem = (MODE != MODE_DENSE && MT == 2) ? Stages<MT>::SMEM_PAIRED : Stages<MT>::SMEM;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return cuda_status(e);
  const int tiles = p.m_tiles * p.n_tiles;
  const int grid = tiles < sms ? tiles : sms;
  if (LaunchFacts* sink = observe_sink())
    return record_launch(sink, reinterpret_cast<const void*>(kernel),
                         MT == 2 ? "w4a16_gemm_kernel single CTA, 256x256 tiles" : "w4a16_gemm_kernel single CTA, 128x256 tiles",
                         grid, THREADS, smem, 1);
  kernel<<<grid, THREADS, smem, stream>>>(map_x, p);
  note_launch();
  return launch_status();
}

template <typename T>
int run(View2 x, View2 w, View2 s, View2 y, int group_size, int zero_point, cudaStream_t stream,
        bool prelaid = false) {
  const int64_t M = x.d0, K = x.d1, N = w.d1;
  if (group_size != 32 && group_size != 64 && group_size != 128) return INTENT_B200_ERR_UNSUPPORTED;
  if (zero_point != -1 && zero_point != 8) return INTENT_B200_ERR_UNSUPPORTED;
  if (K % group_size != 0 || w.d0 * 8 != K || s.d0 * group_size != K || s.d1 != N || y.d0 != M || y.d1 != N)
    return INTENT_B200_ERR_SHAPE;
  if (M == 0 || N == 0) return INTENT_B200_OK;
  if (!x.p || !w.p || !s.p || !y.p) return INTENT_B200_ERR_NULL;
  if (!contiguous(x) || !contiguous(w) || !contiguous(s) || !contiguous(y)) return INTENT_B200_ERR_LAYOUT;
  if (!aligned16(x.p) || !aligned16(w.p) || !aligned16(s.p) || !aligned16(y.p)) return INTENT_B200_ERR_LAYOUT;
  if (K == 0 || N % 8 != 0 || M > (1 << 24) || K > (1 << 24) || N > (1 << 24)) return INTENT_B200_ERR_UNSUPPORTED;
  {  // large M: CTA pairs, each CTA dequantises half of every weight tile
    const int status = w4a16_gemm_pair<T>(x.p, M, K, w.p, s.p, N, y.p, group_size, zero_point, stream, prelaid);
    if (status != INTENT_B200_ERR_UNSUPPORTED) return status;
  }
  if (M > BM)   // two row blocks per tile share every dequantised weight tile
    return launch_gemm<T, MODE_DENSE, 2>(x.p, M, K, w.p, s.p, N, y.p, N, group_size, zero_point, nullptr, nullptr,
                                         stream, false, 1, nullptr, nullptr, 0, 1, prelaid);
  return launch_gemm<T, MODE_DENSE, 1>(x.p, M, K, w.p, s.p, N, y.p, N, group_size, zero_point, nullptr, nullptr,
                                       stream, false, 1, nullptr, nullptr, 0, 1, prelaid);
}

// Grouped contractions over expert-sorted rows padded to `block_rows` (128 or 256) per expert; with 256
// two row blocks share every dequantised weight tile.
//   x [P, K]; tile_expert [>= P/block_rows]; total [1]; w [E, K/8, WN]; s [E, K/G, WN]; out [P, out_cols]
template <typename T, int MODE>
int run_grouped(View2 x, View1 tile_expert, View1 total, View3 w, View3 s, View2 out, int group_size, int zero_point,
                int block_rows, cudaStream_t stream, bool prelaid = false) {
  const int64_t P = x.d0, K = x.d1, E = w.d0, WN = w.d2;
  const int64_t out_cols = MODE == MODE_UPGATE_SILU ? WN / 2 : WN;
  if (group_size != 32 && group_size != 64 && group_size != 128) return INTENT_B200_ERR_UNSUPPORTED;
  if (zero_point != -1 && zero_point != 8) return INTENT_B200_ERR_UNSUPPORTED;
  if (K % group_size != 0 || w.d1 * 8 != K || s.d0 != E || s.d1 * group_size != K || s.d2 != WN || out.d0 != P ||
      out.d1 != out_cols || total.d0 < 1 || (block_rows != BM && block_rows != 2 * BM) ||
      tile_expert.d0 * block_rows < P)
    return INTENT_B200_ERR_SHAPE;
  if (P == 0 || WN == 0 || E == 0) return INTENT_B200_OK;
  if (!x.p || !w.p || !s.p || !out.p || !tile_expert.p || !total.p) return INTENT_B200_ERR_NULL;
  if (!contiguous(x) || !contiguous(w) || !contiguous(s) || !contiguous(out) || !contiguous(tile_expert))
    return INTENT_B200_ERR_LAYOUT;
  if (!aligned16(x.p) || !aligned16(w.p) || !aligned16(s.p) || !aligned16(out.p)) return INTENT_B200_ERR_LAYOUT;
  if (K == 0 || WN % 8 != 0 || (MODE == MODE_UPGATE_SILU && (WN % 256 != 0)) ||
      P > (1 << 24) || K > (1 << 24) || WN > (1 << 24))
    return INTENT_B200_ERR_UNSUPPORTED;
  if (block_rows == 2 * BM || (P + BM - 1) / BM <= PAIR_LIST_BLOCKS)   // 128-row blocks are paired by the kernel
    return launch_gemm<T, MODE, 2>(x.p, P, K, w.p, s.p, WN, out.p, out_cols, group_size, zero_point,
                                   static_cast<const int*>(total.p), static_cast<const int*>(tile_expert.p), stream,
                                   block_rows == BM, E, nullptr, nullptr, 0, 1, prelaid);
  return launch_gemm<T, MODE, 1>(x.p, P, K, w.p, s.p, WN, out.p, out_cols, group_size, zero_point,
                                 static_cast<const int*>(total.p), static_cast<const int*>(tile_expert.p), stream,
                                 false, E, nullptr, nullptr, 0, 1, prelaid);
}

// Down projection with the weighted combine in the epilogue (MODE 3).
//   x [P, K]; tile_expert; total [1]; w [E, K/8, WN]; s [E, K/G, WN]; sorted_routes [>= P]; weights [T, TOP_K]; y [T, WN]
template <typename T>
int run_down_scatter(View2 x, View1 tile_expert, View1 total, View3 w, View3 s, View1 sorted_routes, View2 weights,
                     View2 y, int group_size, int zero_point, int block_rows, cudaStream_t stream,
                     bool prelaid = false) {
  const int64_t P = x.d0, K = x.d1, E = w.d0, WN = w.d2, tokens = weights.d0, top_k = weights.d1;
  if (group_size != 32 && group_size != 64 && group_size != 128) return INTENT_B200_ERR_UNSUPPORTED;
  if (zero_point != -1 && zero_point != 8) return INTENT_B200_ERR_UNSUPPORTED;
  if (K % group_size != 0 || w.d1 * 8 != K || s.d0 != E || s.d1 * group_size != K || s.d2 != WN || y.d0 != tokens ||
      y.d1 != WN || total.d0 < 1 || (block_rows != BM && block_rows != 2 * BM) || tile_expert.d0 * block_rows < P ||
      sorted_routes.d0 < P || top_k <= 0)
    return INTENT_B200_ERR_SHAPE;
  if (P == 0 || WN == 0 || E == 0 || tokens == 0) return INTENT_B200_OK;
  if (!x.p || !w.p || !s.p || !y.p || !tile_expert.p || !total.p || !sorted_routes.p || !weights.p)
    return INTENT_B200_ERR_NULL;
  if (!contiguous(x) || !contiguous(w) || !contiguous(s) || !contiguous(y) || !contiguous(tile_expert) ||
      !contiguous(sorted_routes) || !contiguous(weights))
    return INTENT_B200_ERR_LAYOUT;
  if (!aligned16(x.p) || !aligned16(w.p) || !aligned16(s.p) || !aligned16(y.p)) return INTENT_B200_ERR_LAYOUT;
  if (K == 0 || WN % 8 != 0 || P > (1 << 24) || K > (1 << 24) || WN > (1 << 24) || tokens * top_k > (1 << 30))
    return INTENT_B200_ERR_UNSUPPORTED;
  const int* routes = static_cast<const int*>(sorted_routes.p);
  const float* route_weight = static_cast<const float*>(weights.p);
  if (block_rows == 2 * BM || (P + BM - 1) / BM <= PAIR_LIST_BLOCKS)
    return launch_gemm<T, MODE_DOWN_SCATTER, 2>(x.p, P, K, w.p, s.p, WN, y.p, WN, group_size, zero_point,
                                                static_cast<const int*>(total.p),
                                                static_cast<const int*>(tile_expert.p), stream, block_rows == BM, E,
                                                routes, route_weight, tokens * top_k, int(top_k), prelaid);
  return launch_gemm<T, MODE_DOWN_SCATTER, 1>(x.p, P, K, w.p, s.p, WN, y.p, WN, group_size, zero_point,
                                              static_cast<const int*>(total.p),
                                              static_cast<const int*>(tile_expert.p), stream, false, E, routes,
                                              route_weight, tokens * top_k, int(top_k), prelaid);
}

// The tiled copy stands in for the [K/8, N] matrix: K comes from the activation, N from the scales.
inline bool tiled_as_matrix(View1 tiled, int64_t K, int64_t N, View2* w) {
  if (K <= 0 || N <= 0 || K % 8 != 0 || tiled.d0 != w4a16_prelayout_words(K, N) || !contiguous(tiled)) return false;
  *w = View2{tiled.p, K / 8, N, N, 1};
  return true;
}
inline bool tiled_as_experts(View2 tiled, int64_t K, int64_t WN, View3* w) {
  if (K <= 0 || WN <= 0 || K % 8 != 0 || tiled.d1 != w4a16_prelayout_words(K, WN) || !contiguous(tiled)) return false;
  *w = View3{tiled.p, tiled.d0, K / 8, WN, (K / 8) * WN, WN, 1};
  return true;
}

}  // namespace
}  // namespace ib200

namespace ib200 {
int w4a16_gemm_f16(View2 x, View2 w, View2 s, View2 y, int g, int zp, cudaStream_t stream) {
  return run<__half>(x, w, s, y, g, zp, stream);
}
int w4a16_gemm_bf16(View2 x, View2 w, View2 s, View2 y, int g, int zp, cudaStream_t stream) {
  return run<__nv_bfloat16>(x, w, s, y, g, zp, stream);
}
}  // namespace ib200

// Reads (and clears) the status words of the tensor-core W4A16 kernels - the single-CTA kernel of this
// file and the CTA-pair kernel, which keeps its own word - and synchronises the device.
extern "C" int intent_b200_w4a16_gemm_device_status(void) {
  int value = 0, pair_value = 0, zero = 0;
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return ib200::cuda_status(e);
  e = cudaMemcpyFromSymbol(&value, ib200::g_w4a16_gemm_status, sizeof(int));
  if (e != cudaSuccess) return ib200::cuda_status(e);
  if (value != 0) cudaMemcpyToSymbol(ib200::g_w4a16_gemm_status, &zero, sizeof(int));
  const int status = ib200::w4a16_gemm_pair_take_status(&pair_value);
  if (status != INTENT_B200_OK) return status;
  return value != 0 ? value : pair_value;
}

#define IB200_GROUPED_ENTRY(NAME, TYPE, MODE)                                                                   \
  extern "C" int NAME(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW3(a3), \
                      INTENT_B200_VIEW3(a4), INTENT_B200_VIEW2(a5), int32_t group_size, int32_t zero_point,      \
                      int32_t block_rows, void* stream) {                                                        \
    return ib200::run_grouped<TYPE, ib200::MODE>(IB200_VIEW2_ARG(a0), IB200_VIEW1_ARG(a1), IB200_VIEW1_ARG(a2),  \
                                                 IB200_VIEW3_ARG(a3), IB200_VIEW3_ARG(a4), IB200_VIEW2_ARG(a5),  \
                                                 group_size, zero_point, block_rows,                             \
                                                 static_cast<cudaStream_t>(stream));                             \
  }
IB200_GROUPED_ENTRY(intent_b200_moe_grouped_w4a16_upgate_silu_bf16, __nv_bfloat16, MODE_UPGATE_SILU)
IB200_GROUPED_ENTRY(intent_b200_moe_grouped_w4a16_upgate_silu_f16, __half, MODE_UPGATE_SILU)
IB200_GROUPED_ENTRY(intent_b200_moe_grouped_w4a16_down_f32_bf16, __nv_bfloat16, MODE_GROUPED_F32)
IB200_GROUPED_ENTRY(intent_b200_moe_grouped_w4a16_down_f32_f16, __half, MODE_GROUPED_F32)

#define IB200_DOWN_SCATTER_ENTRY(NAME, TYPE)                                                                        \
  extern "C" int NAME(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW3(a3),     \
                      INTENT_B200_VIEW3(a4), INTENT_B200_VIEW1(a5), INTENT_B200_VIEW2(a6), INTENT_B200_VIEW2(a7),     \
                      int32_t group_size, int32_t zero_point, int32_t block_rows, void* stream) {                    \
    return ib200::run_down_scatter<TYPE>(IB200_VIEW2_ARG(a0), IB200_VIEW1_ARG(a1), IB200_VIEW1_ARG(a2),              \
                                         IB200_VIEW3_ARG(a3), IB200_VIEW3_ARG(a4), IB200_VIEW1_ARG(a5),              \
                                         IB200_VIEW2_ARG(a6), IB200_VIEW2_ARG(a7), group_size, zero_point,           \
                                         block_rows, static_cast<cudaStream_t>(stream));                             \
  }
IB200_DOWN_SCATTER_ENTRY(intent_b200_moe_grouped_w4a16_down_scatter_bf16, __nv_bfloat16)
IB200_DOWN_SCATTER_ENTRY(intent_b200_moe_grouped_w4a16_down_scatter_f16, __half)

// ---- the same entries on a tiled copy of the weight (w4a16_prelayout.cu) -------------------------------------
#define IB200_TILED_GEMM_ENTRY(NAME, TYPE)                                                                        \
  extern "C" int NAME(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW2(a2), INTENT_B200_VIEW2(a3),   \
                      int32_t group_size, int32_t zero_point, void* stream) {                                      \
    ib200::View2 w;                                                                                                \
    if (!ib200::tiled_as_matrix(IB200_VIEW1_ARG(a1), a0_d1, a2_d1, &w)) return INTENT_B200_ERR_SHAPE;              \
    return ib200::run<TYPE>(IB200_VIEW2_ARG(a0), w, IB200_VIEW2_ARG(a2), IB200_VIEW2_ARG(a3), group_size,          \
                            zero_point, static_cast<cudaStream_t>(stream), true);                                  \
  }
IB200_TILED_GEMM_ENTRY(intent_b200_w4a16_gemm_tiled_f16, __half)
IB200_TILED_GEMM_ENTRY(intent_b200_w4a16_gemm_tiled_bf16, __nv_bfloat16)

#define IB200_TILED_GROUPED_ENTRY(NAME, TYPE, MODE)                                                              \
  extern "C" int NAME(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW2(a3), \
                      INTENT_B200_VIEW3(a4), INTENT_B200_VIEW2(a5), int32_t group_size, int32_t zero_point,      \
                      int32_t block_rows, void* stream) {                                                        \
    ib200::View3 w;                                                                                              \
    if (a4_d0 != a3_d0 || !ib200::tiled_as_experts(IB200_VIEW2_ARG(a3), a0_d1, a4_d2, &w))                       \
      return INTENT_B200_ERR_SHAPE;                                                                              \
    return ib200::run_grouped<TYPE, ib200::MODE>(IB200_VIEW2_ARG(a0), IB200_VIEW1_ARG(a1), IB200_VIEW1_ARG(a2),  \
                                                 w, IB200_VIEW3_ARG(a4), IB200_VIEW2_ARG(a5), group_size,        \
                                                 zero_point, block_rows, static_cast<cudaStream_t>(stream),      \
                                                 true);                                                          \
  }
IB200_TILED_GROUPED_ENTRY(intent_b200_moe_grouped_w4a16_upgate_silu_tiled_bf16, __nv_bfloat16, MODE_UPGATE_SILU)
IB200_TILED_GROUPED_ENTRY(intent_b200_moe_grouped_w4a16_upgate_silu_tiled_f16, __half, MODE_UPGATE_SILU)
IB200_TILED_GROUPED_ENTRY(intent_b200_moe_grouped_w4a16_down_f32_tiled_bf16, __nv_bfloat16, MODE_GROUPED_F32)
IB200_TILED_GROUPED_ENTRY(intent_b200_moe_grouped_w4a16_down_f32_tiled_f16, __half, MODE_GROUPED_F32)

#define IB200_TILED_DOWN_SCATTER_ENTRY(NAME, TYPE)                                                                  \
  extern "C" int NAME(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), INTENT_B200_VIEW1(a2), INTENT_B200_VIEW2(a3),     \
                      INTENT_B200_VIEW3(a4), INTENT_B200_VIEW1(a5), INTENT_B200_VIEW2(a6), INTENT_B200_VIEW2(a7),     \
                      int32_t group_size, int32_t zero_point, int32_t block_rows, void* stream) {                    \
    ib200::View3 w;                                                                                                  \
    if (a4_d0 != a3_d0 || !ib200::tiled_as_experts(IB200_VIEW2_ARG(a3), a0_d1, a4_d2, &w))                           \
      return INTENT_B200_ERR_SHAPE;                                                                                  \
    return ib200::run_down_scatter<TYPE>(IB200_VIEW2_ARG(a0), IB200_VIEW1_ARG(a1), IB200_VIEW1_ARG(a2), w,           \
                                         IB200_VIEW3_ARG(a4), IB200_VIEW1_ARG(a5), IB200_VIEW2_ARG(a6),              \
                                         IB200_VIEW2_ARG(a7), group_size, zero_point, block_rows,                    \
                                         static_cast<cudaStream_t>(stream), true);                                   \
  }
IB200_TILED_DOWN_SCATTER_ENTRY(intent_b200_moe_grouped_w4a16_down_scatter_tiled_bf16, __nv_bfloat16)
IB200_TILED_DOWN_SCATTER_ENTRY(intent_b200_moe_grouped_w4a16_down_scatter_tiled_f16, __half)
