// Tiled copy of a packed int4 weight for the tensor-core W4A16 kernels.
//
// The caller-visible weight format is the reference's: packed [K/8, N] int32, N contiguous, nibble j of a
// word = k % 8 == j (examples/kernels/contraction/weight_only_int4.py:31-39).  In that layout a
// dequantiser thread of the GEMM kernels - it owns one weight column and half of a 64-wide k block - needs
// four words that lie N * 4 bytes apart: four 32-bit loads, four address computations.  A weight that is
// static model state can be re-laid once so that those four words are adjacent:
//
//   tiled[column block cb = n / 128][k block kb = k / 64][part = (k % 64) / 32][n % 128][4 words]
//
// with rows past K/8 and columns past N stored as zeros.  One thread then issues one 16-byte load per k
// block and a warp reads 512 contiguous bytes.  The reference has the same idea at the level of whole
// programs: generated programs and native builds are cached and persisted so that their cost is paid once
// (python/intent/compiler/artifact.py:105-157, python/intent/runtime/native_artifact.py:151-190).
#include "common.cuh"

namespace ib200 {
namespace {

constexpr int kBlockCols = 128, kBlockRows = 8, kParts = 2, kWords = 4;   // 64 k per k block, two parts of 32 k

__global__ void w4a16_prelayout_kernel(const uint32_t* __restrict__ packed, int packed_rows, int N, int k_blocks,
                                       size_t plane_in, size_t plane_out, uint4* __restrict__ tiled) {
  // one thread per output 16-byte group: (plane, cb, kb, part, column)
  const size_t per_plane = plane_out / kWords;
  const size_t total = per_plane * gridDim.y;
  const int plane = blockIdx.y;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < per_plane; i += size_t(gridDim.x) * blockDim.x) {
    const int column = int(i % kBlockCols);
    size_t rest = i / kBlockCols;
    const int part = int(rest % kParts);
    rest /= kParts;
    const int kb = int(rest % k_blocks);
    const int cb = int(rest / k_blocks);
    const int n = cb * kBlockCols + column;
    const int row0 = kb * kBlockRows + part * kWords;
    uint32_t w[kWords];
#pragma unroll
    for (int r = 0; r < kWords; ++r)
      w[r] = (n < N && row0 + r < packed_rows) ? packed[size_t(plane) * plane_in + size_t(row0 + r) * N + n] : 0u;
    tiled[size_t(plane) * per_plane + i] = make_uint4(w[0], w[1], w[2], w[3]);
  }
  (void)total;
}

}  // namespace

// 32-bit words of the tiled copy of one [K/8, N] weight.
int64_t w4a16_prelayout_words(int64_t K, int64_t N) {
  if (K <= 0 || N <= 0 || K % 8 != 0) return 0;
  const int64_t k_blocks = (K + 63) / 64, column_blocks = (N + kBlockCols - 1) / kBlockCols;
  return column_blocks * k_blocks * kParts * kBlockCols * kWords;
}

int w4a16_prelayout(const void* packed, int64_t planes, int64_t K, int64_t N, void* tiled, int64_t tiled_words,
                    cudaStream_t stream) {
  const int64_t words = w4a16_prelayout_words(K, N);
  if (words <= 0 || planes < 0) return INTENT_B200_ERR_SHAPE;
  if (tiled_words < words * planes) return INTENT_B200_ERR_SHAPE;
  if (planes == 0) return INTENT_B200_OK;
  if (!packed || !tiled) return INTENT_B200_ERR_NULL;
  if (!aligned16(packed) || !aligned16(tiled)) return INTENT_B200_ERR_LAYOUT;
  if (K > (1 << 24) || N > (1 << 24) || planes > 65535) return INTENT_B200_ERR_UNSUPPORTED;
  const int64_t groups = words / kWords;
  const int grid = int(groups / 256 < 148 * 8 ? (groups + 255) / 256 : 148 * 8);
  w4a16_prelayout_kernel<<<dim3(grid, unsigned(planes)), 256, 0, stream>>>(
      static_cast<const uint32_t*>(packed), int(K / 8), int(N), int((K + 63) / 64), size_t(K / 8) * size_t(N),
      size_t(words), static_cast<uint4*>(tiled));
  note_launch();
  return launch_status();
}

}  // namespace ib200

extern "C" int64_t intent_b200_w4a16_prelayout_words(int64_t K, int64_t N) {
  return ib200::w4a16_prelayout_words(K, N);
}

// a0 packed [K/8, N] i32 -> a1 tiled [words] i32
extern "C" int intent_b200_w4a16_prelayout(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW1(a1), void* stream) {
  using namespace ib200;
  if (!contiguous(IB200_VIEW2_ARG(a0)) || !contiguous(IB200_VIEW1_ARG(a1))) return INTENT_B200_ERR_LAYOUT;
  return w4a16_prelayout(a0, 1, a0_d0 * 8, a0_d1, a1, a1_d0, static_cast<cudaStream_t>(stream));
}

// a0 packed [E, K/8, N] i32 -> a1 tiled [E, words] i32 (every expert's weight tiled on its own)
extern "C" int intent_b200_w4a16_prelayout_grouped(INTENT_B200_VIEW3(a0), INTENT_B200_VIEW2(a1), void* stream) {
  using namespace ib200;
  if (!contiguous(IB200_VIEW3_ARG(a0)) || !contiguous(IB200_VIEW2_ARG(a1))) return INTENT_B200_ERR_LAYOUT;
  if (a1_d0 != a0_d0) return INTENT_B200_ERR_SHAPE;
  const int64_t words = w4a16_prelayout_words(a0_d1 * 8, a0_d2);
  if (a1_d1 != words) return INTENT_B200_ERR_SHAPE;
  return w4a16_prelayout(a0, a0_d0, a0_d1 * 8, a0_d2, a1, a1_d0 * a1_d1, static_cast<cudaStream_t>(stream));
}
