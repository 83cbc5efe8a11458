// Measurement only: what a per-SM ring of TMA loads streams from HBM, and what a memory fence or an atomic
// inside the consuming loop costs.  This is the bare skeleton of the decode kernels (w4a16_table.cu) with no
// arithmetic: one CTA per SM, `slots` shared-memory slots of 4 KiB, every slot refilled by the warp that
// consumed it.  The matrix is [planes][rows][cols] int32; a unit is a box of 32 x 32 words, numbered column
// tile first, then row chunk, and split evenly over the CTAs plane by plane - the access pattern of the
// packed weights of a decode projection.
//
// sync_mode (every `sync_every`-th unit of a CTA, after the slot has been given back):
//   0 nothing                         3 eight 16-byte stores + a relaxed atomic with a returned value
//   1 __threadfence()                 4 the stores + atom.release.gpu
//   2 the stores + atom.acq_rel.gpu   5 the stores + a relaxed reduction without a returned value
#include "common.cuh"
#include "tma.cuh"

namespace ib200 {
namespace {

struct RingProbe {
  int slots, planes, tiles, chunks, units;
  int sync_mode, sync_every;
  int* counters;      // 1024 ints
  float* scratch;     // gridDim.x * 64 * 32 floats
  int* status;
};

__global__ void __launch_bounds__(512, 1) ring_probe_kernel(const __grid_constant__ CUtensorMap map, const RingProbe p) {
  constexpr int WARPS = 16;
  extern __shared__ unsigned char raw[];
  const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
  const int S = p.slots;
  const uint32_t bars = base + uint32_t(S) * 4096u;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < S; i += WARPS * 32) mbar_init(bars + uint32_t(i) * 8u, 1);
  if (tid == 0) fence_mbar_init();
  __syncthreads();
  const int cta = int(blockIdx.x), ctas = int(gridDim.x);
  const int each = p.units / ctas, extra = p.units % ctas;
  const int u0 = cta * each + min(cta, extra), n = each + (cta < extra ? 1 : 0);
  const int total = n * p.planes;
  auto issue = [&](int seq) {
    const int plane = seq / n, u = u0 + seq % n;
    const uint32_t slot = uint32_t(seq % S), bar = bars + slot * 8u;
    mbar_expect_tx(bar, 4096);
    tma_load_3d(base + slot * 4096u, &map, (u / p.chunks) * 32, (u % p.chunks) * 32, plane, bar);
  };
  if (lane == 0)
    for (int seq = warp; seq < min(total, S); seq += WARPS) issue(seq);
  unsigned acc = 0;
  for (int seq = warp; seq < total; seq += WARPS) {   // slots is a multiple of WARPS: a slot always has the same warp
    const uint32_t slot = uint32_t(seq % S);
    if (!__all_sync(0xffffffffu, mbar_wait(bars + slot * 8u, uint32_t(seq / S) & 1u))) {
      if (lane == 0) atomicExch(p.status, INTENT_B200_ERR_TIMEOUT);
      return;
    }
    const uint4 v = lds128(base + slot * 4096u + uint32_t(lane) * 128u);
    acc ^= v.x ^ v.y ^ v.z ^ v.w;
    if (seq + S < total) {
      __syncwarp();
      fence_proxy_async();
      if (lane == 0) issue(seq + S);
    }
    if (p.sync_mode && (seq % p.sync_every) == 0) {
      float* dst = p.scratch + (size_t(cta) * 64 + (seq & 63)) * 32;
      if (p.sync_mode >= 2 && lane < 8) reinterpret_cast<float4*>(dst)[lane] = make_float4(float(acc), 1.f, 2.f, 3.f);
      __syncwarp();
      int old = 0;
      if (lane == 0) {
        int* c = p.counters + ((cta * 7 + seq) & 1023);
        if (p.sync_mode == 1) __threadfence();
        else if (p.sync_mode == 2) asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(c) : "memory");
        else if (p.sync_mode == 3) old = atomicAdd(c, 1);
        else if (p.sync_mode == 4) asm volatile("atom.release.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(c) : "memory");
        else if (p.sync_mode == 5) asm volatile("red.relaxed.gpu.global.add.s32 [%0], 1;" ::"l"(c) : "memory");
      }
      acc ^= unsigned(__shfl_sync(0xffffffffu, old, 0));
    }
  }
  if (acc == 0x12345678u) atomicAdd(p.counters, 1);   // keeps the reads alive
}

}  // namespace
}  // namespace ib200

// Streams `planes` matrices of [rows][cols] int32 (contiguous, one after another in `matrices`) once through the
// ring and returns the milliseconds of the launch (CUDA events on `stream`), or minus a status code.
// rows and cols must be multiples of 32, slots a multiple of 16 up to 48.  `scratch` is at least
// 8192 + sms * 64 * 32 * 4 bytes of zero-filled device memory; its first word is non-zero afterwards if a
// bounded wait gave up.  No counterpart in the reference.
extern "C" double intent_b200_ring_probe_ms(const void* matrices, int32_t planes, int32_t rows, int32_t cols,
                                            int32_t slots, int32_t sync_mode, int32_t sync_every, void* scratch,
                                            void* stream_handle) {
  using namespace ib200;
  if (!matrices || !scratch) return -double(INTENT_B200_ERR_NULL);
  if (planes < 1 || rows < 32 || cols < 32 || rows % 32 || cols % 32 || slots < 16 || slots > 48 || slots % 16 ||
      sync_mode < 0 || sync_mode > 5 || sync_every < 1)
    return -double(INTENT_B200_ERR_UNSUPPORTED);
  int device = 0, sms = 0;
  if (cudaGetDevice(&device) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
    return -double(INTENT_B200_ERR_UNSUPPORTED);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  CUtensorMap map;
  if (!make_tensor_map_3d(&map, CU_TENSOR_MAP_DATA_TYPE_INT32, matrices, uint64_t(planes), uint64_t(rows), uint64_t(cols),
                          uint64_t(cols) * 4, uint64_t(rows) * uint64_t(cols) * 4, 32, 32, CU_TENSOR_MAP_SWIZZLE_NONE))
    return -double(INTENT_B200_ERR_UNSUPPORTED);
  RingProbe p{};
  p.slots = slots;
  p.planes = planes;
  p.tiles = cols / 32;
  p.chunks = rows / 32;
  p.units = p.tiles * p.chunks;
  p.sync_mode = sync_mode;
  p.sync_every = sync_every;
  p.status = static_cast<int*>(scratch);                  // word 0; non-zero after a bounded wait gave up
  p.counters = static_cast<int*>(scratch) + 16;
  p.scratch = reinterpret_cast<float*>(static_cast<unsigned char*>(scratch) + 8192);
  const int smem = 1024 + slots * 4096 + slots * 8;
  cudaError_t e = cudaFuncSetAttribute(ring_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return -double(cuda_status(e));
  cudaEvent_t start = nullptr, stop = nullptr;
  if (cudaEventCreate(&start) != cudaSuccess || cudaEventCreate(&stop) != cudaSuccess) return -double(INTENT_B200_ERR_UNSUPPORTED);
  cudaEventRecord(start, stream);
  ring_probe_kernel<<<sms, 512, smem, stream>>>(map, p);
  cudaEventRecord(stop, stream);
  e = cudaEventSynchronize(stop);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, start, stop);
  cudaEventDestroy(start);
  cudaEventDestroy(stop);
  if (e != cudaSuccess) return -double(cuda_status(e));
  note_launch();
  return double(ms);
}
