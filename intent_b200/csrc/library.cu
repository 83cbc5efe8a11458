// Library identity, status strings, launch counter, and the shape-dispatching
// entry points that choose between the bandwidth and the tensor-core kernels.
#include <atomic>

#include "common.cuh"

namespace ib200 {

static std::atomic<int64_t> g_launches{0};
void note_launch(int count) { g_launches.fetch_add(count, std::memory_order_relaxed); }

int w4a16_stream_f16(View2, View2, View2, View2, int, int, void*, int64_t, cudaStream_t);
int w4a16_stream_bf16(View2, View2, View2, View2, int, int, void*, int64_t, cudaStream_t);
int64_t w4a16_stream_workspace_bytes(int64_t M, int64_t K, int64_t N);
int w4a16_gemm_f16(View2, View2, View2, View2, int, int, cudaStream_t);
int w4a16_gemm_bf16(View2, View2, View2, View2, int, int, cudaStream_t);

// Rows of activation up to which the bandwidth kernel is used.
constexpr int64_t kSkinnyMaxM = 16;

}  // namespace ib200

namespace ib200 {
static thread_local LaunchFacts* t_sink = nullptr;
LaunchFacts* observe_sink() { return t_sink; }
int record_launch(LaunchFacts* sink, const void* kernel, const char* name, int grid, int threads, int dynamic_smem,
                  int cluster) {
  cudaFuncAttributes attributes;
  const cudaError_t e = cudaFuncGetAttributes(&attributes, kernel);
  if (e != cudaSuccess) return cuda_status(e);
  if (sink->valid) return INTENT_B200_OK;    // an entry of several kernels reports its first (dominant) one
  sink->valid = 1;
  sink->registers = attributes.numRegs;
  sink->local_bytes = int(attributes.localSizeBytes);
  sink->static_smem = int(attributes.sharedSizeBytes);
  sink->dynamic_smem = dynamic_smem;
  sink->threads = threads;
  sink->grid = grid;
  sink->cluster = cluster;
  int i = 0;
  for (; name[i] && i < int(sizeof(sink->kernel)) - 1; ++i) sink->kernel[i] = name[i];
  sink->kernel[i] = 0;
  return INTENT_B200_OK;
}
}  // namespace ib200

// Observation of a call without launching it: between begin and end, on the calling thread, the entries of the
// dense / grouped / bandwidth kernels record the launch they would make into `facts` (layout: eight int32 -
// valid, registers per thread, local bytes per thread, static shared bytes, dynamic shared bytes, threads per
// CTA, CTAs, CTAs per cluster - then 64 bytes of kernel name) and return without launching.
extern "C" int intent_b200_observe_begin(void* facts) {
  if (!facts) return INTENT_B200_ERR_NULL;
  ib200::LaunchFacts* sink = static_cast<ib200::LaunchFacts*>(facts);
  *sink = ib200::LaunchFacts{};
  ib200::t_sink = sink;
  return INTENT_B200_OK;
}
extern "C" int intent_b200_observe_end(void) {
  ib200::t_sink = nullptr;
  return INTENT_B200_OK;
}

extern "C" const char* intent_b200_version(void) { return "intent_b200 0.1 sm_100a"; }

extern "C" const char* intent_b200_status_string(int status) {
  switch (status) {
    case INTENT_B200_OK: return "ok";
    case INTENT_B200_ERR_SHAPE: return "extent mismatch";
    case INTENT_B200_ERR_LAYOUT: return "view is not contiguous or not 16-byte aligned";
    case INTENT_B200_ERR_UNSUPPORTED: return "no kernel specialisation for these arguments";
    case INTENT_B200_ERR_TIMEOUT: return "bounded device wait expired";
    case INTENT_B200_ERR_WORKSPACE: return "workspace missing or too small";
    case INTENT_B200_ERR_NULL: return "null pointer";
    case INTENT_B200_ERR_SCRATCH_LIMIT: return "problem exceeds the built-in scratch of the no-allocation entry";
    case INTENT_B200_ERR_INDEX: return "an index read from device memory was out of range";
    default: break;
  }
  if (status >= INTENT_B200_ERR_CUDA) return cudaGetErrorString(static_cast<cudaError_t>(status - INTENT_B200_ERR_CUDA));
  return "unknown status";
}

extern "C" int64_t intent_b200_launch_count(void) { return ib200::g_launches.load(std::memory_order_relaxed); }

#define IB200_W4A16_ENTRY(NAME, TYPE, SELECT, TABLE)                                                              \
  extern "C" int NAME(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),                \
                      INTENT_B200_VIEW2(a3), int32_t group_size, int32_t zero_point, void* workspace,     \
                      int64_t workspace_bytes, void* stream) {                                            \
    const bool skinny = SELECT;                                                                           \
    if (skinny && (TABLE)) {                                                                              \
      const int status = ib200::w4a16_table_single_##TYPE(                                                \
          IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2), IB200_VIEW2_ARG(a3), group_size, \
          zero_point, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));                     \
      if (status != ib200::kTableDeclined) return status;                                                 \
    }                                                                                                     \
    if (skinny)                                                                                           \
      return ib200::w4a16_stream_##TYPE(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2),    \
                                        IB200_VIEW2_ARG(a3), group_size, zero_point, workspace,           \
                                        workspace_bytes, static_cast<cudaStream_t>(stream));              \
    return ib200::w4a16_gemm_##TYPE(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2),        \
                                    IB200_VIEW2_ARG(a3), group_size, zero_point,                          \
                                    static_cast<cudaStream_t>(stream));                                   \
  }

IB200_W4A16_ENTRY(intent_b200_weight_only_int4_matmul_f16, f16, a0_d0 <= ib200::kSkinnyMaxM, a0_d0 >= 2)
IB200_W4A16_ENTRY(intent_b200_weight_only_int4_matmul_bf16, bf16, a0_d0 <= ib200::kSkinnyMaxM, a0_d0 >= 2)
IB200_W4A16_ENTRY(intent_b200_w4a16_gemv_f16, f16, true, false)
IB200_W4A16_ENTRY(intent_b200_w4a16_gemv_bf16, bf16, true, false)
IB200_W4A16_ENTRY(intent_b200_w4a16_gemm_f16, f16, false, false)
IB200_W4A16_ENTRY(intent_b200_w4a16_gemm_bf16, bf16, false, false)

extern "C" int64_t intent_b200_weight_only_int4_matmul_workspace_bytes(int64_t M, int64_t K, int64_t N) {
  if (M > ib200::kSkinnyMaxM) return 0;
  const int64_t stream_bytes = ib200::w4a16_stream_workspace_bytes(M, K, N);
  const int64_t table_bytes = ib200::w4a16_table_single_workspace_bytes(M, K, N);   // 0 unless it can run as a table of one
  return stream_bytes > table_bytes ? stream_bytes : table_bytes;
}

// ---------------------------------------------------------------------------------------------
// entry_benchmark counterparts.  The reference's native ABI exports, beside every `entry(slots...)`,
// `double entry_benchmark(slots..., int64 repetitions)` so that a harness can time a compiled program
// without going through Python (python/intent/runtime/mojo/compilation.py:54-96,
// python/intent/runtime/mojo/program.py:253-257).  Here: the same slots as the entry, then `repetitions`,
// then the stream.  One untimed call comes first (it also validates the arguments), then `repetitions`
// calls are bracketed by two CUDA events on `stream`; the events are the only synchronisation.  Returns
// the mean milliseconds per call, or minus the status code of a failed call.
// ---------------------------------------------------------------------------------------------
namespace ib200 {
template <typename Launch>
double benchmark_entry(int64_t repetitions, void* stream_handle, Launch launch) {
  if (repetitions <= 0) return -double(INTENT_B200_ERR_SHAPE);
  cudaStream_t stream = static_cast<cudaStream_t>(stream_handle);
  int status = launch();
  if (status != INTENT_B200_OK) return -double(status);
  cudaEvent_t start = nullptr, stop = nullptr;
  cudaError_t e = cudaEventCreate(&start);
  if (e == cudaSuccess) e = cudaEventCreate(&stop);
  if (e == cudaSuccess) e = cudaEventRecord(start, stream);
  for (int64_t i = 0; e == cudaSuccess && status == INTENT_B200_OK && i < repetitions; ++i) status = launch();
  if (e == cudaSuccess) e = cudaEventRecord(stop, stream);
  if (e == cudaSuccess) e = cudaEventSynchronize(stop);
  float ms = 0.f;
  if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, start, stop);
  if (start) cudaEventDestroy(start);
  if (stop) cudaEventDestroy(stop);
  if (status != INTENT_B200_OK) return -double(status);
  if (e != cudaSuccess) return -double(cuda_status(e));
  return double(ms) / double(repetitions);
}
}  // namespace ib200

#define IB200_W4A16_BENCHMARK(NAME, ENTRY)                                                                   \
  extern "C" double NAME(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),               \
                         INTENT_B200_VIEW2(a3), int32_t group_size, int32_t zero_point, void* workspace,    \
                         int64_t workspace_bytes, int64_t repetitions, void* stream) {                      \
    return ib200::benchmark_entry(repetitions, stream, [&] {                                                \
      return ENTRY(a0, a0_d0, a0_d1, a0_s0, a0_s1, a1, a1_d0, a1_d1, a1_s0, a1_s1, a2, a2_d0, a2_d1, a2_s0,  \
                   a2_s1, a3, a3_d0, a3_d1, a3_s0, a3_s1, group_size, zero_point, workspace, workspace_bytes, \
                   stream);                                                                                  \
    });                                                                                                     \
  }
IB200_W4A16_BENCHMARK(intent_b200_weight_only_int4_matmul_f16_benchmark, intent_b200_weight_only_int4_matmul_f16)
IB200_W4A16_BENCHMARK(intent_b200_weight_only_int4_matmul_bf16_benchmark, intent_b200_weight_only_int4_matmul_bf16)

extern "C" double intent_b200_gemm_i8_benchmark(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW1(a2),
                                                INTENT_B200_VIEW2(a3), int64_t repetitions, void* stream) {
  return ib200::benchmark_entry(repetitions, stream, [&] {
    return intent_b200_gemm_i8(a0, a0_d0, a0_d1, a0_s0, a0_s1, a1, a1_d0, a1_d1, a1_s0, a1_s1, a2, a2_d0, a2_s0, a3,
                               a3_d0, a3_d1, a3_s0, a3_s1, stream);
  });
}

extern "C" double intent_b200_w8a8_gemm_bf16_benchmark(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                       INTENT_B200_VIEW1(a2), INTENT_B200_VIEW1(a3),
                                                       INTENT_B200_VIEW2(a4), int64_t repetitions, void* stream) {
  return ib200::benchmark_entry(repetitions, stream, [&] {
    return intent_b200_w8a8_gemm_bf16(a0, a0_d0, a0_d1, a0_s0, a0_s1, a1, a1_d0, a1_d1, a1_s0, a1_s1, a2, a2_d0,
                                      a2_s0, a3, a3_d0, a3_s0, a4, a4_d0, a4_d1, a4_s0, a4_s1, stream);
  });
}
