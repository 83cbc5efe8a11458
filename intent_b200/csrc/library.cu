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

#define IB200_W4A16_ENTRY(NAME, TYPE, SELECT)                                                              \
  extern "C" int NAME(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1), INTENT_B200_VIEW2(a2),                \
                      INTENT_B200_VIEW2(a3), int32_t group_size, int32_t zero_point, void* workspace,     \
                      int64_t workspace_bytes, void* stream) {                                            \
    const bool skinny = SELECT;                                                                           \
    if (skinny)                                                                                           \
      return ib200::w4a16_stream_##TYPE(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2),    \
                                        IB200_VIEW2_ARG(a3), group_size, zero_point, workspace,           \
                                        workspace_bytes, static_cast<cudaStream_t>(stream));              \
    return ib200::w4a16_gemm_##TYPE(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2),        \
                                    IB200_VIEW2_ARG(a3), group_size, zero_point,                          \
                                    static_cast<cudaStream_t>(stream));                                   \
  }

IB200_W4A16_ENTRY(intent_b200_weight_only_int4_matmul_f16, f16, a0_d0 <= ib200::kSkinnyMaxM)
IB200_W4A16_ENTRY(intent_b200_weight_only_int4_matmul_bf16, bf16, a0_d0 <= ib200::kSkinnyMaxM)
IB200_W4A16_ENTRY(intent_b200_w4a16_gemv_f16, f16, true)
IB200_W4A16_ENTRY(intent_b200_w4a16_gemv_bf16, bf16, true)
IB200_W4A16_ENTRY(intent_b200_w4a16_gemm_f16, f16, false)
IB200_W4A16_ENTRY(intent_b200_w4a16_gemm_bf16, bf16, false)

extern "C" int64_t intent_b200_weight_only_int4_matmul_workspace_bytes(int64_t M, int64_t K, int64_t N) {
  return M <= ib200::kSkinnyMaxM ? ib200::w4a16_stream_workspace_bytes(M, K, N) : 0;
}
