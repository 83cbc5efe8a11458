// Library identity, status strings, launch counter, and the shape-dispatching
// entry points that choose between the bandwidth and the tensor-core kernels.
#include <atomic>

#include "common.cuh"

namespace ib200 {

static std::atomic<int64_t> g_launches{0};
void note_launch(int count) { g_launches.fetch_add(count, std::memory_order_relaxed); }

int w4a16_skinny_f16(View2, View2, View2, View2, int, int, cudaStream_t);
int w4a16_skinny_bf16(View2, View2, View2, View2, int, int, cudaStream_t);
int w4a16_gemm_f16(View2, View2, View2, View2, int, int, cudaStream_t);
int w4a16_gemm_bf16(View2, View2, View2, View2, int, int, cudaStream_t);

// Rows of activation up to which the bandwidth kernel is used.
constexpr int64_t kSkinnyMaxM = 32;

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
    default: break;
  }
  if (status >= INTENT_B200_ERR_CUDA) return cudaGetErrorString(static_cast<cudaError_t>(status - INTENT_B200_ERR_CUDA));
  return "unknown status";
}

extern "C" int64_t intent_b200_launch_count(void) { return ib200::g_launches.load(std::memory_order_relaxed); }

extern "C" int intent_b200_weight_only_int4_matmul_f16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                       INTENT_B200_VIEW2(a2), INTENT_B200_VIEW2(a3),
                                                       int32_t group_size, int32_t zero_point, void* stream) {
  auto fn = a0_d0 <= ib200::kSkinnyMaxM ? ib200::w4a16_skinny_f16 : ib200::w4a16_gemm_f16;
  return fn(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2), IB200_VIEW2_ARG(a3), group_size,
            zero_point, static_cast<cudaStream_t>(stream));
}

extern "C" int intent_b200_weight_only_int4_matmul_bf16(INTENT_B200_VIEW2(a0), INTENT_B200_VIEW2(a1),
                                                        INTENT_B200_VIEW2(a2), INTENT_B200_VIEW2(a3),
                                                        int32_t group_size, int32_t zero_point, void* stream) {
  auto fn = a0_d0 <= ib200::kSkinnyMaxM ? ib200::w4a16_skinny_bf16 : ib200::w4a16_gemm_bf16;
  return fn(IB200_VIEW2_ARG(a0), IB200_VIEW2_ARG(a1), IB200_VIEW2_ARG(a2), IB200_VIEW2_ARG(a3), group_size,
            zero_point, static_cast<cudaStream_t>(stream));
}
