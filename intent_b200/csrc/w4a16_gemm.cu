// placeholder until the tcgen05 kernel lands
#include "common.cuh"
namespace ib200 {
int w4a16_gemm_f16(View2, View2, View2, View2, int, int, cudaStream_t) { return INTENT_B200_ERR_UNSUPPORTED; }
int w4a16_gemm_bf16(View2, View2, View2, View2, int, int, cudaStream_t) { return INTENT_B200_ERR_UNSUPPORTED; }
}
