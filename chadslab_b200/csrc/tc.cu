// placeholder until the tcgen05 kernels land
#include "common.cuh"
namespace bq {
bool tc_supported(int, int64_t, int64_t, int, int64_t) { return false; }
int launch_qlinear_tc(const uint8_t*, const __half*, int, int64_t, int64_t, const void*, int, int64_t, void*, int,
                      int64_t, cudaStream_t) { return fail(BQ_ERR_UNSUPPORTED, "tensor path not built"); }
bool moe_tc_supported(const Moe*) { return false; }
int launch_moe_experts_tc(const Moe*, const void*, const int32_t*, int64_t, void*, float*, cudaStream_t) {
  return fail(BQ_ERR_UNSUPPORTED, "tensor path not built");
}
}
