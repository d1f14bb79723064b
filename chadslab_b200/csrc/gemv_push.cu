// Dispatch of the tensor-core GEMV (gemv_mma.cuh) for the row-parallel shard of a tensor-parallel linear: the fp32
// partial sums are stored straight into every rank's receive slot (peer memory over NVLink) instead of a local y.
#include "gemv_mma.cuh"

namespace bq {

int launch_qlinear_mma_push(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K, const void* x,
                            int x_dtype, int64_t M, const CommDev* comm_dev, cudaStream_t s) {
  if (!gemv_mma_supported(fmt, N, K, x_dtype, M)) return fail(BQ_ERR_UNSUPPORTED, "shape not supported by the MMA GEMV");
  const int m = (int)M;
  float* y = reinterpret_cast<float*>(const_cast<CommDev*>(comm_dev));
#define BQ_GM_CASE(F, XT) return gm_pick_nv<F, XT, float, GM_OUT_PUSH>(codes, scales, (const XT*)x, y, N, K, m, N, s)
  if (fmt == BQ_FMT_Q8G32) {
    if (x_dtype == BQ_DT_BF16) BQ_GM_CASE(BQ_FMT_Q8G32, __nv_bfloat16);
    if (x_dtype == BQ_DT_F32) BQ_GM_CASE(BQ_FMT_Q8G32, float);
  } else {
    if (x_dtype == BQ_DT_BF16) BQ_GM_CASE(BQ_FMT_Q4G32, __nv_bfloat16);
    if (x_dtype == BQ_DT_F32) BQ_GM_CASE(BQ_FMT_Q4G32, float);
  }
#undef BQ_GM_CASE
  return fail(BQ_ERR_ARG, "bad dtype");
}

}  // namespace bq
