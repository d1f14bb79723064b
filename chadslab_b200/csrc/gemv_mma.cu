// Dispatch of the tensor-core GEMV (kernel and launch templates: gemv_mma.cuh) for plain outputs.
#include "gemv_mma.cuh"

namespace bq {

bool gemv_mma_supported(int fmt, int64_t N, int64_t K, int x_dtype, int64_t M) {
  (void)fmt;
  const int nv = (int)M * (x_dtype == BQ_DT_F32 ? 2 : 1);
  return N >= 1 && M >= 1 && nv <= 4 && (K % 128) == 0 && (int64_t)nv * K * 2 <= 160 * 1024;
}

int launch_qlinear_mma(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K, const void* x,
                       int x_dtype, int64_t M, void* y, int y_dtype, int64_t ldy, cudaStream_t s) {
  if (!gemv_mma_supported(fmt, N, K, x_dtype, M)) return fail(BQ_ERR_UNSUPPORTED, "shape not supported by the MMA GEMV");
  const int m = (int)M;
#define BQ_GM_CASE(F, XT, YT) return gm_pick_nv<F, XT, YT, GM_OUT_PLAIN>(codes, scales, (const XT*)x, (YT*)y, N, K, m, ldy, s)
  if (fmt == BQ_FMT_Q8G32) {
    if (x_dtype == BQ_DT_BF16 && y_dtype == BQ_DT_F32) BQ_GM_CASE(BQ_FMT_Q8G32, __nv_bfloat16, float);
    if (x_dtype == BQ_DT_BF16 && y_dtype == BQ_DT_BF16) BQ_GM_CASE(BQ_FMT_Q8G32, __nv_bfloat16, __nv_bfloat16);
    if (x_dtype == BQ_DT_F32 && y_dtype == BQ_DT_F32) BQ_GM_CASE(BQ_FMT_Q8G32, float, float);
    if (x_dtype == BQ_DT_F32 && y_dtype == BQ_DT_BF16) BQ_GM_CASE(BQ_FMT_Q8G32, float, __nv_bfloat16);
  } else {
    if (x_dtype == BQ_DT_BF16 && y_dtype == BQ_DT_F32) BQ_GM_CASE(BQ_FMT_Q4G32, __nv_bfloat16, float);
    if (x_dtype == BQ_DT_BF16 && y_dtype == BQ_DT_BF16) BQ_GM_CASE(BQ_FMT_Q4G32, __nv_bfloat16, __nv_bfloat16);
    if (x_dtype == BQ_DT_F32 && y_dtype == BQ_DT_F32) BQ_GM_CASE(BQ_FMT_Q4G32, float, float);
    if (x_dtype == BQ_DT_F32 && y_dtype == BQ_DT_BF16) BQ_GM_CASE(BQ_FMT_Q4G32, float, __nv_bfloat16);
  }
#undef BQ_GM_CASE
  return fail(BQ_ERR_ARG, "bad dtype");
}

}  // namespace bq
