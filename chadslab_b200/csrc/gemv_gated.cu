// Dispatch of the tensor-core GEMV (gemv_mma.cuh) for a fused gate|up projection with the gated activation applied in
// the epilogue: the weight's 16-row blocks hold 8 gate rows followed by the 8 up rows of the same output columns.
#include "gemv_mma.cuh"

namespace bq {

int launch_qlinear_mma_gated(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K, const void* x,
                             int x_dtype, int64_t M, void* out, int act, cudaStream_t s) {
  if (!gemv_mma_supported(fmt, N, K, x_dtype, M) || (N % 16) != 0)
    return fail(BQ_ERR_UNSUPPORTED, "shape not supported by the MMA GEMV");
  const int m = (int)M;
  const int64_t ldo = N / 2;
#define BQ_GM_CASE(F, XT, O) return gm_pick_nv<F, XT, XT, O>(codes, scales, (const XT*)x, (XT*)out, N, K, m, ldo, s)
#define BQ_GM_ACT(F, XT)                        \
  do {                                          \
    if (act == 0) BQ_GM_CASE(F, XT, GM_OUT_GELU); \
    BQ_GM_CASE(F, XT, GM_OUT_SILU);             \
  } while (0)
  if (fmt == BQ_FMT_Q8G32) {
    if (x_dtype == BQ_DT_BF16) BQ_GM_ACT(BQ_FMT_Q8G32, __nv_bfloat16);
    if (x_dtype == BQ_DT_F32) BQ_GM_ACT(BQ_FMT_Q8G32, float);
  } else {
    if (x_dtype == BQ_DT_BF16) BQ_GM_ACT(BQ_FMT_Q4G32, __nv_bfloat16);
    if (x_dtype == BQ_DT_F32) BQ_GM_ACT(BQ_FMT_Q4G32, float);
  }
#undef BQ_GM_ACT
#undef BQ_GM_CASE
  return fail(BQ_ERR_ARG, "bad dtype");
}

}  // namespace bq
