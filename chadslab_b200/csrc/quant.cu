// Device-side quantizer: fp32 / bf16 weights [N, K] -> the interface layout of the packed formats, bit for bit what
// the host packer produces:
//   scale = fp16_rn(min(absmax / qmax, 65504))          (fp32 division, round to nearest even)
//   code  = clip(rint(w / f32(scale)), -qmax, qmax)      (rint = round half to even; divide by the ROUNDED scale)
//   a group whose scale is 0 (all zero, or absmax / qmax underflows fp16) gets codes 0
//   Q4: nibble = code + 8, element 2j in the low nibble of byte j, element 2j+1 in the high nibble
// One warp per quantization group (32 consecutive k of one row): lane = element.
#include "common.cuh"

namespace bq {

template <typename T, int FMT>
__global__ void __launch_bounds__(256) quantize_kernel(const T* __restrict__ w, uint8_t* __restrict__ codes,
                                                       __half* __restrict__ scales, int64_t n_groups) {
  constexpr float QMAX = FMT == BQ_FMT_Q8G32 ? 127.0f : 7.0f;
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t g = warp0; g < n_groups; g += warps) {
    const float v = to_float<T>(w[g * GROUP + lane]);
    float amax = fabsf(v);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    const __half sh = __float2half_rn(fminf(__fdiv_rn(amax, QMAX), 65504.0f));
    const float s = __half2float(sh);
    float q = 0.0f;
    if (s != 0.0f) q = fminf(fmaxf(rintf(__fdiv_rn(v, s)), -QMAX), QMAX);
    const int c = (int)q;
    if (lane == 0) scales[g] = sh;
    if (FMT == BQ_FMT_Q8G32) {
      codes[g * GROUP + lane] = (uint8_t)(int8_t)c;
    } else {
      const int nib = c + 8;
      const int hi = __shfl_down_sync(0xffffffffu, nib, 1);
      if ((lane & 1) == 0) codes[g * (GROUP / 2) + (lane >> 1)] = (uint8_t)(nib | (hi << 4));
    }
  }
}

}  // namespace bq

using namespace bq;

extern "C" {

int bq_quantize(const void* w, int w_dtype, int64_t N, int64_t K, int fmt, void* codes_out, void* scales_out, void* stream) {
  if (device_id() < 0) return fail(BQ_ERR_STATE, "bq_init() has not been called");
  if (fmt != BQ_FMT_Q8G32 && fmt != BQ_FMT_Q4G32) return fail(BQ_ERR_ARG, "unknown weight format");
  if (w_dtype != BQ_DT_F32 && w_dtype != BQ_DT_BF16) return fail(BQ_ERR_ARG, "w dtype must be BQ_DT_F32 or BQ_DT_BF16");
  if (N < 0 || K <= 0 || K % GROUP) return fail(BQ_ERR_ARG, "K must be a positive multiple of 32");
  if (N == 0) return BQ_OK;
  if (!w || !codes_out || !scales_out) return fail(BQ_ERR_ARG, "null pointer");
  const int64_t groups = N * (K / GROUP);
  int64_t grid = (groups + 7) / 8;
  if (grid > (int64_t)sm_count() * 16) grid = (int64_t)sm_count() * 16;
  cudaStream_t s = (cudaStream_t)stream;
  uint8_t* c = static_cast<uint8_t*>(codes_out);
  __half* sc = static_cast<__half*>(scales_out);
#define BQ_Q_CASE(TT, F) quantize_kernel<TT, F><<<(unsigned)grid, 256, 0, s>>>(static_cast<const TT*>(w), c, sc, groups)
  if (w_dtype == BQ_DT_F32) {
    if (fmt == BQ_FMT_Q8G32) BQ_Q_CASE(float, BQ_FMT_Q8G32); else BQ_Q_CASE(float, BQ_FMT_Q4G32);
  } else {
    if (fmt == BQ_FMT_Q8G32) BQ_Q_CASE(__nv_bfloat16, BQ_FMT_Q8G32); else BQ_Q_CASE(__nv_bfloat16, BQ_FMT_Q4G32);
  }
#undef BQ_Q_CASE
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

}  // extern "C"
