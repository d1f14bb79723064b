// MoE bookkeeping kernels: router softmax/top-k, stable counting-sort permute, row gather,
// deterministic weighted combine, and the CUDA-core grouped SwiGLU expert FFN (exact fp32
// arithmetic; the tensor-core grouped kernel lives in tc.cu).
#include <mutex>

#include "common.cuh"

namespace bq {

// -------------------------------------------------------------------------------------------
// route: one warp per token
// -------------------------------------------------------------------------------------------
template <int VPL>
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, int64_t T, int E,
                                                        int top_k, int renorm, int32_t* __restrict__ idx_out,
                                                        float* __restrict__ w_out) {
  const int lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  float v[VPL];
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int e = lane + 32 * j;
    v[j] = e < E ? logits[t * E + e] : -INFINITY;
    mx = fmaxf(mx, v[j]);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  float all = 0.0f;
  if (!renorm) {
#pragma unroll
    for (int j = 0; j < VPL; ++j) all += (lane + 32 * j < E) ? expf(v[j] - mx) : 0.0f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) all += __shfl_xor_sync(0xffffffffu, all, off);
  }
  float my_e = 0.0f;      // lane s keeps exp of the s-th selected logit
  int my_i = 0;
  float top_sum = 0.0f;
  for (int s = 0; s < top_k; ++s) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int e = lane + 32 * j;   // ascending in j, so strict > keeps the lower index on ties
      if (e < E && v[j] > best) { best = v[j]; bi = e; }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, off);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;  // fewer finite logits than top_k (all -inf / NaN rows)
    const float ex = expf(best - mx);
    top_sum += ex;
    if (lane == s) { my_e = ex; my_i = bi; }
#pragma unroll
    for (int j = 0; j < VPL; ++j)
      if (lane + 32 * j == bi) v[j] = -INFINITY;
  }
  if (lane < top_k) {
    idx_out[t * top_k + lane] = my_i;
    w_out[t * top_k + lane] = my_e / (renorm ? top_sum : all);
  }
}

// -------------------------------------------------------------------------------------------
// permute: stable counting sort of A = T*k assignments by expert id.
// scratch layout: int32 counts[nchunks][E].  One warp owns one contiguous chunk.
// -------------------------------------------------------------------------------------------
constexpr int PERM_WARPS = 4;
static int perm_chunks(int64_t A) {
  int64_t n = (A + 255) / 256;
  if (n > 1024) n = 1024;
  if (n < 1) n = 1;
  return (int)n;
}

__global__ void __launch_bounds__(PERM_WARPS * 32)
moe_hist_kernel(const int32_t* __restrict__ idx, int64_t A, int E, int nchunks, int64_t chunk,
                int32_t* __restrict__ counts) {
  extern __shared__ int32_t cnt[];  // [PERM_WARPS][E]
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int w = blockIdx.x * PERM_WARPS + wib;
  int32_t* c = cnt + wib * E;
  for (int e = lane; e < E; e += 32) c[e] = 0;
  __syncwarp();
  if (w < nchunks) {
    const int64_t a = (int64_t)w * chunk, b = min(A, a + chunk);
    for (int64_t i = a + lane; i < b; i += 32) {
      const int e = idx[i];
      if (e >= 0 && e < E) atomicAdd(&c[e], 1);
    }
    __syncwarp();
    for (int e = lane; e < E; e += 32) counts[(int64_t)w * E + e] = c[e];
  }
}

// one block, E <= 1024 threads: per-expert exclusive scan over chunks, then over experts
__global__ void __launch_bounds__(1024)
moe_scan_kernel(int32_t* __restrict__ counts, int E, int nchunks, int32_t* __restrict__ offsets, int32_t* __restrict__ perm,
                int64_t A) {
  __shared__ int32_t tot[1024];
  const int e = threadIdx.x;
  int32_t run = 0;
  if (e < E) {
    int w = 0;
    for (; w + 4 <= nchunks; w += 4) {
      const int32_t c0 = counts[(int64_t)(w + 0) * E + e], c1 = counts[(int64_t)(w + 1) * E + e];
      const int32_t c2 = counts[(int64_t)(w + 2) * E + e], c3 = counts[(int64_t)(w + 3) * E + e];
      counts[(int64_t)(w + 0) * E + e] = run; run += c0;
      counts[(int64_t)(w + 1) * E + e] = run; run += c1;
      counts[(int64_t)(w + 2) * E + e] = run; run += c2;
      counts[(int64_t)(w + 3) * E + e] = run; run += c3;
    }
    for (; w < nchunks; ++w) {
      const int32_t c0 = counts[(int64_t)w * E + e];
      counts[(int64_t)w * E + e] = run; run += c0;
    }
  }
  tot[e] = e < E ? run : 0;
  __syncthreads();
  // Hillis-Steele inclusive scan over up to 1024 totals
  for (int off = 1; off < 1024; off <<= 1) {
    const int32_t add = e >= off ? tot[e - off] : 0;
    __syncthreads();
    tot[e] += add;
    __syncthreads();
  }
  if (e < E) offsets[e + 1] = tot[e];
  if (e == 0) offsets[0] = 0;
  // assignments with an expert id outside [0, E) are dropped: the sorted positions behind the last segment hold -1
  for (int64_t p = (int64_t)tot[E - 1] + e; p < A; p += 1024) perm[p] = -1;
}

__global__ void __launch_bounds__(PERM_WARPS * 32)
moe_scatter_kernel(const int32_t* __restrict__ idx, int64_t A, int E, int nchunks, int64_t chunk,
                   const int32_t* __restrict__ counts, const int32_t* __restrict__ offsets,
                   int32_t* __restrict__ perm, int32_t* __restrict__ inv) {
  extern __shared__ int32_t cnt[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int w = blockIdx.x * PERM_WARPS + wib;
  if (w >= nchunks) return;
  int32_t* c = cnt + wib * E;
  for (int e = lane; e < E; e += 32) c[e] = counts[(int64_t)w * E + e] + offsets[e];
  __syncwarp();
  const int64_t a = (int64_t)w * chunk, b = min(A, a + chunk);
  for (int64_t base = a; base < b; base += 32) {
    const int64_t i = base + lane;
    const bool valid = i < b;
    int e = valid ? idx[i] : -1;
    const bool ok = valid && e >= 0 && e < E;
    const unsigned act = __ballot_sync(0xffffffffu, ok);
    if (ok) {
      const unsigned same = __match_any_sync(act, e);
      const int rank = __popc(same & ((1u << lane) - 1u));
      const int pos = c[e] + rank;
      __syncwarp(act);
      if (rank == 0) c[e] += __popc(same);
      perm[pos] = (int32_t)i;
      if (inv) inv[i] = pos;
    } else if (valid && inv) {
      inv[i] = -1;  // out-of-range expert id: assignment dropped
    }
    __syncwarp();
  }
}

// Decode-sized sorts (A <= PERM_SMALL_A, E <= PERM_SMALL_E): the three kernels above as ONE single-CTA kernel --
// totals, scan and the stable placement all happen in shared memory, so the sort costs one launch instead of three
// latency-bound ones.  Same results bit for bit (stable: by expert, then by assignment index); needs no scratch.
constexpr int PERM_SMALL_A = 16384;
constexpr int PERM_SMALL_E = 256;
__global__ void __launch_bounds__(1024)
moe_permute_small_kernel(const int32_t* __restrict__ idx, int A, int E, int32_t* __restrict__ perm, int32_t* __restrict__ inv,
                         int32_t* __restrict__ offsets) {
  __shared__ int32_t base[PERM_SMALL_E];          // next free sorted position of every expert
  __shared__ int32_t scan[1024];
  __shared__ int32_t wcnt[32][PERM_SMALL_E];      // per warp: assignments of the current chunk that go to expert e
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  pdl_launch_dependents();
  pdl_wait();
  for (int e = t; e < E; e += 1024) base[e] = 0;
  __syncthreads();
  for (int i = t; i < A; i += 1024) {
    const int e = idx[i];
    if (e >= 0 && e < E) atomicAdd(&base[e], 1);
  }
  __syncthreads();
  const int32_t cnt = t < E ? base[t] : 0;
  scan[t] = cnt;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int32_t add = t >= off ? scan[t - off] : 0;
    __syncthreads();
    scan[t] += add;
    __syncthreads();
  }
  if (t < E) { offsets[t + 1] = scan[t]; base[t] = scan[t] - cnt; }
  if (t == 0) offsets[0] = 0;
  const int32_t valid = scan[E - 1];
  __syncthreads();
  for (int p = valid + t; p < A; p += 1024) perm[p] = -1;      // dropped assignments (expert id outside [0, E))
  for (int c0 = 0; c0 < A; c0 += 1024) {                       // chunks of 1024 assignments, in order
    for (int j = lane; j < E; j += 32) wcnt[warp][j] = 0;
    __syncwarp();
    const int i = c0 + t;
    const int e = i < A ? idx[i] : -1;
    const bool ok = e >= 0 && e < E;
    const unsigned act = __ballot_sync(0xffffffffu, ok);
    int rank = 0;
    if (ok) {
      const unsigned same = __match_any_sync(act, e);
      rank = __popc(same & ((1u << lane) - 1u));
      if (rank == 0) wcnt[warp][e] = __popc(same);
    }
    __syncthreads();
    if (t < E) {                                               // exclusive prefix over the warps, chunk total to base
      int32_t run = 0;
#pragma unroll 4
      for (int w = 0; w < 32; ++w) {
        const int32_t c = wcnt[w][t];
        wcnt[w][t] = run;
        run += c;
      }
      scan[t] = run;                                           // this chunk's count of expert t
    }
    __syncthreads();
    if (ok) {
      const int pos = base[e] + wcnt[warp][e] + rank;
      perm[pos] = i;
      if (inv) inv[i] = pos;
    } else if (i < A && inv) {
      inv[i] = -1;
    }
    __syncthreads();
    if (t < E) base[t] += scan[t];
    __syncthreads();
  }
}

// -------------------------------------------------------------------------------------------
// gather / combine
// -------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_gather_kernel(const uint4* __restrict__ x, int64_t row_vec,
                                                         const int32_t* __restrict__ perm, int64_t P, int top_k,
                                                         uint4* __restrict__ xp) {
  const int64_t total = P * row_vec;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = i / row_vec, c = i - p * row_vec;
    const int32_t a = perm[p];                       // -1: a dropped assignment (expert id out of range) -> zero row
    xp[i] = a >= 0 ? x[(int64_t)(a / top_k) * row_vec + c] : make_uint4(0u, 0u, 0u, 0u);
  }
}

template <typename YT>
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* __restrict__ out,
                                                          const int32_t* __restrict__ inv,
                                                          const float* __restrict__ w, int64_t T, int top_k,
                                                          int64_t H, YT* __restrict__ y) {
  const int64_t total = T * H;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / H, c = i - t * H;
    float acc = 0.0f;
    for (int s = 0; s < top_k; ++s) {      // fixed slot order, separate multiply and add
      const int32_t p = inv[t * top_k + s];
      if (p >= 0) acc = __fadd_rn(acc, __fmul_rn(w[t * top_k + s], out[(int64_t)p * H + c]));
    }
    y[i] = from_float<YT>(acc);
  }
}

// -------------------------------------------------------------------------------------------
// grouped expert FFN, CUDA-core version.  grid = (row tiles, E).  GATED: h = silu(g)*u -> bf16;
// otherwise plain linear -> f32.  Activations are bf16 rows offsets[e]..offsets[e+1].
// -------------------------------------------------------------------------------------------
template <int FMT> struct WordDotM;
template <> struct WordDotM<BQ_FMT_Q8G32> {
  static constexpr int WPW = 4;
  __device__ static __forceinline__ void cvt(uint32_t word, float* f) {
    const uint32_t v = word;   // device bytes are code + 128
    f[0] = q8_byte_to_float<0>(v); f[1] = q8_byte_to_float<1>(v);
    f[2] = q8_byte_to_float<2>(v); f[3] = q8_byte_to_float<3>(v);
  }
};
template <> struct WordDotM<BQ_FMT_Q4G32> {
  static constexpr int WPW = 8;
  __device__ static __forceinline__ void cvt(uint32_t v, float* f) {
    f[q4_elem(0)] = q4_nibble_to_float<0>(v); f[q4_elem(1)] = q4_nibble_to_float<1>(v);
    f[q4_elem(2)] = q4_nibble_to_float<2>(v); f[q4_elem(3)] = q4_nibble_to_float<3>(v);
    f[q4_elem(4)] = q4_nibble_to_float<4>(v); f[q4_elem(5)] = q4_nibble_to_float<5>(v);
    f[q4_elem(6)] = q4_nibble_to_float<6>(v); f[q4_elem(7)] = q4_nibble_to_float<7>(v);
  }
};

constexpr int MOE_MT = 4;
constexpr int MOE_WARPS = 8;

template <int FMT, bool GATED>
__global__ void __launch_bounds__(MOE_WARPS * 32)
moe_ffn_simt_kernel(const uint8_t* const* __restrict__ codesA, const __half* const* __restrict__ scalesA,
                    const uint8_t* const* __restrict__ codesB, const __half* const* __restrict__ scalesB,
                    const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ offsets, int64_t N,
                    int64_t K, void* __restrict__ outp) {
  extern __shared__ __align__(16) float xs[];  // [MOE_MT][K]
  constexpr int WPW = WordDotM<FMT>::WPW;
  constexpr int WPC = WPW * 4;
  const int e = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t a = offsets[e], b = offsets[e + 1];
  if (a >= b) return;
  const uint8_t* cA = codesA[e];
  const __half* sA = scalesA[e];
  const uint8_t* cB = GATED ? codesB[e] : nullptr;
  const __half* sB = GATED ? scalesB[e] : nullptr;
  const int64_t row_bytes = (FMT == BQ_FMT_Q8G32) ? K : K / 2;
  const int64_t groups = K / GROUP;
  const int pieces = (int)(K / WPC);

  for (int64_t m0 = a; m0 < b; m0 += MOE_MT) {
    const int mv = (int)min((int64_t)MOE_MT, b - m0);
    __syncthreads();
    for (int64_t i = threadIdx.x; i < (int64_t)MOE_MT * K; i += blockDim.x) {
      const int m = (int)(i / K);
      const int64_t k = i - (int64_t)m * K;
      xs[i] = m < mv ? __bfloat162float(x[(m0 + m) * K + k]) : 0.0f;
    }
    __syncthreads();
    for (int64_t row = (int64_t)blockIdx.x * MOE_WARPS + warp; row < N; row += (int64_t)gridDim.x * MOE_WARPS) {
      float accA[MOE_MT], accB[MOE_MT];
#pragma unroll
      for (int m = 0; m < MOE_MT; ++m) accA[m] = accB[m] = 0.0f;
      for (int c = lane; c < pieces; c += 32) {
        const uint4 wa = ldg_stream16(cA + row * row_bytes + (int64_t)c * 16);
        uint4 wb = make_uint4(0, 0, 0, 0);
        if (GATED) wb = ldg_stream16(cB + row * row_bytes + (int64_t)c * 16);
        const int g = (c * WPC) / GROUP;
        const float sa = __half2float(sA[row * groups + g]);
        const float sb = GATED ? __half2float(sB[row * groups + g]) : 0.0f;
        float pa[MOE_MT], pb[MOE_MT];
#pragma unroll
        for (int m = 0; m < MOE_MT; ++m) pa[m] = pb[m] = 0.0f;
        const uint32_t wwa[4] = {wa.x, wa.y, wa.z, wa.w};
        const uint32_t wwb[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float fa[WPW], fb[WPW];
          WordDotM<FMT>::cvt(wwa[q], fa);
          if (GATED) WordDotM<FMT>::cvt(wwb[q], fb);
#pragma unroll
          for (int m = 0; m < MOE_MT; ++m) {
            const float* xm = xs + (int64_t)m * K + c * WPC + q * WPW;
#pragma unroll
            for (int j = 0; j < WPW; ++j) {
              pa[m] = fmaf(fa[j], xm[j], pa[m]);
              if (GATED) pb[m] = fmaf(fb[j], xm[j], pb[m]);
            }
          }
        }
#pragma unroll
        for (int m = 0; m < MOE_MT; ++m) {
          accA[m] = fmaf(sa, pa[m], accA[m]);
          if (GATED) accB[m] = fmaf(sb, pb[m], accB[m]);
        }
      }
#pragma unroll
      for (int m = 0; m < MOE_MT; ++m) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          accA[m] += __shfl_xor_sync(0xffffffffu, accA[m], off);
          if (GATED) accB[m] += __shfl_xor_sync(0xffffffffu, accB[m], off);
        }
      }
      if (lane == 0) {
        for (int m = 0; m < mv; ++m) {
          if (GATED) {
            const float gte = accA[m];
            const float h = gte / (1.0f + expf(-gte)) * accB[m];
            ((__nv_bfloat16*)outp)[(m0 + m) * N + row] = __float2bfloat16_rn(h);
          } else {
            ((float*)outp)[(m0 + m) * N + row] = accA[m];
          }
        }
      }
    }
  }
}

static int moe_ffn_simt(const Moe* m, bool gated, const void* x, const int32_t* offsets, void* out,
                        cudaStream_t s) {
  const int64_t N = gated ? m->F : m->H, K = gated ? m->H : m->F;
  const size_t smem = (size_t)MOE_MT * K * sizeof(float);
  if (smem > 200 * 1024) return fail(BQ_ERR_UNSUPPORTED, "expert K too large for the shared-memory stage");
  int64_t gx = (N + MOE_WARPS - 1) / MOE_WARPS;
  const int64_t cap = (sm_count() * 4 + m->E - 1) / m->E;
  if (gx > cap) gx = cap;
  if (gx < 1) gx = 1;
  dim3 grid((unsigned)gx, (unsigned)m->E);
#define BQ_MOE_LAUNCH(F, G)                                                                              \
  do {                                                                                                   \
    auto kern = moe_ffn_simt_kernel<F, G>;                                                               \
    if (smem > 48 * 1024)                                                                                \
      BQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));      \
    kern<<<grid, MOE_WARPS * 32, smem, s>>>(G ? m->gate_codes : m->down_codes,                           \
                                            G ? m->gate_scales : m->down_scales, m->up_codes,            \
                                            m->up_scales, (const __nv_bfloat16*)x, offsets, N, K, out);  \
  } while (0)
  if (m->fmt == BQ_FMT_Q8G32) { if (gated) BQ_MOE_LAUNCH(BQ_FMT_Q8G32, true); else BQ_MOE_LAUNCH(BQ_FMT_Q8G32, false); }
  else                        { if (gated) BQ_MOE_LAUNCH(BQ_FMT_Q4G32, true); else BQ_MOE_LAUNCH(BQ_FMT_Q4G32, false); }
#undef BQ_MOE_LAUNCH
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}


}  // namespace bq

using namespace bq;

static int ready() {
  if (device_id() < 0) return fail(BQ_ERR_STATE, "bq_init() has not been called");
  return BQ_OK;
}

extern "C" {

int bq_moe_route(const float* logits, int64_t T, int E, int top_k, int renormalise, int32_t* idx_out,
                 float* w_out, void* stream) {
  int rc = ready();
  if (rc) return rc;
  if (T < 0 || E <= 0 || E > 1024 || top_k <= 0 || top_k > 32 || top_k > E)
    return fail(BQ_ERR_ARG, "need T >= 0, 1 <= E <= 1024, 1 <= top_k <= min(32, E)");
  if (T == 0) return BQ_OK;
  if (!logits || !idx_out || !w_out) return fail(BQ_ERR_ARG, "null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int wpb = 4;
  const int grid = (int)((T + wpb - 1) / wpb);
  if (E <= 128)      moe_route_kernel<4><<<grid, wpb * 32, 0, s>>>(logits, T, E, top_k, renormalise, idx_out, w_out);
  else if (E <= 256) moe_route_kernel<8><<<grid, wpb * 32, 0, s>>>(logits, T, E, top_k, renormalise, idx_out, w_out);
  else               moe_route_kernel<32><<<grid, wpb * 32, 0, s>>>(logits, T, E, top_k, renormalise, idx_out, w_out);
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

int bq_moe_route_linear(bq_weight_t router, const void* x_bf16, int64_t T, int top_k, int renormalise, int32_t* idx_out,
                        float* w_out, void* stream) {
  int rc = ready();
  if (rc) return rc;
  Weight* w = get_weight(router);
  if (!w) return BQ_ERR_HANDLE;
  if (T < 0 || top_k <= 0 || top_k > 32 || top_k > w->N) return fail(BQ_ERR_ARG, "need T >= 0, 1 <= top_k <= min(32, E)");
  if (T >= ((int64_t)1 << 31)) return fail(BQ_ERR_ARG, "T out of range");
  if (T == 0) return BQ_OK;
  if (!x_bf16 || !idx_out || !w_out) return fail(BQ_ERR_ARG, "null pointer");
  if (!moe_route_linear_supported(w->fmt, w->N, w->K, top_k))
    return fail(BQ_ERR_UNSUPPORTED, "fused router needs E <= 128 and K a multiple of 128: use bq_qlinear + bq_moe_route");
  return launch_moe_route_linear(w->codes, w->scales, w->fmt, w->N, w->K, x_bf16, T, top_k, renormalise, idx_out, w_out,
                                 (cudaStream_t)stream);
}

int64_t bq_moe_permute_scratch_bytes(int64_t T, int top_k, int E) {
  if (T < 0 || top_k <= 0 || E <= 0) return 0;
  return (int64_t)perm_chunks(T * top_k) * E * (int64_t)sizeof(int32_t);
}

int bq_moe_permute(const int32_t* idx, int64_t T, int top_k, int E, int32_t* perm, int32_t* inv,
                   int32_t* offsets, void* scratch, void* stream) {
  int rc = ready();
  if (rc) return rc;
  if (T < 0 || E <= 0 || E > 1024 || top_k <= 0) return fail(BQ_ERR_ARG, "need T >= 0, 1 <= E <= 1024, top_k >= 1");
  if (T * top_k > 0x7fffffff) return fail(BQ_ERR_ARG, "T * top_k exceeds int32 range");
  if (!offsets) return fail(BQ_ERR_ARG, "offsets must not be null");
  cudaStream_t s = (cudaStream_t)stream;
  const int64_t A = T * top_k;
  if (A == 0) {
    BQ_CUDA(cudaMemsetAsync(offsets, 0, sizeof(int32_t) * (E + 1), s));
    return BQ_OK;
  }
  if (!idx || !perm || !scratch) return fail(BQ_ERR_ARG, "null pointer");
  if (A <= PERM_SMALL_A && E <= PERM_SMALL_E) {      // decode-sized: one single-CTA launch (the scratch is not needed)
    BQ_CUDA(launch_chain(moe_permute_small_kernel, dim3(1), dim3(1024), 0, s, 1, idx, (int)A, E, perm, inv, offsets));
    count_launch();
    BQ_CUDA(cudaGetLastError());
    return BQ_OK;
  }
  const int nchunks = perm_chunks(A);
  const int64_t chunk = (A + nchunks - 1) / nchunks;
  const int blocks = (nchunks + PERM_WARPS - 1) / PERM_WARPS;
  const size_t smem = (size_t)PERM_WARPS * E * sizeof(int32_t);
  int32_t* counts = (int32_t*)scratch;
  moe_hist_kernel<<<blocks, PERM_WARPS * 32, smem, s>>>(idx, A, E, nchunks, chunk, counts);
  moe_scan_kernel<<<1, 1024, 0, s>>>(counts, E, nchunks, offsets, perm, A);
  moe_scatter_kernel<<<blocks, PERM_WARPS * 32, smem, s>>>(idx, A, E, nchunks, chunk, counts, offsets, perm, inv);
  count_launch(3);
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

// ---- permute without any allocation ---------------------------------------------------------------------
// Some hosts of this library may not allocate device memory at the point where they sort tokens: a serving
// loop that has handed every free byte of HBM to its KV-cache pool, a plugin that runs under an allocator
// it does not own, or a latency-critical section where a cudaMalloc (which synchronises the device) is
// forbidden.  For them the per-chunk histograms of the counting sort live in this fixed array, which every
// GPU that loads the library holds (512 KiB) until the process exits.
constexpr int64_t PERMUTE_STATIC_INTS = 131072;   // 512 KiB: chunks * experts may not exceed this
static __device__ __align__(256) int32_t g_permute_scratch[PERMUTE_STATIC_INTS];
// The array's name is only a host-side handle; kernels need its device address, fetched once per device.
static int32_t* g_permute_scratch_addr[64] = {nullptr};
static std::mutex g_permute_scratch_mu;

int64_t bq_moe_permute_noalloc_max_bytes(void) { return PERMUTE_STATIC_INTS * (int64_t)sizeof(int32_t); }

int bq_moe_permute_noalloc(const int32_t* idx, int64_t T, int top_k, int E, int32_t* perm, int32_t* inv,
                           int32_t* offsets, void* stream) {
  int rc = ready();
  if (rc) return rc;
  if (T < 0 || E <= 0 || E > 1024 || top_k <= 0) return fail(BQ_ERR_ARG, "need T >= 0, 1 <= E <= 1024, top_k >= 1");
  if (T * top_k > 0x7fffffff) return fail(BQ_ERR_ARG, "T * top_k exceeds int32 range");
  const int64_t need = bq_moe_permute_scratch_bytes(T, top_k, E);
  if (need > bq_moe_permute_noalloc_max_bytes())
    return fail(BQ_ERR_ARG, "bq_moe_permute_noalloc: this T*top_k and E need " + std::to_string(need) +
                                " bytes of histogram scratch, the built-in array holds " +
                                std::to_string(bq_moe_permute_noalloc_max_bytes()) +
                                "; use bq_moe_permute with caller-provided scratch");
  const int dev = device_id();
  if (dev < 0 || dev >= 64) return fail(BQ_ERR_STATE, "device index out of range for the built-in scratch table");
  int32_t* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_permute_scratch_mu);
    if (!g_permute_scratch_addr[dev]) {     // first call on this device: resolve the symbol's device address
      int cur = -1;
      BQ_CUDA(cudaGetDevice(&cur));
      if (cur != dev) BQ_CUDA(cudaSetDevice(dev));       // the look-up answers for the current device
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_permute_scratch);
      if (cur != dev && cur >= 0) cudaSetDevice(cur);    // leave the caller's device selection as it was
      if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(built-in permute scratch)");
      g_permute_scratch_addr[dev] = static_cast<int32_t*>(p);
    }
    scratch = g_permute_scratch_addr[dev];
  }
  // Nothing in the array has to start at zero: the histogram kernel writes every cell the later kernels read.
  return bq_moe_permute(idx, T, top_k, E, perm, inv, offsets, scratch, stream);
}

int bq_moe_gather(const void* x, int dtype, int64_t H, const int32_t* perm, int64_t P, int top_k, void* xp,
                  void* stream) {
  int rc = ready();
  if (rc) return rc;
  if (dtype != BQ_DT_F32 && dtype != BQ_DT_BF16) return fail(BQ_ERR_ARG, "bad dtype");
  const int64_t row_bytes = H * (dtype == BQ_DT_F32 ? 4 : 2);
  if (H <= 0 || row_bytes % 16 != 0) return fail(BQ_ERR_ARG, "row size must be a positive multiple of 16 bytes");
  if (P < 0 || top_k <= 0) return fail(BQ_ERR_ARG, "bad P or top_k");
  if (P == 0) return BQ_OK;
  if (!x || !perm || !xp) return fail(BQ_ERR_ARG, "null pointer");
  const int64_t row_vec = row_bytes / 16;
  int64_t grid = (P * row_vec + 255) / 256;
  if (grid > (int64_t)sm_count() * 16) grid = (int64_t)sm_count() * 16;
  moe_gather_kernel<<<(int)grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)x, row_vec, perm, P, top_k, (uint4*)xp);
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

int bq_moe_experts(bq_moe_t h, const void* xp_bf16, const int32_t* offsets, int64_t P, void* hbuf_bf16,
                   float* out, int path, void* stream) {
  return bq_moe_experts_ex(h, xp_bf16, offsets, P, P, hbuf_bf16, out, path, stream);
}

int bq_moe_experts_ex(bq_moe_t h, const void* xp_bf16, const int32_t* offsets, int64_t P, int64_t rows_hint,
                      void* hbuf_bf16, float* out, int path, void* stream) {
  int rc = ready();
  if (rc) return rc;
  Moe* m = get_moe(h);
  if (!m) return BQ_ERR_HANDLE;
  if (P < 0 || rows_hint < 0 || rows_hint > P) return fail(BQ_ERR_ARG, "need 0 <= rows_hint <= P");
  if (P == 0) return BQ_OK;
  if (!xp_bf16 || !offsets || !hbuf_bf16 || !out) return fail(BQ_ERR_ARG, "null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const bool tc_ok = m->tc_state != nullptr;
  if (path == BQ_PATH_TENSOR && !tc_ok) return fail(BQ_ERR_UNSUPPORTED, "tensor path unavailable for this expert shape");
  // decode sizes (an expert sees about a dozen rows): the batched GEMV streams every expert's weights once per
  // 16-row tile straight from HBM into registers; larger segments amortise the tcgen05 pipeline
  const bool batch_ok = moe_batch_supported(m) && ((reinterpret_cast<uintptr_t>(xp_bf16) | reinterpret_cast<uintptr_t>(hbuf_bf16)) & 15) == 0;
  if (path == BQ_PATH_MMA && !batch_ok) return fail(BQ_ERR_UNSUPPORTED, "batched-GEMV path unavailable for this expert shape");
  if (path == BQ_PATH_MMA || (path == BQ_PATH_AUTO && batch_ok && rows_hint <= (int64_t)m->E * 20)) {
    set_last_path(BQ_PATH_MMA);
    return launch_moe_experts_batch(m, xp_bf16, nullptr, 1, offsets, P, rows_hint, hbuf_bf16, out, s);
  }
  if ((path == BQ_PATH_AUTO && tc_ok) || path == BQ_PATH_TENSOR) {
    set_last_path(BQ_PATH_TENSOR);
    return launch_moe_experts_tc(m, xp_bf16, offsets, P, rows_hint, hbuf_bf16, out, s);
  }
  set_last_path(BQ_PATH_SIMT);
  if ((rc = moe_ffn_simt(m, true, xp_bf16, offsets, hbuf_bf16, s))) return rc;
  return moe_ffn_simt(m, false, hbuf_bf16, offsets, out, s);
}

int bq_moe_experts_tokens(bq_moe_t h, const void* x_bf16, const int32_t* perm, int top_k, const int32_t* offsets, int64_t P,
                          int64_t rows_hint, void* xp_work, void* hbuf_bf16, float* out, int path, void* stream) {
  int rc = ready();
  if (rc) return rc;
  Moe* m = get_moe(h);
  if (!m) return BQ_ERR_HANDLE;
  if (P < 0 || rows_hint < 0 || rows_hint > P || top_k <= 0) return fail(BQ_ERR_ARG, "need 0 <= rows_hint <= P and top_k >= 1");
  if (P == 0) return BQ_OK;
  if (!x_bf16 || !perm || !offsets || !hbuf_bf16 || !out) return fail(BQ_ERR_ARG, "null pointer");
  const bool batch_ok = moe_batch_supported(m) && ((reinterpret_cast<uintptr_t>(x_bf16) | reinterpret_cast<uintptr_t>(hbuf_bf16)) & 15) == 0;
  if (path == BQ_PATH_MMA && !batch_ok) return fail(BQ_ERR_UNSUPPORTED, "batched-GEMV path unavailable for this expert shape");
  if (path == BQ_PATH_MMA || (path == BQ_PATH_AUTO && batch_ok && rows_hint <= (int64_t)m->E * 20)) {
    set_last_path(BQ_PATH_MMA);             // the kernel reads the token rows through perm: no gathered copy
    return launch_moe_experts_batch(m, x_bf16, perm, top_k, offsets, P, rows_hint, hbuf_bf16, out, (cudaStream_t)stream);
  }
  if (!xp_work) return fail(BQ_ERR_ARG, "this path needs the gathered rows: xp_work must not be null");
  if ((rc = bq_moe_gather(x_bf16, BQ_DT_BF16, m->H, perm, P, top_k, xp_work, stream))) return rc;
  return bq_moe_experts_ex(h, xp_work, offsets, P, rows_hint, hbuf_bf16, out, path, stream);
}

int bq_moe_combine(const float* out, const int32_t* inv, const float* w, int64_t T, int top_k, int64_t H,
                   void* y, int y_dtype, void* stream) {
  int rc = ready();
  if (rc) return rc;
  if (T < 0 || top_k <= 0 || H <= 0) return fail(BQ_ERR_ARG, "bad sizes");
  if (y_dtype != BQ_DT_F32 && y_dtype != BQ_DT_BF16) return fail(BQ_ERR_ARG, "bad dtype");
  if (T == 0) return BQ_OK;
  if (!out || !inv || !w || !y) return fail(BQ_ERR_ARG, "null pointer");
  int64_t grid = (T * H + 255) / 256;
  if (grid > (int64_t)sm_count() * 16) grid = (int64_t)sm_count() * 16;
  cudaStream_t s = (cudaStream_t)stream;
  if (y_dtype == BQ_DT_F32)
    moe_combine_kernel<float><<<(int)grid, 256, 0, s>>>(out, inv, w, T, top_k, H, (float*)y);
  else
    moe_combine_kernel<__nv_bfloat16><<<(int)grid, 256, 0, s>>>(out, inv, w, T, top_k, H, (__nv_bfloat16*)y);
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

}  // extern "C"
