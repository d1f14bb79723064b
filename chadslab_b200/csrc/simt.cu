// CUDA-core kernels: exact dequantize / unpack, the decode-shaped GEMV (M = 1..4 per pass,
// fp32 arithmetic throughout) and the lm_head argmax.
//
// GEMV data flow (HBM-bound): every lane streams 16-byte pieces of packed codes with
// 128-bit non-allocating loads (a warp instruction covers 512 contiguous bytes of one row),
// unpacks them to fp32 in registers with mantissa-insertion tricks (no I2F), multiplies
// against the activation vector held as fp32 in shared memory, applies the fp16 group scale
// once per 16 (Q8) or 32 (Q4) weights, and reduces across the warp with shuffles.
// A warp works on R rows at a time so each activation fetched from shared memory is used R
// times and R independent 16-byte loads per lane are in flight.
#include "common.cuh"

namespace bq {

// -------------------------------------------------------------------------------------------
// dequantize / unpack : one thread per 16-byte piece of codes
// -------------------------------------------------------------------------------------------
template <int FMT, typename OT>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ codes,
                                                      const __half* __restrict__ scales,
                                                      OT* __restrict__ out, int64_t N, int64_t K) {
  constexpr int WPC = (FMT == BQ_FMT_Q8G32) ? 16 : 32;  // weights per 16-byte piece
  const int64_t pieces_per_row = K / WPC;
  const int64_t total = N * pieces_per_row;
  for (int64_t p = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; p < total;
       p += (int64_t)gridDim.x * blockDim.x) {
    const int64_t row = p / pieces_per_row;
    const int64_t c = p - row * pieces_per_row;
    const uint4 w = *reinterpret_cast<const uint4*>(codes + p * 16);
    const int64_t k0 = c * WPC;
    const float s = __half2float(scales[row * (K / GROUP) + k0 / GROUP]);
    OT* o = out + row * K + k0;
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (FMT == BQ_FMT_Q8G32) {
        const uint32_t v = words[q];   // device bytes are code + 128
        o[4 * q + 0] = from_float<OT>(q8_byte_to_float<0>(v) * s);
        o[4 * q + 1] = from_float<OT>(q8_byte_to_float<1>(v) * s);
        o[4 * q + 2] = from_float<OT>(q8_byte_to_float<2>(v) * s);
        o[4 * q + 3] = from_float<OT>(q8_byte_to_float<3>(v) * s);
      } else {
        const uint32_t v = words[q];
        o[8 * q + q4_elem(0)] = from_float<OT>(q4_nibble_to_float<0>(v) * s);
        o[8 * q + q4_elem(1)] = from_float<OT>(q4_nibble_to_float<1>(v) * s);
        o[8 * q + q4_elem(2)] = from_float<OT>(q4_nibble_to_float<2>(v) * s);
        o[8 * q + q4_elem(3)] = from_float<OT>(q4_nibble_to_float<3>(v) * s);
        o[8 * q + q4_elem(4)] = from_float<OT>(q4_nibble_to_float<4>(v) * s);
        o[8 * q + q4_elem(5)] = from_float<OT>(q4_nibble_to_float<5>(v) * s);
        o[8 * q + q4_elem(6)] = from_float<OT>(q4_nibble_to_float<6>(v) * s);
        o[8 * q + q4_elem(7)] = from_float<OT>(q4_nibble_to_float<7>(v) * s);
      }
    }
  }
}

// one thread per 32-bit word of codes (row sizes are multiples of 16 bytes)
template <int FMT>
__global__ void __launch_bounds__(256) unpack_kernel(const uint8_t* __restrict__ codes,
                                                     int8_t* __restrict__ out, int64_t total_bytes) {
  const int64_t words = total_bytes / 4;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < words;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t v = reinterpret_cast<const uint32_t*>(codes)[i];
    if (FMT == BQ_FMT_Q8G32) {
      reinterpret_cast<uint32_t*>(out)[i] = v ^ 0x80808080u;   // device bytes are code + 128
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) out[8 * i + q4_elem(j)] = (int8_t)((int)((v >> (4 * j)) & 0xF) - 8);
    }
  }
}

// interface encoding <-> device encoding, in place, one thread per word.
// Q8: every byte is stored as code + 128 (flip the sign bit), so unpacking needs no sign fix-up.
// Q4: nibble order inside the word (see q4_elem).
__global__ void __launch_bounds__(256) q4_repack_kernel(uint32_t* __restrict__ words, int64_t n, int to_device, int q8) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t v = words[i];
    if (q8) { words[i] = v ^ 0x80808080u; continue; }
    uint32_t o = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (to_device) o |= ((v >> (4 * q4_elem(j))) & 0xFu) << (4 * j);   // device nibble j <- element q4_elem(j)
      else           o |= ((v >> (4 * j)) & 0xFu) << (4 * q4_elem(j));
    }
    words[i] = o;
  }
}

static int grid_for(int64_t work_items, int block) {
  int64_t g = (work_items + block - 1) / block;
  int64_t cap = (int64_t)sm_count() * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

int launch_dequant(const Weight* w, void* out, int out_dtype, cudaStream_t s) {
  const int wpc = w->fmt == BQ_FMT_Q8G32 ? 16 : 32;
  const int64_t pieces = w->N * (w->K / wpc);
  if (pieces == 0) return BQ_OK;
  const int grid = grid_for(pieces, 256);
  if (w->fmt == BQ_FMT_Q8G32) {
    if (out_dtype == BQ_DT_F32)
      dequant_kernel<BQ_FMT_Q8G32, float><<<grid, 256, 0, s>>>(w->codes, w->scales, (float*)out, w->N, w->K);
    else
      dequant_kernel<BQ_FMT_Q8G32, __nv_bfloat16><<<grid, 256, 0, s>>>(w->codes, w->scales, (__nv_bfloat16*)out, w->N, w->K);
  } else {
    if (out_dtype == BQ_DT_F32)
      dequant_kernel<BQ_FMT_Q4G32, float><<<grid, 256, 0, s>>>(w->codes, w->scales, (float*)out, w->N, w->K);
    else
      dequant_kernel<BQ_FMT_Q4G32, __nv_bfloat16><<<grid, 256, 0, s>>>(w->codes, w->scales, (__nv_bfloat16*)out, w->N, w->K);
  }
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

int launch_device_encode(uint8_t* codes, size_t bytes, int fmt, bool to_device_layout, cudaStream_t s) {
  if (bytes == 0) return BQ_OK;
  const int64_t n = (int64_t)(bytes / 4);
  q4_repack_kernel<<<grid_for(n, 256), 256, 0, s>>>(reinterpret_cast<uint32_t*>(codes), n, to_device_layout ? 1 : 0,
                                                    fmt == BQ_FMT_Q8G32 ? 1 : 0);
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

int launch_unpack(const Weight* w, int8_t* out, cudaStream_t s) {
  const int64_t bytes = (int64_t)w->codes_bytes;
  if (bytes == 0) return BQ_OK;
  const int grid = grid_for(bytes / 4, 256);
  if (w->fmt == BQ_FMT_Q8G32)
    unpack_kernel<BQ_FMT_Q8G32><<<grid, 256, 0, s>>>(w->codes, out, bytes);
  else
    unpack_kernel<BQ_FMT_Q4G32><<<grid, 256, 0, s>>>(w->codes, out, bytes);
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

// -------------------------------------------------------------------------------------------
// GEMV
// -------------------------------------------------------------------------------------------
constexpr int GEMV_WARPS = 8;

// dot of one 32-bit word of codes against fp32 activations
template <int FMT> struct WordDot;
template <> struct WordDot<BQ_FMT_Q8G32> {
  static constexpr int WPW = 4;  // weights per word
  __device__ static __forceinline__ float run(uint32_t word, const float* xv, float acc) {
    const uint32_t v = word;   // device bytes are code + 128
    acc = fmaf(q8_byte_to_float<0>(v), xv[0], acc);
    acc = fmaf(q8_byte_to_float<1>(v), xv[1], acc);
    acc = fmaf(q8_byte_to_float<2>(v), xv[2], acc);
    acc = fmaf(q8_byte_to_float<3>(v), xv[3], acc);
    return acc;
  }
};
template <> struct WordDot<BQ_FMT_Q4G32> {
  static constexpr int WPW = 8;
  __device__ static __forceinline__ float run(uint32_t v, const float* xv, float acc) {
    acc = fmaf(q4_nibble_to_float<0>(v), xv[q4_elem(0)], acc);
    acc = fmaf(q4_nibble_to_float<1>(v), xv[q4_elem(1)], acc);
    acc = fmaf(q4_nibble_to_float<2>(v), xv[q4_elem(2)], acc);
    acc = fmaf(q4_nibble_to_float<3>(v), xv[q4_elem(3)], acc);
    acc = fmaf(q4_nibble_to_float<4>(v), xv[q4_elem(4)], acc);
    acc = fmaf(q4_nibble_to_float<5>(v), xv[q4_elem(5)], acc);
    acc = fmaf(q4_nibble_to_float<6>(v), xv[q4_elem(6)], acc);
    acc = fmaf(q4_nibble_to_float<7>(v), xv[q4_elem(7)], acc);
    return acc;
  }
};

// x: [MT rows, K] of XT (row stride ldx); y: [MT rows, N] of YT (row stride ldy).
template <int FMT, typename XT, typename YT, int MT, int R>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
qgemv_simt_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ scales,
                  const XT* __restrict__ x, YT* __restrict__ y, int64_t N, int64_t K, int m_valid,
                  int64_t ldx, int64_t ldy) {
  extern __shared__ __align__(16) float xs[];  // [MT][K] fp32
  constexpr int WPW = WordDot<FMT>::WPW;
  constexpr int WPC = WPW * 4;                 // weights per 16-byte piece
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;

  for (int64_t i = threadIdx.x; i < (int64_t)MT * K; i += blockDim.x) {
    const int m = (int)(i / K);
    const int64_t k = i - (int64_t)m * K;
    xs[i] = (m < m_valid) ? to_float<XT>(x[(int64_t)m * ldx + k]) : 0.0f;
  }
  __syncthreads();

  const int64_t row_bytes = (FMT == BQ_FMT_Q8G32) ? K : K / 2;
  const int64_t groups = K / GROUP;
  const int pieces = (int)(K / WPC);           // 16-byte pieces per row

  for (int64_t rowbase = ((int64_t)blockIdx.x * GEMV_WARPS + warp) * R; rowbase < N;
       rowbase += (int64_t)gridDim.x * GEMV_WARPS * R) {
    float acc[R][MT];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) acc[r][m] = 0.0f;

    const uint8_t* rowp[R];
    const __half* scp[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      int64_t row = rowbase + r;
      if (row >= N) row = N - 1;               // clamp: result discarded below
      rowp[r] = codes + row * row_bytes;
      scp[r] = scales + row * groups;
    }

#pragma unroll 2
    for (int c = lane; c < pieces; c += 32) {
      uint4 w[R];
      float sc[R];
#pragma unroll
      for (int r = 0; r < R; ++r) w[r] = ldg_stream16(rowp[r] + (int64_t)c * 16);
      const int g = (c * WPC) / GROUP;
#pragma unroll
      for (int r = 0; r < R; ++r) sc[r] = __half2float(__ldg(scp[r] + g));
      const int k0 = c * WPC;
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float part[R];
#pragma unroll
        for (int r = 0; r < R; ++r) part[r] = 0.0f;
        const float* xm = xs + (int64_t)m * K + k0;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float xv[WPW];
#pragma unroll
          for (int v4 = 0; v4 < WPW / 4; ++v4) {
            const float4 t = *reinterpret_cast<const float4*>(xm + q * WPW + v4 * 4);
            xv[v4 * 4 + 0] = t.x; xv[v4 * 4 + 1] = t.y; xv[v4 * 4 + 2] = t.z; xv[v4 * 4 + 3] = t.w;
          }
#pragma unroll
          for (int r = 0; r < R; ++r) {
            const uint32_t word = q == 0 ? w[r].x : q == 1 ? w[r].y : q == 2 ? w[r].z : w[r].w;
            part[r] = WordDot<FMT>::run(word, xv, part[r]);
          }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r][m] = fmaf(sc[r], part[r], acc[r][m]);
      }
    }

#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int m = 0; m < MT; ++m) {
        float v = acc[r][m];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        acc[r][m] = v;
      }
    if (lane == 0) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int64_t row = rowbase + r;
        if (row < N) {
#pragma unroll
          for (int m = 0; m < MT; ++m)
            if (m < m_valid) y[(int64_t)m * ldy + row] = from_float<YT>(acc[r][m]);
        }
      }
    }
  }
}

template <int FMT, typename XT, typename YT, int MT, int R>
static int launch_simt_tile(const uint8_t* codes, const __half* scales, int64_t N, int64_t K,
                            const XT* x, YT* y, int m_valid, int64_t ldx, int64_t ldy, cudaStream_t s) {
  auto kern = qgemv_simt_kernel<FMT, XT, YT, MT, R>;
  const size_t smem = (size_t)MT * K * sizeof(float);
  if (smem > 200 * 1024) return fail(BQ_ERR_UNSUPPORTED, "K too large for the shared-memory activation stage");
  static thread_local size_t configured = 0;  // per instantiation
  if (smem > 48 * 1024 && smem > configured) {
    BQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024)));
    configured = 200 * 1024;
  }
  const int64_t rows_per_cta = (int64_t)GEMV_WARPS * R;
  int64_t grid = (N + rows_per_cta - 1) / rows_per_cta;
  // resident CTAs per SM are limited by shared memory; keep the grid a multiple of the SM count
  int per_sm = 8;
  if (smem > 0) {
    int by_smem = (int)((220 * 1024) / (smem + 1024));
    if (by_smem < per_sm) per_sm = by_smem < 1 ? 1 : by_smem;
  }
  const int64_t cap = (int64_t)sm_count() * per_sm;
  if (grid > cap) grid = cap;
  kern<<<(int)grid, GEMV_WARPS * 32, smem, s>>>(codes, scales, x, y, N, K, m_valid, ldx, ldy);
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

template <int FMT, typename XT, typename YT>
static int simt_dispatch(const uint8_t* codes, const __half* scales, int64_t N, int64_t K, const XT* x,
                         int64_t M, YT* y, int64_t ldy, cudaStream_t s) {
  int64_t m0 = 0;
  while (m0 < M) {
    const int64_t left = M - m0;
    int rc;
    // keep the fp32 activation stage within shared memory: MT*K*4 bytes
    if (left >= 4 && 4 * K * 4 <= 200 * 1024)
      rc = launch_simt_tile<FMT, XT, YT, 4, 2>(codes, scales, N, K, x + m0 * K, y + m0 * ldy, 4, K, ldy, s), m0 += 4;
    else if (left >= 2 && 2 * K * 4 <= 200 * 1024)
      rc = launch_simt_tile<FMT, XT, YT, 2, 2>(codes, scales, N, K, x + m0 * K, y + m0 * ldy, 2, K, ldy, s), m0 += 2;
    else
      rc = launch_simt_tile<FMT, XT, YT, 1, 4>(codes, scales, N, K, x + m0 * K, y + m0 * ldy, 1, K, ldy, s), m0 += 1;
    if (rc != BQ_OK) return rc;
  }
  return BQ_OK;
}

int launch_qlinear_simt(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K,
                        const void* x, int x_dtype, int64_t M, void* y, int y_dtype, int64_t ldy,
                        cudaStream_t s) {
  if (N == 0 || M == 0) return BQ_OK;
#define BQ_SIMT_CASE(F, XT, YT) \
  return simt_dispatch<F, XT, YT>(codes, scales, N, K, (const XT*)x, M, (YT*)y, ldy, s)
  if (fmt == BQ_FMT_Q8G32) {
    if (x_dtype == BQ_DT_F32 && y_dtype == BQ_DT_F32) BQ_SIMT_CASE(BQ_FMT_Q8G32, float, float);
    if (x_dtype == BQ_DT_BF16 && y_dtype == BQ_DT_F32) BQ_SIMT_CASE(BQ_FMT_Q8G32, __nv_bfloat16, float);
    if (x_dtype == BQ_DT_F32 && y_dtype == BQ_DT_BF16) BQ_SIMT_CASE(BQ_FMT_Q8G32, float, __nv_bfloat16);
    if (x_dtype == BQ_DT_BF16 && y_dtype == BQ_DT_BF16) BQ_SIMT_CASE(BQ_FMT_Q8G32, __nv_bfloat16, __nv_bfloat16);
  } else {
    if (x_dtype == BQ_DT_F32 && y_dtype == BQ_DT_F32) BQ_SIMT_CASE(BQ_FMT_Q4G32, float, float);
    if (x_dtype == BQ_DT_BF16 && y_dtype == BQ_DT_F32) BQ_SIMT_CASE(BQ_FMT_Q4G32, __nv_bfloat16, float);
    if (x_dtype == BQ_DT_F32 && y_dtype == BQ_DT_BF16) BQ_SIMT_CASE(BQ_FMT_Q4G32, float, __nv_bfloat16);
    if (x_dtype == BQ_DT_BF16 && y_dtype == BQ_DT_BF16) BQ_SIMT_CASE(BQ_FMT_Q4G32, __nv_bfloat16, __nv_bfloat16);
  }
#undef BQ_SIMT_CASE
  return fail(BQ_ERR_ARG, "bad dtype");
}

// -------------------------------------------------------------------------------------------
// argmax over each row of logits[M,N]; ties resolve to the lower index
// -------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T* __restrict__ logits, int64_t N,
                                                      int32_t* __restrict__ out, float* __restrict__ vout) {
  const T* row = logits + (int64_t)blockIdx.x * N;
  float best = -INFINITY;
  int32_t bi = 0x7fffffff;
  for (int64_t i = threadIdx.x; i < N; i += blockDim.x) {
    const float v = to_float<T>(row[i]);
    if (v > best || (v == best && (int32_t)i < bi)) { best = v; bi = (int32_t)i; }
  }
  __shared__ float sv[32];
  __shared__ int32_t si[32];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const int32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, off);
      const int32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (threadIdx.x == 0) {
      out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
      if (vout) vout[blockIdx.x] = best;
    }
  }
}

// Large vocabularies: stage 1 reduces ARG_CHUNKS slices of every row to (value, index) pairs, stage 2 reduces the pairs.
constexpr int ARG_CHUNKS = 128;
template <typename T>
__global__ void __launch_bounds__(256) argmax_partial_kernel(const T* __restrict__ logits, int64_t N, float* __restrict__ pv,
                                                             int32_t* __restrict__ pi) {
  pdl_launch_dependents();
  pdl_wait();
  const T* row = logits + (int64_t)blockIdx.y * N;
  const int64_t per = (N + ARG_CHUNKS - 1) / ARG_CHUNKS;
  const int64_t lo = (int64_t)blockIdx.x * per, hi = min(N, lo + per);
  float best = -INFINITY;
  int32_t bi = 0x7fffffff;
  for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = to_float<T>(row[i]);
    if (v > best || (v == best && (int32_t)i < bi)) { best = v; bi = (int32_t)i; }
  }
  __shared__ float sv[8];
  __shared__ int32_t si[8];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const int32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    pv[(int64_t)blockIdx.y * ARG_CHUNKS + blockIdx.x] = best;
    pi[(int64_t)blockIdx.y * ARG_CHUNKS + blockIdx.x] = bi;
  }
}
__global__ void __launch_bounds__(ARG_CHUNKS) argmax_final_kernel(const float* __restrict__ pv, const int32_t* __restrict__ pi,
                                                                  int32_t* __restrict__ out, float* __restrict__ vout) {
  pdl_launch_dependents();
  pdl_wait();
  float best = pv[(int64_t)blockIdx.x * ARG_CHUNKS + threadIdx.x];
  int32_t bi = pi[(int64_t)blockIdx.x * ARG_CHUNKS + threadIdx.x];
  __shared__ float sv[ARG_CHUNKS / 32];
  __shared__ int32_t si[ARG_CHUNKS / 32];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
    const int32_t oi = __shfl_xor_sync(0xffffffffu, bi, off);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < ARG_CHUNKS / 32; ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
    if (vout) vout[blockIdx.x] = best;
  }
}

static Scratch g_arg_sv, g_arg_si;         // stage-1 (value, index) pairs (library scratch: see common.cuh)

int launch_argmax(const void* logits, int dtype, int64_t M, int64_t N, int32_t* out, cudaStream_t s, float* vout) {
  if (M == 0) return BQ_OK;
  if (N >= 32768 && M <= 65535) {
    int rc = scratch_ensure(&g_arg_sv, sizeof(float) * (size_t)M * ARG_CHUNKS, s, "argmax");
    if (!rc) rc = scratch_ensure(&g_arg_si, sizeof(int32_t) * (size_t)M * ARG_CHUNKS, s, "argmax");
    if (rc) return rc;
    float* g_arg_pv = (float*)g_arg_sv.ptr;
    int32_t* g_arg_pi = (int32_t*)g_arg_si.ptr;
    dim3 grid(ARG_CHUNKS, (unsigned)M);
    if (dtype == BQ_DT_F32)
      BQ_CUDA(launch_chain(argmax_partial_kernel<float>, grid, dim3(256), 0, s, 1, (const float*)logits, N, g_arg_pv, g_arg_pi));
    else
      BQ_CUDA(launch_chain(argmax_partial_kernel<__nv_bfloat16>, grid, dim3(256), 0, s, 1, (const __nv_bfloat16*)logits, N, g_arg_pv,
                           g_arg_pi));
    BQ_CUDA(launch_chain(argmax_final_kernel, dim3((unsigned)M), dim3(ARG_CHUNKS), 0, s, 1, (const float*)g_arg_pv,
                         (const int32_t*)g_arg_pi, out, vout));
    count_launch(2);
    BQ_CUDA(cudaGetLastError());
    return BQ_OK;
  }
  if (dtype == BQ_DT_F32)
    argmax_kernel<float><<<(int)M, 1024, 0, s>>>((const float*)logits, N, out, vout);
  else
    argmax_kernel<__nv_bfloat16><<<(int)M, 1024, 0, s>>>((const __nv_bfloat16*)logits, N, out, vout);
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

}  // namespace bq
