// Decode-step glue between the quantized matmuls, as a handful of kernels so that one token is ~10 launches
// per layer instead of ~40 framework ops: residual add + RMSNorm, rotate-half RoPE + KV-cache append,
// single-query (decode) attention over the KV cache, and the gated activation (GeGLU / SwiGLU).
// All arithmetic is fp32; T is the activation storage type (float or bf16).
#include "common.cuh"

namespace bq {

// x[r,:] += delta[r,:] (if delta), then out[r,:] = x[r,:] * rsqrt(mean(x^2) + eps) * w[:]
// One block per row; each thread keeps up to RN_CACHE of its elements in registers, so x and delta are read once.
constexpr int RN_THREADS = 256;
constexpr int RN_CACHE = 16;
template <typename T>
__global__ void __launch_bounds__(RN_THREADS) add_rmsnorm_kernel(T* __restrict__ x, const float* __restrict__ delta,
                                                                 const float* __restrict__ w, T* __restrict__ out,
                                                                 int64_t H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  T* xr = x + (int64_t)blockIdx.x * H;
  const float* dr = delta ? delta + (int64_t)blockIdx.x * H : nullptr;
  T* orow = out + (int64_t)blockIdx.x * H;
  float cache[RN_CACHE];
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < RN_CACHE; ++j) {
    const int64_t i = threadIdx.x + (int64_t)j * RN_THREADS;
    float v = 0.0f;
    if (i < H) {
      v = to_float<T>(xr[i]);
      if (dr) {
        v = to_float<T>(from_float<T>(v + dr[i]));   // the residual stream is stored in T
        xr[i] = from_float<T>(v);
      }
    }
    cache[j] = v;
    ss += v * v;
  }
  for (int64_t i = threadIdx.x + (int64_t)RN_CACHE * RN_THREADS; i < H; i += RN_THREADS) {   // rows longer than the cache
    float v = to_float<T>(xr[i]);
    if (dr) {
      v = to_float<T>(from_float<T>(v + dr[i]));
      xr[i] = from_float<T>(v);
    }
    ss += v * v;
  }
  __shared__ float red[RN_THREADS / 32];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int i = 0; i < RN_THREADS / 32; ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)H + eps);
#pragma unroll
  for (int j = 0; j < RN_CACHE; ++j) {
    const int64_t i = threadIdx.x + (int64_t)j * RN_THREADS;
    if (i < H) orow[i] = from_float<T>(cache[j] * inv * w[i]);
  }
  for (int64_t i = threadIdx.x + (int64_t)RN_CACHE * RN_THREADS; i < H; i += RN_THREADS)
    orow[i] = from_float<T>(to_float<T>(xr[i]) * inv * w[i]);
}

// Same operation for rows of up to RN_VEC_MAX elements whose length is a multiple of 8 and whose pointers are
// 16-byte aligned (every decoder shape): a thread owns chunks of 8 consecutive elements, so x, delta and the norm
// weights arrive as a few 16-byte loads issued together before the reduction.  The per-thread order of the
// sum of squares (chunk by chunk, element by element) is shared with allreduce_add_rmsnorm_kernel (comm.cu).
constexpr int RN_VCHUNKS = 2;
constexpr int RN_VEC_MAX = RN_VCHUNKS * RN_THREADS * 8;
template <typename T>
__global__ void __launch_bounds__(RN_THREADS) add_rmsnorm_vec_kernel(T* __restrict__ x, const float* __restrict__ delta,
                                                                     const float* __restrict__ w, T* __restrict__ out,
                                                                     int64_t H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  T* xr = x + (int64_t)blockIdx.x * H;
  const float* dr = delta ? delta + (int64_t)blockIdx.x * H : nullptr;
  T* orow = out + (int64_t)blockIdx.x * H;
  float v[RN_VCHUNKS][8], g[RN_VCHUNKS][8];
  float ss = 0.0f;
#pragma unroll
  for (int c = 0; c < RN_VCHUNKS; ++c) {
    const int64_t i0 = ((int64_t)threadIdx.x + c * RN_THREADS) * 8;
    if (i0 < H) {
      float d[8];
      load8<T>(xr + i0, v[c]);
      load8<float>(w + i0, g[c]);
      if (dr) load8<float>(dr + i0, d);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (dr) v[c][i] = to_float<T>(from_float<T>(v[c][i] + d[i]));   // the residual stream is stored in T
        ss += v[c][i] * v[c][i];
      }
      if (dr) store8<T>(xr + i0, v[c]);
    }
  }
  __shared__ float red[RN_THREADS / 32];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int i = 0; i < RN_THREADS / 32; ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)H + eps);
#pragma unroll
  for (int c = 0; c < RN_VCHUNKS; ++c) {
    const int64_t i0 = ((int64_t)threadIdx.x + c * RN_THREADS) * 8;
    if (i0 < H) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = v[c][i] * inv * g[c][i];
      store8<T>(orow + i0, o);
    }
  }
}

// qkv: fp32 [B, (Hq + 2*Hkv) * D] (output of the fused q|k|v projection).  Writes q (rotated) as T [B, Hq, D],
// and k (rotated), v into the caches [B, S, Hkv, D] at position *pos.  One block per (b, head).
template <typename T>
__global__ void __launch_bounds__(128) rope_kv_append_kernel(const float* __restrict__ qkv, const int64_t* __restrict__ pos_p,
                                                             T* __restrict__ q_out, T* __restrict__ k_cache,
                                                             T* __restrict__ v_cache, int Hq, int Hkv, int D, int64_t S,
                                                             float base, int* __restrict__ status) {
  const int b = blockIdx.y, h = blockIdx.x;            // h in [0, Hq + 2*Hkv)
  pdl_launch_dependents();
  pdl_wait();
  const int64_t pos = *pos_p;
  if (pos < 0 || pos >= S) {                           // the cache has no row for this position: record it, write nothing
    if (threadIdx.x == 0) atomicExch(status, (int)BQ_ERR_ARG);
    return;
  }
  const float* src = qkv + ((int64_t)b * (Hq + 2 * Hkv) + h) * D;
  const int half = D / 2;
  T* dst;
  bool rot = true;
  if (h < Hq) dst = q_out + ((int64_t)b * Hq + h) * D;
  else if (h < Hq + Hkv) dst = k_cache + (((int64_t)b * S + pos) * Hkv + (h - Hq)) * D;
  else { dst = v_cache + (((int64_t)b * S + pos) * Hkv + (h - Hq - Hkv)) * D; rot = false; }
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    // values pass through T once before the rotation, as a runtime that stores q/k in T would do
    const float x1 = to_float<T>(from_float<T>(src[i])), x2 = to_float<T>(from_float<T>(src[i + half]));
    if (rot) {
      const float inv = 1.0f / powf(base, (float)(2 * i) / (float)D);
      float sn, cs;
      sincosf((float)pos * inv, &sn, &cs);
      dst[i] = from_float<T>(x1 * cs - x2 * sn);
      dst[i + half] = from_float<T>(x2 * cs + x1 * sn);
    } else {
      dst[i] = from_float<T>(x1);
      dst[i + half] = from_float<T>(x2);
    }
  }
}

// Single-query attention: out[b, h, :] = softmax(q[b,h,:] . K[b, 0..pos, kv(h), :] / sqrt(D)) . V[b, 0..pos, kv(h), :]
// One block (8 warps) per (b, h).  A lane owns 8 consecutive head-dim elements (D <= 256, D % 8 == 0), so a warp
// reads one K or V row with a single coalesced vector load per lane; a warp takes PB positions per trip (PB K rows and
// PB V rows in flight: 4, or 8 for bf16 caches on grids of at least a full wave of heads, where two CTAs of 120
// registers per SM stream faster than three of 80) and keeps an online softmax; the 8 partial (max, sum, acc) states
// merge through shared memory.
constexpr int ATT_WARPS = 8;
constexpr int ATT_MAXD = 256;
constexpr int ATT_EPL = 8;
// a row's 8 elements as loaded (converted to fp32 only where they are used, so that the K and V rows of a whole
// trip can be in flight together without a register per element)
template <typename T> struct RawRow;
template <> struct RawRow<float> { float4 a, b; };
template <> struct RawRow<__nv_bfloat16> { uint4 r; };
__device__ __forceinline__ RawRow<float> load_raw(const float* p) {
  RawRow<float> v;
  v.a = *reinterpret_cast<const float4*>(p);
  v.b = *reinterpret_cast<const float4*>(p + 4);
  return v;
}
__device__ __forceinline__ RawRow<__nv_bfloat16> load_raw(const __nv_bfloat16* p) {
  RawRow<__nv_bfloat16> v;
  v.r = *reinterpret_cast<const uint4*>(p);
  return v;
}
__device__ __forceinline__ void unpack_raw(const RawRow<float>& v, float* f) {
  f[0] = v.a.x; f[1] = v.a.y; f[2] = v.a.z; f[3] = v.a.w; f[4] = v.b.x; f[5] = v.b.y; f[6] = v.b.z; f[7] = v.b.w;
}
__device__ __forceinline__ void unpack_raw(const RawRow<__nv_bfloat16>& v, float* f) {
  const uint32_t wds[4] = {v.r.x, v.r.y, v.r.z, v.r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(wds[i] << 16);
    f[2 * i + 1] = __uint_as_float(wds[i] & 0xFFFF0000u);
  }
}
// Elements d0 .. d0+7 of one head taken from the fp32 projection output, RoPE-rotated (rotate-half pairs d, d + D/2)
// with the roundings of rope_kv_append_kernel: through T before the rotation and T after it.  cs / sn: the cosines
// and sines of the D/2 rotation angles of this position (same expressions as rope_kv_append_kernel).
template <typename T>
__device__ __forceinline__ void rope8(const float* __restrict__ src, int d0, int D, const float* cs, const float* sn,
                                      bool rotate, float* o) {
  const int half = D / 2;
#pragma unroll
  for (int i = 0; i < ATT_EPL; ++i) {
    const int d = d0 + i;
    if (!rotate) {
      o[i] = to_float<T>(from_float<T>(src[d]));
    } else {
      const int j = d < half ? d : d - half;
      const float x1 = to_float<T>(from_float<T>(src[j])), x2 = to_float<T>(from_float<T>(src[j + half]));
      o[i] = to_float<T>(from_float<T>(d < half ? x1 * cs[j] - x2 * sn[j] : x2 * cs[j] + x1 * sn[j]));
    }
  }
}
// FUSED: `q` is unused; the query, and the K / V rows of the current position, come straight from `qkv` (fp32
// [B, (Hq + 2 Hkv) D], the fused projection's output), rotated here; the cache supplies positions < pos only and
// the CTA of the first query head of each KV group appends the new rows to it.  One launch instead of
// rope_kv_append_kernel + this kernel.
template <typename T, bool FUSED, int PB>
__global__ void __launch_bounds__(ATT_WARPS * 32, (PB == 8 || sizeof(T) == 4) ? 2 : 3)
decode_attention_kernel(const T* __restrict__ q, const float* __restrict__ qkv, T* __restrict__ k_cache,
                        T* __restrict__ v_cache, const int64_t* __restrict__ pos_p, T* __restrict__ out, int Hq, int Hkv,
                        int D, int64_t S, float rope_base, float* __restrict__ part, unsigned* __restrict__ counters,
                        int* __restrict__ status) {
  const int b = blockIdx.y, h = blockIdx.x;
  // gridDim.z > 1: the positions are split over gridDim.z CTAs (long contexts, few heads); each leaves its
  // (max, sum, unnormalised output) in `part` and the last one to arrive merges them in split order
  const int nsplit = gridDim.z, z = blockIdx.z;
  const int kv = h / (Hq / Hkv);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n_all = *pos_p + 1;
  if (n_all < 1 || n_all > S) {        // position outside the cache (same for every CTA of the launch): record it and
    if (threadIdx.x == 0) atomicExch(status, (int)BQ_ERR_ARG);      // leave the cache, `out` and the counters untouched
    return;
  }
  __shared__ float s_cos[ATT_MAXD / 2], s_sin[ATT_MAXD / 2];
  if (FUSED) {                         // the rotation angles of the current position, once per CTA
    for (int j = threadIdx.x; j < D / 2; j += blockDim.x) {
      const float inv = 1.0f / powf(rope_base, (float)(2 * j) / (float)D);
      sincosf((float)(n_all - 1) * inv, &s_sin[j], &s_cos[j]);
    }
    __syncthreads();
  }
  const int64_t per = ((n_all + nsplit - 1) / nsplit + PB - 1) / PB * PB;
  const int64_t p_lo = (int64_t)z * per;
  const int64_t n_own = p_lo + per < n_all ? p_lo + per : n_all;        // this CTA covers [p_lo, n_own)
  // FUSED: the current position (n_all - 1) is not in the cache yet; the CTA that owns it adds it after the loop
  const int64_t n_pos = FUSED && n_own == n_all ? n_all - 1 : n_own;
  const int d0 = lane * ATT_EPL;
  const bool live = d0 < D;
  float qv[ATT_EPL], acc[ATT_EPL];
  const float scale = rsqrtf((float)D);
#pragma unroll
  for (int i = 0; i < ATT_EPL; ++i) { qv[i] = 0.0f; acc[i] = 0.0f; }
  if (live) {
    if (FUSED) rope8<T>(qkv + ((int64_t)b * (Hq + 2 * Hkv) + h) * D, d0, D, s_cos, s_sin, true, qv);
    else load8<T>(q + ((int64_t)b * Hq + h) * D + d0, qv);
#pragma unroll
    for (int i = 0; i < ATT_EPL; ++i) qv[i] *= scale;
  }
  float mx = -INFINITY, sum = 0.0f;
  const int64_t row_stride = (int64_t)Hkv * D;
  const T* kbase = k_cache + ((int64_t)b * S * Hkv + kv) * D + d0;
  const T* vbase = v_cache + ((int64_t)b * S * Hkv + kv) * D + d0;
  // positions and the row stride as 32-bit values: one widening multiply-add per row address
  const int n_pos32 = (int)n_pos, rs32 = (int)row_stride;
  const bool b16 = (lane & 16) != 0, b8 = (lane & 8) != 0;
  for (int s0 = (int)p_lo + warp * PB; s0 < n_pos32; s0 += ATT_WARPS * PB) {
    // all K and V rows of the trip are requested before anything is computed
    RawRow<T> kr[PB], vr[PB];
    float dot[PB];
    if (live) {
#pragma unroll
      for (int j = 0; j < PB; ++j) {
        const int sidx = s0 + j < n_pos32 ? s0 + j : n_pos32 - 1;       // clamp: masked below
        kr[j] = load_raw(kbase + (int64_t)sidx * rs32);
      }
#pragma unroll
      for (int j = 0; j < PB; ++j) {
        const int sidx = s0 + j < n_pos32 ? s0 + j : n_pos32 - 1;
        vr[j] = load_raw(vbase + (int64_t)sidx * rs32);
      }
    }
#pragma unroll
    for (int j = 0; j < PB; ++j) {
      float dsum = 0.0f;
      if (live) {
        float kf[ATT_EPL];
        unpack_raw(kr[j], kf);
#pragma unroll
        for (int i = 0; i < ATT_EPL; ++i) dsum += qv[i] * kf[i];
      }
      dot[j] = dsum;
    }
    // The partial dot products of a lane are summed over the warp four rows at a time: two halving exchanges leave
    // each group of 8 lanes with one row, three more steps sum it, four broadcasts hand every lane all 4 sums (10
    // shuffles instead of 20).
    static_assert(PB % 4 == 0, "the warp reduction folds 4 rows at a time");
#pragma unroll
    for (int q4 = 0; q4 < PB; q4 += 4) {
      float a0 = b16 ? dot[q4 + 2] : dot[q4 + 0], a1 = b16 ? dot[q4 + 3] : dot[q4 + 1];
      const float t0 = b16 ? dot[q4 + 0] : dot[q4 + 2], t1 = b16 ? dot[q4 + 1] : dot[q4 + 3];
      a0 += __shfl_xor_sync(0xffffffffu, t0, 16);
      a1 += __shfl_xor_sync(0xffffffffu, t1, 16);
      float c = b8 ? a1 : a0;
      const float t = b8 ? a0 : a1;
      c += __shfl_xor_sync(0xffffffffu, t, 8);
      c += __shfl_xor_sync(0xffffffffu, c, 4);
      c += __shfl_xor_sync(0xffffffffu, c, 2);
      c += __shfl_xor_sync(0xffffffffu, c, 1);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float d = __shfl_sync(0xffffffffu, c, (j >> 1) * 16 + (j & 1) * 8);
        dot[q4 + j] = s0 + q4 + j < n_pos32 ? d : -INFINITY;
      }
    }
    float nm = mx;
#pragma unroll
    for (int j = 0; j < PB; ++j) nm = fmaxf(nm, dot[j]);
    const float corr = __expf(mx - nm);
    sum *= corr;
#pragma unroll
    for (int i = 0; i < ATT_EPL; ++i) acc[i] *= corr;
#pragma unroll
    for (int j = 0; j < PB; ++j) {
      const float p = __expf(dot[j] - nm);                                   // 0 for masked positions
      sum += p;
      if (live) {
        float vf[ATT_EPL];
        unpack_raw(vr[j], vf);
#pragma unroll
        for (int i = 0; i < ATT_EPL; ++i) acc[i] += p * vf[i];
      }
    }
    mx = nm;
  }
  if (FUSED && warp == 0 && p_lo < n_all && n_own == n_all) {
    // the current position: K (rotated) and V from the projection output, one more online-softmax step
    const int64_t pos = n_all - 1;
    float kn[ATT_EPL], vn[ATT_EPL];
    float dsum = 0.0f;
    if (live) {
      rope8<T>(qkv + ((int64_t)b * (Hq + 2 * Hkv) + Hq + kv) * D, d0, D, s_cos, s_sin, true, kn);
      rope8<T>(qkv + ((int64_t)b * (Hq + 2 * Hkv) + Hq + Hkv + kv) * D, d0, D, s_cos, s_sin, false, vn);
#pragma unroll
      for (int i = 0; i < ATT_EPL; ++i) dsum += qv[i] * kn[i];
      if (h % (Hq / Hkv) == 0) {                      // first query head of the group appends to the cache
        store8<T>(k_cache + (((int64_t)b * S + pos) * Hkv + kv) * D + d0, kn);
        store8<T>(v_cache + (((int64_t)b * S + pos) * Hkv + kv) * D + d0, vn);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, off);
    const float nm = fmaxf(mx, dsum);
    const float corr = __expf(mx - nm), p = __expf(dsum - nm);
    sum = sum * corr + p;
    if (live) {
#pragma unroll
      for (int i = 0; i < ATT_EPL; ++i) acc[i] = acc[i] * corr + p * vn[i];
    }
    mx = nm;
  }
  __shared__ float s_mx[ATT_WARPS], s_sum[ATT_WARPS], s_acc[ATT_WARPS][ATT_MAXD];
  if (lane == 0) { s_mx[warp] = mx; s_sum[warp] = sum; }
#pragma unroll
  for (int i = 0; i < ATT_EPL; ++i) s_acc[warp][d0 + i] = acc[i];
  __syncthreads();
  float gm = -INFINITY;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) gm = fmaxf(gm, s_mx[w]);
  float gs = 0.0f;
#pragma unroll
  for (int w = 0; w < ATT_WARPS; ++w) gs += s_mx[w] == -INFINITY ? 0.0f : s_sum[w] * __expf(s_mx[w] - gm);
  if (nsplit == 1) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float o = 0.0f;
#pragma unroll
      for (int w = 0; w < ATT_WARPS; ++w) o += s_mx[w] == -INFINITY ? 0.0f : s_acc[w][d] * __expf(s_mx[w] - gm);
      out[((int64_t)b * Hq + h) * D + d] = from_float<T>(o / gs);
    }
    return;
  }
  const int64_t bh = (int64_t)b * Hq + h;
  float* mine = part + (bh * nsplit + z) * (D + 2);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.0f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) o += s_mx[w] == -INFINITY ? 0.0f : s_acc[w][d] * __expf(s_mx[w] - gm);
    mine[2 + d] = o;
  }
  if (threadIdx.x == 0) { mine[0] = gm; mine[1] = gs; }
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&counters[bh], 1u);
    s_last = prev == (unsigned)nsplit - 1;
    if (s_last) counters[bh] = 0;                       // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* all = part + bh * nsplit * (D + 2);
  float tm = -INFINITY;
  for (int i = 0; i < nsplit; ++i) tm = fmaxf(tm, __ldcg(all + (int64_t)i * (D + 2)));
  float ts = 0.0f;
  for (int i = 0; i < nsplit; ++i) {
    const float m_i = __ldcg(all + (int64_t)i * (D + 2));
    ts += m_i == -INFINITY ? 0.0f : __ldcg(all + (int64_t)i * (D + 2) + 1) * __expf(m_i - tm);
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float o = 0.0f;
    for (int i = 0; i < nsplit; ++i) {
      const float m_i = __ldcg(all + (int64_t)i * (D + 2));
      o += m_i == -INFINITY ? 0.0f : __ldcg(all + (int64_t)i * (D + 2) + 2 + d) * __expf(m_i - tm);
    }
    out[bh * D + d] = from_float<T>(o / ts);
  }
}

// Grouped-query variant: one CTA serves `hpw` query heads of one KV head, so a K / V row is fetched once for all of
// them instead of once per query head.  A warp's lanes are split as (head hl, chunk c): lane = hl * (32 / hpw) + c
// owns EPLN = D * hpw / 32 consecutive head-dim elements of head hl; the lanes of different heads read the same K / V
// bytes (one transaction).  Positions are walked as in the kernel above (a warp takes PB per trip, online softmax,
// the 8 warps' states merge through shared memory, optional split over gridDim.z with a last-arrival merge).
// grid.x = Hkv * (rep / hpw): KV head kv = blockIdx.x / (rep / hpw), query heads kv * rep + hg * hpw + hl.
template <typename T, int N> struct RawVec { uint4 v[N * (int)sizeof(T) / 16]; };
template <typename T, int N> __device__ __forceinline__ RawVec<T, N> load_rawvec(const T* p) {
  RawVec<T, N> r;
#pragma unroll
  for (int i = 0; i < N * (int)sizeof(T) / 16; ++i) r.v[i] = reinterpret_cast<const uint4*>(p)[i];
  return r;
}
template <int N> __device__ __forceinline__ void unpack_rawvec(const RawVec<float, N>& r, float* f) {
#pragma unroll
  for (int i = 0; i < N / 4; ++i) {
    f[4 * i] = __uint_as_float(r.v[i].x); f[4 * i + 1] = __uint_as_float(r.v[i].y);
    f[4 * i + 2] = __uint_as_float(r.v[i].z); f[4 * i + 3] = __uint_as_float(r.v[i].w);
  }
}
template <int N> __device__ __forceinline__ void unpack_rawvec(const RawVec<__nv_bfloat16, N>& r, float* f) {
#pragma unroll
  for (int i = 0; i < N / 8; ++i) {
    const uint32_t wds[4] = {r.v[i].x, r.v[i].y, r.v[i].z, r.v[i].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f[8 * i + 2 * j] = __uint_as_float(wds[j] << 16);
      f[8 * i + 2 * j + 1] = __uint_as_float(wds[j] & 0xFFFF0000u);
    }
  }
}
constexpr int GQA_MAX_HD = 512;          // hpw * D handled by one warp (EPLN <= 16)
template <typename T, bool FUSED, int EPLN, int PB>      // PB positions per warp and trip (K and V rows of a trip in flight)
__global__ void __launch_bounds__(ATT_WARPS * 32)
decode_attention_gqa_kernel(const T* __restrict__ q, const float* __restrict__ qkv, T* __restrict__ k_cache,
                            T* __restrict__ v_cache, const int64_t* __restrict__ pos_p, T* __restrict__ out, int Hq, int Hkv,
                            int D, int64_t S, float rope_base, float* __restrict__ part, unsigned* __restrict__ counters,
                            int* __restrict__ status, int hpw) {
  const int rep = Hq / Hkv, gpk = rep / hpw;
  const int b = blockIdx.y, kv = blockIdx.x / gpk, hg = blockIdx.x % gpk;
  const int nsplit = gridDim.z, z = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lph = 32 / hpw;                      // lanes per head = D / EPLN
  const int hl = lane / lph, c = lane % lph;
  const int h = kv * rep + hg * hpw + hl;        // this lane's query head
  const int d0 = c * EPLN;
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n_all = *pos_p + 1;
  if (n_all < 1 || n_all > S) {
    if (threadIdx.x == 0) atomicExch(status, (int)BQ_ERR_ARG);
    return;
  }
  __shared__ float s_cos[ATT_MAXD / 2], s_sin[ATT_MAXD / 2];
  if (FUSED) {
    for (int j = threadIdx.x; j < D / 2; j += blockDim.x) {
      const float inv = 1.0f / powf(rope_base, (float)(2 * j) / (float)D);
      sincosf((float)(n_all - 1) * inv, &s_sin[j], &s_cos[j]);
    }
    __syncthreads();
  }
  const int64_t per = ((n_all + nsplit - 1) / nsplit + PB - 1) / PB * PB;
  const int64_t p_lo = (int64_t)z * per;
  const int64_t n_own = p_lo + per < n_all ? p_lo + per : n_all;
  const int64_t n_pos = FUSED && n_own == n_all ? n_all - 1 : n_own;
  float qv[EPLN], acc[EPLN];
  const float scale = rsqrtf((float)D);
  if (FUSED) {
    const float* src = qkv + ((int64_t)b * (Hq + 2 * Hkv) + h) * D;
#pragma unroll
    for (int i = 0; i < EPLN; ++i) qv[i] = rope_elem<T>(src, d0 + i, D, s_cos, s_sin, true) * scale;
  } else {
    const RawVec<T, EPLN> r = load_rawvec<T, EPLN>(q + ((int64_t)b * Hq + h) * D + d0);
    unpack_rawvec<EPLN>(r, qv);
#pragma unroll
    for (int i = 0; i < EPLN; ++i) qv[i] *= scale;
  }
#pragma unroll
  for (int i = 0; i < EPLN; ++i) acc[i] = 0.0f;
  float mx = -INFINITY, sum = 0.0f;
  const int64_t row_stride = (int64_t)Hkv * D;
  const T* kbase = k_cache + ((int64_t)b * S * Hkv + kv) * D + d0;
  const T* vbase = v_cache + ((int64_t)b * S * Hkv + kv) * D + d0;
  for (int64_t s0 = p_lo + (int64_t)warp * PB; s0 < n_pos; s0 += ATT_WARPS * PB) {
    RawVec<T, EPLN> kr[PB], vr[PB];
    float dot[PB];
#pragma unroll
    for (int j = 0; j < PB; ++j) {
      const int64_t sidx = s0 + j < n_pos ? s0 + j : n_pos - 1;       // clamp: masked below
      kr[j] = load_rawvec<T, EPLN>(kbase + sidx * row_stride);
    }
#pragma unroll
    for (int j = 0; j < PB; ++j) {
      const int64_t sidx = s0 + j < n_pos ? s0 + j : n_pos - 1;
      vr[j] = load_rawvec<T, EPLN>(vbase + sidx * row_stride);
    }
#pragma unroll
    for (int j = 0; j < PB; ++j) {
      float kf[EPLN], dsum = 0.0f;
      unpack_rawvec<EPLN>(kr[j], kf);
#pragma unroll
      for (int i = 0; i < EPLN; ++i) dsum += qv[i] * kf[i];
      for (int off = lph >> 1; off > 0; off >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, off);   // over the head's lanes
      dot[j] = s0 + j < n_pos ? dsum : -INFINITY;
    }
    float nm = mx;
#pragma unroll
    for (int j = 0; j < PB; ++j) nm = fmaxf(nm, dot[j]);
    const float corr = __expf(mx - nm);
    sum *= corr;
#pragma unroll
    for (int i = 0; i < EPLN; ++i) acc[i] *= corr;
#pragma unroll
    for (int j = 0; j < PB; ++j) {
      const float p = __expf(dot[j] - nm);
      sum += p;
      float vf[EPLN];
      unpack_rawvec<EPLN>(vr[j], vf);
#pragma unroll
      for (int i = 0; i < EPLN; ++i) acc[i] += p * vf[i];
    }
    mx = nm;
  }
  if (FUSED && warp == 0 && p_lo < n_all && n_own == n_all) {
    const int64_t pos = n_all - 1;
    float kn[EPLN], vn[EPLN], dsum = 0.0f;
    const float* ksrc = qkv + ((int64_t)b * (Hq + 2 * Hkv) + Hq + kv) * D;
    const float* vsrc = qkv + ((int64_t)b * (Hq + 2 * Hkv) + Hq + Hkv + kv) * D;
#pragma unroll
    for (int i = 0; i < EPLN; ++i) {
      kn[i] = rope_elem<T>(ksrc, d0 + i, D, s_cos, s_sin, true);
      vn[i] = rope_elem<T>(vsrc, d0 + i, D, s_cos, s_sin, false);
      dsum += qv[i] * kn[i];
    }
    if (hg == 0 && hl == 0) {                       // one head's lanes append the new rows to the cache
      T* kd = k_cache + (((int64_t)b * S + pos) * Hkv + kv) * D + d0;
      T* vd = v_cache + (((int64_t)b * S + pos) * Hkv + kv) * D + d0;
#pragma unroll
      for (int i = 0; i < EPLN; i += 8) { store8<T>(kd + i, kn + i); store8<T>(vd + i, vn + i); }
    }
    for (int off = lph >> 1; off > 0; off >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, off);
    const float nm = fmaxf(mx, dsum);
    const float corr = __expf(mx - nm), p = __expf(dsum - nm);
    sum = sum * corr + p;
#pragma unroll
    for (int i = 0; i < EPLN; ++i) acc[i] = acc[i] * corr + p * vn[i];
    mx = nm;
  }
  // ---- merge the 8 warps (per head), then the position splits ----------------------------------------------------
  __shared__ float s_mx[ATT_WARPS][32], s_sum[ATT_WARPS][32], s_acc[ATT_WARPS][GQA_MAX_HD];
  s_mx[warp][lane] = mx;
  s_sum[warp][lane] = sum;
#pragma unroll
  for (int i = 0; i < EPLN; ++i) s_acc[warp][lane * EPLN + i] = acc[i];        // = [hl][d0 + i] since lane = hl * lph + c
  __syncthreads();
  const int HD = hpw * D;
  const int64_t bh0 = (int64_t)b * Hq + kv * rep + hg * hpw;                    // first query head of this CTA
  for (int e = threadIdx.x; e < HD; e += blockDim.x) {
    const int eh = e / D, ed = e - eh * D, el = eh * lph;                       // a lane of head eh holds its (max, sum)
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) gm = fmaxf(gm, s_mx[w][el]);
    float gs = 0.0f, o = 0.0f;
#pragma unroll
    for (int w = 0; w < ATT_WARPS; ++w) {
      const float f = s_mx[w][el] == -INFINITY ? 0.0f : __expf(s_mx[w][el] - gm);
      gs += s_sum[w][el] * f;
      o += s_acc[w][e] * f;
    }
    if (nsplit == 1) {
      out[(bh0 + eh) * D + ed] = from_float<T>(o / gs);
    } else {
      float* mine = part + ((bh0 + eh) * nsplit + z) * (D + 2);
      mine[2 + ed] = o;
      if (ed == 0) { mine[0] = gm; mine[1] = gs; }
    }
  }
  if (nsplit == 1) return;
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  const int64_t cidx = (int64_t)b * (Hkv * gpk) + blockIdx.x;                   // one arrival counter per (batch, head group)
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&counters[cidx], 1u);
    s_last = prev == (unsigned)nsplit - 1;
    if (s_last) counters[cidx] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int e = threadIdx.x; e < HD; e += blockDim.x) {
    const int eh = e / D, ed = e - eh * D;
    const float* all = part + (bh0 + eh) * nsplit * (D + 2);
    float tm = -INFINITY;
    for (int i = 0; i < nsplit; ++i) tm = fmaxf(tm, __ldcg(all + (int64_t)i * (D + 2)));
    float ts = 0.0f, o = 0.0f;
    for (int i = 0; i < nsplit; ++i) {
      const float m_i = __ldcg(all + (int64_t)i * (D + 2));
      const float f = m_i == -INFINITY ? 0.0f : __expf(m_i - tm);
      ts += __ldcg(all + (int64_t)i * (D + 2) + 1) * f;
      o += __ldcg(all + (int64_t)i * (D + 2) + 2 + ed) * f;
    }
    out[(bh0 + eh) * D + ed] = from_float<T>(o / ts);
  }
}

// gu: fp32 [rows, 2F] = (gate | up) from the fused projection; out[r, f] = act(gate) * up, stored as T.
// act: 0 = gelu (tanh approximation), 1 = silu
template <typename T>
__global__ void __launch_bounds__(256) gated_act_kernel(const float* __restrict__ gu, T* __restrict__ out, int64_t rows,
                                                        int64_t F, int act, int blocked) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = rows * F;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / F, f = i - r * F;
    // blocked: 16-column blocks of gu hold 8 gate values followed by the 8 up values of the same outputs
    const int64_t gi = blocked ? (f >> 3) * 16 + (f & 7) : f, ui = blocked ? gi + 8 : F + f;
    const float g = gu[r * 2 * F + gi], u = gu[r * 2 * F + ui];
    float a;
    if (act == 0) a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    else a = g / (1.0f + __expf(-g));
    out[i] = from_float<T>(a * u);
  }
}

}  // namespace bq

using namespace bq;

// library-owned scratch (see Scratch in common.cuh: never freed, growth refused during stream capture)
static Scratch g_gu;            // bq_qlinear_gated, large batches: the gate|up product before the activation
static Scratch g_att_part;      // split-position attention: partial (max, sum, output) states
static Scratch g_att_count;     // its arrival counters, one per (batch, head): all zero between launches

namespace bq {
int glue_reserve(int64_t rows, int64_t N) { return scratch_ensure(&g_gu, (size_t)rows * N * sizeof(float), 0, "bq_reserve"); }
}  // namespace bq

static int glue_ready(int dtype) {
  if (device_id() < 0) return fail(BQ_ERR_STATE, "bq_init() has not been called");
  if (dtype != BQ_DT_F32 && dtype != BQ_DT_BF16) return fail(BQ_ERR_ARG, "dtype must be BQ_DT_F32 or BQ_DT_BF16");
  return BQ_OK;
}

static int launch_attention(const void* q, const float* qkv, void* k_cache, void* v_cache, const int64_t* pos, void* out,
                            int64_t B, int Hq, int Hkv, int D, int64_t S, float rope_base, int dtype, void* stream) {
  int rc = glue_ready(dtype);
  if (rc) return rc;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv || D <= 0 || D > ATT_MAXD || (D % 8) || S <= 0 || S >= ((int64_t)1 << 31) ||
      (int64_t)Hkv * D >= ((int64_t)1 << 31))
    return fail(BQ_ERR_ARG, "bad sizes (head_dim <= 256 and a multiple of 8, Hq a multiple of Hkv, fewer than 2^31 positions)");
  if (!k_cache || !v_cache || !pos || !out) return fail(BQ_ERR_ARG, "null pointer");
  // grouped-query attention: one CTA serves hpw query heads of a KV head (K / V rows fetched once for all of them)
  const int rep = Hq / Hkv;
  int hpw = 1;
  while (hpw * 2 <= rep && rep % (hpw * 2) == 0 && hpw * 2 * D <= GQA_MAX_HD && hpw * 2 <= 32) hpw *= 2;
  const int epln = D * hpw / 32;
  const bool gqa = hpw > 1 && (D * hpw) % 32 == 0 && (epln == 8 || epln == 16) &&
                   ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(q) |
                     reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  // bf16 caches with several query heads per KV head: the tensor-path kernel (attn_mma.cu), which keeps up with HBM
  int hp = 0;
  const bool mma = dtype == BQ_DT_BF16 && attention_mma_supported(Hq, Hkv, D, &hp) &&
                   ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(q) |
                     reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  const int64_t ctas_xy = mma ? B * Hkv * (rep / hp) : gqa ? B * Hkv * (rep / hpw) : B * Hq;
  // Positions are split over nsplit CTAs per (batch row, head group).  A partly filled last wave costs (nearly) a whole
  // wave - fully so for the latency-bound tensor-path kernel - and every CTA pays a fixed prologue + merge worth about 96
  // positions (256 for the tensor-path kernel: with 96 the sparse-MoE decoder, batch 256 x 512 positions, took two
  // slices and its step grew from 17.7 to 18.5 ms), so the slice count minimises waves x (positions per slice + fixed).
  // Measured on batch 64 x 2048
  // positions: 16 heads x 256 -> 2-3 slices (367-371 us against 377 with one), 2 heads x 256 (a tensor-parallel rank)
  // -> 3 slices (71 us against 78 with the 5 that merely fill the machine).  At least 128 positions per slice (64 for
  // the tensor-path kernel, which has half the warps).
  const int64_t min_pos = mma ? 64 : 128, max_split = mma ? 64 : 32;
  int64_t ns_max = S / min_pos < max_split ? S / min_pos : max_split;
  if (ns_max < 1) ns_max = 1;
  // The one-head-per-CTA kernel on bf16 caches with at least a full wave of (batch row, head) pairs keeps 8 positions
  // (16 rows) per warp in flight: 120 registers, two CTAs per SM, and being bound by memory then it pays for a partly
  // filled wave only while there are fewer than two of them.  Same box, step of the 7B shape at 2048 positions:
  // batch 64 13.15 -> 12.90 ms, batch 32 8.27 -> 8.21; smaller grids lose with it (batch 16 5.85 -> 5.97, batch 8
  // 3.88 -> 4.32: fewer warps to overlap arithmetic with loads) and keep 4 positions per trip, three CTAs per SM.
  const bool wide = !mma && !gqa && dtype == BQ_DT_BF16 && ctas_xy >= 3 * (int64_t)sm_count();
  const int64_t slots = (int64_t)sm_count() * (mma ? attention_mma_ctas_per_sm(qkv != nullptr, D, hp > 8) : wide ? 2 : 3);
  const int64_t fixed = mma ? 256 : 96;      // the tensor-path CTA rotates and stages up to 16 query heads and merges 4 warps x 16 heads
  int64_t nsplit = 1;
  double best_cost = -1.0;
  for (int64_t ns = 1; ns <= ns_max; ++ns) {
    const int64_t whole = (ctas_xy * ns + slots - 1) / slots;
    const double frac = (double)(ctas_xy * ns) / (double)slots;
    const double waves = wide && frac >= 2.0 ? frac : (double)whole;
    const double cost = waves * (double)((S + ns - 1) / ns + fixed);
    if (best_cost < 0.0 || cost < best_cost) { nsplit = ns; best_cost = cost; }
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (nsplit > 1) {
    if ((rc = scratch_ensure(&g_att_part, (size_t)B * Hq * nsplit * (D + 2) * sizeof(float), s, "split-position attention")))
      return rc;
    if ((rc = scratch_ensure(&g_att_count, (size_t)B * Hq * sizeof(unsigned), s, "split-position attention", true))) return rc;
  }
  float* part = (float*)g_att_part.ptr;
  unsigned* counters = (unsigned*)g_att_count.ptr;
  if (mma) return launch_attention_mma(q, qkv, k_cache, v_cache, pos, out, B, Hq, Hkv, D, S, rope_base, hp, (int)nsplit, part, counters, s);
  if (gqa) {
    dim3 grid((unsigned)(Hkv * (rep / hpw)), (unsigned)B, (unsigned)nsplit);
#define BQ_GQA_LAUNCH(TT, FUSED, EP)                                                                                       \
  BQ_CUDA(launch_chain(decode_attention_gqa_kernel<TT, FUSED, EP, (sizeof(TT) * EP > 32 ? 2 : 4)>, grid, dim3(ATT_WARPS * 32), 0, s, 1, (const TT*)q, qkv,   \
                       (TT*)k_cache, (TT*)v_cache, pos, (TT*)out, Hq, Hkv, D, S, rope_base, part, counters, status_word(), hpw))
#define BQ_GQA_PICK(TT)                                                                            \
  do {                                                                                             \
    if (epln == 8) { if (qkv) BQ_GQA_LAUNCH(TT, true, 8); else BQ_GQA_LAUNCH(TT, false, 8); }      \
    else           { if (qkv) BQ_GQA_LAUNCH(TT, true, 16); else BQ_GQA_LAUNCH(TT, false, 16); }    \
  } while (0)
    if (dtype == BQ_DT_F32) BQ_GQA_PICK(float); else BQ_GQA_PICK(__nv_bfloat16);
#undef BQ_GQA_PICK
#undef BQ_GQA_LAUNCH
    count_launch();
    BQ_CUDA(cudaGetLastError());
    return BQ_OK;
  }
  dim3 grid((unsigned)Hq, (unsigned)B, (unsigned)nsplit);
#define BQ_ATT_LAUNCH(TT, FUSED, PB)                                                                                    \
  BQ_CUDA(launch_chain(decode_attention_kernel<TT, FUSED, PB>, grid, dim3(ATT_WARPS * 32), 0, s, 1, (const TT*)q, qkv, (TT*)k_cache, \
                       (TT*)v_cache, pos, (TT*)out, Hq, Hkv, D, S, rope_base, part, counters, status_word()))
  if (dtype == BQ_DT_F32) {
    if (qkv) BQ_ATT_LAUNCH(float, true, 4); else BQ_ATT_LAUNCH(float, false, 4);
  } else if (wide) {
    if (qkv) BQ_ATT_LAUNCH(__nv_bfloat16, true, 8); else BQ_ATT_LAUNCH(__nv_bfloat16, false, 8);
  } else {
    if (qkv) BQ_ATT_LAUNCH(__nv_bfloat16, true, 4); else BQ_ATT_LAUNCH(__nv_bfloat16, false, 4);
  }
#undef BQ_ATT_LAUNCH
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}


extern "C" {

int bq_add_rmsnorm(void* x, const float* delta, const float* weight, void* out, int64_t rows, int64_t H, float eps,
                   int dtype, void* stream) {
  int rc = glue_ready(dtype);
  if (rc) return rc;
  if (rows < 0 || H <= 0) return fail(BQ_ERR_ARG, "bad sizes");
  if (rows == 0) return BQ_OK;
  if (!x || !weight || !out) return fail(BQ_ERR_ARG, "null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const uintptr_t align = reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(delta) | reinterpret_cast<uintptr_t>(weight) |
                          reinterpret_cast<uintptr_t>(out);
  const bool vec = H % 8 == 0 && H <= RN_VEC_MAX && (align & 15) == 0;
  if (dtype == BQ_DT_F32)
    BQ_CUDA(launch_chain(vec ? add_rmsnorm_vec_kernel<float> : add_rmsnorm_kernel<float>, dim3((unsigned)rows), dim3(RN_THREADS), 0, s,
                         1, (float*)x, delta, weight, (float*)out, H, eps));
  else
    BQ_CUDA(launch_chain(vec ? add_rmsnorm_vec_kernel<__nv_bfloat16> : add_rmsnorm_kernel<__nv_bfloat16>, dim3((unsigned)rows),
                         dim3(RN_THREADS), 0, s, 1, (__nv_bfloat16*)x, delta, weight, (__nv_bfloat16*)out, H, eps));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

int bq_rope_kv_append(const float* qkv, const int64_t* pos, void* q_out, void* k_cache, void* v_cache, int64_t B, int Hq,
                      int Hkv, int D, int64_t S, float rope_base, int dtype, void* stream) {
  int rc = glue_ready(dtype);
  if (rc) return rc;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || (D & 1) || S <= 0) return fail(BQ_ERR_ARG, "bad sizes");
  if (!qkv || !pos || !q_out || !k_cache || !v_cache) return fail(BQ_ERR_ARG, "null pointer");
  dim3 grid((unsigned)(Hq + 2 * Hkv), (unsigned)B);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == BQ_DT_F32)
    BQ_CUDA(launch_chain(rope_kv_append_kernel<float>, grid, dim3(128), 0, s, 1, qkv, pos, (float*)q_out, (float*)k_cache,
                         (float*)v_cache, Hq, Hkv, D, S, rope_base, status_word()));
  else
    BQ_CUDA(launch_chain(rope_kv_append_kernel<__nv_bfloat16>, grid, dim3(128), 0, s, 1, qkv, pos, (__nv_bfloat16*)q_out,
                         (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, Hq, Hkv, D, S, rope_base, status_word()));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

int bq_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int64_t* pos, void* out, int64_t B,
                        int Hq, int Hkv, int D, int64_t S, int dtype, void* stream) {
  if (!q) return fail(BQ_ERR_ARG, "null pointer");
  return launch_attention(q, nullptr, const_cast<void*>(k_cache), const_cast<void*>(v_cache), pos, out, B, Hq, Hkv, D, S, 0.0f,
                          dtype, stream);
}

int bq_decode_attention_rope(const float* qkv, void* k_cache, void* v_cache, const int64_t* pos, void* out, int64_t B,
                             int Hq, int Hkv, int D, int64_t S, float rope_base, int dtype, void* stream) {
  if (!qkv) return fail(BQ_ERR_ARG, "null pointer");
  return launch_attention(nullptr, qkv, k_cache, v_cache, pos, out, B, Hq, Hkv, D, S, rope_base, dtype, stream);
}

static int launch_gated_act(const float* gate_up, void* out, int64_t rows, int64_t F, int act, int dtype, int blocked,
                            cudaStream_t s) {
  int64_t grid = (rows * F + 255) / 256;
  if (grid > (int64_t)sm_count() * 8) grid = (int64_t)sm_count() * 8;
  if (dtype == BQ_DT_F32)
    BQ_CUDA(launch_chain(gated_act_kernel<float>, dim3((unsigned)grid), dim3(256), 0, s, 1, gate_up, (float*)out, rows, F, act,
                         blocked));
  else
    BQ_CUDA(launch_chain(gated_act_kernel<__nv_bfloat16>, dim3((unsigned)grid), dim3(256), 0, s, 1, gate_up, (__nv_bfloat16*)out,
                         rows, F, act, blocked));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

int bq_gated_act(const float* gate_up, void* out, int64_t rows, int64_t F, int act, int dtype, void* stream) {
  int rc = glue_ready(dtype);
  if (rc) return rc;
  if (rows < 0 || F <= 0 || (act != 0 && act != 1)) return fail(BQ_ERR_ARG, "bad arguments");
  if (rows == 0) return BQ_OK;
  if (!gate_up || !out) return fail(BQ_ERR_ARG, "null pointer");
  return launch_gated_act(gate_up, out, rows, F, act, dtype, 0, (cudaStream_t)stream);
}

int bq_qlinear_gated(bq_weight_t weight, const void* x, int x_dtype, int64_t M, void* out, int act, void* stream) {
  int rc = glue_ready(x_dtype);
  if (rc) return rc;
  Weight* w = get_weight(weight);
  if (!w) return BQ_ERR_HANDLE;
  if (M < 0 || (act != 0 && act != 1)) return fail(BQ_ERR_ARG, "bad arguments");
  if (w->N % 16) return fail(BQ_ERR_ARG, "a fused gate|up weight has a multiple of 16 rows");
  if (M == 0) return BQ_OK;
  if (!x || !out) return fail(BQ_ERR_ARG, "null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const bool batch_ok = x_dtype == BQ_DT_BF16 && gemv_batch_supported(w->fmt, w->N, w->K, x_dtype, M) &&
                        (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  if (batch_ok && M >= 3) {                                             // 3..16 rows: the batched GEMV, same epilogue
    set_last_path(BQ_PATH_MMA);
    return launch_qlinear_batch(w->codes, w->scales, w->fmt, w->N, w->K, x, x_dtype, M, out, BQ_DT_BF16, w->N / 2, act, s);
  }
  if (gemv_mma_supported(w->fmt, w->N, w->K, x_dtype, M)) {      // decode-sized: activation in the GEMV's epilogue
    set_last_path(BQ_PATH_MMA);
    return launch_qlinear_mma_gated(w->codes, w->scales, w->fmt, w->N, w->K, x, x_dtype, M, out, act, s);
  }
  // larger bf16 batches: the tcgen05 kernel applies the activation in its epilogue (a gate row and its up row sit 8
  // lanes apart in one warp), no intermediate product
  if (x_dtype == BQ_DT_BF16 && tc_supported(w->fmt, w->N, w->K, x_dtype, M) && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    set_last_path(BQ_PATH_TENSOR);
    return launch_qlinear_tc(w->codes, w->scales, w->fmt, w->N, w->K, x, x_dtype, M, out, BQ_DT_BF16, w->N / 2, s, act);
  }
  // anything else: plain product into a scratch owned by the library (sized on the first call: before any graph
  // capture), then the activation kernel reading the blocked layout
  if ((rc = scratch_ensure(&g_gu, (size_t)M * w->N * sizeof(float), s, "bq_qlinear_gated"))) return rc;
  rc = bq_qlinear(weight, x, x_dtype, M, g_gu.ptr, BQ_DT_F32, stream);
  if (rc) return rc;
  return launch_gated_act((const float*)g_gu.ptr, out, M, w->N / 2, act, x_dtype, 1, s);
}

}  // extern "C"
