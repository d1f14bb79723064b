// Single-query (decode) attention for grouped-query layouts on the warp-level tensor path, bf16 caches.
//
// With `rep` query heads per KV head every cache row meets `rep` queries: 4 * rep multiply-adds per cached bf16
// element.  From rep = 4 on that is more arithmetic than the fp32 pipe delivers at HBM speed (rep = 8, head_dim 128:
// 2048 FMAs per 512 bytes of K + V), so the CUDA-core kernel of glue.cu reads the cache at a fraction of the memory
// rate.  Here the query heads of one KV head are the M dimension of mma.sync.m16n8k16 (bf16 in, fp32 accumulate):
//
//   scores  S[head, pos] = Q[head, :] . K[pos, :]      A = Q (heads x d), B = K rows as they lie in the cache
//   output  O[head, :]  += P[head, pos] * V[pos, :]    A = P (the score fragment, rounded to bf16), B = V
//
// One CTA = (batch row, KV head, up to 16 query heads, one slice of the positions); its 4 warps take 16-position
// blocks in turn and keep their own running (max, sum, O); shared memory merges the warps, and - when positions are
// split over CTAs - the last CTA to arrive merges the slices (same scheme as the CUDA-core kernel).
//
// Operand fragments are filled with 16-byte loads straight from the cache, no shared-memory staging:
//   * the k index of S is a permutation of d (lane t of a quad owns d = 32 L + 8 t .. + 7 of every 32-wide chunk L and
//     feeds two k16 steps from one load); Q sits in shared memory under the same permutation, so the sum is the same;
//   * for O the lane loads 8 consecutive d of cache rows 2t, 2t+1, 2t+8, 2t+9 of the block and pairs rows with PRMT
//     (B wants two consecutive k = positions per register); n-tile j = 8 i + e of the output then holds
//     d = 64 i + 8 n + e at column n, which is undone when the accumulators go to shared memory.
// Softmax runs in the exp2 domain (scores scaled by log2(e) / sqrt(d)).  Heads beyond `hp` are zero rows of Q.
#include "common.cuh"

namespace bq {

constexpr int AM_WARPS = 4;
constexpr int AM_THREADS = AM_WARPS * 32;

// d[0..1] (+ d[2..3] when HI) += A x B; without HI the rows 8..15 of A are zero and their sums are dropped
template <bool HI>
__device__ __forceinline__ void am_mma(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  if (HI) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    float x2, x3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%9,%9};"
                 : "+f"(d[0]), "+f"(d[1]), "=f"(x2), "=f"(x3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1), "f"(0.0f));
  }
}
__device__ __forceinline__ uint32_t am_word(const uint4& v, int w) { return w == 0 ? v.x : w == 1 ? v.y : w == 2 ? v.z : v.w; }
__device__ __forceinline__ uint32_t am_pack(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

template <bool FUSED, int D, bool HI>
__global__ void __launch_bounds__(AM_THREADS, (D > 128 ? 2 : 3))
decode_attention_mma_kernel(const __nv_bfloat16* __restrict__ q, const float* __restrict__ qkv, __nv_bfloat16* k_cache,
                            __nv_bfloat16* v_cache, const int64_t* __restrict__ pos_p, __nv_bfloat16* __restrict__ out, int Hq,
                            int Hkv, int64_t S, float rope_base, float* __restrict__ part, unsigned* __restrict__ counters,
                            int* __restrict__ status, int hp) {
  constexpr int ROWS = HI ? 16 : 8;
  constexpr int NC = HI ? 4 : 2;             // accumulator registers per n-tile
  constexpr int QSTR = D + 32;               // q row pitch in shared memory (64 bytes of padding: conflict-free 16-byte reads)
  constexpr int NT = D / 8;
  __shared__ __align__(16) __nv_bfloat16 qs[ROWS * QSTR];
  __shared__ float s_cos[D / 2], s_sin[D / 2];
  __shared__ float s_mx[AM_WARPS][ROWS], s_sum[AM_WARPS][ROWS];
  __shared__ float s_acc[AM_WARPS][ROWS][D];

  const int rep = Hq / Hkv, gpk = rep / hp;
  const int b = blockIdx.y, kv = blockIdx.x / gpk, hg = blockIdx.x % gpk;
  const int nsplit = gridDim.z, z = blockIdx.z;
  // position slices leave (max, sum) pairs behind the [B * Hq][nsplit][D] accumulators of `part`
  float* stats = part + (int64_t)gridDim.y * Hq * nsplit * D;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int h0 = kv * rep + hg * hp;                       // first query head of this CTA
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n_all = *pos_p + 1;
  if (n_all < 1 || n_all > S) {        // position outside the cache (the same for every CTA): record it, touch nothing
    if (threadIdx.x == 0) atomicExch(status, (int)BQ_ERR_ARG);
    return;
  }
  const int64_t per = ((n_all + nsplit - 1) / nsplit + 15) / 16 * 16;
  const int64_t p_lo = (int64_t)z * per;
  const int64_t n_pos = p_lo + per < n_all ? p_lo + per : n_all;      // this CTA covers [p_lo, n_pos)

  if (FUSED) {
    for (int j = threadIdx.x; j < D / 2; j += AM_THREADS) {
      const float inv = 1.0f / powf(rope_base, (float)(2 * j) / (float)D);
      sincosf((float)(n_all - 1) * inv, &s_sin[j], &s_cos[j]);
    }
    __syncthreads();
#pragma unroll 4
    for (int e = threadIdx.x; e < ROWS * D; e += AM_THREADS) {
      const int hl = e / D, d = e - hl * D;
      float v = 0.0f;
      if (hl < hp) v = rope_elem<__nv_bfloat16>(qkv + ((int64_t)b * (Hq + 2 * Hkv) + h0 + hl) * D, d, D, s_cos, s_sin, true);
      qs[hl * QSTR + d] = __float2bfloat16_rn(v);
    }
    if (n_pos == n_all && p_lo < n_all) {
      // this CTA covers the newest position: its K / V rows go into the cache first and are then read back like every
      // other row (CTAs of other head groups of the same KV head store the same bytes)
      const float* ksrc = qkv + ((int64_t)b * (Hq + 2 * Hkv) + Hq + kv) * D;
      const float* vsrc = qkv + ((int64_t)b * (Hq + 2 * Hkv) + Hq + Hkv + kv) * D;
      __nv_bfloat16* kd = k_cache + (((int64_t)b * S + (n_all - 1)) * Hkv + kv) * D;
      __nv_bfloat16* vd = v_cache + (((int64_t)b * S + (n_all - 1)) * Hkv + kv) * D;
      for (int d = threadIdx.x; d < D; d += AM_THREADS) {
        kd[d] = __float2bfloat16_rn(rope_elem<__nv_bfloat16>(ksrc, d, D, s_cos, s_sin, true));
        vd[d] = __float2bfloat16_rn(rope_elem<__nv_bfloat16>(vsrc, d, D, s_cos, s_sin, false));
      }
    }
  } else {
    for (int e = threadIdx.x; e < ROWS * (D / 8); e += AM_THREADS) {
      const int hl = e / (D / 8), c = e - hl * (D / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (hl < hp) v = *reinterpret_cast<const uint4*>(q + ((int64_t)b * Hq + h0 + hl) * D + c * 8);
      *reinterpret_cast<uint4*>(&qs[hl * QSTR + c * 8]) = v;
    }
  }
  __syncthreads();

  float acc[NT][NC];
#pragma unroll
  for (int j = 0; j < NT; ++j)
#pragma unroll
    for (int c = 0; c < NC; ++c) acc[j][c] = 0.0f;
  float mx[2] = {-INFINITY, -INFINITY}, sum[2] = {0.0f, 0.0f};        // rows g and g + 8; sum is this lane's share
  const float sl2 = rsqrtf((float)D) * 1.4426950408889634f;
  const int64_t row_stride = (int64_t)Hkv * D;
  const __nv_bfloat16* kb = k_cache + ((int64_t)b * S * Hkv + kv) * D + 8 * t;
  const __nv_bfloat16* vb = v_cache + ((int64_t)b * S * Hkv + kv) * D + 8 * g;

  // Software pipeline without extra registers: the K rows of the next block are requested as soon as the scores of this
  // one are done (their registers are free then), the V rows of the next block as soon as this block's P V is done, so
  // one of the two is always in flight while the warp computes.
  uint4 kr[2][D / 32], vr[4][D / 64];
  auto load_k = [&](int64_t p0) {
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
      int64_t row = p0 + 8 * nt + g;
      if (row >= n_pos) row = n_pos - 1;                  // masked below; a row that exists is read instead
#pragma unroll
      for (int L = 0; L < D / 32; ++L) kr[nt][L] = *reinterpret_cast<const uint4*>(kb + row * row_stride + 32 * L);
    }
  };
  auto load_v = [&](int64_t p0) {
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      int64_t row = p0 + 2 * t + (r & 1) + 8 * (r >> 1);
      if (row >= n_pos) row = n_pos - 1;
#pragma unroll
      for (int i = 0; i < D / 64; ++i) vr[r][i] = *reinterpret_cast<const uint4*>(vb + row * row_stride + 64 * i);
    }
  };
  const int64_t p_first = p_lo + (int64_t)warp * 16;
  if (p_first < n_pos) { load_k(p_first); load_v(p_first); }
  for (int64_t p0 = p_first; p0 < n_pos; p0 += AM_WARPS * 16) {
    const int64_t p_next = p0 + AM_WARPS * 16;
    // ---- scores of 16 positions x the CTA's heads -------------------------------------------------------------
    float sc[2][NC];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int c = 0; c < NC; ++c) sc[nt][c] = 0.0f;
#pragma unroll
    for (int L = 0; L < D / 32; ++L) {
      const uint4 qa = *reinterpret_cast<const uint4*>(&qs[g * QSTR + 32 * L + 8 * t]);
      uint4 qb = make_uint4(0u, 0u, 0u, 0u);
      if (HI) qb = *reinterpret_cast<const uint4*>(&qs[(g + 8) * QSTR + 32 * L + 8 * t]);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        am_mma<HI>(sc[nt], qa.x, qb.x, qa.y, qb.y, kr[nt][L].x, kr[nt][L].y);
        am_mma<HI>(sc[nt], qa.z, qb.z, qa.w, qb.w, kr[nt][L].z, kr[nt][L].w);
      }
    }
    if (p_next < n_pos) load_k(p_next);
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        const int64_t pos = p0 + 8 * nt + 2 * t + (c & 1);
        sc[nt][c] = pos < n_pos ? sc[nt][c] * sl2 : -INFINITY;
      }
    // ---- running softmax per head row (a quad of lanes holds one row's 16 scores) ---------------------------------
    uint32_t pa[4] = {0u, 0u, 0u, 0u};
    float corr[2] = {1.0f, 1.0f};
#pragma unroll
    for (int hr = 0; hr < (HI ? 2 : 1); ++hr) {
      float m = fmaxf(fmaxf(sc[0][2 * hr], sc[0][2 * hr + 1]), fmaxf(sc[1][2 * hr], sc[1][2 * hr + 1]));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      const float nm = fmaxf(mx[hr], m);                  // finite: the block holds at least one position below n_pos
      corr[hr] = exp2f(mx[hr] - nm);
      const float p00 = exp2f(sc[0][2 * hr] - nm), p01 = exp2f(sc[0][2 * hr + 1] - nm);
      const float p10 = exp2f(sc[1][2 * hr] - nm), p11 = exp2f(sc[1][2 * hr + 1] - nm);
      sum[hr] = sum[hr] * corr[hr] + ((p00 + p01) + (p10 + p11));
      pa[hr] = am_pack(p00, p01);                         // a0 / a1: positions 2t, 2t+1
      pa[2 + hr] = am_pack(p10, p11);                     // a2 / a3: positions 2t+8, 2t+9
      mx[hr] = nm;
    }
    // ---- O += P V ----------------------------------------------------------------------------------------------------
#pragma unroll
    for (int i = 0; i < D / 64; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int j = 8 * i + e;
        const uint32_t sel = (e & 1) ? 0x7632u : 0x5410u;
        const uint32_t b0 = __byte_perm(am_word(vr[0][i], e >> 1), am_word(vr[1][i], e >> 1), sel);
        const uint32_t b1 = __byte_perm(am_word(vr[2][i], e >> 1), am_word(vr[3][i], e >> 1), sel);
        acc[j][0] *= corr[0];
        acc[j][1] *= corr[0];
        if (HI) { acc[j][2] *= corr[1]; acc[j][3] *= corr[1]; }
        am_mma<HI>(acc[j], pa[0], pa[1], pa[2], pa[3], b0, b1);
      }
    if (p_next < n_pos) load_v(p_next);
  }

  // ---- merge the warps (per head), then the position slices -------------------------------------------------------------
#pragma unroll
  for (int hr = 0; hr < (HI ? 2 : 1); ++hr) {
    float s = sum[hr];
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (t == 0) { s_mx[warp][g + 8 * hr] = mx[hr]; s_sum[warp][g + 8 * hr] = s; }
  }
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int d = 64 * (j >> 3) + 16 * t + (j & 7);         // column 2t of n-tile j; column 2t + 1 is d + 8
    s_acc[warp][g][d] = acc[j][0];
    s_acc[warp][g][d + 8] = acc[j][1];
    if (HI) { s_acc[warp][g + 8][d] = acc[j][2]; s_acc[warp][g + 8][d + 8] = acc[j][3]; }
  }
  __syncthreads();
  const int HD = hp * D;
  const int64_t bh0 = (int64_t)b * Hq + h0;
  for (int e = threadIdx.x; e < HD; e += AM_THREADS) {
    const int eh = e / D, ed = e - eh * D;
    float gm = -INFINITY;
#pragma unroll
    for (int w = 0; w < AM_WARPS; ++w) gm = fmaxf(gm, s_mx[w][eh]);
    float gs = 0.0f, o = 0.0f;
#pragma unroll
    for (int w = 0; w < AM_WARPS; ++w) {
      const float f = s_mx[w][eh] == -INFINITY ? 0.0f : exp2f(s_mx[w][eh] - gm);
      gs += s_sum[w][eh] * f;
      o += s_acc[w][eh][ed] * f;
    }
    if (nsplit == 1) {
      out[(bh0 + eh) * D + ed] = __float2bfloat16_rn(o / gs);
    } else {
      part[((bh0 + eh) * nsplit + z) * D + ed] = o;
      if (ed == 0) {
        float* st = stats + ((bh0 + eh) * nsplit + z) * 2;
        st[0] = gm;
        st[1] = gs;
      }
    }
  }
  if (nsplit == 1) return;
  __threadfence();
  __syncthreads();
  __shared__ int s_last;
  const int64_t cidx = (int64_t)b * gridDim.x + blockIdx.x;             // one arrival counter per (batch row, head group)
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(&counters[cidx], 1u);
    s_last = prev == (unsigned)nsplit - 1;
    if (s_last) counters[cidx] = 0;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // the last slice to arrive merges: per head the weights exp2(m_i - max) / sum first (shared memory, reusing the
  // warps' accumulator area), then every output element is a weighted sum of nsplit independent loads
  float* s_f = &s_acc[0][0][0];                                         // [hp][nsplit]; hp * nsplit <= 16 * 64 floats
  for (int eh = warp; eh < hp; eh += AM_WARPS) {
    const float* st = stats + (bh0 + eh) * nsplit * 2;
    float tm = -INFINITY;
    for (int i = lane; i < nsplit; i += 32) tm = fmaxf(tm, __ldcg(st + 2 * i));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, off));
    float ts = 0.0f;
    for (int i = lane; i < nsplit; i += 32) {
      const float m_i = __ldcg(st + 2 * i);
      const float f = m_i == -INFINITY ? 0.0f : exp2f(m_i - tm);
      s_f[eh * nsplit + i] = f;
      ts += __ldcg(st + 2 * i + 1) * f;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ts += __shfl_xor_sync(0xffffffffu, ts, off);
    __syncwarp();
    const float inv = 1.0f / ts;
    for (int i = lane; i < nsplit; i += 32) s_f[eh * nsplit + i] *= inv;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < HD / 4; e += AM_THREADS) {
    const int eh = e / (D / 4), e4 = e - eh * (D / 4);
    const float4* all = reinterpret_cast<const float4*>(part + (bh0 + eh) * nsplit * D) + e4;
    float4 o = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
    for (int i = 0; i < nsplit; ++i) {
      const float4 v = __ldcg(all + (int64_t)i * (D / 4));
      const float f = s_f[eh * nsplit + i];
      o.x += v.x * f; o.y += v.y * f; o.z += v.z * f; o.w += v.w * f;
    }
    __nv_bfloat16* dst = out + (bh0 + eh) * D + 4 * e4;
    *reinterpret_cast<uint2*>(dst) = make_uint2(am_pack(o.x, o.y), am_pack(o.z, o.w));
  }
}

bool attention_mma_supported(int Hq, int Hkv, int D, int* hp_out) {
  const int rep = Hq / Hkv;
  if (rep < 2 || (D != 64 && D != 128 && D != 256)) return false;
  const int cap = D == 256 ? 8 : 16;                     // 16 head rows x 256 would need 128 accumulator registers
  int hp = rep;
  if (rep > cap) {
    if (rep % cap) return false;
    hp = cap;
  }
  *hp_out = hp;
  return true;
}

// CTAs of the kernel instance that are resident on an SM (registers decide), asked once per instance
int attention_mma_ctas_per_sm(bool fused, int D, bool hi) {
  static int cache[2][3][2] = {};
  const int di = D == 64 ? 0 : D == 128 ? 1 : 2;
  int& c = cache[fused ? 1 : 0][di][hi ? 1 : 0];
  if (c == 0) {
    int n = 0;
    cudaError_t e = cudaErrorInvalidValue;
#define BQ_AM_OCC(FUSED, DD, HI) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_attention_mma_kernel<FUSED, DD, HI>, AM_THREADS, 0)
#define BQ_AM_OCC_PICK(FUSED)                                                                    \
  do {                                                                                           \
    if (D == 64) { if (hi) BQ_AM_OCC(FUSED, 64, true); else BQ_AM_OCC(FUSED, 64, false); }        \
    else if (D == 128) { if (hi) BQ_AM_OCC(FUSED, 128, true); else BQ_AM_OCC(FUSED, 128, false); } \
    else BQ_AM_OCC(FUSED, 256, false);                                                           \
  } while (0)
    if (fused) BQ_AM_OCC_PICK(true); else BQ_AM_OCC_PICK(false);
#undef BQ_AM_OCC_PICK
#undef BQ_AM_OCC
    c = (e == cudaSuccess && n >= 1) ? n : 1;
  }
  return c;
}

int launch_attention_mma(const void* q, const float* qkv, void* k_cache, void* v_cache, const int64_t* pos, void* out, int64_t B,
                         int Hq, int Hkv, int D, int64_t S, float rope_base, int hp, int nsplit, float* part, unsigned* counters,
                         cudaStream_t s) {
  const int gpk = (Hq / Hkv) / hp;
  dim3 grid((unsigned)(Hkv * gpk), (unsigned)B, (unsigned)nsplit);
  const bool hi = hp > 8;
#define BQ_AM_LAUNCH(FUSED, DD, HI)                                                                                        \
  BQ_CUDA(launch_chain(decode_attention_mma_kernel<FUSED, DD, HI>, grid, dim3(AM_THREADS), 0, s, 1, (const __nv_bfloat16*)q, qkv, \
                       (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, pos, (__nv_bfloat16*)out, Hq, Hkv, S, rope_base, part,    \
                       counters, status_word(), hp))
#define BQ_AM_PICK(FUSED)                                                          \
  do {                                                                             \
    if (D == 64) { if (hi) BQ_AM_LAUNCH(FUSED, 64, true); else BQ_AM_LAUNCH(FUSED, 64, false); }        \
    else if (D == 128) { if (hi) BQ_AM_LAUNCH(FUSED, 128, true); else BQ_AM_LAUNCH(FUSED, 128, false); } \
    else BQ_AM_LAUNCH(FUSED, 256, false);                                          \
  } while (0)
  if (qkv) BQ_AM_PICK(true); else BQ_AM_PICK(false);
#undef BQ_AM_PICK
#undef BQ_AM_LAUNCH
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

}  // namespace bq
