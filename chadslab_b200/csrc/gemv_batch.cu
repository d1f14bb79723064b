// Batched decode GEMV: 5..16 activation rows (and the grouped MoE experts at decode sizes, where an expert sees a
// dozen rows) on the tensor cores without the shared-memory / tensor-memory pipeline of the large-batch kernel.
//
// Same data path as the 1..4-row GEMV (gemv_mma.cuh): a warp owns 16 weight rows, every lane streams 16 contiguous
// bytes of "its" row per step straight from HBM into registers (ld.global.nc, 128-bit), unpacks them with the
// mantissa-insertion trick and feeds mma.sync.m16n8k16.  What differs is the exactness model: here the A operand holds
// code * scale rounded once to fp16 (as in the tcgen05 kernel; max-normalised error ~2e-4 against the fp32 oracle),
// so all 8 columns of the B operand are activation rows and one pass over the weights serves 8 rows per column set
// (NB sets: 8 or 16 rows) with accumulators that live across the whole K loop.
//
// Activations: every CTA converts its (at most 16) rows to fp16 in shared memory, each row scaled by the power of two
// that puts its maximum in [2^14, 2^15) (undone in the epilogue).  Within every k-step the row is stored so that the
// four lanes of a quad read consecutive 16-byte pieces, and rows are padded by 64 bytes: the B-fragment loads of a
// warp are then free of bank conflicts.
//
// GB_ROUTE: the MoE router in one launch -- a CTA takes 16 tokens, its 8 warps the (at most 128) expert rows of the
// router weight, the logits meet in shared memory and a warp per token does softmax + top-k (the arithmetic of
// moe_route_kernel).
// Modes: plain y = x W^T; fused gate|up weight with the gated activation in the epilogue (16-row blocks = 8 gate rows +
// the 8 up rows of the same outputs); MoE gate|up (two weights of one expert, rows of a 16-row tile of the expert's
// segment, optionally gathered through the sort permutation, h = silu(g) * u as bf16); MoE down (fp32 rows out).
#include "gemv_mma.cuh"

namespace bq {

constexpr int GB_WARPS = 8;
constexpr int GB_THREADS = GB_WARPS * 32;
constexpr int GB_DENSE = 0, GB_GATED = 1, GB_MOE_GU = 2, GB_MOE_DOWN = 3, GB_ROUTE = 4;

struct GbArgs {
  const uint8_t* codes;              // dense / gated: the weight
  const __half* scales;
  const uint8_t* const* codesA;      // MoE: per-expert pointers (gate or down)
  const __half* const* scalesA;
  const uint8_t* const* codesB;      // MoE gate|up: the up matrices
  const __half* const* scalesB;
  const __nv_bfloat16* x;            // activations (bf16): [m_rows, K]; MoE: rows addressed through the tile
  const int32_t* perm;               // MoE gate|up: x holds TOKEN rows, sorted position p reads row perm[p] / top_k
  const int32_t* offsets;            // MoE: expert row ranges
  const int32_t* tiles;              // MoE: tiles[0] = count, then (expert, first row) pairs of 16-row tiles
  void* y;                           // GB_ROUTE: int32 idx_out [T, top_k]
  float* w_out;                      // GB_ROUTE: f32 routing weights [T, top_k]
  int64_t ldy, N, K;
  int m_rows, top_k, act;            // GB_ROUTE: m_rows = T (all tokens), act = renormalise
};

// 8 fp16 values of a row, k = 8c .. 8c+7, go to this offset (in halves) of the row's shared-memory image: inside a
// k-step the pieces are ordered (piece i, lane t) instead of (lane t, piece i)
template <bool Q8> __device__ __forceinline__ int64_t gb_xoffset(int64_t c) {
  if (Q8) {   // step = 64 k = 8 pieces; lane t owns pieces 2t, 2t+1
    const int64_t s = c >> 3;
    const int r = (int)(c & 7), t = r >> 1, i = r & 1;
    return s * 64 + i * 32 + t * 8;
  } else {    // step = 128 k = 16 pieces; lane t owns pieces 4t .. 4t+3
    const int64_t s = c >> 4;
    const int r = (int)(c & 15), t = r >> 2, i = r & 3;
    return s * 128 + i * 32 + t * 8;
  }
}

template <int FMT, int NB, int KSPLIT, int MODE, typename YT, bool PIPE>
__global__ void __launch_bounds__(GB_THREADS) qgemv_batch_kernel(const __grid_constant__ GbArgs a) {
  constexpr bool Q8 = FMT == BQ_FMT_Q8G32;
  constexpr int KSTEP = Q8 ? 64 : 128;
  constexpr int MMAS = Q8 ? 4 : 8;
  constexpr int MP = 8 * NB;                       // activation rows a CTA holds (padded)
  constexpr int RB_PER_CTA = GB_WARPS / KSPLIT;
  constexpr bool MOE = MODE == GB_MOE_GU || MODE == GB_MOE_DOWN;
  constexpr bool TWO = MODE == GB_MOE_GU;          // two weight matrices share the activations
  constexpr int NACC = TWO ? 2 : 1;
  extern __shared__ __align__(16) uint8_t gb_smem[];
  const int64_t K = a.K, N = a.N;
  const int64_t xstride = K + 32;                  // halves: rows 64 bytes apart modulo 128
  __half* xs = reinterpret_cast<__half*>(gb_smem);
  float* xscale = reinterpret_cast<float*>(gb_smem + (size_t)MP * xstride * 2);     // [MP]
  float* red = xscale + MP;                                                         // [NACC][GB_WARPS][16][MP]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;

  const int64_t row_bytes = Q8 ? K : K / 2;
  const int64_t groups = K / GROUP;
  const int rb_in_cta = warp / KSPLIT;
  const int ksp = warp % KSPLIT;
  const int64_t steps_total = K / KSTEP;
  const int64_t s_begin = steps_total * ksp / KSPLIT, s_end = steps_total * (ksp + 1) / KSPLIT;
  const int64_t cta_rb0 = (MODE == GB_ROUTE ? 0 : MOE ? (int64_t)blockIdx.y : (int64_t)blockIdx.x) * RB_PER_CTA;
  const int64_t cta_rb_stride = (MODE == GB_ROUTE ? 1 : MOE ? (int64_t)gridDim.y : (int64_t)gridDim.x) * RB_PER_CTA;

  // One step of a warp's weight stream in registers: 16 bytes of codes of rows g and g + 8 of each matrix and the two
  // rows' scale of this lane's group.  PIPE (4-bit weights; 12 and more steps per warp, or an expert tile): the stream is software-
  // pipelined one step deep (loads and MMAs are `asm volatile` and keep their program order), and the first step of the
  // first row block is requested before the activation rows are staged - for the dense modes even before
  // griddepcontrol.wait, weights being constants.  Measured: (256000, 2048) at 4-8 rows 70 -> 63 us, the 128-expert
  // layer's gate|up 174 -> 162 us; with a handful of steps per warp (16384 x 2048: 9.4 -> 10.7 us) and for int8 (the
  // exact GEMV lost 10-50% with the extra registers) the plain loop is faster.
  struct StepRegs { uint4 wq[NACC][2]; __half sc[NACC][2]; };
  constexpr int PD = (!Q8 && PIPE) ? 1 : 0;
  StepRegs ring[PD + 1];
  auto fetch = [&](const uint8_t* cA, const __half* sA, const uint8_t* cB, const __half* sB, int64_t r0, int64_t r1, int64_t st,
                   StepRegs& r) {
    const int64_t so = st * (Q8 ? 2 : 4) + (Q8 ? (t >> 1) : t);
    r.wq[0][0] = ldg_stream16(cA + r0 * row_bytes + t * 16 + st * 64);
    r.wq[0][1] = ldg_stream16(cA + r1 * row_bytes + t * 16 + st * 64);
    r.sc[0][0] = sA[r0 * groups + so];
    r.sc[0][1] = sA[r1 * groups + so];
    if (TWO) {
      r.wq[NACC - 1][0] = ldg_stream16(cB + r0 * row_bytes + t * 16 + st * 64);
      r.wq[NACC - 1][1] = ldg_stream16(cB + r1 * row_bytes + t * 16 + st * 64);
      r.sc[NACC - 1][0] = sB[r0 * groups + so];
      r.sc[NACC - 1][1] = sB[r1 * groups + so];
    }
  };
  auto preload_first = [&](const uint8_t* cA, const __half* sA, const uint8_t* cB, const __half* sB) {
    const int64_t rb = cta_rb0 + rb_in_cta;
    if (PD > 0 && rb * 16 < N && s_begin < s_end) {
      int64_t r0 = rb * 16 + g, r1 = r0 + 8;
      if (r0 >= N) r0 = N - 1;
      if (r1 >= N) r1 = N - 1;
      fetch(cA, sA, cB, sB, r0, r1, s_begin, ring[0]);
    }
  };
  if (!MOE) preload_first(a.codes, a.scales, nullptr, nullptr);

  pdl_wait();                                      // activations, tile list and row ranges come from preceding kernels
  const uint8_t* codesA = a.codes;
  const __half* scalesA = a.scales;
  const uint8_t* codesB = nullptr;
  const __half* scalesB = nullptr;
  int64_t m0 = 0;
  int m_rows = a.m_rows;
  if (MODE == GB_ROUTE) {                          // 16 tokens per CTA
    m0 = (int64_t)blockIdx.x * MP;
    m_rows = (int)(a.m_rows - m0 < MP ? a.m_rows - m0 : MP);
  }
  if (MOE) {
    if ((int)blockIdx.x >= a.tiles[0]) return;     // uniform across the CTA, before any barrier
    const int e = a.tiles[1 + 2 * blockIdx.x];
    m0 = a.tiles[2 + 2 * blockIdx.x];
    const int64_t m_end = a.offsets[e + 1];
    m_rows = (int)(m_end - m0 < MP ? m_end - m0 : MP);
    codesA = a.codesA[e]; scalesA = a.scalesA[e];
    if (TWO) { codesB = a.codesB[e]; scalesB = a.scalesB[e]; }
    preload_first(codesA, scalesA, codesB, scalesB);      // the expert is known: its first step travels while the rows are staged
  }

  // ---- activations -> scaled fp16 rows in shared memory (one warp per row, two passes over the row) ----------
  for (int r = warp; r < MP; r += GB_WARPS) {
    if (r >= m_rows) {                              // warp-uniform; unused columns only feed outputs nobody stores
      if (lane == 0) xscale[r] = 0.0f;
      continue;
    }
    int64_t src = (MOE || MODE == GB_ROUTE) ? m0 + r : r;
    if (MODE == GB_MOE_GU && a.perm) {
      const int32_t p = a.perm[src];
      src = p >= 0 ? p / a.top_k : 0;
    }
    const __nv_bfloat16* xrow = a.x + src * K;
    // the row arrives in batches of GB_PC 16-byte pieces per lane, all requested before any is used (a loop with one
    // load in flight per trip made this prologue longer than the weight stream of a small expert tile); rows of up
    // to 32 * 8 * GB_PC elements stay in registers between the maximum and the conversion
    constexpr int GB_PC = 8;
    const int64_t nchunks = K / 8;
    uint4 raw[GB_PC];
    float mx = 0.0f;
    for (int64_t c0 = 0; c0 < nchunks; c0 += 32 * GB_PC) {
#pragma unroll
      for (int i = 0; i < GB_PC; ++i) {
        const int64_t c = c0 + i * 32 + lane;
        raw[i] = c < nchunks ? *reinterpret_cast<const uint4*>(xrow + c * 8) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int i = 0; i < GB_PC; ++i) {
        const uint32_t wds[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          mx = fmaxf(mx, fabsf(__uint_as_float(wds[j] << 16)));
          mx = fmaxf(mx, fabsf(__uint_as_float(wds[j] & 0xFFFF0000u)));
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    int e = 0;
    if (mx > 0.0f && mx < INFINITY) e = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 - 14;
    if (e < -100) e = -100;
    const float down = __uint_as_float((uint32_t)(127 - e) << 23);
    __half* xr = xs + (int64_t)r * xstride;
    const bool cached = nchunks <= 32 * GB_PC;           // the single batch above is still in `raw`
    for (int64_t c0 = 0; c0 < nchunks; c0 += 32 * GB_PC) {
      if (!cached) {
#pragma unroll
        for (int i = 0; i < GB_PC; ++i) {
          const int64_t c = c0 + i * 32 + lane;
          raw[i] = c < nchunks ? *reinterpret_cast<const uint4*>(xrow + c * 8) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int i = 0; i < GB_PC; ++i) {
        const int64_t c = c0 + i * 32 + lane;
        if (c < nchunks) {
          const uint32_t wds[4] = {raw[i].x, raw[i].y, raw[i].z, raw[i].w};
          __half2 h[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            h[j] = __floats2half2_rn(__uint_as_float(wds[j] << 16) * down, __uint_as_float(wds[j] & 0xFFFF0000u) * down);
          *reinterpret_cast<uint4*>(xr + gb_xoffset<Q8>(c)) = *reinterpret_cast<const uint4*>(h);
        }
      }
    }
    if (lane == 0) xscale[r] = __uint_as_float((uint32_t)(127 + e) << 23);
  }
  __syncthreads();

  for (int64_t rb_base = cta_rb0; rb_base * 16 < N; rb_base += cta_rb_stride) {
    const int64_t rb = rb_base + rb_in_cta;
    const bool active = rb * 16 < N;               // warp-uniform
    int64_t r0 = rb * 16 + g, r1 = r0 + 8;
    if (r0 >= N) r0 = N - 1;
    if (r1 >= N) r1 = N - 1;
    float d[NACC][NB][4];
#pragma unroll
    for (int w = 0; w < NACC; ++w)
#pragma unroll
      for (int b = 0; b < NB; ++b) d[w][b][0] = d[w][b][1] = d[w][b][2] = d[w][b][3] = 0.0f;

    if (PD > 0 && active && rb_base != cta_rb0 && s_begin < s_end) fetch(codesA, scalesA, codesB, scalesB, r0, r1, s_begin, ring[0]);
    auto consume = [&](int64_t s, const StepRegs& rg) {
      uint4 wq[NACC][2];
      __half2 sc[NACC][2];
#pragma unroll
      for (int w = 0; w < NACC; ++w)
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) { wq[w][rr] = rg.wq[w][rr]; sc[w][rr] = __half2half2(rg.sc[w][rr]); }
      // A fragments (code * scale as fp16): afr[j] = {row g slots 2t..; row g+8 slots 2t..; row g slots 2t+8..; row g+8 ..}
      uint32_t afr[NACC][MMAS][4];
#pragma unroll
      for (int w = 0; w < NACC; ++w) {
#pragma unroll
        for (int rr = 0; rr < 2; ++rr) {
          const uint32_t ww[4] = {wq[w][rr].x, wq[w][rr].y, wq[w][rr].z, wq[w][rr].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if (Q8) {
              uint32_t lo, hi;
              q8_word_to_h2(ww[q], lo, hi);
              __half2 l2 = __hmul2(*reinterpret_cast<__half2*>(&lo), sc[w][rr]);
              __half2 h2 = __hmul2(*reinterpret_cast<__half2*>(&hi), sc[w][rr]);
              afr[w][q][rr] = *reinterpret_cast<uint32_t*>(&l2);
              afr[w][q][2 + rr] = *reinterpret_cast<uint32_t*>(&h2);
            } else {
              uint32_t h[4];
              q4_word_to_h2(ww[q], h);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                __half2 v = __hmul2(*reinterpret_cast<__half2*>(&h[i]), sc[w][rr]);
                h[i] = *reinterpret_cast<uint32_t*>(&v);
              }
              afr[w][2 * q][rr] = h[0]; afr[w][2 * q][2 + rr] = h[1];
              afr[w][2 * q + 1][rr] = h[2]; afr[w][2 * q + 1][2 + rr] = h[3];
            }
          }
        }
      }
      // B fragments: column n = g is activation row 8 b + g; MMA j takes this lane's 4 consecutive k
      const __half* xlane = xs + s * KSTEP + 8 * t;
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const uint4* xp = reinterpret_cast<const uint4*>(xlane + (int64_t)(8 * b + g) * xstride);
        uint32_t bfr[MMAS][2];
#pragma unroll
        for (int i = 0; i < MMAS / 2; ++i) {
          const uint4 xv = xp[4 * i];                // pieces of a lane are 32 halves (4 x 16 bytes) apart
          bfr[2 * i][0] = xv.x; bfr[2 * i][1] = xv.y; bfr[2 * i + 1][0] = xv.z; bfr[2 * i + 1][1] = xv.w;
        }
#pragma unroll
        for (int w = 0; w < NACC; ++w)
#pragma unroll
          for (int j = 0; j < MMAS; ++j) mma_f16_16816(d[w][b], afr[w][j], bfr[j][0], bfr[j][1]);
      }
    };
    if (PD == 0) {
#pragma unroll 2
      for (int64_t s = active ? s_begin : s_end; s < s_end; ++s) {
        fetch(codesA, scalesA, codesB, scalesB, r0, r1, s, ring[0]);
        consume(s, ring[0]);
      }
    } else {
      for (int64_t s = active ? s_begin : s_end; s < s_end; s += PD + 1) {
#pragma unroll
        for (int u = 0; u <= PD; ++u) {
          if (s + u < s_end) {
            if (s + u + PD < s_end) fetch(codesA, scalesA, codesB, scalesB, r0, r1, s + u + PD, ring[(u + PD) % (PD + 1)]);
            consume(s + u, ring[u]);
          }
        }
      }
    }

    // ---- K-split partials meet in shared memory (fixed order), then scale back and store -------------------------
    // d[w][b] = {(row g, m = 8b+2t), (row g, m+1), (row g+8, m), (row g+8, m+1)}
    if (KSPLIT > 1) {
#pragma unroll
      for (int w = 0; w < NACC; ++w)
#pragma unroll
        for (int b = 0; b < NB; ++b) {
          float* rw = red + ((size_t)(w * GB_WARPS + warp) * 16) * MP;
          rw[g * MP + 8 * b + 2 * t] = d[w][b][0];
          rw[g * MP + 8 * b + 2 * t + 1] = d[w][b][1];
          rw[(g + 8) * MP + 8 * b + 2 * t] = d[w][b][2];
          rw[(g + 8) * MP + 8 * b + 2 * t + 1] = d[w][b][3];
        }
      __syncthreads();
      if (ksp == 0) {
#pragma unroll
        for (int w = 0; w < NACC; ++w)
#pragma unroll
          for (int b = 0; b < NB; ++b) {
            float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
            for (int i = 0; i < KSPLIT; ++i) {
              const float* rw = red + ((size_t)(w * GB_WARPS + rb_in_cta * KSPLIT + i) * 16) * MP;
              s0 += rw[g * MP + 8 * b + 2 * t];
              s1 += rw[g * MP + 8 * b + 2 * t + 1];
              s2 += rw[(g + 8) * MP + 8 * b + 2 * t];
              s3 += rw[(g + 8) * MP + 8 * b + 2 * t + 1];
            }
            d[w][b][0] = s0; d[w][b][1] = s1; d[w][b][2] = s2; d[w][b][3] = s3;
          }
      }
    }
    if (active && (KSPLIT == 1 || ksp == 0)) {
      const int64_t ra = rb * 16 + g, rbb = ra + 8;
#pragma unroll
      for (int b = 0; b < NB; ++b) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const int m = 8 * b + 2 * t + j;
          if (m < m_rows) {
            const float back = xscale[m];
            const float v0 = d[0][b][j] * back, v1 = d[0][b][2 + j] * back;        // rows g and g + 8
            if (MODE == GB_ROUTE) {                 // logits of the CTA's tokens meet in shared memory: [token][expert]
              if (ra < N) red[m * N + ra] = v0;
              if (rbb < N) red[m * N + rbb] = v1;
              continue;
            }
            YT* yrow = reinterpret_cast<YT*>(a.y) + (m0 + m) * a.ldy;
            if (MODE == GB_DENSE || MODE == GB_MOE_DOWN) {
              if (ra < N) yrow[ra] = from_float<YT>(v0);
              if (rbb < N) yrow[rbb] = from_float<YT>(v1);
            } else if (MODE == GB_GATED) {        // v0 = gate, v1 = up of output column rb * 8 + g
              if (rbb < N) {
                float act;
                if (a.act == 0) act = 0.5f * v0 * (1.0f + tanhf(0.7978845608028654f * (v0 + 0.044715f * v0 * v0 * v0)));
                else act = v0 / (1.0f + __expf(-v0));
                yrow[rb * 8 + g] = from_float<YT>(act * v1);
              }
            } else {                               // MoE gate|up: h = silu(gate) * up, same rows of both matrices
              const float u0 = d[NACC - 1][b][j] * back, u1 = d[NACC - 1][b][2 + j] * back;
              if (ra < N) yrow[ra] = from_float<YT>(v0 / (1.0f + __expf(-v0)) * u0);
              if (rbb < N) yrow[rbb] = from_float<YT>(v1 / (1.0f + __expf(-v1)) * u1);
            }
          }
        }
      }
    }
    if (KSPLIT > 1) __syncthreads();
  }
  if (MODE == GB_ROUTE) {
    // softmax over the E logits of a token, k rounds of arg-max (ties to the lower expert id), optional renormalisation:
    // one warp per token, lane l holds experts l, l + 32, l + 64, l + 96
    __syncthreads();
    const int E = (int)N, top_k = a.top_k;
    int32_t* idx_out = reinterpret_cast<int32_t*>(a.y);
    for (int m = warp; m < m_rows; m += GB_WARPS) {
      float v[4];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int e = lane + 32 * j;
        v[j] = e < E ? red[m * E + e] : -INFINITY;
        mx = fmaxf(mx, v[j]);
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      float all = 0.0f;
      if (!a.act) {
#pragma unroll
        for (int j = 0; j < 4; ++j) all += (lane + 32 * j < E) ? expf(v[j] - mx) : 0.0f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) all += __shfl_xor_sync(0xffffffffu, all, off);
      }
      float my_e = 0.0f, top_sum = 0.0f;
      int my_i = 0;
      for (int sl = 0; sl < top_k; ++sl) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int e = lane + 32 * j;
          if (e < E && v[j] > best) { best = v[j]; bi = e; }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
          const float ov = __shfl_xor_sync(0xffffffffu, best, off);
          const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
          if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;
        const float ex = expf(best - mx);
        top_sum += ex;
        if (lane == sl) { my_e = ex; my_i = bi; }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (lane + 32 * j == bi) v[j] = -INFINITY;
      }
      if (lane < top_k) {
        idx_out[(m0 + m) * top_k + lane] = my_i;
        a.w_out[(m0 + m) * top_k + lane] = my_e / (a.act ? top_sum : all);
      }
    }
  }
}

// ---- host side ------------------------------------------------------------------------------------------------
// (The area where K-split partials meet is part of every launch's request, also of the expert modes that never split K:
// without it the 16-row expert tile asked for 67 instead of 83 KB, landed on another shared-memory / L1 split and ran
// 163 -> 210 us on the 128-expert layer at 256 tokens, with either way of rounding the carve-out request.)
static size_t gb_smem_bytes(int nb, int64_t K, bool two) {
  const int mp = 8 * nb;
  return (size_t)mp * (K + 32) * 2 + (size_t)mp * 4 + (size_t)(two ? 2 : 1) * GB_WARPS * 16 * mp * 4;
}

bool gemv_batch_supported(int fmt, int64_t N, int64_t K, int x_dtype, int64_t M) {
  if (x_dtype != BQ_DT_BF16 || M < 1 || M > 16 || N < 1 || (K % 128) != 0) return false;
  if (M > 8) {
    // 9..16 rows need two column sets and twice the shared memory, which costs resident CTAs and L1: measured against
    // the tcgen05 kernel it wins for 4-bit weights while the rows stay short (K <= 2048) or the matrix small, and
    // loses for int8
    if (fmt != BQ_FMT_Q4G32 || (K > 2048 && N > 16384)) return false;
    return gb_smem_bytes(2, K, false) <= 200 * 1024;
  }
  return gb_smem_bytes(1, K, false) <= 200 * 1024;
}

// CTAs of this kernel that should share an SM: as many as the registers allow (3), fewer when the activation rows are large
static int gb_ctas_per_sm(size_t smem) {
  int n = (int)((200 * 1024) / (smem + 1024));
  return n > 3 ? 3 : (n < 1 ? 1 : n);
}

template <int FMT, int NB, int KSPLIT, int MODE, typename YT, bool PIPE>
static int gb_launch_impl(const GbArgs& a, dim3 grid, bool two, cudaStream_t s);

// PIPE (4-bit weights only): the pipelined variant pays off from about 12 steps per warp, and for the expert modes at
// any length, because there the first step travels while the 16 token rows are gathered and converted
template <int FMT, int NB, int KSPLIT, int MODE, typename YT>
static int gb_launch(const GbArgs& a, dim3 grid, bool two, cudaStream_t s) {
  if constexpr (FMT == BQ_FMT_Q4G32) {
    if (MODE == GB_MOE_GU || MODE == GB_MOE_DOWN || a.K / 128 / KSPLIT >= 12)
      return gb_launch_impl<FMT, NB, KSPLIT, MODE, YT, true>(a, grid, two, s);
  }
  return gb_launch_impl<FMT, NB, KSPLIT, MODE, YT, false>(a, grid, two, s);
}

template <int FMT, int NB, int KSPLIT, int MODE, typename YT, bool PIPE>
static int gb_launch_impl(const GbArgs& a, dim3 grid, bool two, cudaStream_t s) {
  auto kern = qgemv_batch_kernel<FMT, NB, KSPLIT, MODE, YT, PIPE>;
  const size_t smem = gb_smem_bytes(NB, a.K, two);
  // Shared memory and L1 share one array.  The kernel wants both: room for gb_ctas_per_sm CTAs' activation rows AND
  // as much L1 as is left (scales and activations are re-read through it; with the carve-out at its maximum the
  // kernel ran at half speed, with the default one CTA per SM was resident above 48 KB).  So the carve-out asked for
  // is exactly what those CTAs need.
  static size_t cfg_smem = 0;
  static int cfg_pct = -1;
  if (smem > cfg_smem) {
    BQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cfg_smem = smem;
  }
  int pct = (int)((gb_ctas_per_sm(smem) * (smem + 1024) * 100 + 227 * 1024 - 1) / (227 * 1024));
  if (pct > 100) pct = 100;
  if (pct != cfg_pct) {
    BQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, pct));
    cfg_pct = pct;
  }
  BQ_CUDA(launch_chain(kern, grid, dim3(GB_THREADS), smem, s, 1, a));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

// dense / gated: pick the K split like the 1..4-row GEMV does (enough warps to keep the memory system busy)
template <int FMT, int NB, int MODE, typename YT>
static int gb_dense(const GbArgs& a, cudaStream_t s) {
  const int64_t rb = (a.N + 15) / 16;
  const int64_t want = (int64_t)sm_count() * 16;
  const int64_t cap = (int64_t)sm_count() * gb_ctas_per_sm(gb_smem_bytes(NB, a.K, false));
  auto grid_for = [&](int ksplit) {
    int64_t gx = (rb + GB_WARPS / ksplit - 1) / (GB_WARPS / ksplit);
    return dim3((unsigned)(gx > cap ? cap : gx));
  };
  if (rb >= want || a.K < 1024) return gb_launch<FMT, NB, 1, MODE, YT>(a, grid_for(1), false, s);
  if (rb * 2 >= want || a.K < 2048) return gb_launch<FMT, NB, 2, MODE, YT>(a, grid_for(2), false, s);
  if (rb * 4 >= want || a.K < 4096) return gb_launch<FMT, NB, 4, MODE, YT>(a, grid_for(4), false, s);
  return gb_launch<FMT, NB, 8, MODE, YT>(a, grid_for(8), false, s);
}

int launch_qlinear_batch(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K, const void* x,
                         int x_dtype, int64_t M, void* y, int y_dtype, int64_t ldy, int gated_act, cudaStream_t s) {
  if (!gemv_batch_supported(fmt, N, K, x_dtype, M)) return fail(BQ_ERR_UNSUPPORTED, "shape not supported by the batched GEMV");
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return fail(BQ_ERR_ARG, "activations must be 16-byte aligned");
  GbArgs a;
  memset(&a, 0, sizeof(a));
  a.codes = codes; a.scales = scales; a.x = (const __nv_bfloat16*)x; a.y = y; a.ldy = ldy; a.N = N; a.K = K;
  a.m_rows = (int)M; a.act = gated_act < 0 ? 0 : gated_act;
  const bool gated = gated_act >= 0;
#define BQ_GB_CASE(F, NBV)                                                                                      \
  do {                                                                                                          \
    if (gated) return gb_dense<F, NBV, GB_GATED, __nv_bfloat16>(a, s);                                          \
    if (y_dtype == BQ_DT_F32) return gb_dense<F, NBV, GB_DENSE, float>(a, s);                                   \
    return gb_dense<F, NBV, GB_DENSE, __nv_bfloat16>(a, s);                                                     \
  } while (0)
  if (fmt == BQ_FMT_Q8G32) { if (M <= 8) BQ_GB_CASE(BQ_FMT_Q8G32, 1); BQ_GB_CASE(BQ_FMT_Q8G32, 2); }
  else                     { if (M <= 8) BQ_GB_CASE(BQ_FMT_Q4G32, 1); BQ_GB_CASE(BQ_FMT_Q4G32, 2); }
#undef BQ_GB_CASE
  return fail(BQ_ERR_ARG, "bad format");
}

bool moe_route_linear_supported(int fmt, int64_t E, int64_t K, int top_k) {
  (void)fmt;
  return E >= 1 && E <= 128 && top_k >= 1 && top_k <= 32 && top_k <= E && (K % 128) == 0 &&
         gb_smem_bytes(2, K, false) <= 200 * 1024;
}

int launch_moe_route_linear(const uint8_t* codes, const __half* scales, int fmt, int64_t E, int64_t K, const void* x, int64_t T,
                            int top_k, int renorm, int32_t* idx_out, float* w_out, cudaStream_t s) {
  if (!moe_route_linear_supported(fmt, E, K, top_k)) return fail(BQ_ERR_UNSUPPORTED, "fused router: E <= 128, K % 128 == 0");
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return fail(BQ_ERR_ARG, "activations must be 16-byte aligned");
  GbArgs a;
  memset(&a, 0, sizeof(a));
  a.codes = codes; a.scales = scales; a.x = (const __nv_bfloat16*)x; a.y = idx_out; a.w_out = w_out; a.N = E; a.K = K;
  a.m_rows = (int)T; a.top_k = top_k; a.act = renorm;
  dim3 grid((unsigned)((T + 15) / 16));
  return fmt == BQ_FMT_Q8G32 ? gb_launch<BQ_FMT_Q8G32, 2, 1, GB_ROUTE, float>(a, grid, false, s)
                             : gb_launch<BQ_FMT_Q4G32, 2, 1, GB_ROUTE, float>(a, grid, false, s);
}

// ---- MoE grouped experts at decode sizes: 8- or 16-row tiles of every expert's segment ------------------------------
__global__ void __launch_bounds__(1024) moe_tile_kernel(const int32_t* __restrict__ offsets, int E, int tile_rows,
                                                        int32_t* __restrict__ tiles) {
  __shared__ int32_t pre[1024];
  const int e = threadIdx.x;
  pdl_launch_dependents();
  pdl_wait();
  int32_t cnt = 0;
  if (e < E) cnt = (offsets[e + 1] - offsets[e] + tile_rows - 1) / tile_rows;
  pre[e] = cnt;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int32_t add = e >= off ? pre[e - off] : 0;
    __syncthreads();
    pre[e] += add;
    __syncthreads();
  }
  if (e < E) {
    const int32_t base = pre[e] - cnt, first = offsets[e];
    for (int i = 0; i < cnt; ++i) {
      tiles[1 + 2 * (base + i)] = e;
      tiles[2 + 2 * (base + i)] = first + i * tile_rows;
    }
  }
  if (e == E - 1) tiles[0] = pre[e];
}

bool moe_batch_supported(const Moe* m) {
  return (m->H % 128) == 0 && (m->F % 128) == 0 && gb_smem_bytes(2, m->H, true) <= 200 * 1024 &&
         gb_smem_bytes(2, m->F, false) <= 200 * 1024 && m->E <= 1024;
}

static Scratch g_tiles16;      // tile list of the current call (library scratch: see common.cuh)

template <int NB>
static int moe_batch_launch(const Moe* m, const GbArgs& a, const GbArgs& b, int64_t max_tiles, cudaStream_t s) {
  int rc;
  {
    // gate|up: a warp streams 16 gate rows and the 16 up rows of the same outputs; 8 row blocks per CTA pass
    const int64_t rb = (m->F + 15) / 16;
    dim3 grid((unsigned)max_tiles, (unsigned)((rb + GB_WARPS - 1) / GB_WARPS));
    rc = m->fmt == BQ_FMT_Q8G32 ? gb_launch<BQ_FMT_Q8G32, NB, 1, GB_MOE_GU, __nv_bfloat16>(a, grid, true, s)
                                : gb_launch<BQ_FMT_Q4G32, NB, 1, GB_MOE_GU, __nv_bfloat16>(a, grid, true, s);
    if (rc) return rc;
  }
  {
    // down: short K (a handful of steps per warp): every warp walks several row blocks
    const int64_t rb = (m->H + 15) / 16;
    int64_t gy = (rb + GB_WARPS * 4 - 1) / (GB_WARPS * 4);
    if (gy < 1) gy = 1;
    dim3 grid((unsigned)max_tiles, (unsigned)gy);
    rc = m->fmt == BQ_FMT_Q8G32 ? gb_launch<BQ_FMT_Q8G32, NB, 1, GB_MOE_DOWN, float>(b, grid, false, s)
                                : gb_launch<BQ_FMT_Q4G32, NB, 1, GB_MOE_DOWN, float>(b, grid, false, s);
  }
  return rc;
}

// rows_hint: rows the experts are expected to hold in total (<= P, the rows the buffers hold).  It picks the tile
// height: a tile streams its expert's weights and pays the whole unpack arithmetic once whatever it holds, and the MMA
// work grows with its height: 8 rows up to an average of 5 rows per expert (64 tokens, 128 experts, top-8: experts stage
// 121 -> 103 us), 16 rows beyond.  24-row tiles lost (256 tokens: 162 -> 193 us): two such CTAs take 200 KB of the
// shared-memory / L1 array and 127 registers.
int launch_moe_experts_batch(const Moe* m, const void* x, const int32_t* perm, int top_k, const int32_t* offsets, int64_t P,
                             int64_t rows_hint, void* hbuf, float* out, cudaStream_t s) {
  if (!moe_batch_supported(m)) return fail(BQ_ERR_UNSUPPORTED, "batched-GEMV expert path unavailable for this expert shape");
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (reinterpret_cast<uintptr_t>(hbuf) & 15) != 0)
    return fail(BQ_ERR_ARG, "activation buffers must be 16-byte aligned");
  const int64_t avg = (rows_hint + m->E - 1) / m->E;
  const int nb = avg <= 5 ? 1 : 2;
  const int tile_rows = 8 * nb;
  const int64_t max_tiles = (P + tile_rows - 1) / tile_rows + m->E;
  int rc = scratch_ensure(&g_tiles16, sizeof(int32_t) * (size_t)(2 * ((P + 7) / 8 + m->E) + 1 + 64), s, "bq_moe_experts (tile list)");
  if (rc) return rc;
  int32_t* tiles = (int32_t*)g_tiles16.ptr;
  BQ_CUDA(launch_chain(moe_tile_kernel, dim3(1), dim3(1024), 0, s, 1, offsets, m->E, tile_rows, tiles));
  count_launch();
  GbArgs a;
  memset(&a, 0, sizeof(a));
  a.codesA = m->gate_codes; a.scalesA = m->gate_scales; a.codesB = m->up_codes; a.scalesB = m->up_scales;
  a.x = (const __nv_bfloat16*)x; a.perm = perm; a.top_k = top_k > 0 ? top_k : 1; a.offsets = offsets; a.tiles = tiles;
  a.y = hbuf; a.ldy = m->F; a.N = m->F; a.K = m->H;
  GbArgs b;
  memset(&b, 0, sizeof(b));
  b.codesA = m->down_codes; b.scalesA = m->down_scales; b.x = (const __nv_bfloat16*)hbuf; b.offsets = offsets; b.tiles = tiles;
  b.y = out; b.ldy = m->H; b.N = m->H; b.K = m->F; b.top_k = 1;
  return nb == 1 ? moe_batch_launch<1>(m, a, b, max_tiles, s) : moe_batch_launch<2>(m, a, b, max_tiles, s);
}

}  // namespace bq
