// Decode-shaped GEMV (1..4 activation rows) that streams packed weights straight from HBM into
// registers and contracts them on the tensor cores with *exact* group scaling.
//
// Why tensor cores for a GEMV: at HBM speed a B200 SM receives ~45 packed bytes per ns; unpacking a
// weight to fp32 and issuing one FMA per weight needs more integer-pipe issue slots than the SM has
// (measured: the CUDA-core kernel stalls at ~45% ALU-pipe utilisation and 30-70% of HBM).  Here a
// weight costs ~0.6-0.75 integer-pipe instructions: codes become exact fp16 integers with one
// PRMT/LOP3 per pair (mantissa insertion) and one HSUB2/HFMA2, and mma.sync.m16n8k16 does the
// multiply-adds with fp32 accumulation.
//
// Exactness: the A operand holds the integer codes (exact in fp16), not code*scale.  The 8 columns of
// the B operand are (activation vector, quantization group) pairs: column c is non-zero only on the
// k-slots that belong to its group, so D[row][c] is that group's integer-weighted partial sum.  The fp16
// group scale is applied afterwards in fp32, exactly as dequantize-then-multiply would.
//
// Activations are turned into fp16 inside the kernel: every row is scaled by the power of two that puts
// its largest magnitude in [2^14, 2^15) (exact for bf16 inputs down to 2^-29 of the row maximum); fp32
// rows are split into two fp16 vectors hi + lo * 2^-11, which keeps 22 significant bits.
//
// Work split: a warp owns 16 weight rows (lanes g = lane/4 and g+8) and a K range; each lane loads 16
// contiguous bytes of "its" row per step (a quad covers 64 bytes), so the load pattern is 8 rows x 64
// contiguous bytes per warp instruction.  KSPLIT warps of a CTA share a row block and split K (their
// partial sums meet in shared memory), which keeps all SMs busy when N is small.
#pragma once
#include "common.cuh"

namespace bq {

constexpr int GM_OUT_PLAIN = 0, GM_OUT_PUSH = 1, GM_OUT_GELU = 2, GM_OUT_SILU = 3;
constexpr int GM_WARPS = 8;
constexpr int GM_THREADS = GM_WARPS * 32;

// ---- thread-block cluster helpers (split-K across the CTAs of a cluster, summed through distributed shared memory)
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_cluster_f32(const float* local_ptr, uint32_t rank) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(local_ptr);
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(a), "r"(rank));
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}

__device__ __forceinline__ void mma_f16_16816(float* d, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 4 int8 codes (one word, stored as code + 128 on the device) -> two fp16x2 registers holding the exact
// codes (c0,c1), (c2,c3): 0x6400 | byte = 1024 + byte, minus 1152
__device__ __forceinline__ void q8_word_to_h2(uint32_t v, uint32_t& lo, uint32_t& hi) {
  uint32_t p0 = __byte_perm(v, 0x64646464u, 0x4140);
  uint32_t p1 = __byte_perm(v, 0x64646464u, 0x4342);
  const __half2 off = __float2half2_rn(1152.0f);
  __half2 h0 = __hsub2(*reinterpret_cast<__half2*>(&p0), off);
  __half2 h1 = __hsub2(*reinterpret_cast<__half2*>(&p1), off);
  lo = *reinterpret_cast<uint32_t*>(&h0);
  hi = *reinterpret_cast<uint32_t*>(&h1);
}
// 8 4-bit codes (one word, device nibble order) -> four fp16x2 registers (e0,e1),(e2,e3),(e4,e5),(e6,e7)
__device__ __forceinline__ void q4_word_to_h2(uint32_t v, uint32_t* o) {
  const __half2 off = __float2half2_rn(1032.0f);
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  const __half2 off16 = __float2half2_rn(-72.0f);
  const uint32_t v8 = v >> 8;
  uint32_t t0 = lop3_and_or(v, 0x000F000Fu, 0x64006400u);
  uint32_t t1 = lop3_and_or(v, 0x00F000F0u, 0x64006400u);
  uint32_t t2 = lop3_and_or(v8, 0x000F000Fu, 0x64006400u);
  uint32_t t3 = lop3_and_or(v8, 0x00F000F0u, 0x64006400u);
  __half2 h0 = __hsub2(*reinterpret_cast<__half2*>(&t0), off);
  __half2 h1 = __hfma2(*reinterpret_cast<__half2*>(&t1), sixteenth, off16);
  __half2 h2 = __hsub2(*reinterpret_cast<__half2*>(&t2), off);
  __half2 h3 = __hfma2(*reinterpret_cast<__half2*>(&t3), sixteenth, off16);
  o[0] = *reinterpret_cast<uint32_t*>(&h0);
  o[1] = *reinterpret_cast<uint32_t*>(&h1);
  o[2] = *reinterpret_cast<uint32_t*>(&h2);
  o[3] = *reinterpret_cast<uint32_t*>(&h3);
}

// FMT        weight format
// NV         fp16 activation vectors held in shared memory (bf16: one per row; fp32: two per row)
// KSPLIT     warps that split K for one 16-row block (1, 2, 4 or 8); GM_WARPS/KSPLIT row blocks per CTA
// Columns of an MMA: Q8 -> 2 groups per 64-k step, so 4 vectors per MMA; Q4 -> 4 groups per 128-k step,
// so 2 vectors per MMA.  NB = MMAs (column sets) needed for NV vectors.
// CL         launched as a thread-block cluster of kc_arg CTAs that split K (compile-time switch so the plain
//            instantiation carries no cluster code at all)
// PUSH       row-parallel shard of a tensor-parallel linear: `y` is not an output array but the device descriptor
//            of a peer-memory communicator (CommDev, comm.cu); every partial sum is stored into the receive slot
//            of every rank (plain stores over NVLink), and the kernel that follows on the stream waits for the
//            values and sums the slots.  YT must be float.
// OUT        GM_OUT_PLAIN: y[m, row]; GM_OUT_PUSH: as above; GM_OUT_GELU / GM_OUT_SILU: the weight is a fused
//            gate|up projection whose 16-row blocks hold 8 gate rows followed by the 8 up rows of the same output
//            columns, so a lane owns both halves of a column: y[m, block*8 + g] = act(gate) * up, ldy = N / 2.
template <int FMT, int NV, int KSPLIT, typename XT, typename YT, bool CL, int OUT>
__global__ void __launch_bounds__(GM_THREADS)
qgemv_mma_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ scales, const XT* __restrict__ x,
                 YT* __restrict__ y, int64_t N, int64_t K, int m_rows, int64_t ldy, int kc_arg) {
  const int kc = CL ? kc_arg : 1;
  constexpr bool PUSH = OUT == GM_OUT_PUSH;
  constexpr bool Q8 = FMT == BQ_FMT_Q8G32;
  constexpr bool XF32 = sizeof(XT) == 4;
  constexpr int GROUPS_PER_STEP = Q8 ? 2 : 4;          // groups covered by a quad per step
  constexpr int KSTEP = GROUPS_PER_STEP * GROUP;       // 64 or 128 k per step
  constexpr int VPM = 8 / GROUPS_PER_STEP;             // vectors per MMA column set (4 or 2)
  constexpr int NB = (NV + VPM - 1) / VPM;
  constexpr int MMAS = Q8 ? 4 : 8;                     // MMAs per step per column set
  constexpr int RB_PER_CTA = GM_WARPS / KSPLIT;

  extern __shared__ __align__(16) uint8_t gm_smem[];
  __half* xs = reinterpret_cast<__half*>(gm_smem);                       // [NV][K]
  float* xscale = reinterpret_cast<float*>(gm_smem + (size_t)NV * K * 2);  // [NV] power-of-two back-scale
  float* red = xscale + 8;                                                 // [GM_WARPS][16][NV] partials
  float* cred = red + GM_WARPS * 16 * NV;                                  // [RB_PER_CTA][16][NV] per-CTA sums (cluster)
  // kc > 1: the kc CTAs of a cluster (gridDim.y = kc) split K; rank 0 adds the others' sums through DSMEM
  const int cy = CL ? (int)cluster_ctarank() : 0;

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  // Launched with programmatic stream serialization: it may start while a preceding (small, early-triggering) kernel
  // still runs, so wait before touching x / y.  It never triggers its own successor early: a successor whose CTAs
  // become resident while this grid streams takes registers and shared memory away from it, and measured (256000-row
  // head, q4: 58 against 63 us) that costs more than the launch latency it hides.
  const int64_t row_bytes = Q8 ? K : K / 2;
  const int64_t groups = K / GROUP;
  const int rb_in_cta = warp / KSPLIT;
  const int ksp = warp % KSPLIT;
  const int64_t steps_total = K / KSTEP;
  const int64_t cs_begin = steps_total * cy / kc, cs_end = steps_total * (cy + 1) / kc;   // this CTA's steps
  const int64_t s_begin = cs_begin + (cs_end - cs_begin) * ksp / KSPLIT;
  const int64_t s_end = cs_begin + (cs_end - cs_begin) * (ksp + 1) / KSPLIT;

  // One step of a warp's weight stream as it sits in registers: 16 bytes of codes of rows g and g + 8 and the rows' group
  // scales of the step (Q8: 2 fp16 = one word per row; Q4: 4 fp16 = two words per row).
  struct StepRegs { uint4 w0, w1; uint32_t sa[2], sb[2]; };
  auto fetch = [&](const uint8_t* p0, const uint8_t* p1, const __half* sc0, const __half* sc1, int64_t st, StepRegs& r) {
    r.w0 = ldg_stream16(p0 + st * 64);
    r.w1 = ldg_stream16(p1 + st * 64);
    if (Q8) {
      r.sa[0] = *reinterpret_cast<const uint32_t*>(sc0 + st * 2);
      r.sb[0] = *reinterpret_cast<const uint32_t*>(sc1 + st * 2);
    } else {
      const uint2 a = *reinterpret_cast<const uint2*>(sc0 + st * 4), b = *reinterpret_cast<const uint2*>(sc1 + st * 4);
      r.sa[0] = a.x; r.sa[1] = a.y; r.sb[0] = b.x; r.sb[1] = b.y;
    }
  };
  // 4-bit weights: the weight stream is software-pipelined one step deep (the loads and the MMAs are `asm volatile` and
  // keep their program order, so otherwise a warp requests the codes of a step only after it has issued the MMAs of the
  // step before), and the first step of the CTA's first row block is requested here, BEFORE griddepcontrol.wait:
  // weights are constants of the model, so their first trip to HBM overlaps the tail of the preceding kernel and the
  // activation staging below.  Measured: head shape 0.78 -> 0.80 of HBM, batch-1 decode step of the 7B shape -3%.
  // int8 weights keep the plain loop: with any pipelining depth the extra registers cost a resident CTA and the
  // kernel lost 10-50% (depths 1-3 measured on the same box); deeper than one step also lost for 4-bit.
  constexpr int PD = Q8 ? 0 : 1;
  StepRegs ring[PD + 1];
  if (PD > 0) {
    const int64_t rb = (int64_t)blockIdx.x * RB_PER_CTA + rb_in_cta;
    if (rb * 16 < N) {
      int64_t r0 = rb * 16 + g, r1 = r0 + 8;
      if (r0 >= N) r0 = N - 1;
      if (r1 >= N) r1 = N - 1;
#pragma unroll
      for (int j = 0; j < PD; ++j)
        if (s_begin + j < s_end)
          fetch(codes + r0 * row_bytes + t * 16, codes + r1 * row_bytes + t * 16, scales + r0 * groups, scales + r1 * groups, s_begin + j, ring[j]);
    }
  }
  pdl_wait();
  // PUSH: the receive-slot addresses of this call, one per rank, parked behind the reduction buffers
  float** push_dst = reinterpret_cast<float**>(cred + GM_WARPS * 16 * NV);
  if (PUSH && threadIdx.x < comm_world(y)) push_dst[threadIdx.x] = comm_push_base(y, threadIdx.x);
  float* push_stage = reinterpret_cast<float*>(push_dst + 16);      // PUSH: [row block of the CTA][activation row][16 outputs]

  // ---- activations -> scaled fp16 vectors in shared memory ------------------------------------------
  {
    __shared__ float wmax[GM_WARPS];
    constexpr int ROWS = XF32 ? NV / 2 : NV;
    for (int r = 0; r < ROWS; ++r) {
      // 16-byte loads: 8 bf16 or 4 fp32 per thread and trip (rows start 16-byte aligned: K % 128 == 0)
      constexpr int VEC = XF32 ? 4 : 8;
      const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
      const XT* xrow = x + (int64_t)r * K;
      float mx = 0.0f;
      if (r < m_rows) {
        if (vec_ok) {
          for (int64_t k = (int64_t)threadIdx.x * VEC; k < K; k += GM_THREADS * VEC) {
            const uint4 raw = *reinterpret_cast<const uint4*>(xrow + k);
            const XT* e = reinterpret_cast<const XT*>(&raw);
#pragma unroll
            for (int i = 0; i < VEC; ++i) mx = fmaxf(mx, fabsf(to_float<XT>(e[i])));
          }
        } else {
          for (int64_t k = threadIdx.x; k < K; k += GM_THREADS) mx = fmaxf(mx, fabsf(to_float<XT>(xrow[k])));
        }
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      __syncthreads();
      if (lane == 0) wmax[warp] = mx;
      __syncthreads();
      mx = wmax[0];
#pragma unroll
      for (int i = 1; i < GM_WARPS; ++i) mx = fmaxf(mx, wmax[i]);
      int e = 0;
      if (mx > 0.0f && mx < INFINITY) e = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 - 14;
      if (e < -100) e = -100;
      const float down = __uint_as_float((uint32_t)(127 - e) << 23);
      const int64_t steps_all = K / KSTEP;
      const int64_t k_lo = (steps_all * cy / kc) * KSTEP, k_hi = (steps_all * (cy + 1) / kc) * KSTEP;   // this CTA's K slice
      if (vec_ok && r < m_rows) {
        for (int64_t k = k_lo + (int64_t)threadIdx.x * VEC; k < k_hi; k += GM_THREADS * VEC) {
          const uint4 raw = *reinterpret_cast<const uint4*>(xrow + k);
          const XT* el = reinterpret_cast<const XT*>(&raw);
          __half hi[VEC], lo[VEC];
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            const float v = to_float<XT>(el[i]) * down;
            hi[i] = __float2half_rn(v);
            if (XF32) lo[i] = __float2half_rn((v - __half2float(hi[i])) * 2048.0f);
          }
          if (XF32) {
            *reinterpret_cast<uint2*>(xs + (int64_t)(2 * r) * K + k) = *reinterpret_cast<const uint2*>(hi);
            *reinterpret_cast<uint2*>(xs + (int64_t)(2 * r + 1) * K + k) = *reinterpret_cast<const uint2*>(lo);
          } else {
            *reinterpret_cast<uint4*>(xs + (int64_t)r * K + k) = *reinterpret_cast<const uint4*>(hi);
          }
        }
      } else {
        for (int64_t k = k_lo + threadIdx.x; k < k_hi; k += GM_THREADS) {
          const float v = r < m_rows ? to_float<XT>(xrow[k]) * down : 0.0f;
          if (XF32) {
            const __half hi = __float2half_rn(v);
            const float rem = (v - __half2float(hi)) * 2048.0f;
            xs[(int64_t)(2 * r) * K + k] = hi;
            xs[(int64_t)(2 * r + 1) * K + k] = __float2half_rn(rem);
          } else {
            xs[(int64_t)r * K + k] = __float2half_rn(v);
          }
        }
      }
      if (threadIdx.x == 0) {
        const float up = __uint_as_float((uint32_t)(127 + e) << 23);
        if (XF32) { xscale[2 * r] = up; xscale[2 * r + 1] = up * (1.0f / 2048.0f); }
        else      { xscale[r] = up; }
      }
    }
    __syncthreads();
  }

  // which activation vector / group-column this lane feeds into B: column n = g.
  //   Q8: column n = 2*v + h, h = group half (0/1); this lane's k-slots are in half (t >> 1)
  //   Q4: column n = 4*v + q, q = group (0..3);     this lane's k-slots are in group t
  const int col_sub = Q8 ? (g & 1) : (g & 3);
  const int my_sub = Q8 ? (t >> 1) : t;
  const int v_of_g = Q8 ? (g >> 1) : (g >> 2);
  const bool feeds = col_sub == my_sub;

  for (int64_t rb_base = (int64_t)blockIdx.x * RB_PER_CTA; rb_base * 16 < N; rb_base += (int64_t)gridDim.x * RB_PER_CTA) {
    const int64_t rb = rb_base + rb_in_cta;
    const bool active = rb * 16 < N;            // warp-uniform; inactive warps only keep the barriers company
    int64_t r0 = rb * 16 + g, r1 = r0 + 8;
    if (r0 >= N) r0 = N - 1;
    if (r1 >= N) r1 = N - 1;
    const bool push_vec = PUSH && rb * 16 + 16 <= N && (ldy & 3) == 0;      // warp-uniform
    const uint8_t* p0 = codes + r0 * row_bytes + t * 16;
    const uint8_t* p1 = codes + r1 * row_bytes + t * 16;
    const __half* sc0 = scales + r0 * groups;
    const __half* sc1 = scales + r1 * groups;
    // acc0 / acc1: row g / row g+8, one value per column set: this lane's two C columns (one activation
    // vector, two groups) already multiplied by their group scales and summed
    float acc0[NB][1], acc1[NB][1];
#pragma unroll
    for (int b = 0; b < NB; ++b) acc0[b][0] = acc1[b][0] = 0.0f;

    const bool first_block = rb_base == (int64_t)blockIdx.x * RB_PER_CTA;      // its first PD steps are already in flight
    if (PD > 0 && active && !first_block) {
#pragma unroll
      for (int j = 0; j < PD; ++j)
        if (s_begin + j < s_end) fetch(p0, p1, sc0, sc1, s_begin + j, ring[j]);
    }
    auto consume = [&](int64_t s, const StepRegs& rg) {
      const uint4 w0 = rg.w0, w1 = rg.w1;
      float s0[GROUPS_PER_STEP], s1[GROUPS_PER_STEP];
      if (Q8) {
        const __half2 a = *reinterpret_cast<const __half2*>(&rg.sa[0]);
        const __half2 b = *reinterpret_cast<const __half2*>(&rg.sb[0]);
        s0[0] = __low2float(a); s0[1] = __high2float(a);
        s1[0] = __low2float(b); s1[1] = __high2float(b);
      } else {
        const __half2 a0 = *reinterpret_cast<const __half2*>(&rg.sa[0]), a1 = *reinterpret_cast<const __half2*>(&rg.sa[1]);
        const __half2 b0 = *reinterpret_cast<const __half2*>(&rg.sb[0]), b1 = *reinterpret_cast<const __half2*>(&rg.sb[1]);
        s0[0] = __low2float(a0); s0[1] = __high2float(a0); s0[2] = __low2float(a1); s0[3] = __high2float(a1);
        s1[0] = __low2float(b0); s1[1] = __high2float(b0); s1[2] = __low2float(b1); s1[3] = __high2float(b1);
      }
      // A fragments: afr[j] = {row g slots 2t..; row g+8 slots 2t..; row g slots 2t+8..; row g+8 slots 2t+8..}
      uint32_t afr[MMAS][4];
      {
        const uint32_t ww0[4] = {w0.x, w0.y, w0.z, w0.w};
        const uint32_t ww1[4] = {w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (Q8) {
            q8_word_to_h2(ww0[q], afr[q][0], afr[q][2]);
            q8_word_to_h2(ww1[q], afr[q][1], afr[q][3]);
          } else {
            uint32_t h0[4], h1[4];
            q4_word_to_h2(ww0[q], h0);
            q4_word_to_h2(ww1[q], h1);
            afr[2 * q][0] = h0[0]; afr[2 * q][2] = h0[1]; afr[2 * q + 1][0] = h0[2]; afr[2 * q + 1][2] = h0[3];
            afr[2 * q][1] = h1[0]; afr[2 * q][3] = h1[1]; afr[2 * q + 1][1] = h1[2]; afr[2 * q + 1][3] = h1[3];
          }
        }
      }
      // this lane's k range in the step: Q8 16 k at 16*t, Q4 32 k at 32*t
      const int64_t kbase = s * KSTEP + (Q8 ? 16 : 32) * t;
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int v = b * VPM + v_of_g;
        const bool on = feeds && v < NV;
        // B fragments: MMA j takes 4 consecutive k (two fp16x2 registers)
        uint32_t bfr[MMAS][2];
        if (on) {
          const uint4* xp = reinterpret_cast<const uint4*>(xs + (int64_t)v * K + kbase);
#pragma unroll
          for (int i = 0; i < MMAS / 2; ++i) {
            const uint4 xv = xp[i];
            bfr[2 * i][0] = xv.x; bfr[2 * i][1] = xv.y; bfr[2 * i + 1][0] = xv.z; bfr[2 * i + 1][1] = xv.w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < MMAS; ++j) bfr[j][0] = bfr[j][1] = 0u;
        }
        float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < MMAS; ++j) mma_f16_16816(d, afr[j], bfr[j][0], bfr[j][1]);
        // this lane's C columns are 2t and 2t+1: (vector, group) pairs of column set b
        //   Q8: col 2t   = (v = t, half 0), col 2t+1 = (v = t, half 1)         -> one vector, two groups
        //   Q4: col 2t   = (v = t>>1, group 2*(t&1)), col 2t+1 = group 2*(t&1)+1 -> one vector, two groups
        if (Q8) {
          acc0[b][0] = fmaf(s0[0], d[0], acc0[b][0]);
          acc0[b][0] = fmaf(s0[1], d[1], acc0[b][0]);
          acc1[b][0] = fmaf(s1[0], d[2], acc1[b][0]);
          acc1[b][0] = fmaf(s1[1], d[3], acc1[b][0]);
        } else {
          const int q0 = 2 * (t & 1);
          acc0[b][0] = fmaf(q0 ? s0[2] : s0[0], d[0], acc0[b][0]);
          acc0[b][0] = fmaf(q0 ? s0[3] : s0[1], d[1], acc0[b][0]);
          acc1[b][0] = fmaf(q0 ? s1[2] : s1[0], d[2], acc1[b][0]);
          acc1[b][0] = fmaf(q0 ? s1[3] : s1[1], d[3], acc1[b][0]);
        }
      }
    };
    if (PD == 0) {
      // KSPLIT == 8 is the small-N / long-K case: a warp has only a dozen steps, so the loop is unrolled further
      constexpr int UNR = KSPLIT == 8 ? 4 : 2;
#pragma unroll UNR
      for (int64_t s = active ? s_begin : s_end; s < s_end; ++s) {
        fetch(p0, p1, sc0, sc1, s, ring[0]);
        consume(s, ring[0]);
      }
    } else {
      for (int64_t s = active ? s_begin : s_end; s < s_end; s += PD + 1) {
#pragma unroll
        for (int u = 0; u <= PD; ++u) {
          if (s + u < s_end) {
            if (s + u + PD < s_end) fetch(p0, p1, sc0, sc1, s + u + PD, ring[(u + PD) % (PD + 1)]);
            consume(s + u, ring[u]);
          }
        }
      }
    }

    // ---- fold: Q4 has the two group pairs of a vector in lanes t and t^1 ------------------------------
    if (!Q8) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        acc0[b][0] += __shfl_xor_sync(0xffffffffu, acc0[b][0], 1);
        acc1[b][0] += __shfl_xor_sync(0xffffffffu, acc1[b][0], 1);
      }
    }
    // lane (g, t) now holds, for column set b: Q8 vector b*4 + t; Q4 vector b*2 + (t >> 1) (in both lanes of a pair)
    // ---- K-split partials meet in shared memory (summed in a fixed order), then scale back and store ----
    if (KSPLIT > 1) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int v = Q8 ? (b * VPM + t) : (b * VPM + (t >> 1));
        if (v < NV && (Q8 || (t & 1) == 0)) {
          red[(warp * 16 + g) * NV + v] = acc0[b][0];
          red[(warp * 16 + g + 8) * NV + v] = acc1[b][0];
        }
      }
      __syncthreads();
    }
    float racc0[NB], racc1[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) racc0[b] = racc1[b] = 0.0f;
    if (KSPLIT == 1 || ksp == 0) {      // warp-uniform
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int v = Q8 ? (b * VPM + t) : (b * VPM + (t >> 1));
        float a0 = acc0[b][0], a1 = acc1[b][0];
        if (KSPLIT > 1) {
          a0 = 0.0f; a1 = 0.0f;
          if (v < NV) {
#pragma unroll
            for (int i = 0; i < KSPLIT; ++i) {
              a0 += red[((rb_in_cta * KSPLIT + i) * 16 + g) * NV + v];
              a1 += red[((rb_in_cta * KSPLIT + i) * 16 + g + 8) * NV + v];
            }
          }
        }
        if (CL) {                           // park this CTA's sums where the cluster's rank 0 can read them
          if (v < NV && (Q8 || (t & 1) == 0)) {
            cred[(rb_in_cta * 16 + g) * NV + v] = a0;
            cred[(rb_in_cta * 16 + g + 8) * NV + v] = a1;
          }
        }
        racc0[b] = a0;
        racc1[b] = a1;
      }
    }
    if (CL) cluster_sync_all();             // every CTA of the cluster runs the same number of trips
    if ((KSPLIT == 1 || ksp == 0) && cy == 0) {
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        const int v = Q8 ? (b * VPM + t) : (b * VPM + (t >> 1));
        float a0 = racc0[b], a1 = racc1[b];
        if (CL && v < NV) {
          for (int r = 1; r < kc; ++r) {    // fixed order: deterministic
            a0 += ld_cluster_f32(&cred[(rb_in_cta * 16 + g) * NV + v], (uint32_t)r);
            a1 += ld_cluster_f32(&cred[(rb_in_cta * 16 + g + 8) * NV + v], (uint32_t)r);
          }
        }
        const float back = v < NV ? xscale[v] : 0.0f;
        a0 *= back;
        a1 *= back;
        if (XF32) {   // hi and lo vectors of an fp32 row: neighbouring lanes (Q8) / neighbouring pairs (Q4)
          a0 += __shfl_xor_sync(0xffffffffu, a0, Q8 ? 1 : 2);
          a1 += __shfl_xor_sync(0xffffffffu, a1, Q8 ? 1 : 2);
        }
        const int m = XF32 ? (v >> 1) : v;
        const bool writer = XF32 ? (Q8 ? (t & 1) == 0 : t == 0) : (Q8 ? true : (t & 1) == 0);
        if (active && writer && v < NV && m < m_rows) {
          const int64_t ra = rb * 16 + g, rbb = ra + 8;
          if (PUSH) {       // y is a CommDev: the partial sums go straight into every rank's receive slot
            if (push_vec) {   // whole 16-row block: staged, then stored as 16-byte vectors (below)
              push_stage[(rb_in_cta * 4 + m) * 16 + g] = a0;
              push_stage[(rb_in_cta * 4 + m) * 16 + g + 8] = a1;
            } else {
              const int world = comm_world(y);
              for (int r = 0; r < world; ++r) {
                if (ra < N) comm_deposit(push_dst[r] + (int64_t)m * ldy + ra, a0);
                if (rbb < N) comm_deposit(push_dst[r] + (int64_t)m * ldy + rbb, a1);
              }
            }
          } else if (OUT == GM_OUT_GELU || OUT == GM_OUT_SILU) {
            if (rbb < N) {   // a0 = gate, a1 = up of output column rb*8 + g (same formulas as gated_act_kernel)
              float a;
              if (OUT == GM_OUT_GELU) a = 0.5f * a0 * (1.0f + tanhf(0.7978845608028654f * (a0 + 0.044715f * a0 * a0 * a0)));
              else a = a0 / (1.0f + __expf(-a0));
              y[(int64_t)m * ldy + rb * 8 + g] = from_float<YT>(a * a1);
            }
          } else {
            if (ra < N) y[(int64_t)m * ldy + ra] = from_float<YT>(a0);
            if (rbb < N) y[(int64_t)m * ldy + rbb] = from_float<YT>(a1);
          }
        }
      }
    }
    if (PUSH && (KSPLIT == 1 || ksp == 0) && cy == 0 && active && push_vec) {
      // lane = (rank, 16-byte piece of the block's 16 outputs): one vector store per lane and activation row covers
      // every rank (world <= 8)
      __syncwarp();
      const int world = comm_world(y);
      const int r = lane >> 2, piece = lane & 3;
      if (r < world) {
        for (int m = 0; m < m_rows; ++m) {
          const float4 v = *reinterpret_cast<const float4*>(&push_stage[(rb_in_cta * 4 + m) * 16 + piece * 4]);
          comm_deposit4(push_dst[r] + (int64_t)m * ldy + rb * 16 + piece * 4, v);
        }
      }
      __syncwarp();
    }
    if (KSPLIT > 1) __syncthreads();
    if (CL) cluster_sync_all();             // rank 0 is done reading before anybody overwrites or exits
  }
}

// ---- host side ------------------------------------------------------------------------------------------
template <int FMT, int NV, int KSPLIT, typename XT, typename YT, int OUT>
static int gm_launch(const uint8_t* codes, const __half* scales, const XT* x, YT* y, int64_t N, int64_t K, int m_rows,
                     int64_t ldy, cudaStream_t s) {
  auto kern = qgemv_mma_kernel<FMT, NV, KSPLIT, XT, YT, false, OUT>;
  auto kern_cl = qgemv_mma_kernel<FMT, NV, KSPLIT, XT, YT, true, OUT>;
  const size_t smem = (size_t)NV * K * 2 + 32 + 2 * (size_t)GM_WARPS * 16 * NV * sizeof(float) + (OUT == GM_OUT_PUSH ? 128 + GM_WARPS * 4 * 16 * sizeof(float) : 0);
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    BQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    BQ_CUDA(cudaFuncSetAttribute(kern_cl, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    configured = 200 * 1024;
  }
  const int64_t rb = (N + 15) / 16;
  const int rb_per_cta = GM_WARPS / KSPLIT;
  int64_t grid = (rb + rb_per_cta - 1) / rb_per_cta;
  // CTAs that are resident at once (registers and shared memory decide; asked once per shared-memory size): the grid
  // is capped there and the CTAs walk the row blocks, so the kernel is one wave whatever N is
  static size_t occ_smem = (size_t)-1;
  static int occ = 1;
  if (smem != occ_smem) {
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, GM_THREADS, smem) != cudaSuccess || n < 1) n = 1;
    occ = n > 6 ? 6 : n;
    occ_smem = smem;
  }
  const int64_t cap = (int64_t)sm_count() * occ;
  // Few row blocks but a long K (e.g. 2048 x 16384): the CTAs above cannot fill the machine.  Split K further
  // across a thread-block cluster of kc CTAs (summed through distributed shared memory, fixed order) while every
  // warp keeps at least 4 steps to stream.
  const int64_t steps_per_warp = K / (FMT == BQ_FMT_Q8G32 ? 64 : 128) / KSPLIT;
  int kc = 1;
  while (kc < 8 && grid * kc * 2 <= (int64_t)sm_count() * 3 && steps_per_warp / (kc * 2) >= 4) kc *= 2;
  if (grid > cap) grid = cap;
  if (kc == 1)
    BQ_CUDA(launch_chain(kern, dim3((unsigned)grid), dim3(GM_THREADS), smem, s, 1, codes, scales, x, y, N, K, m_rows, ldy, 1));
  else
    BQ_CUDA(launch_chain(kern_cl, dim3((unsigned)grid, (unsigned)kc), dim3(GM_THREADS), smem, s, kc, codes, scales, x, y, N, K,
                         m_rows, ldy, kc));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

template <int FMT, int NV, typename XT, typename YT, int OUT>
static int gm_pick_split(const uint8_t* codes, const __half* scales, const XT* x, YT* y, int64_t N, int64_t K,
                         int m_rows, int64_t ldy, cudaStream_t s) {
  // enough 16-row blocks for every SM to hold several warps -> no K split; otherwise split K in the CTA
  const int64_t rb = (N + 15) / 16;
  const int64_t want = (int64_t)sm_count() * 16;      // warps that keep the memory system busy
  if (rb >= want || K < 1024) return gm_launch<FMT, NV, 1, XT, YT, OUT>(codes, scales, x, y, N, K, m_rows, ldy, s);
  if (rb * 2 >= want || K < 2048) return gm_launch<FMT, NV, 2, XT, YT, OUT>(codes, scales, x, y, N, K, m_rows, ldy, s);
  if (rb * 4 >= want || K < 4096) return gm_launch<FMT, NV, 4, XT, YT, OUT>(codes, scales, x, y, N, K, m_rows, ldy, s);
  return gm_launch<FMT, NV, 8, XT, YT, OUT>(codes, scales, x, y, N, K, m_rows, ldy, s);
}

template <int FMT, typename XT, typename YT, int OUT>
static int gm_pick_nv(const uint8_t* codes, const __half* scales, const XT* x, YT* y, int64_t N, int64_t K, int m_rows,
                      int64_t ldy, cudaStream_t s) {
  const int nv = m_rows * (sizeof(XT) == 4 ? 2 : 1);
  if (sizeof(XT) == 4) {
    if (nv <= 2) return gm_pick_split<FMT, 2, XT, YT, OUT>(codes, scales, x, y, N, K, m_rows, ldy, s);
    return gm_pick_split<FMT, 4, XT, YT, OUT>(codes, scales, x, y, N, K, m_rows, ldy, s);
  }
  if (nv == 1) return gm_pick_split<FMT, 1, XT, YT, OUT>(codes, scales, x, y, N, K, m_rows, ldy, s);
  if (nv == 2) return gm_pick_split<FMT, 2, XT, YT, OUT>(codes, scales, x, y, N, K, m_rows, ldy, s);
  return gm_pick_split<FMT, 4, XT, YT, OUT>(codes, scales, x, y, N, K, m_rows, ldy, s);
}

}  // namespace bq
