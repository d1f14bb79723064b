// Tensor-core path (sm_100a): tcgen05.mma with the dequantized weights as the A operand in tensor memory and the
// accumulator in tensor memory.
//
// Formulation ("swap-AB"): D[n, m] = sum_k W[n, k] * x[m, k].  The 128 weight rows of a tile are the MMA M
// dimension, the batch (activation rows) is the MMA N dimension (BN = 16..256), so decode-sized batches waste no
// tensor work on padding weight rows and the accumulator lane == output column n.
//
// Per CTA (one 128 x BN output tile, or two weight tiles sharing one activation tile; 320 threads), one pipeline
// step = 128 k:
//   warp 0      producer : TMA (cp.async.bulk.tensor.2d, no multicast) of the packed codes [128 rows x 128 k]
//                          (swizzled so that "one thread reads one row" is free of bank conflicts), two activation
//                          atoms [BN x 64 k, 128-byte swizzle = the UMMA K-major layout] and, every second step, the
//                          fp16 scales [128 x 8 groups] into a ring of stages with mbarrier transaction counts
//   warps 2..9  converter: every thread owns one weight row (= its TMEM lane): packed codes + scale -> fp16 =
//                          code * scale (exact product rounded once to fp16) in registers, written with tcgen05.st
//                          into one of two A buffers in tensor memory; later the epilogue
//   warp 1      issuer   : one thread issues 8 x tcgen05.mma (K = 16 each, kind::f16, A from TMEM, B = fp16
//                          activations from shared memory, D = fp32 in TMEM) per step and commits to the barriers
//                          that free the A buffer and the stage
//   epilogue             : tcgen05.ld of the 128 x BN fp32 tile, row back-scale, transposed into the (idle) stage ring
//                          and written with one bulk tensor store (cp.async.bulk.tensor, shared -> global); plain
//                          st.global for MoE tiles and outputs whose rows are not 16-byte aligned
// A dense call requests the codes and scales of its first stages before griddepcontrol.wait (weights do not depend
// on the preceding kernel).  Every mbarrier wait is bounded; on expiry a status word is set and all roles drain and exit.
//
// Activations reach the tensor core as fp16: a pre-pass kernel scales every activation row by a power of two that
// puts its largest magnitude in [2^14, 2^15) and rounds to fp16 (exact for bf16 inputs down to 2^-29 of the row
// maximum); the epilogue multiplies the row back.  Both MMA operands then have the same type (an fp16 A with a bf16 B
// in one kind::f16 MMA raises an illegal-instruction error on this GPU).
//
// MODE 1 (GATED; MoE experts / SwiGLU): the gate and up matrices share the activation tile, two accumulators, the
// epilogue writes silu(g) * u as bf16.  MODE 2 (DUAL): rows n0.. and n0+128.. of one matrix share the activation tile.
#include <cuda.h>

#include "common.cuh"

namespace bq {

constexpr int TC_ROWS = 128;        // weight rows per tile (UMMA M)
// Converter warps: 4 * KQ per CTA, KQ per tensor-memory lane quarter, each converting 128 / KQ k of its 32 rows per step.
// Tiles of 128 batch rows and more use KQ = 4 (16 warps): with 8 warps a step took ~3000 cycles although no unit was
// busy, because a converter warp issues one instruction per ~5 cycles (dependent PRMT / HSUB2 / HMUL2 chains) and two
// warps per scheduler cannot hide that.  Smaller tiles (two CTAs per SM, little to convert per MMA) keep KQ = 2:
// measured, 16 warps made M = 64 slower.
__host__ __device__ constexpr int tc_kq(int bn) { return bn >= 128 ? 4 : 2; }
__host__ __device__ constexpr int tc_threads(int kq) { return 64 + 128 * kq; }
constexpr int TC_SC_SLOTS = 3;      // scale tiles in flight (each covers 2 k-steps)
constexpr size_t TC_PART_BYTES = (size_t)64 << 20;   // split-K partial tiles never exceed this
constexpr uint64_t TC_WAIT_NS = 2000000000ull;   // every device-side wait gives up after 2 s

// ---- PTX wrappers -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One try: the hardware may suspend the thread up to `hint_ns` while the phase is incomplete.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait by one thread (at most ~TC_WAIT_NS).  Returns false if the wait expired or another
// role already gave up; on expiry the CTA-wide abort flag is raised.
__device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const uint64_t t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 16; ++i)
      if (mbar_try(bar, parity, 2000u)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > TC_WAIT_NS) { *abort_flag = 1; return false; }
  }
}
// One poll without suspending the thread.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// The hand-offs of the pipeline (stage landed -> convert -> A buffer full -> MMA -> buffer free) are short waits on the
// critical path: polling them costs a few issue slots of one lane, while a thread suspended in try_wait resumed late
// enough to cost 14-20% of the whole kernel (int8, measured at M = 64 and M = 4096).  So: poll for a while (~100 us),
// then suspend.
constexpr int TC_SPIN = 8192;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (int i = 0; i < TC_SPIN; ++i)
    if (mbar_test(bar, parity)) return true;
  if (mbar_try(bar, parity, 2000u)) return true;
  return mbar_wait_slow(bar, parity, abort_flag);
}
// Warp-collective wait: lane 0 does the waiting (32 lanes polling one mbarrier word serialise on it and
// cost ~300 cycles even when the phase is complete); __syncwarp orders the other lanes' later reads of
// the data behind lane 0's observation of the phase.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile int* abort_flag, int lane) {
  uint32_t ok = 0;
  if (lane == 0) ok = mbar_wait(bar, parity, abort_flag) ? 1u : 0u;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int c0, int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
// Tile store shared -> global (bulk async group of the issuing thread).  Rows / columns of the box that fall outside
// the tensor are not written.
__device__ __forceinline__ void tma_store_2d(const void* tmap, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(tmap), "r"(c0), "r"(c1), "r"(src)
               : "memory");
}
// ends the group and waits until the stores issued so far have READ their shared-memory source
__device__ __forceinline__ void tma_store_drain() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major, 128-byte-swizzled shared-memory matrix descriptor: rows of 128 bytes, 8-row groups 1024
// bytes apart; tile base 1024-byte aligned.  Advancing K by 16 elements = +32 bytes on the address.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);       // start address
  d |= (uint64_t)1 << 16;                          // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;                // stride byte offset: 8 rows * 128 B
  d |= (uint64_t)1 << 46;                          // descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                          // SWIZZLE_128B
  return d;
}
// kind::f16 instruction descriptor: D = f32, A = B = f16, both K-major, M = 128, N = BN.
__host__ __device__ constexpr uint32_t umma_idesc(int bn) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(TC_ROWS >> 4) << 24);
}


// ---- converters: 16 bytes of codes -> fp16 (code * scale) -------------------------------------------
// Q8: 16 codes -> two 16-byte pieces of the A row.
__device__ __forceinline__ void cvt_q8_chunk(const uint4 w, const __half2 s2, uint4& lo, uint4& hi) {
  const uint32_t words[4] = {w.x, w.y, w.z, w.w};
  uint32_t o[8];
  const __half2 off = __float2half2_rn(1152.0f);   // 1024 (magic) + 128 (sign offset)
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const uint32_t v = words[q];   // device bytes are code + 128
    uint32_t p0 = __byte_perm(v, 0x64646464u, 0x4140);   // (1024 + b0, 1024 + b1) as fp16x2
    uint32_t p1 = __byte_perm(v, 0x64646464u, 0x4342);   // (1024 + b2, 1024 + b3)
    __half2 h0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p0), off), s2);
    __half2 h1 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p1), off), s2);
    o[2 * q] = *reinterpret_cast<uint32_t*>(&h0);
    o[2 * q + 1] = *reinterpret_cast<uint32_t*>(&h1);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}
// Q4: one 32-bit word in the device nibble order (e0,e2,e4,e6,e1,e3,e5,e7) -> 8 fp16 in element
// order.  Masks 0x000F000F / 0x00F000F0 pick the adjacent element pairs (e0,e1) / (e2,e3) straight
// into fp16 mantissas (1024 + n, resp. 1024 + 16 n); one shift serves the upper half of the word.
__device__ __forceinline__ uint4 cvt_q4_word(const uint32_t v, const __half2 s2) {
  const __half2 off = __float2half2_rn(1032.0f);       // 1024 (magic) + 8 (zero point)
  const __half2 sixteenth = __float2half2_rn(0.0625f);
  const __half2 off16 = __float2half2_rn(-72.0f);      // -(1024/16 + 8)
  const uint32_t v8 = v >> 8;
  uint32_t t0 = lop3_and_or(v, 0x000F000Fu, 0x64006400u);    // 1024 + (e0, e1)
  uint32_t t1 = lop3_and_or(v, 0x00F000F0u, 0x64006400u);    // 1024 + 16 * (e2, e3)
  uint32_t t2 = lop3_and_or(v8, 0x000F000Fu, 0x64006400u);   // 1024 + (e4, e5)
  uint32_t t3 = lop3_and_or(v8, 0x00F000F0u, 0x64006400u);   // 1024 + 16 * (e6, e7)
  __half2 h01 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t0), off), s2);
  __half2 h23 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&t1), sixteenth, off16), s2);
  __half2 h45 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t2), off), s2);
  __half2 h67 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&t3), sixteenth, off16), s2);
  return make_uint4(*reinterpret_cast<uint32_t*>(&h01), *reinterpret_cast<uint32_t*>(&h23),
                    *reinterpret_cast<uint32_t*>(&h45), *reinterpret_cast<uint32_t*>(&h67));
}

// One converter thread's share of a 128-k step of its weight row: 128 / KQ codes -> code * scale as fp16 pairs.
// `raw` = the row's packed codes of the step in the (swizzled) stage, `scw` = its 4 scales of the step.
template <int FMT, int KQ>
__device__ __forceinline__ void convert_row_slice(const uint8_t* raw, const __half* scw, int row, int kq, uint32_t* regs) {
  if (FMT == BQ_FMT_Q8G32) {
    // 16 codes per 16-byte chunk; chunk c of the row sits at 16-byte slot c ^ (row & 7)
#pragma unroll
    for (int i = 0; i < 8 / KQ; ++i) {
      const int c = (8 / KQ) * kq + i;
      const uint4 wv = *reinterpret_cast<const uint4*>(raw + ((c ^ (row & 7)) << 4));
      uint4 lo, hi;
      cvt_q8_chunk(wv, __half2half2(scw[c >> 1]), lo, hi);
      regs[8 * i + 0] = lo.x; regs[8 * i + 1] = lo.y; regs[8 * i + 2] = lo.z; regs[8 * i + 3] = lo.w;
      regs[8 * i + 4] = hi.x; regs[8 * i + 5] = hi.y; regs[8 * i + 6] = hi.z; regs[8 * i + 7] = hi.w;
    }
  } else {
    // 32 codes (one group) per 16-byte chunk; chunk c sits at 16-byte slot c ^ ((row >> 1) & 3)
#pragma unroll
    for (int i = 0; i < 4 / KQ; ++i) {
      const int c = (4 / KQ) * kq + i;
      const uint4 wv = *reinterpret_cast<const uint4*>(raw + ((c ^ ((row >> 1) & 3)) << 4));
      const __half2 s2 = __half2half2(scw[c]);
      const uint4 q0 = cvt_q4_word(wv.x, s2), q1 = cvt_q4_word(wv.y, s2), q2 = cvt_q4_word(wv.z, s2),
                  q3 = cvt_q4_word(wv.w, s2);
      uint32_t* r = regs + 16 * i;
      r[0] = q0.x; r[1] = q0.y; r[2] = q0.z; r[3] = q0.w; r[4] = q1.x; r[5] = q1.y; r[6] = q1.z; r[7] = q1.w;
      r[8] = q2.x; r[9] = q2.y; r[10] = q2.z; r[11] = q2.w; r[12] = q3.x; r[13] = q3.y; r[14] = q3.z; r[15] = q3.w;
    }
  }
}

// =================================================================================================
// The converted fp16 weights never touch shared memory: shared memory only holds packed codes, activations and
// scales, so two CTAs fit on an SM up to BN = 128.
// TMEM columns: [0, NW*BN) accumulators, then NW x 2 A buffers of 64 columns (= 128 k) from column 128 (NW*BN <= 128)
// or 256; 256 columns are allocated (two CTAs per SM) when that fits below 256, else all 512.
// =================================================================================================
constexpr int T2_BK = 128;
constexpr int T2_ACOLS = 64;

// NW = 2: the CTA converts two 128-row weight tiles (rows n0.. and n0+128..) per activation tile, which halves
// the activation bytes fetched per multiply-add (the activation tiles come from L2, the scarcer resource of
// large batches); then BN = 128 and all 512 TMEM columns are in use (2 accumulators + 2 x 2 A buffers).
template <int FMT, int BN, int MODE> struct T2Plan {
  static constexpr int NW = MODE ? 2 : 1;                                 // MODE: 0 single, 1 gated (gate|up), 2 dual
  static constexpr int RAW_ROW = (FMT == BQ_FMT_Q8G32) ? 128 : 64;      // code bytes per row per step
  static constexpr int RAW = TC_ROWS * RAW_ROW;
  static constexpr int XT = 2 * BN * 128;                                 // two 64-k swizzle atoms
  static constexpr int SCT = TC_ROWS * 16;                                // 8 fp16 scales per row = 256 k = 2 steps
  static constexpr int STAGE = ((NW * RAW + XT + 1023) / 1024) * 1024;
  static constexpr int FIXED = TC_SC_SLOTS * NW * SCT + 1024 + 1024;
  // tensor memory: NW accumulators of BN columns from column 0, then NW x 2 A buffers of 64 columns from ACOL0.
  // (One accumulator per weight tile: rotating the 8 MMAs of a step over several independent accumulators was
  // measured and gave nothing at any batch size -- small MMAs do not serialise on the accumulator -- while it made
  // the k-summation order, hence the low bits of the result, depend on the tile size.)
  // 256 columns (two CTAs per SM) only when everything fits below 256; two weight tiles always need 512.
  static constexpr int ACOL0 = NW * BN <= 128 ? 128 : 256;                // first A-buffer column
  static constexpr int TMEM_NEED = ACOL0 + NW * 2 * T2_ACOLS;
  static constexpr int TMEM_COLS = TMEM_NEED <= 256 ? 256 : 512;
  static constexpr int BUDGET = (TMEM_COLS == 256 ? 100 : 200) * 1024;    // shared memory follows: two CTAs per SM or one
  static constexpr int S_RAW = (BUDGET - FIXED) / STAGE;
  static constexpr int S = S_RAW > 4 ? 4 : (S_RAW < 2 ? 2 : S_RAW);       // S <= 2*SC_SLOTS - 1 = 5
  static constexpr int SMEM = FIXED + S * STAGE;
  static_assert(TMEM_NEED <= 512, "tensor memory plan too large");
  static_assert(NW * BN <= ACOL0 && BN % 16 == 0, "accumulators must fit below the A buffers");
  static_assert(SMEM <= 227 * 1024, "shared memory plan too large");
};

struct T2Args {
  CUtensorMap tm_x;      // fp16 activations [M, K], box 64 x BN, 128B swizzle
  CUtensorMap tm_w;      // codes: Q8 box 128 B x 128 rows (128B swizzle); Q4 box 64 B x 128 rows (64B swizzle)
  CUtensorMap tm_s;      // scales fp16 [N, K/32], box 8 x 128
  const float* xscale;
  void* out;
  int64_t ldy, N, K, M;
  int out_dtype;
  int* status;
  // MoE (grouped experts): per expert {codes0, scales0, codes1, scales1} descriptors, row ranges, tile list
  const CUtensorMap* tm_list;
  const int32_t* offsets;
  const int32_t* tiles;
  int moe;
  // dense split-K (few output tiles, long K): blockIdx.z takes `kper` 128-k steps from kper * blockIdx.z and leaves
  // its fp32 partial tile in part[blockIdx.z][M][N]; splitk_reduce_kernel adds the slices in order.  kper is even
  // (a scale tile covers two steps).  0 = no split.
  int kper;
  float* part;
  // >= 0 (dense only): the weight is a fused gate|up projection whose 16-row blocks hold 8 gate rows followed by the 8
  // up rows of the same outputs; the epilogue stores act(gate) * up (0 = gelu-tanh, 1 = silu) as bf16 [M, N / 2]
  int gated_act;
  int tile_order;        // pair kernel: which tile index varies fastest over the grid (see the kernel)
  // Output through a tile store (dense calls whose output rows are 16-byte aligned): the epilogue transposes the
  // accumulator into shared memory ([batch row][weight row], the layout of y) and one thread stores the tile with
  // cp.async.bulk.tensor.  tm_y covers y [M, N] (or [M, N / 2] for a gated call, or the split-K partial slices as
  // [nz * part_rows, N]); box = 128 (64 gated) x batch rows of a tile.  Plain st.global from the epilogue warps
  // cost ~130 cycles per warp store (the SM keeps few writes in flight), 2.6 us of a 128 x 64 tile.
  CUtensorMap tm_y;
  int tma_store;
  int64_t part_rows;     // rows per split-K slice in `part` (M rounded up to whole batch tiles when tma_store)
};

__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
// one converter thread's CPT (32 or 16) columns of a step
template <int CPT> __device__ __forceinline__ void tc_st_cols(uint32_t taddr, const uint32_t* v) {
  if (CPT == 32) tc_st32(taddr, v); else tc_st16(taddr, v);
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int FMT, int BN, int MODE>
__global__ void __launch_bounds__(tc_threads(tc_kq(BN)), (T2Plan<FMT, BN, MODE>::TMEM_COLS == 256 ? 2 : 1)) qgemm_tmem_kernel(const __grid_constant__ T2Args args) {
  using P = T2Plan<FMT, BN, MODE>;
  constexpr int S = P::S, NA = 2, NW = P::NW;
  constexpr int KQ = tc_kq(BN), CONV_WARPS = 4 * KQ, CPT = 64 / KQ;
  constexpr bool GATED = MODE == 1, DUAL = MODE == 2;
  static_assert(GATED || NW * BN * 512 <= S * P::STAGE, "the output tile is staged in the stage ring");
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stages = smem;                                  // per stage: [x atom 0][x atom 1][codes tile 0][codes tile 1]
  uint8_t* sc_tiles = stages + S * P::STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sc_tiles + TC_SC_SLOTS * NW * P::SCT);
  uint64_t* full = bars;               // [S]  TMA landed
  uint64_t* empty = bars + S;          // [S]  converter warps (8) + MMA commit (1)
  uint64_t* a_full = bars + 2 * S;     // [NA] converter warps (8)
  uint64_t* a_empty = a_full + NA;     // [NA] MMA commit (1)
  uint64_t* acc_full = a_empty + NA;   // [1]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(acc_full + 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t n0 = (int64_t)blockIdx.y * TC_ROWS * (DUAL ? 2 : 1);
  int64_t m0 = (int64_t)blockIdx.x * BN, m_end = args.M;
  const CUtensorMap* tmw[2] = {&args.tm_w, &args.tm_w};
  const CUtensorMap* tms[2] = {&args.tm_s, &args.tm_s};
  if (args.moe) {
    pdl_wait();                                       // the tile list and the row ranges come from preceding kernels
    if ((int)blockIdx.x >= args.tiles[0]) return;     // uniform across the CTA, before any barrier
    const int e = args.tiles[1 + 2 * blockIdx.x];
    m0 = args.tiles[2 + 2 * blockIdx.x];
    m_end = args.offsets[e + 1];
    const CUtensorMap* l = args.tm_list + (int64_t)e * 4;
    tmw[0] = l; tms[0] = l + 1; tmw[1] = GATED ? l + 2 : l; tms[1] = GATED ? l + 3 : l + 1;
  }
  const int ksteps_all = (int)(args.K / T2_BK);
  const int k0 = args.kper ? (int)blockIdx.z * args.kper : 0;                 // first 128-k step of this CTA
  const int ksteps = args.kper ? (ksteps_all - k0 < args.kper ? ksteps_all - k0 : args.kper) : ksteps_all;

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) { mbar_init(smem_u32(&full[i]), 1); mbar_init(smem_u32(&empty[i]), CONV_WARPS + 1); }
    for (int i = 0; i < NA; ++i) { mbar_init(smem_u32(&a_full[i]), CONV_WARPS); mbar_init(smem_u32(&a_empty[i]), 1); }
    mbar_init(smem_u32(acc_full), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)P::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Programmatic dependent launch: barriers and tensor memory are set up while the preceding kernel drains; nothing
  // it wrote (activations, tile list) has been read yet, and nothing is written before this point.
  pdl_launch_dependents();
  // The weights do not depend on the preceding kernel: a dense call requests the codes and scales of its first stages
  // before waiting for it, so that their latency runs under its tail (the activations follow after the wait).
  auto load_weights = [&](int ks, uint32_t fb) {
    const int s = ks % S, kg = k0 + ks;               // kg: step index in the whole K (k0 is even)
    uint8_t* st = stages + s * P::STAGE;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const int nrow = (int)n0 + (DUAL ? w * TC_ROWS : 0);
      tma_load_2d(smem_u32(st + P::XT + w * P::RAW), tmw[w], kg * P::RAW_ROW, nrow, fb);
      if ((ks & 1) == 0)
        tma_load_2d(smem_u32(sc_tiles + (((ks >> 1) % TC_SC_SLOTS) * NW + w) * P::SCT), tms[w], (kg >> 1) * 8, nrow, fb);
    }
  };
  auto stage_bytes = [&](int ks) { return (uint32_t)(NW * P::RAW + P::XT + ((ks & 1) == 0 ? NW * P::SCT : 0)); };
  int early = 0;
  if (warp == 0 && lane == 0 && !args.moe) {
    early = ksteps < S ? ksteps : S;
    for (int ks = 0; ks < early; ++ks) {
      const uint32_t fb = smem_u32(&full[ks % S]);
      mbar_expect_tx(fb, stage_bytes(ks));
      load_weights(ks, fb);
    }
  }
  pdl_wait();

  if (warp == 0) {
    // ================= producer =================
    if (lane == 0) {
      for (int ks = 0; ks < ksteps; ++ks) {
        const int s = ks % S;
        const uint32_t ph = (uint32_t)(ks / S) & 1u;
        const uint32_t fb = smem_u32(&full[s]);
        if (ks >= early) {
          if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1u, abort_flag)) break;
          mbar_expect_tx(fb, stage_bytes(ks));
        }
        uint8_t* st = stages + s * P::STAGE;
        const int kg = k0 + ks;
        tma_load_2d(smem_u32(st), &args.tm_x, kg * T2_BK, (int)m0, fb);
        tma_load_2d(smem_u32(st + BN * 128), &args.tm_x, kg * T2_BK + 64, (int)m0, fb);
        if (ks >= early) load_weights(ks, fb);
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(BN);
      const uint64_t bdesc_stage0 = umma_desc_sw128(smem_u32(stages));
      bool ok = true;
      for (int ks = 0; ks < ksteps && ok; ++ks) {
        const int s = ks % S, a = ks & 1;
        const uint32_t aph = (uint32_t)(ks >> 1) & 1u;
        ok = mbar_wait(smem_u32(&a_full[a]), aph, abort_flag);   // implies the stage (and its activations) landed
        if (!ok) break;
        tc_fence_after();
        const uint64_t bdesc0 = bdesc_stage0 + (uint64_t)((uint32_t)(s * P::STAGE) >> 4);   // stage offsets are < 256 KB
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          const uint32_t a_tmem = tmem_base + (uint32_t)(P::ACOL0 + (w * NA + a) * T2_ACOLS);
          const uint32_t d_tmem = tmem_base + (uint32_t)(w * BN);
#pragma unroll
          for (int kk = 0; kk < T2_BK / 16; ++kk)
            tc_mma_f16_ts(d_tmem, a_tmem + (uint32_t)(8 * kk),
                          bdesc0 + (uint64_t)((((kk >> 2) * BN * 128) >> 4) + 2 * (kk & 3)), idesc, (ks > 0 || kk > 0) ? 1u : 0u);
        }
        tc_commit(smem_u32(&a_empty[a]));
        tc_commit(smem_u32(&empty[s]));
      }
      if (ok) tc_commit(smem_u32(acc_full));
    }
  } else {
    // ================= converters (one weight row per thread), then epilogue =================
    const int lg = warp & 3;                 // TMEM lane group this warp may touch
    const int kq = (warp - 2) >> 2;          // which slice of the 128-k step this warp converts
    const int row = lg * 32 + lane;
    bool ok = true;
    for (int ks = 0; ks < ksteps && ok; ++ks) {
      const int s = ks % S, a = ks & 1;
      const uint32_t ph = (uint32_t)(ks / S) & 1u, aph = (uint32_t)(ks >> 1) & 1u;
      ok = mbar_wait_warp(smem_u32(&full[s]), ph, abort_flag, lane);
      ok = ok && mbar_wait_warp(smem_u32(&a_empty[a]), aph ^ 1u, abort_flag, lane);
      if (!ok) break;
#pragma unroll
      for (int w = 0; w < NW; ++w) {
      const uint8_t* raw = stages + s * P::STAGE + P::XT + w * P::RAW + row * P::RAW_ROW;
      const __half* scw = reinterpret_cast<const __half*>(sc_tiles + (((ks >> 1) % TC_SC_SLOTS) * NW + w) * P::SCT) + row * 8 + (ks & 1) * 4;
      uint32_t regs[CPT];
      convert_row_slice<FMT, KQ>(raw, scw, row, kq, regs);
      tc_st_cols<CPT>(tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(P::ACOL0 + (w * NA + a) * T2_ACOLS + CPT * kq), regs);
      }
      tc_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&a_full[a]));
        mbar_arrive(smem_u32(&empty[s]));
      }
    }
    if (ok) ok = mbar_wait_warp(smem_u32(acc_full), 0u, abort_flag, lane);
    if (ok) {
      tc_fence_after();
      const int64_t n = n0 + row;
      const uint32_t tbase = tmem_base + ((uint32_t)(lg * 32) << 16);
      if (!GATED && args.tma_store) {
        // Transposed tile(s) in the stage ring, which is idle by now (every load has landed and every MMA has
        // completed): [batch row][128 weight rows] in the output type, or [batch row][64 outputs] bf16 for a gated
        // call.  Consecutive lanes write consecutive words: no bank conflicts.  One thread stores the tile below.
        const bool gated = args.gated_act >= 0, f32 = args.kper || args.out_dtype == BQ_DT_F32;
#pragma unroll 1
        for (int c0 = 16 * kq; c0 < BN; c0 += 16 * KQ) {
          if (m0 + c0 >= m_end) break;
          float xs[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) xs[j] = m0 + c0 + j < m_end ? __ldg(args.xscale + m0 + c0 + j) : 0.0f;
#pragma unroll
          for (int w = 0; w < NW; ++w) {
            uint32_t v[16];
            tc_ld16(tbase + (uint32_t)(w * BN + c0), v);
            tc_ld_wait();
            uint8_t* tile = stages + (size_t)w * BN * 512;
            if (gated) {
              __nv_bfloat16* t16 = reinterpret_cast<__nv_bfloat16*>(tile) + (size_t)c0 * 64 + ((row >> 4) * 8 + (row & 7));
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float f = __uint_as_float(v[j]) * xs[j];
                const float up = __shfl_xor_sync(0xffffffffu, f, 8);
                if ((lane & 8) == 0) {
                  float a;
                  if (args.gated_act == 0) a = 0.5f * f * (1.0f + tanhf(0.7978845608028654f * (f + 0.044715f * f * f * f)));
                  else a = f / (1.0f + __expf(-f));
                  t16[j * 64] = __float2bfloat16_rn(a * up);
                }
              }
            } else if (f32) {
              float* t32 = reinterpret_cast<float*>(tile) + (size_t)c0 * 128 + row;
#pragma unroll
              for (int j = 0; j < 16; ++j) t32[j * 128] = __uint_as_float(v[j]) * xs[j];
            } else {
              __nv_bfloat16* t16 = reinterpret_cast<__nv_bfloat16*>(tile) + (size_t)c0 * 128 + row;
#pragma unroll
              for (int j = 0; j < 16; ++j) t16[j * 128] = __float2bfloat16_rn(__uint_as_float(v[j]) * xs[j]);
            }
          }
        }
        fence_async_smem();                     // the tile store below reads these writes through the async proxy
      } else {
#pragma unroll 1
      for (int c0 = 16 * kq; c0 < BN; c0 += 16 * KQ) {
        if (m0 + c0 >= m_end) break;
        // the 16 row back-scales of this chunk, loaded before any store (a load behind a store to memory that may
        // alias cannot be hoisted by the compiler, and 16 exposed load latencies tripled the epilogue time)
        float xs[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) xs[j] = m0 + c0 + j < m_end ? __ldg(args.xscale + m0 + c0 + j) : 0.0f;
        if (GATED) {                               // h = silu(gate) * up, rounded to bf16
          uint32_t v[16], u[16];
          tc_ld16(tbase + (uint32_t)c0, v);
          tc_ld16(tbase + (uint32_t)(BN + c0), u);
          tc_ld_wait();
          if (n < args.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int64_t m = m0 + c0 + j;
              if (m < m_end) {
                const float rs = xs[j];
                const float f = __uint_as_float(v[j]) * rs;
                const float h = f / (1.0f + __expf(-f)) * (__uint_as_float(u[j]) * rs);
                reinterpret_cast<__nv_bfloat16*>(args.out)[m * args.ldy + n] = __float2bfloat16_rn(h);
              }
            }
          }
          continue;
        }
#pragma unroll
        for (int w = 0; w < NW; ++w) {
          uint32_t v[16];
          tc_ld16(tbase + (uint32_t)(w * BN + c0), v);
          tc_ld_wait();
          const int64_t nn = n + w * TC_ROWS;
          if (args.gated_act >= 0) {
            // this lane's row is a gate row (row & 8 == 0) or the up row of the same output (lane + 8): the pair
            // meets through a shuffle and the gate lane stores act(gate) * up
            const int64_t ncol = (nn >> 4) * 8 + (nn & 7);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int64_t m = m0 + c0 + j;
              const float f = m < m_end ? __uint_as_float(v[j]) * xs[j] : 0.0f;
              const float up = __shfl_xor_sync(0xffffffffu, f, 8);
              if ((lane & 8) == 0 && m < m_end && nn < args.N) {
                float a;
                if (args.gated_act == 0) a = 0.5f * f * (1.0f + tanhf(0.7978845608028654f * (f + 0.044715f * f * f * f)));
                else a = f / (1.0f + __expf(-f));
                reinterpret_cast<__nv_bfloat16*>(args.out)[m * args.ldy + ncol] = __float2bfloat16_rn(a * up);
              }
            }
            continue;
          }
          if (nn < args.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int64_t m = m0 + c0 + j;
              if (m < m_end) {
                const float f = __uint_as_float(v[j]) * xs[j];
                if (args.kper) args.part[((int64_t)blockIdx.z * args.part_rows + m) * args.N + nn] = f;
                else if (args.out_dtype == BQ_DT_F32) reinterpret_cast<float*>(args.out)[m * args.ldy + nn] = f;
                else reinterpret_cast<__nv_bfloat16*>(args.out)[m * args.ldy + nn] = __float2bfloat16_rn(f);
              }
            }
          }
        }
      }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(args.status, BQ_ERR_TIMEOUT);
  if (!GATED && args.tma_store && threadIdx.x == 64 && !*abort_flag) {
    // rows past M and weight rows past N are clipped by the tensor map; a split-K slice keeps whole batch tiles
    const int ydiv = args.gated_act >= 0 ? 2 : 1;
    const int yrow = (int)((args.kper ? (int64_t)blockIdx.z * args.part_rows : 0) + m0);
#pragma unroll
    for (int w = 0; w < NW; ++w)
      tma_store_2d(&args.tm_y, smem_u32(stages + (size_t)w * BN * 512), (int)((n0 + w * TC_ROWS) / ydiv), yrow);
    tma_store_drain();                          // the shared-memory tile must outlive the store's reads
  }
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)P::TMEM_COLS)
                 : "memory");
  }
}

// =================================================================================================
// 2-SM variant for large batches (M >= 512): the two CTAs of a cluster form one 256 x 256 UMMA tile.
//
// Large batches are bound by the bytes a CTA must stage per multiply-add (codes + activation tile): a 128 x 256 tile
// needs 80 KB per 128-k step for int8 and only two stages fit.  Here CTA r of the pair converts weight rows
// n0 + 128 r .. + 127 into ITS tensor memory and stages only ITS half of the activation tile (batch rows m0 + 128 r ..),
// 48 KB per step, four stages; one thread of the leader (rank 0) issues tcgen05.mma.cta_group::2 (M = 256, N = 256):
// A from each CTA's tensor memory, B = the two halves in the two CTAs' shared memory, D = 128 lanes x 256 columns in
// each CTA's tensor memory.  No multicast anywhere: every CTA loads its own operands with plain TMA loads; the
// leader learns that the peer's operands are ready through one remote mbarrier arrival per step, forwarded by a thread
// of the peer once the peer's converter warps have arrived on a barrier of their own CTA (the barrier the issuer waits
// on lives in the leader's shared memory), and tells the peer that its buffers are free / its accumulator is complete
// with a second tcgen05.commit aimed at the peer's barrier.
// Tensor memory: [0, 256) accumulator, 4 x 64 columns of A from column 256 (the converters run up to three k-steps
// ahead of the MMAs, so that their latency - wake-up, unpack, tcgen05.st, arrive - is off the critical path); allocated
// with cta_group::2 by warp 1 of both CTAs.
// =================================================================================================
template <int FMT> struct PairPlan {
  static constexpr int RAW_ROW = (FMT == BQ_FMT_Q8G32) ? 128 : 64;
  static constexpr int RAW = TC_ROWS * RAW_ROW;
  static constexpr int XT = 2 * 128 * 128;                               // this CTA's 128 batch rows, two 64-k atoms
  static constexpr int SCT = TC_ROWS * 16;
  static constexpr int STAGE = ((RAW + XT + 1023) / 1024) * 1024;
  static constexpr int FIXED = TC_SC_SLOTS * SCT + 1024 + 1024;
  static constexpr int S = 4;
  static constexpr int NA = 4;                                           // A buffers in tensor memory (64 columns each)
  static constexpr int SMEM = FIXED + S * STAGE;
  static constexpr int ACOL0 = 256;
  static constexpr int TMEM_COLS = 512;
  static_assert(ACOL0 + NA * T2_ACOLS <= TMEM_COLS, "tensor memory plan too large");
  static_assert(SMEM <= 227 * 1024, "shared memory plan too large");
};

__device__ __forceinline__ uint32_t pair_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void pair_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t pair_map(uint32_t local_addr, uint32_t rank) {
  uint32_t ra;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_addr), "r"(rank));
  return ra;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_test_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __noinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (int i = 0; i < TC_SPIN; ++i)
    if (mbar_test_cluster(bar, parity)) return true;
  if (mbar_try_cluster(bar, parity, 2000u)) return true;
  const uint64_t t0 = global_ns();
  for (;;) {
    for (int i = 0; i < 16; ++i)
      if (mbar_try_cluster(bar, parity, 2000u)) return true;
    if (*abort_flag) return false;
    if (global_ns() - t0 > TC_WAIT_NS) { *abort_flag = 1; return false; }
  }
}
__device__ __forceinline__ void tc_commit2(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tc_mma2_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// kind::f16 instruction descriptor of the pair: D = f32, A = B = f16, K-major, M = 256 (128 per CTA), N = 256
__host__ __device__ constexpr uint32_t umma_idesc_pair() {
  return (1u << 4) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

template <int FMT>
__global__ void __launch_bounds__(tc_threads(4), 1) qgemm_pair_kernel(const __grid_constant__ T2Args args) {
  using P = PairPlan<FMT>;
  constexpr int S = P::S, NA = P::NA;
  static_assert(256 * 512 <= S * P::STAGE, "the output tile is staged in the stage ring");
  constexpr int KQ = 4, CONV_WARPS = 4 * KQ, CPT = 64 / KQ;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* stages = smem;                                  // per stage: [x atom 0][x atom 1][codes tile]
  uint8_t* sc_tiles = stages + S * P::STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sc_tiles + TC_SC_SLOTS * P::SCT);
  uint64_t* full = bars;               // [S]  this CTA's TMA landed
  uint64_t* empty = bars + S;          // [S]  this CTA's converter warps (8) + the leader's MMA commit (1)
  uint64_t* a_full = bars + 2 * S;     // [NA] LEADER's copy is the one in use: 8 converter warps of each CTA
  uint64_t* a_empty = a_full + NA;     // [NA] the leader's MMA commit (1)
  uint64_t* acc_full = a_empty + NA;   // [1]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(acc_full + 1);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = pair_rank();                       // 0 = leader (issues the MMAs), 1 = peer
  // Cluster dimension x = 2: rank = blockIdx.x & 1.  grid.x / 2 is the index that varies fastest among the pairs that
  // run together: the 256-row weight tile (tile_order 0: they share an activation tile, right when the weights fit in
  // L2) or the 256-row batch tile (tile_order 1: they share weight rows, right for a matrix larger than L2 - the head)
  const int64_t fast = (int64_t)(blockIdx.x >> 1), slow = (int64_t)blockIdx.y;
  const int64_t n0 = ((args.tile_order ? slow : fast) * 2 + rank) * TC_ROWS;      // this CTA's weight rows
  const int64_t m0 = (args.tile_order ? fast : slow) * 256, m_end = args.M;       // the pair's batch rows
  const int64_t mx0 = m0 + 128 * (int64_t)rank;                            // the half of them this CTA stages
  const int ksteps = (int)(args.K / T2_BK);

  if (threadIdx.x == 0) {
    for (int i = 0; i < S; ++i) { mbar_init(smem_u32(&full[i]), 1); mbar_init(smem_u32(&empty[i]), CONV_WARPS + 1); }
    // a_full: the leader's copy gates the MMAs (its own converter warps + one arrival forwarded from the peer); the
    // peer's copy collects the peer's converter warps for its forwarder
    for (int i = 0; i < NA; ++i) {
      mbar_init(smem_u32(&a_full[i]), rank == 0 ? CONV_WARPS + 1 : CONV_WARPS);
      mbar_init(smem_u32(&a_empty[i]), 1);
    }
    mbar_init(smem_u32(acc_full), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"((uint32_t)P::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  pair_sync();                          // both CTAs' barriers are initialised before anybody arrives on them remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();
  // codes and scales of the first stages are requested before the wait for the preceding kernel (see the single-CTA kernel)
  auto load_weights = [&](int ks, uint32_t fb) {
    tma_load_2d(smem_u32(stages + (ks % S) * P::STAGE + P::XT), &args.tm_w, ks * P::RAW_ROW, (int)n0, fb);
    if ((ks & 1) == 0)
      tma_load_2d(smem_u32(sc_tiles + ((ks >> 1) % TC_SC_SLOTS) * P::SCT), &args.tm_s, (ks >> 1) * 8, (int)n0, fb);
  };
  auto stage_bytes = [&](int ks) { return (uint32_t)(P::RAW + P::XT + ((ks & 1) == 0 ? P::SCT : 0)); };
  int early = 0;
  if (warp == 0 && lane == 0) {
    early = ksteps < S ? ksteps : S;
    for (int ks = 0; ks < early; ++ks) {
      const uint32_t fb = smem_u32(&full[ks % S]);
      mbar_expect_tx(fb, stage_bytes(ks));
      load_weights(ks, fb);
    }
  }
  pdl_wait();

  if (warp == 0) {
    // ================= producer: this CTA's codes, scales and its half of the activation tile =================
    if (lane == 0) {
      for (int ks = 0; ks < ksteps; ++ks) {
        const int s = ks % S;
        const uint32_t ph = (uint32_t)(ks / S) & 1u;
        const uint32_t fb = smem_u32(&full[s]);
        if (ks >= early) {
          if (!mbar_wait_cluster(smem_u32(&empty[s]), ph ^ 1u, abort_flag)) break;
          mbar_expect_tx(fb, stage_bytes(ks));
        }
        uint8_t* st = stages + s * P::STAGE;
        tma_load_2d(smem_u32(st), &args.tm_x, ks * T2_BK, (int)mx0, fb);
        tma_load_2d(smem_u32(st + 128 * 128), &args.tm_x, ks * T2_BK + 64, (int)mx0, fb);
        if (ks >= early) load_weights(ks, fb);
      }
      if (*abort_flag) {
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer (leader only) =================
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = umma_idesc_pair();
      const uint64_t bdesc_stage0 = umma_desc_sw128(smem_u32(stages));
      const uint32_t peer_a_empty = pair_map(smem_u32(&a_empty[0]), 1u), peer_empty = pair_map(smem_u32(&empty[0]), 1u);
      const uint32_t peer_acc = pair_map(smem_u32(acc_full), 1u);
      bool ok = true;
      for (int ks = 0; ks < ksteps && ok; ++ks) {
        const int s = ks % S, a = ks % NA;
        const uint32_t aph = (uint32_t)(ks / NA) & 1u;
        ok = mbar_wait_cluster(smem_u32(&a_full[a]), aph, abort_flag);   // both CTAs converted (hence both stages landed)
        if (!ok) break;
        tc_fence_after();
        const uint64_t bdesc0 = bdesc_stage0 + (uint64_t)((uint32_t)(s * P::STAGE) >> 4);
        const uint32_t a_tmem = tmem_base + (uint32_t)(P::ACOL0 + a * T2_ACOLS);
#pragma unroll
        for (int kk = 0; kk < T2_BK / 16; ++kk)
          tc_mma2_f16_ts(tmem_base, a_tmem + (uint32_t)(8 * kk),
                         bdesc0 + (uint64_t)((((kk >> 2) * 128 * 128) >> 4) + 2 * (kk & 3)), idesc, (ks > 0 || kk > 0) ? 1u : 0u);
        tc_commit2(smem_u32(&a_empty[a]));
        tc_commit2(peer_a_empty + (uint32_t)(a * 8));
        tc_commit2(smem_u32(&empty[s]));
        tc_commit2(peer_empty + (uint32_t)(s * 8));
      }
      if (ok) {
        tc_commit2(smem_u32(acc_full));
        tc_commit2(peer_acc);
      }
    } else if (lane == 0) {
      // ================= forwarder (peer only) =================
      // The peer's converter warps arrive on a barrier of their own CTA; this thread passes each completed phase on to
      // the leader as ONE cluster-scope arrival.  (With every converter warp arriving remotely, the release fence of
      // a cluster-scope arrive sat in the converter loop 16 times per step: ncu showed the warps stalled on it.)
      const uint32_t leader_a_full = pair_map(smem_u32(&a_full[0]), 0u);
      for (int ks = 0; ks < ksteps; ++ks) {
        const int a = ks % NA;
        const uint32_t aph = (uint32_t)(ks / NA) & 1u;
        if (!mbar_wait(smem_u32(&a_full[a]), aph, abort_flag)) break;
        tc_fence_after();
        tc_fence_before();
        mbar_arrive_cluster(leader_a_full + (uint32_t)(a * 8));
      }
    }
  } else {
    // ================= converters (one weight row per thread), then epilogue =================
    const int lg = warp & 3;
    const int kq = (warp - 2) >> 2;
    const int row = lg * 32 + lane;
    bool ok = true;
    for (int ks = 0; ks < ksteps && ok; ++ks) {
      const int s = ks % S, a = ks % NA;
      const uint32_t ph = (uint32_t)(ks / S) & 1u, aph = (uint32_t)(ks / NA) & 1u;
      ok = mbar_wait_warp(smem_u32(&full[s]), ph, abort_flag, lane);
      if (ok) {
        uint32_t fine = 0;
        if (lane == 0) fine = mbar_wait_cluster(smem_u32(&a_empty[a]), aph ^ 1u, abort_flag) ? 1u : 0u;
        ok = __shfl_sync(0xffffffffu, fine, 0) != 0;
      }
      if (!ok) break;
      const uint8_t* raw = stages + s * P::STAGE + P::XT + row * P::RAW_ROW;
      const __half* scw = reinterpret_cast<const __half*>(sc_tiles + ((ks >> 1) % TC_SC_SLOTS) * P::SCT) + row * 8 + (ks & 1) * 4;
      uint32_t regs[CPT];
      convert_row_slice<FMT, KQ>(raw, scw, row, kq, regs);
      tc_st_cols<CPT>(tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(P::ACOL0 + a * T2_ACOLS + CPT * kq), regs);
      tc_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(smem_u32(&a_full[a]));        // own CTA's barrier: the leader's gates the MMAs, the peer's its forwarder
        mbar_arrive(smem_u32(&empty[s]));
      }
    }
    if (ok) {
      uint32_t fine = 0;
      if (lane == 0) fine = mbar_wait_cluster(smem_u32(acc_full), 0u, abort_flag) ? 1u : 0u;
      ok = __shfl_sync(0xffffffffu, fine, 0) != 0;
    }
    if (ok) {
      tc_fence_after();
      const int64_t nn = n0 + row;
      const uint32_t tbase = tmem_base + ((uint32_t)(lg * 32) << 16);
      if (args.tma_store) {
        // transposed tile in the idle stage ring ([256 batch rows][this CTA's 128 weight rows], or [256][64] bf16 for a
        // gated call), stored by one thread below: see the single-CTA kernel
        const bool gated = args.gated_act >= 0, f32 = args.out_dtype == BQ_DT_F32;
#pragma unroll 1
        for (int c0 = 16 * kq; c0 < 256; c0 += 16 * KQ) {
          if (m0 + c0 >= m_end) break;
          float xs[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) xs[j] = m0 + c0 + j < m_end ? __ldg(args.xscale + m0 + c0 + j) : 0.0f;
          uint32_t v[16];
          tc_ld16(tbase + (uint32_t)c0, v);
          tc_ld_wait();
          if (gated) {
            __nv_bfloat16* t16 = reinterpret_cast<__nv_bfloat16*>(stages) + (size_t)c0 * 64 + ((row >> 4) * 8 + (row & 7));
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float f = __uint_as_float(v[j]) * xs[j];
              const float up = __shfl_xor_sync(0xffffffffu, f, 8);
              if ((lane & 8) == 0) {
                float act;
                if (args.gated_act == 0) act = 0.5f * f * (1.0f + tanhf(0.7978845608028654f * (f + 0.044715f * f * f * f)));
                else act = f / (1.0f + __expf(-f));
                t16[j * 64] = __float2bfloat16_rn(act * up);
              }
            }
          } else if (f32) {
            float* t32 = reinterpret_cast<float*>(stages) + (size_t)c0 * 128 + row;
#pragma unroll
            for (int j = 0; j < 16; ++j) t32[j * 128] = __uint_as_float(v[j]) * xs[j];
          } else {
            __nv_bfloat16* t16 = reinterpret_cast<__nv_bfloat16*>(stages) + (size_t)c0 * 128 + row;
#pragma unroll
            for (int j = 0; j < 16; ++j) t16[j * 128] = __float2bfloat16_rn(__uint_as_float(v[j]) * xs[j]);
          }
        }
        fence_async_smem();
      } else {
#pragma unroll 1
      for (int c0 = 16 * kq; c0 < 256; c0 += 16 * KQ) {
        if (m0 + c0 >= m_end) break;
        float xs[16];                            // back-scales first: see the single-CTA kernel
#pragma unroll
        for (int j = 0; j < 16; ++j) xs[j] = m0 + c0 + j < m_end ? __ldg(args.xscale + m0 + c0 + j) : 0.0f;
        uint32_t v[16];
        tc_ld16(tbase + (uint32_t)c0, v);
        tc_ld_wait();
        if (args.gated_act >= 0) {
          const int64_t ncol = (nn >> 4) * 8 + (nn & 7);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int64_t m = m0 + c0 + j;
            const float f = m < m_end ? __uint_as_float(v[j]) * xs[j] : 0.0f;
            const float up = __shfl_xor_sync(0xffffffffu, f, 8);
            if ((lane & 8) == 0 && m < m_end && nn < args.N) {
              float act;
              if (args.gated_act == 0) act = 0.5f * f * (1.0f + tanhf(0.7978845608028654f * (f + 0.044715f * f * f * f)));
              else act = f / (1.0f + __expf(-f));
              reinterpret_cast<__nv_bfloat16*>(args.out)[m * args.ldy + ncol] = __float2bfloat16_rn(act * up);
            }
          }
          continue;
        }
        if (nn < args.N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int64_t m = m0 + c0 + j;
            if (m < m_end) {
              const float f = __uint_as_float(v[j]) * xs[j];
              if (args.out_dtype == BQ_DT_F32) reinterpret_cast<float*>(args.out)[m * args.ldy + nn] = f;
              else reinterpret_cast<__nv_bfloat16*>(args.out)[m * args.ldy + nn] = __float2bfloat16_rn(f);
            }
          }
        }
      }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(args.status, BQ_ERR_TIMEOUT);
  if (args.tma_store && threadIdx.x == 64 && !*abort_flag) {
    tma_store_2d(&args.tm_y, smem_u32(stages), (int)(n0 / (args.gated_act >= 0 ? 2 : 1)), (int)m0);
    tma_store_drain();
  }
  pair_sync();                          // neither CTA frees tensor memory or leaves while the other may still use it
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)P::TMEM_COLS)
                 : "memory");
  }
}

// Activation pre-pass: one block per row.  scale_back[m] = 2^e with e = floor(log2(rowmax)) - 14, and
// x16[m, k] = fp16(x[m, k] * 2^-e).  Rows that are all zero (or hold inf / nan) use e = 0.
template <typename XT>
__global__ void __launch_bounds__(256) x_prep_kernel(const XT* __restrict__ x, int64_t K, __half* __restrict__ x16,
                                                     float* __restrict__ scale_back, const int32_t* __restrict__ nrows_dev) {
  pdl_launch_dependents();
  pdl_wait();
  if (nrows_dev && (int64_t)blockIdx.x >= (int64_t)*nrows_dev) return;     // rows in use are only known on the device
  const XT* row = x + (int64_t)blockIdx.x * K;
  __half* orow = x16 + (int64_t)blockIdx.x * K;
  // K is a multiple of 256 and rows are 16-byte aligned: a thread owns chunks of 8 elements; the first XP_CACHE chunks
  // stay in registers between the two passes (rows up to 8192 elements are read once)
  constexpr int XP_CACHE = 4;
  float v[XP_CACHE][8];
  float mx = 0.0f;
  const int64_t chunks = K / 8;
#pragma unroll
  for (int c = 0; c < XP_CACHE; ++c) {
    const int64_t i = (int64_t)threadIdx.x + (int64_t)c * 256;
    if (i < chunks) {
      load8<XT>(row + i * 8, v[c]);
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(v[c][j]));
    }
  }
  for (int64_t i = (int64_t)threadIdx.x + (int64_t)XP_CACHE * 256; i < chunks; i += 256) {
    float t[8];
    load8<XT>(row + i * 8, t);
#pragma unroll
    for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fabsf(t[j]));
  }
  __shared__ float red[8];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  mx = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
  int e = 0;
  if (mx > 0.0f && mx < INFINITY) e = (int)((__float_as_uint(mx) >> 23) & 0xFF) - 127 - 14;   // floor(log2) - 14
  if (e < -100) e = -100;                                   // denormal row maxima: keep 2^-e finite
  const float down = __uint_as_float((uint32_t)(127 - e) << 23);   // 2^-e
  auto emit = [&](int64_t i, const float* f) {
    __half h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) h[j] = __float2half_rn(f[j] * down);
    *reinterpret_cast<uint4*>(orow + i * 8) = *reinterpret_cast<const uint4*>(h);
  };
#pragma unroll
  for (int c = 0; c < XP_CACHE; ++c) {
    const int64_t i = (int64_t)threadIdx.x + (int64_t)c * 256;
    if (i < chunks) emit(i, v[c]);
  }
  for (int64_t i = (int64_t)threadIdx.x + (int64_t)XP_CACHE * 256; i < chunks; i += 256) {
    float t[8];
    load8<XT>(row + i * 8, t);
    emit(i, t);
  }
  if (threadIdx.x == 0) scale_back[blockIdx.x] = __uint_as_float((uint32_t)(127 + e) << 23);
}

// out[m, n] = sum over z of part[z][m][n], slices added in order (deterministic), stored in the output type
template <typename YT>
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, int nz, int64_t M, int64_t N,
                                                            int64_t part_rows, YT* __restrict__ out, int64_t ldy) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t total = M * N, zstride = part_rows * N;          // a slice holds part_rows >= M rows
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float s = part[i];
    for (int z = 1; z < nz; ++z) s += part[(int64_t)z * zstride + i];
    const int64_t m = i / N, n = i - m * N;
    out[m * ldy + n] = from_float<YT>(s);
  }
}

// Same for a fused gate|up weight (16-column blocks = 8 gate + 8 up values of the same outputs): the slices are added
// in order and out[m, n / 16 * 8 + n % 8] = act(gate) * up is stored as bf16 [M, N / 2].
__global__ void __launch_bounds__(256) splitk_reduce_gated_kernel(const float* __restrict__ part, int nz, int64_t M, int64_t N,
                                                                  int64_t part_rows, __nv_bfloat16* __restrict__ out, int64_t ldy,
                                                                  int act) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t half = N / 2, total = M * half;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / half, c = i - m * half;
    const int64_t ng = (c >> 3) * 16 + (c & 7);
    float g = 0.0f, u = 0.0f;
    for (int z = 0; z < nz; ++z) {
      const float* p = part + ((int64_t)z * part_rows + m) * N + ng;
      g += p[0];
      u += p[8];
    }
    float a;
    if (act == 0) a = 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
    else a = g / (1.0f + __expf(-g));
    out[m * ldy + c] = __float2bfloat16_rn(a * u);
  }
}

// ---- library-owned scratch (see Scratch in common.cuh: never freed, growth refused during capture) -------------
static Scratch g_x16;      // pre-scaled fp16 activations [rows, K]
static Scratch g_xs;       // per-row power-of-two back-scales
static Scratch g_part;     // split-K partial tiles

static int ensure_x_scratch(int64_t rows, int64_t K, cudaStream_t s) {
  int rc = scratch_ensure(&g_x16, ((size_t)rows * K + 64) * sizeof(__half), s, "tcgen05 path (activation pre-pass)");
  if (rc) return rc;
  return scratch_ensure(&g_xs, ((size_t)rows + 64) * sizeof(float), s, "tcgen05 path (activation scales)");
}
int tc_reserve(int64_t rows, int64_t K, int64_t N) {
  int rc = ensure_x_scratch(rows, K, 0);
  if (rc) return rc;
  // split-K partial tiles are bounded by TC_PART_BYTES whatever the shape
  size_t part = (size_t)((rows + 255) / 256 * 256) * N * 4 * sizeof(float);      // slices hold whole batch tiles
  if (part > TC_PART_BYTES) part = TC_PART_BYTES;
  return scratch_ensure(&g_part, part, 0, "tcgen05 path (split-K partial tiles)");
}
static int launch_x_prep(const void* x, int x_dtype, int64_t rows, int64_t K, cudaStream_t s,
                         const int32_t* nrows_dev = nullptr) {
  int rc = ensure_x_scratch(rows, K, s);
  if (rc) return rc;
  if (x_dtype != BQ_DT_BF16) return fail(BQ_ERR_UNSUPPORTED, "tensor path takes bf16 activations");
  BQ_CUDA(launch_chain(x_prep_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(256), 0, s, 1, (const __nv_bfloat16*)x, K,
                       (__half*)g_x16.ptr, (float*)g_xs.ptr, nrows_dev));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

// small kernel: MoE tile list from expert offsets.  tiles[0] = count, then (expert, m0) pairs.
__global__ void __launch_bounds__(1024) moe_tile_list_kernel(const int32_t* __restrict__ offsets, int E, int bn,
                                                             int32_t* __restrict__ tiles) {
  __shared__ int32_t pre[1024];
  const int e = threadIdx.x;
  int32_t cnt = 0;
  pdl_launch_dependents();
  pdl_wait();
  if (e < E) cnt = (offsets[e + 1] - offsets[e] + bn - 1) / bn;
  pre[e] = cnt;
  __syncthreads();
  for (int off = 1; off < 1024; off <<= 1) {
    const int32_t add = e >= off ? pre[e - off] : 0;
    __syncthreads();
    pre[e] += add;
    __syncthreads();
  }
  if (e < E) {
    const int32_t base = pre[e] - cnt;
    const int32_t a = offsets[e];
    for (int i = 0; i < cnt; ++i) {
      tiles[1 + 2 * (base + i)] = e;
      tiles[2 + 2 * (base + i)] = a + i * bn;
    }
  }
  if (e == E - 1) tiles[0] = pre[e];
}


// ---- host side --------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

static int make_map_2d(CUtensorMap* tm, CUtensorMapDataType dt, const void* base, uint64_t inner, uint64_t outer,
                       uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, CUtensorMapSwizzle sw) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(BQ_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(BQ_ERR_CUDA, "cuTensorMapEncodeTiled failed (code " + std::to_string((int)r) + ")");
  return BQ_OK;
}

// Descriptors of one weight: codes box = one 128-k step of 128 rows (int8: 128-byte rows, 128-byte swizzle; 4-bit:
// 64-byte rows, 64-byte swizzle -- either way "one thread reads one row" is free of bank conflicts); scales box =
// 8 groups (256 k) of 128 rows.
static int weight_maps(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K, CUtensorMap* tm_codes,
                       CUtensorMap* tm_scales) {
  const uint64_t rb = fmt == BQ_FMT_Q8G32 ? K : K / 2;
  int rc = make_map_2d(tm_codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, codes, rb, (uint64_t)N, rb,
                       fmt == BQ_FMT_Q8G32 ? 128 : 64, TC_ROWS,
                       fmt == BQ_FMT_Q8G32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
  if (rc) return rc;
  return make_map_2d(tm_scales, CU_TENSOR_MAP_DATA_TYPE_UINT16, scales, (uint64_t)(K / GROUP), (uint64_t)N,
                     (uint64_t)(K / GROUP) * 2, 8, TC_ROWS, CU_TENSOR_MAP_SWIZZLE_NONE);
}

static int x_map(CUtensorMap* tm, const void* x, int64_t rows, int64_t K, int bn) {
  return make_map_2d(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x, (uint64_t)K, (uint64_t)rows, (uint64_t)K * 2, 64,
                     (uint32_t)bn, CU_TENSOR_MAP_SWIZZLE_128B);
}

bool tc_shape_ok(int64_t N, int64_t K) {
  // scale rows must be 16-byte multiples for the TMA descriptor: K % 256 == 0
  return N >= 1 && K >= 256 && (K % 256) == 0 && N < ((int64_t)1 << 31) && K < ((int64_t)1 << 31);
}

bool tc_supported(int fmt, int64_t N, int64_t K, int x_dtype, int64_t M) {
  (void)fmt;
  return x_dtype == BQ_DT_BF16 && M >= 1 && M < ((int64_t)1 << 31) && tc_shape_ok(N, K);
}

static int pick_bn(int64_t M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

template <int FMT, int BN, int MODE>
static int t2_launch(const T2Args& a, dim3 grid, cudaStream_t s) {
  using P = T2Plan<FMT, BN, MODE>;
  auto kern = qgemm_tmem_kernel<FMT, BN, MODE>;
  static bool configured = false;
  if (!configured) {
    BQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P::SMEM));
    configured = true;
  }
  BQ_CUDA(launch_chain(kern, grid, dim3(tc_threads(tc_kq(BN))), (size_t)P::SMEM, s, 1, a));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}
template <int FMT>
static int pair_launch(const T2Args& a, dim3 grid, cudaStream_t s) {
  using P = PairPlan<FMT>;
  auto kern = qgemm_pair_kernel<FMT>;
  static bool configured = false;
  if (!configured) {
    BQ_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, P::SMEM));
    configured = true;
  }
  BQ_CUDA(launch_chain(kern, grid, dim3(tc_threads(4)), (size_t)P::SMEM, s, -2, a));      // clusters of 2 CTAs along grid.x
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}
template <int FMT>
static int t2_dispatch(const T2Args& a, int bn, dim3 grid, cudaStream_t s) {
  switch (bn) {
    case 16:  return t2_launch<FMT, 16, 0>(a, grid, s);
    case 32:  return t2_launch<FMT, 32, 0>(a, grid, s);
    case 64:  return t2_launch<FMT, 64, 0>(a, grid, s);
    case 128: return t2_launch<FMT, 128, 0>(a, grid, s);
    case 256: return t2_launch<FMT, 256, 0>(a, grid, s);
    default:  return t2_launch<FMT, 128, 2>(a, grid, s);      // 512: two weight tiles x 128 batch rows
  }
}

// Tensor map of the output for the epilogue's tile store: `cols` elements per row (fp32 or bf16), row stride ld
// elements, box = box_cols x box_rows.  Returns false (plain stores are used) when the rows are not 16-byte aligned.
static bool out_map(CUtensorMap* tm, void* base, bool f32, int64_t cols, int64_t rows, int64_t ld, int box_cols, int box_rows,
                    int* rc) {
  const int es = f32 ? 4 : 2;
  *rc = BQ_OK;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (ld * es) % 16 != 0) return false;
  *rc = make_map_2d(tm, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, base, (uint64_t)cols,
                    (uint64_t)rows, (uint64_t)ld * es, (uint32_t)box_cols, (uint32_t)box_rows, CU_TENSOR_MAP_SWIZZLE_NONE);
  return *rc == BQ_OK;
}

int launch_qlinear_tc(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K, const void* x,
                      int x_dtype, int64_t M, void* y, int y_dtype, int64_t ldy, cudaStream_t s, int gated_act) {
  if (x_dtype != BQ_DT_BF16) return fail(BQ_ERR_UNSUPPORTED, "tensor path takes bf16 activations");
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return fail(BQ_ERR_ARG, "activations must be 16-byte aligned");
  const int bn = pick_bn(M);
  int rc = launch_x_prep(x, x_dtype, M, K, s);
  if (rc) return rc;
  T2Args t;
  memset(&t, 0, sizeof(t));
  // Large batches: pairs of CTAs on 256 x 256 tiles (each stages half of the activation tile), when the pairs fill at
  // least half the machine.  Measured at M = 4096 against one CTA per tile (int8) / two weight tiles per CTA (4-bit):
  // (12288, 3072) int8 875 TFLOP/s, 4-bit 896 against 823; (16384, 8192) 4-bit 1137 against 1050; the int8 prefill of the
  // 7B shape (8 x 4096 tokens) 860 ms against 1178 ms.
  const int64_t row_tiles = (N + TC_ROWS - 1) / TC_ROWS;
  if (M >= 512 && N >= 2 * TC_ROWS && ((row_tiles + 1) / 2) * ((M + 255) / 256) * 2 >= (int64_t)sm_count()) {
    if ((rc = x_map(&t.tm_x, g_x16.ptr, M, K, 128))) return rc;
    if ((rc = weight_maps(codes, scales, fmt, N, K, &t.tm_w, &t.tm_s))) return rc;
    t.xscale = (const float*)g_xs.ptr; t.out = y; t.ldy = ldy; t.N = N; t.K = K; t.M = M; t.out_dtype = y_dtype;
    t.status = status_word();
    t.gated_act = gated_act;
    t.tma_store = out_map(&t.tm_y, y, gated_act < 0 && y_dtype == BQ_DT_F32, gated_act >= 0 ? N / 2 : N, M, ldy,
                          gated_act >= 0 ? 64 : 128, 256, &rc) ? 1 : 0;
    if (rc) return rc;
    // weights that do not fit in L2 while the activations do: batch tiles vary fastest, so a weight tile is read once
    const int64_t w_bytes = N * (fmt == BQ_FMT_Q8G32 ? K : K / 2), x_bytes = M * K * 2;
    t.tile_order = (w_bytes > ((int64_t)64 << 20) && x_bytes <= ((int64_t)64 << 20)) ? 1 : 0;
    const int64_t pairs_n = (row_tiles + 1) / 2, tiles_m = (M + 255) / 256;
    dim3 gridp((unsigned)(2 * (t.tile_order ? tiles_m : pairs_n)), (unsigned)(t.tile_order ? pairs_n : tiles_m));
    return fmt == BQ_FMT_Q8G32 ? pair_launch<BQ_FMT_Q8G32>(t, gridp, s) : pair_launch<BQ_FMT_Q4G32>(t, gridp, s);
  }
  // large batches are bound by the L2 -> SM traffic of codes + activations per multiply-add: 4-bit weights do
  // better with 256 weight rows x 128 batch rows per CTA, int8 with 128 x 256 (measured)
  // (only when that still gives every SM a CTA; otherwise 128-row tiles, split over K below when they are few)
  const bool two = bn == 256 && fmt == BQ_FMT_Q4G32 && N >= 2 * TC_ROWS &&
                   ((M + 127) / 128) * ((N + 2 * TC_ROWS - 1) / (2 * TC_ROWS)) >= (int64_t)sm_count();
  const int bx = two ? 128 : bn;
  if ((rc = x_map(&t.tm_x, g_x16.ptr, M, K, bx))) return rc;
  if ((rc = weight_maps(codes, scales, fmt, N, K, &t.tm_w, &t.tm_s))) return rc;
  t.xscale = (const float*)g_xs.ptr; t.out = y; t.ldy = ldy; t.N = N; t.K = K; t.M = M; t.out_dtype = y_dtype;
  t.status = status_word();
  t.gated_act = gated_act;
  const int rows_cta = two ? 2 * TC_ROWS : TC_ROWS;
  dim3 grid2((unsigned)((M + bx - 1) / bx), (unsigned)((N + rows_cta - 1) / rows_cta));
  const int sel = two ? 512 : bn;
  // Fewer output tiles than half the resident CTAs and a long K (e.g. 2048 x 16384, a down projection at decode batch
  // sizes, or any projection of a tensor-parallel shard): split K over grid.z into one wave of slices, each with at
  // least 4 steps; partial tiles are summed in order.
  const int64_t ctas = (int64_t)grid2.x * grid2.y, ksteps_all = K / T2_BK;
  int nz = 1;
  const int64_t slots = (int64_t)sm_count() * (bn <= 64 ? 2 : 1);       // CTAs of this tile size that are resident at once
  // a slice of partial products holds whole batch tiles when the tiles are stored with the tile-store epilogue
  const int64_t part_rows = (N % 4 == 0) ? (int64_t)grid2.x * bx : M;
  t.part_rows = part_rows;
  if (!two && slots / ctas >= 2 && ksteps_all >= 8) {
    int64_t want = slots / ctas;                                       // one wave of slices
    if (want > ksteps_all / 4) want = ksteps_all / 4;
    while (want > 1 && (size_t)want * part_rows * N * sizeof(float) > TC_PART_BYTES) --want;
    if (want > 1) {
      int64_t kper = ((ksteps_all + want - 1) / want + 1) & ~(int64_t)1;
      nz = (int)((ksteps_all + kper - 1) / kper);
      if (nz > 1) {
        if ((rc = scratch_ensure(&g_part, (size_t)nz * part_rows * N * sizeof(float), s, "tcgen05 path (split-K partial tiles)")))
          return rc;
        t.kper = (int)kper; t.part = (float*)g_part.ptr; grid2.z = (unsigned)nz;
        t.gated_act = -1;                       // the slices are plain partial products; the reduction applies the activation
        t.tma_store = (N % 4 == 0 && out_map(&t.tm_y, g_part.ptr, true, N, (int64_t)nz * part_rows, N, 128, bx, &rc)) ? 1 : 0;
        if (rc) return rc;
      }
    }
  }
  // (a single wave of 256-row batch tiles ends with one thread storing 128 KB while nothing else runs: measured
  // slower than plain stores there, faster everywhere else)
  if (nz <= 1 && !(bx == 256 && ctas < 2 * slots)) {
    t.tma_store = out_map(&t.tm_y, y, gated_act < 0 && y_dtype == BQ_DT_F32, gated_act >= 0 ? N / 2 : N, M, ldy,
                          gated_act >= 0 ? 64 : 128, bx, &rc) ? 1 : 0;
    if (rc) return rc;
  }
  rc = fmt == BQ_FMT_Q8G32 ? t2_dispatch<BQ_FMT_Q8G32>(t, sel, grid2, s) : t2_dispatch<BQ_FMT_Q4G32>(t, sel, grid2, s);
  if (rc || nz <= 1) return rc;
  int64_t rg = (M * N + 255) / 256;
  if (rg > (int64_t)sm_count() * 8) rg = (int64_t)sm_count() * 8;
  if (gated_act >= 0)
    BQ_CUDA(launch_chain(splitk_reduce_gated_kernel, dim3((unsigned)rg), dim3(256), 0, s, 1, (const float*)g_part.ptr, nz, M, N,
                         part_rows, (__nv_bfloat16*)y, ldy, gated_act));
  else if (y_dtype == BQ_DT_F32)
    BQ_CUDA(launch_chain(splitk_reduce_kernel<float>, dim3((unsigned)rg), dim3(256), 0, s, 1, (const float*)g_part.ptr, nz, M, N,
                         part_rows, (float*)y, ldy));
  else
    BQ_CUDA(launch_chain(splitk_reduce_kernel<__nv_bfloat16>, dim3((unsigned)rg), dim3(256), 0, s, 1, (const float*)g_part.ptr, nz, M,
                         N, part_rows, (__nv_bfloat16*)y, ldy));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

// ---- MoE grouped experts ---------------------------------------------------------------------------------
struct MoeTcState {           // device-side per-expert tensor maps + tile list, owned by the expert set
  CUtensorMap* gate_up;       // [E][4] = {gate codes, gate scales, up codes, up scales}
  CUtensorMap* down;          // [E][4] = {down codes, down scales, (same again)}
  Scratch tiles;              // tile list of the current call (grows with the row count)
};

bool moe_tc_supported(const Moe* m) { return tc_shape_ok(m->F, m->H) && tc_shape_ok(m->H, m->F); }

int moe_tc_prepare(Moe* m, const std::vector<const uint8_t*>* codes, const std::vector<const __half*>* scales) {
  // codes/scales: [0]=gate, [1]=up, [2]=down host-side pointer lists (device addresses)
  if (!moe_tc_supported(m)) { m->tc_state = nullptr; return BQ_OK; }
  MoeTcState* st = new MoeTcState();
  st->gate_up = st->down = nullptr;
  std::vector<CUtensorMap> gu((size_t)m->E * 4), dn((size_t)m->E * 4);
  for (int e = 0; e < m->E; ++e) {
    int rc = weight_maps(codes[0][e], scales[0][e], m->fmt, m->F, m->H, &gu[e * 4 + 0], &gu[e * 4 + 1]);
    if (!rc) rc = weight_maps(codes[1][e], scales[1][e], m->fmt, m->F, m->H, &gu[e * 4 + 2], &gu[e * 4 + 3]);
    if (!rc) rc = weight_maps(codes[2][e], scales[2][e], m->fmt, m->H, m->F, &dn[e * 4 + 0], &dn[e * 4 + 1]);
    if (rc) { delete st; return rc; }
    dn[e * 4 + 2] = dn[e * 4 + 0];
    dn[e * 4 + 3] = dn[e * 4 + 1];
  }
  const size_t bytes = sizeof(CUtensorMap) * (size_t)m->E * 4;
  BQ_CUDA(cudaMalloc((void**)&st->gate_up, bytes));
  BQ_CUDA(cudaMalloc((void**)&st->down, bytes));
  BQ_CUDA(cudaMemcpy(st->gate_up, gu.data(), bytes, cudaMemcpyHostToDevice));
  BQ_CUDA(cudaMemcpy(st->down, dn.data(), bytes, cudaMemcpyHostToDevice));
  m->tc_state = st;
  return BQ_OK;
}

void moe_tc_release(Moe* m) {
  MoeTcState* st = static_cast<MoeTcState*>(m->tc_state);
  if (!st) return;
  cudaFree(st->gate_up); cudaFree(st->down);
  if (st->tiles.ptr) cudaFree(st->tiles.ptr);     // outgrown lists stay in the library's retire list
  delete st;
  m->tc_state = nullptr;
}

template <int FMT, int MODE>
static int t2_moe_dispatch(const T2Args& a, int bn, dim3 grid, cudaStream_t s) {
  switch (bn) {
    case 16:  return t2_launch<FMT, 16, MODE>(a, grid, s);
    case 32:  return t2_launch<FMT, 32, MODE>(a, grid, s);
    case 64:  return t2_launch<FMT, 64, MODE>(a, grid, s);
    default:  return t2_launch<FMT, 128, MODE>(a, grid, s);
  }
}

int launch_moe_experts_tc(const Moe* m, const void* xp, const int32_t* offsets, int64_t P, int64_t rows_hint, void* hbuf,
                          float* out, cudaStream_t s) {
  MoeTcState* st = static_cast<MoeTcState*>(m->tc_state);
  if (!st) return fail(BQ_ERR_UNSUPPORTED, "tensor path unavailable for this expert shape");
  if ((reinterpret_cast<uintptr_t>(xp) & 15) != 0 || (reinterpret_cast<uintptr_t>(hbuf) & 15) != 0)
    return fail(BQ_ERR_ARG, "activation buffers must be 16-byte aligned");
  // rows per expert ~ P / E: pick the batch tile for the average segment.  A tcgen05.mma costs the same to issue
  // for 16 or 64 columns, so the 16-row tile is kept for segments that are mostly below 16 rows (at an average of
  // 16 half the experts would need a second tile that streams the same weights again); up to an average of 20 rows a
  // 32-row tile covers nearly every expert in one piece and stages half the activation bytes of the 64-row one.
  const int64_t avg = (rows_hint + m->E - 1) / m->E;
  const int bn = avg <= 8 ? 16 : avg <= 20 ? 32 : avg <= 64 ? 64 : 128;
  const int64_t max_tiles = (P + bn - 1) / bn + m->E;
  int rc = scratch_ensure(&st->tiles, sizeof(int32_t) * (size_t)(2 * max_tiles + 1 + 64), s, "bq_moe_experts (tile list)");
  if (rc) return rc;
  int32_t* tiles = (int32_t*)st->tiles.ptr;
  BQ_CUDA(launch_chain(moe_tile_list_kernel, dim3(1), dim3(1024), 0, s, 1, offsets, m->E, bn, tiles));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  // gate|up -> h (bf16), then down -> out (f32)
  T2Args a;
  memset(&a, 0, sizeof(a));
  if ((rc = launch_x_prep(xp, BQ_DT_BF16, P, m->H, s, offsets + m->E))) return rc;     // offsets[E] = rows in use
  if ((rc = x_map(&a.tm_x, g_x16.ptr, P, m->H, bn))) return rc;
  a.xscale = (const float*)g_xs.ptr; a.tm_list = st->gate_up; a.offsets = offsets; a.tiles = tiles; a.out = hbuf; a.ldy = m->F;
  a.N = m->F; a.K = m->H; a.M = P; a.out_dtype = BQ_DT_BF16; a.moe = 1; a.status = status_word(); a.gated_act = -1;
  dim3 g1((unsigned)max_tiles, (unsigned)((m->F + TC_ROWS - 1) / TC_ROWS));
  rc = m->fmt == BQ_FMT_Q8G32 ? t2_moe_dispatch<BQ_FMT_Q8G32, 1>(a, bn, g1, s) : t2_moe_dispatch<BQ_FMT_Q4G32, 1>(a, bn, g1, s);
  if (rc) return rc;
  T2Args b;
  memset(&b, 0, sizeof(b));
  if ((rc = launch_x_prep(hbuf, BQ_DT_BF16, P, m->F, s, offsets + m->E))) return rc;   // stream order: the first GEMM is done with the scratch
  if ((rc = x_map(&b.tm_x, g_x16.ptr, P, m->F, bn))) return rc;
  b.xscale = (const float*)g_xs.ptr; b.tm_list = st->down; b.offsets = offsets; b.tiles = tiles; b.out = out; b.ldy = m->H;
  b.N = m->H; b.K = m->F; b.M = P; b.out_dtype = BQ_DT_F32; b.moe = 1; b.status = status_word(); b.gated_act = -1;
  dim3 g2((unsigned)max_tiles, (unsigned)((m->H + TC_ROWS - 1) / TC_ROWS));
  return m->fmt == BQ_FMT_Q8G32 ? t2_moe_dispatch<BQ_FMT_Q8G32, 0>(b, bn, g2, s) : t2_moe_dispatch<BQ_FMT_Q4G32, 0>(b, bn, g2, s);
}

}  // namespace bq
