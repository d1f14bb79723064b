// Shared declarations for libb200q: weight record, error plumbing, small device helpers.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <string>
#include <vector>

#include "../../include/b200q.h"

namespace bq {

constexpr int GROUP = 32;
constexpr int SM_COUNT_B200 = 148;

// A packed weight resident in HBM.  Device layout = interface layout (row-major codes and
// row-major scales, each in its own 256-byte aligned allocation): a block of consecutive
// rows is one contiguous byte range, which is what the bulk-copy (TMA) pipeline wants.
struct Weight {
  uint32_t magic;        // 0xB200C0DE while alive
  int fmt;
  int64_t N, K;
  uint8_t* codes;        // Q8: N*K bytes, Q4: N*K/2 bytes
  __half* scales;        // N*K/32 fp16
  size_t codes_bytes, scales_bytes;
  bool view;             // rows of another weight (bq_weight_slice_rows): the memory is not owned
  int64_t row_bytes() const { return fmt == BQ_FMT_Q8G32 ? K : K / 2; }
};
constexpr uint32_t WEIGHT_MAGIC = 0xB200C0DEu;

struct Moe {
  uint32_t magic;        // 0xB2003E00 while alive
  int E;
  int64_t H, F;
  int fmt;
  // device arrays of per-expert pointers
  const uint8_t** gate_codes; const __half** gate_scales;
  const uint8_t** up_codes;   const __half** up_scales;
  const uint8_t** down_codes; const __half** down_scales;
  void* tc_state;        // tensor-core path: per-expert TMA descriptors + tile list (tc.cu)
};
constexpr uint32_t MOE_MAGIC = 0xB2003E00u;

// Peer-memory communicator (comm.cu): what the kernels read.  Every rank owns one buffer of receive slots that all
// ranks of the node map through CUDA IPC.  Rank s deposits its contribution to a sum in slot [parity][s] of EVERY
// rank's buffer; a slot element holds COMM_EMPTY (the bit pattern of -0.0f, which no deposit ever carries) until
// the value arrives, so the data announces itself: no flags, no fences.  The receiver adds the slots in rank order
// and puts COMM_EMPTY back.  `state[0]` is the call counter (epoch, starts at 1; parity = epoch & 1), `state[1]`
// counts finished CTAs, `state[2]` != 0 marks a communicator on which a wait timed out.
constexpr int COMM_MAX_WORLD = 8;
constexpr uint32_t COMM_EMPTY = 0x80000000u;
struct CommDev {
  float* data[COMM_MAX_WORLD];        // rank r's receive slots: [2][world][slot_elems] floats
  uint32_t* state;                    // this rank's {epoch, finished-CTA counter, failed}
  int64_t slot_elems;
  uint64_t wait_ns;                   // bound of the wait for a value
  int rank, world;
};

// ---- host-side state / error plumbing (api.cu) -----------------------------------------
int fail(int code, const std::string& msg);
int fail_cuda(cudaError_t e, const char* what);
void count_launch(int n = 1);
void set_last_path(int p);
Weight* get_weight(bq_weight_t h);     // nullptr (and error set) if invalid
Moe* get_moe(bq_moe_t h);
int device_id();
int sm_count();
int* status_word();                    // device int, 0 = fine
void comm_mark_all_failed();           // comm.cu: a bounded wait expired somewhere; communicators need bq_comm_reset
void ep_mark_all_failed();             // ep.cu: same for the expert-parallel objects
// api.cu: logits of this weight into library scratch, then per row the argmax id and the maximum itself
int lm_head_local(bq_weight_t w, const void* x, int x_dtype, int64_t M, int32_t* imax, float* vmax, cudaStream_t s);

// Library-owned scratch (activation pre-pass output, split-K partial tiles, attention partial states, ...).
// Grow-only, and a buffer that was ever handed out is never freed while the library is loaded: a CUDA graph
// captured earlier keeps its address (tensor maps included), so growth allocates a larger buffer and retires the old
// one instead of freeing it.  Growth is refused (BQ_ERR_STATE) while `stream` is being captured: make one call of
// the largest size, or bq_reserve(), before capturing.  All calls that use library scratch must be ordered on the
// device (one stream, or events between streams): the buffers are shared.
struct Scratch {
  void* ptr = nullptr;
  size_t bytes = 0;
};
int scratch_ensure(Scratch* s, size_t need, cudaStream_t stream, const char* what, bool zero_new = false);
int tc_reserve(int64_t rows, int64_t K, int64_t N);      // tc.cu: activation pre-pass output, split-K partial tiles
int glue_reserve(int64_t rows, int64_t N);               // glue.cu: gate|up product of bq_qlinear_gated

#define BQ_CUDA(call)                                          \
  do {                                                         \
    cudaError_t e__ = (call);                                  \
    if (e__ != cudaSuccess) return ::bq::fail_cuda(e__, #call); \
  } while (0)

// ---- kernel launchers implemented in the .cu files ----------------------------------------
int launch_dequant(const Weight* w, void* out, int out_dtype, cudaStream_t s);
int launch_unpack(const Weight* w, int8_t* out, cudaStream_t s);
// SIMT (CUDA-core, exact fp32) path: any M (loops over row tiles of the activations)
int launch_qlinear_simt(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K,
                        const void* x, int x_dtype, int64_t M, void* y, int y_dtype, int64_t ldy,
                        cudaStream_t s);
// tensor-core (tcgen05) path: bf16 activations.  gated_act >= 0: fused gate|up weight (16-row blocks = 8 gate + 8 up rows),
// y = act(gate) * up as bf16 [M, N / 2] with ldy = N / 2 (0 = gelu-tanh, 1 = silu)
int launch_qlinear_tc(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K,
                      const void* x, int x_dtype, int64_t M, void* y, int y_dtype, int64_t ldy,
                      cudaStream_t s, int gated_act = -1);
bool tc_supported(int fmt, int64_t N, int64_t K, int x_dtype, int64_t M);
// tensor-core GEMV with exact group scaling (mma.sync), 1..4 activation rows
int launch_qlinear_mma(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K,
                       const void* x, int x_dtype, int64_t M, void* y, int y_dtype, int64_t ldy,
                       cudaStream_t s);
bool gemv_mma_supported(int fmt, int64_t N, int64_t K, int x_dtype, int64_t M);
// same GEMV, fp32 partial sums pushed into every rank's receive slot of a peer-memory communicator (gemv_push.cu)
int launch_qlinear_mma_push(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K,
                            const void* x, int x_dtype, int64_t M, const CommDev* comm_dev, cudaStream_t s);
// same GEMV on a fused gate|up weight (16-row blocks = 8 gate rows + 8 up rows): out[M, N/2] = act(gate) * up in the
// activations' dtype; act 0 = gelu (tanh), 1 = silu (gemv_gated.cu)
int launch_qlinear_mma_gated(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K,
                             const void* x, int x_dtype, int64_t M, void* out, int act, cudaStream_t s);
// batched decode GEMV (gemv_batch.cu): 5..16 bf16 activation rows, code * scale rounded to fp16 like the tcgen05 kernel.
// gated_act < 0: plain product; 0 / 1: fused gate|up weight (16-row blocks = 8 gate + 8 up rows), gelu / silu epilogue,
// out[M, N/2] in bf16.
bool gemv_batch_supported(int fmt, int64_t N, int64_t K, int x_dtype, int64_t M);
int launch_qlinear_batch(const uint8_t* codes, const __half* scales, int fmt, int64_t N, int64_t K, const void* x,
                         int x_dtype, int64_t M, void* y, int y_dtype, int64_t ldy, int gated_act, cudaStream_t s);
// grouped experts at decode sizes on the same kernel: x holds the sorted rows (perm == nullptr) or the TOKEN rows, which
// are then read through perm (row of sorted position p = perm[p] / top_k): no gathered copy is needed
// router linear + softmax + top-k in one launch (E <= 128 experts)
bool moe_route_linear_supported(int fmt, int64_t E, int64_t K, int top_k);
int launch_moe_route_linear(const uint8_t* codes, const __half* scales, int fmt, int64_t E, int64_t K, const void* x, int64_t T,
                            int top_k, int renorm, int32_t* idx_out, float* w_out, cudaStream_t s);
bool moe_batch_supported(const Moe* m);
int launch_moe_experts_batch(const Moe* m, const void* x, const int32_t* perm, int top_k, const int32_t* offsets, int64_t P,
                             int64_t rows_hint, void* hbuf, float* out, cudaStream_t s);
bool moe_tc_supported(const Moe* m);
int moe_tc_prepare(Moe* m, const std::vector<const uint8_t*>* codes, const std::vector<const __half*>* scales);
void moe_tc_release(Moe* m);
int launch_moe_experts_tc(const Moe* m, const void* xp, const int32_t* offsets, int64_t P, int64_t rows_hint, void* hbuf,
                          float* out, cudaStream_t s);
// Device encoding of the codes (a bijection of the interface bytes, undone by bq_weight_export):
//   Q4: within every 32-bit word the 8 nibbles are stored in the order e0,e2,e4,e6,e1,e3,e5,e7 (element
//       e_i of the interface layout), so that masking with 0x000F000F / 0x00F000F0 yields adjacent pairs;
//   Q8: every byte holds code + 128 (sign bit flipped), so mantissa insertion needs no sign fix-up.
int launch_device_encode(uint8_t* codes, size_t bytes, int fmt, bool to_device_layout, cudaStream_t s);
// out[m] = argmax of row m (ties -> lower index); vout (optional): the maximum itself
int launch_argmax(const void* logits, int dtype, int64_t M, int64_t N, int32_t* out, cudaStream_t s, float* vout = nullptr);
// grouped-query decode attention on mma.sync (bf16 caches, head_dim 64 / 128 / 256): hp = query heads per CTA
bool attention_mma_supported(int Hq, int Hkv, int D, int* hp_out);
int attention_mma_ctas_per_sm(bool fused, int D, bool hi);
int launch_attention_mma(const void* q, const float* qkv, void* k_cache, void* v_cache, const int64_t* pos, void* out, int64_t B,
                         int Hq, int Hkv, int D, int64_t S, float rope_base, int hp, int nsplit, float* part, unsigned* counters,
                         cudaStream_t s);
bool pdl_enabled();     // programmatic dependent launch on every launch of the library

#ifdef __CUDACC__
// Launch with the programmatic-stream-serialization attribute (the kernel must call pdl_wait() before it reads or
// writes anything a preceding kernel on the stream may still be using).  `cluster_y` > 1 adds a cluster dimension
// along y; `cluster_y` < -1 one of -cluster_y CTAs along x (CTA pairs of tcgen05 cta_group::2 are neighbours in x).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chain(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, int cluster_y,
                                Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_y > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1; attr[n].val.clusterDim.y = (unsigned)cluster_y; attr[n].val.clusterDim.z = 1;
    ++n;
  } else if (cluster_y < -1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)(-cluster_y); attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr; cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

// ---- device helpers --------------------------------------------------------------------------
#ifdef __CUDACC__
// Where this rank's contribution to the current call goes in rank r's buffer (element 0 of its receive slot).
__device__ __forceinline__ float* comm_push_base(const void* desc, int r) {
  const CommDev* d = reinterpret_cast<const CommDev*>(desc);
  const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(d->state);
  return d->data[r] + ((int64_t)(e & 1u) * d->world + d->rank) * d->slot_elems;
}
__device__ __forceinline__ int comm_world(const void* desc) { return reinterpret_cast<const CommDev*>(desc)->world; }
// One deposit: a system-scope 4-byte store (atomic by size); -0.0f is stored as +0.0f so that it cannot be taken
// for an empty slot.
__device__ __forceinline__ void comm_deposit(float* p, float v) {
  uint32_t b = __float_as_uint(v);
  if (b == COMM_EMPTY) b = 0u;
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(b) : "memory");
}
__device__ __forceinline__ void comm_deposit4(float* p, float4 v) {      // p 16-byte aligned
  uint32_t a = __float_as_uint(v.x), b = __float_as_uint(v.y), c = __float_as_uint(v.z), d = __float_as_uint(v.w);
  if (a == COMM_EMPTY) a = 0u;
  if (b == COMM_EMPTY) b = 0u;
  if (c == COMM_EMPTY) c = 0u;
  if (d == COMM_EMPTY) d = 0u;
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// Programmatic dependent launch: a kernel lets its successor start launching right away and itself waits for its
// predecessor (completion + memory visibility) before it touches anything the predecessor may have written.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ uint4 ldg_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;  // (a & b) | c
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}
__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) {
  return __uint_as_float(((uint32_t)b) << 16);
}
template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// 8 consecutive elements <-> 8 floats with 16-byte accesses (the pointer must be 16-byte aligned)
template <typename T> __device__ __forceinline__ void load8(const T* p, float* f);
template <> __device__ __forceinline__ void load8<float>(const float* p, float* f) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* f) {
  const uint4 r = *reinterpret_cast<const uint4*>(p);
  const uint32_t wds[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(wds[i] << 16);
    f[2 * i + 1] = __uint_as_float(wds[i] & 0xFFFF0000u);
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float* f);
template <> __device__ __forceinline__ void store8<float>(float* p, const float* f) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* f) {
  uint4 r;
  uint32_t* w = &r.x;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
  *reinterpret_cast<uint4*>(p) = r;
}

// element d of a head taken from the fp32 projection output, rotated like rope_kv_append_kernel does
template <typename T>
__device__ __forceinline__ float rope_elem(const float* __restrict__ src, int d, int D, const float* cs, const float* sn, bool rotate) {
  if (!rotate) return to_float<T>(from_float<T>(src[d]));
  const int half = D / 2, j = d < half ? d : d - half;
  const float x1 = to_float<T>(from_float<T>(src[j])), x2 = to_float<T>(from_float<T>(src[j + half]));
  return to_float<T>(from_float<T>(d < half ? x1 * cs[j] - x2 * sn[j] : x2 * cs[j] + x1 * sn[j]));
}

// Exact integer-code -> fp32 conversions without the (slow) I2F pipe.
// Q8: `v` holds four device bytes, each code + 128.
// Byte `I` is dropped into the mantissa of 2^23, giving 8388608 + code + 128 exactly.
template <int I> __device__ __forceinline__ float q8_byte_to_float(uint32_t v_xor80) {
  constexpr uint32_t sel = 0x7650u | (uint32_t)I;
  return __uint_as_float(__byte_perm(v_xor80, 0x4B000000u, sel)) - 8388736.0f;
}
// Q4 (device layout): nibble `I` of the word holds element q4_elem(I) of the 8; stored value is code + 8.
__host__ __device__ constexpr int q4_elem(int nib) { return nib < 4 ? 2 * nib : 2 * (nib - 4) + 1; }
template <int I> __device__ __forceinline__ float q4_nibble_to_float(uint32_t v) {
  uint32_t m = lop3_and_or(I == 0 ? v : (v >> (4 * I)), 0xFu, 0x4B000000u);
  return __uint_as_float(m) - 8388616.0f;
}
#endif

}  // namespace bq
