// C ABI of libb200q.so: state, error plumbing, packed-weight handles, dispatch.
// No CPU fallback exists: every compute entry point launches CUDA kernels or fails.
#include <atomic>
#include <mutex>
#include <unordered_set>
#include <vector>

#include "common.cuh"

namespace bq {

static thread_local std::string t_err;
static thread_local int t_last_path = BQ_PATH_AUTO;
static std::atomic<int64_t> g_launches{0};
static std::mutex g_mu;
static std::unordered_set<void*> g_weights, g_moes;
static int g_device = -1;
static int g_sms = 0;
static int* g_status = nullptr;
// device staging for the host-buffer entry point and for argmax-only lm_head calls
static Scratch g_stage_x, g_stage_y;
static Scratch g_logits;                  // bq_lm_head without a logits buffer (argmax only)
static std::vector<void*> g_retired;      // scratch buffers that were outgrown: kept, a captured graph may still use them

int fail(int code, const std::string& msg) { t_err = msg; return code; }
int fail_cuda(cudaError_t e, const char* what) {
  t_err = std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")";
  return BQ_ERR_CUDA;
}
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }
void set_last_path(int p) { t_last_path = p; }
bool pdl_enabled() { return true; }      // every launch of the library carries the programmatic-serialization attribute
int device_id() { return g_device; }
int sm_count() { return g_sms > 0 ? g_sms : SM_COUNT_B200; }
int* status_word() { return g_status; }

int scratch_ensure(Scratch* sc, size_t need, cudaStream_t stream, const char* what, bool zero_new) {
  if (need <= sc->bytes) return BQ_OK;
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return fail(BQ_ERR_STATE, std::string(what) + ": the library's scratch would have to grow to " + std::to_string(need) +
                                  " bytes during stream capture; make one call of this size, or bq_reserve(), before capturing");
  }
  const size_t cap_bytes = need + need / 4 + 4096;
  void* p = nullptr;
  BQ_CUDA(cudaMalloc(&p, cap_bytes));
  if (zero_new) {
    cudaError_t e = cudaMemset(p, 0, cap_bytes);
    if (e != cudaSuccess) { cudaFree(p); return fail_cuda(e, "cudaMemset(scratch)"); }
  }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (sc->ptr) g_retired.push_back(sc->ptr);
  }
  sc->ptr = p;
  sc->bytes = cap_bytes;
  return BQ_OK;
}

Weight* get_weight(bq_weight_t h) {
  void* p = reinterpret_cast<void*>(static_cast<uintptr_t>(h));
  std::lock_guard<std::mutex> lk(g_mu);
  if (!p || !g_weights.count(p) || static_cast<Weight*>(p)->magic != WEIGHT_MAGIC) {
    fail(BQ_ERR_HANDLE, "invalid weight handle");
    return nullptr;
  }
  return static_cast<Weight*>(p);
}
Moe* get_moe(bq_moe_t h) {
  void* p = reinterpret_cast<void*>(static_cast<uintptr_t>(h));
  std::lock_guard<std::mutex> lk(g_mu);
  if (!p || !g_moes.count(p) || static_cast<Moe*>(p)->magic != MOE_MAGIC) {
    fail(BQ_ERR_HANDLE, "invalid moe handle");
    return nullptr;
  }
  return static_cast<Moe*>(p);
}

static int check_ready() {
  if (g_device < 0) return fail(BQ_ERR_STATE, "bq_init() has not been called");
  int cur = -1;
  BQ_CUDA(cudaGetDevice(&cur));
  if (cur != g_device) BQ_CUDA(cudaSetDevice(g_device));
  return BQ_OK;
}

static int check_shape(int64_t N, int64_t K, int fmt) {
  if (fmt != BQ_FMT_Q8G32 && fmt != BQ_FMT_Q4G32) return fail(BQ_ERR_ARG, "unknown weight format");
  if (N < 0 || K <= 0) return fail(BQ_ERR_ARG, "N must be >= 0 and K > 0");
  if (K % GROUP != 0) return fail(BQ_ERR_ARG, "K must be a multiple of 32 (the quantization group)");
  if (N > (int64_t)1 << 31 || K > (int64_t)1 << 24) return fail(BQ_ERR_ARG, "N or K out of range");
  return BQ_OK;
}

static int alloc_weight(int64_t N, int64_t K, int fmt, Weight** out) {
  Weight* w = new Weight();
  w->magic = WEIGHT_MAGIC;
  w->fmt = fmt; w->N = N; w->K = K;
  w->codes_bytes = (size_t)(N * (fmt == BQ_FMT_Q8G32 ? K : K / 2));
  w->scales_bytes = (size_t)(N * (K / GROUP)) * sizeof(__half);
  w->codes = nullptr; w->scales = nullptr; w->view = false;
  // +256 bytes of slack so whole-16-byte vector reads past a ragged tail stay in bounds
  cudaError_t e = cudaMalloc((void**)&w->codes, w->codes_bytes + 256);
  if (e == cudaSuccess) e = cudaMalloc((void**)&w->scales, w->scales_bytes + 256);
  if (e == cudaSuccess) e = cudaMemset(w->codes + w->codes_bytes, 0, 256);
  if (e == cudaSuccess) e = cudaMemset((uint8_t*)w->scales + w->scales_bytes, 0, 256);
  if (e != cudaSuccess) {
    if (w->codes) cudaFree(w->codes);
    if (w->scales) cudaFree(w->scales);
    delete w;
    return fail_cuda(e, "cudaMalloc(weight)");
  }
  *out = w;
  return BQ_OK;
}

static bq_weight_t publish(Weight* w) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_weights.insert(w);
  return static_cast<bq_weight_t>(reinterpret_cast<uintptr_t>(w));
}


static size_t dt_size(int dt) { return dt == BQ_DT_F32 ? 4 : 2; }
static bool dt_ok(int dt) { return dt == BQ_DT_F32 || dt == BQ_DT_BF16; }

// Kernel-family choice.  MMA = tensor-core GEMV: exact group scaling for 1..4 activation rows, the batched variant
// (weights rounded to fp16 like the tcgen05 kernel) for 5..16 bf16 rows; TENSOR = tcgen05 dequant-GEMM (bf16
// activations, any M); SIMT = CUDA-core exact fp32 (any shape).
static int choose_path(const Weight* w, const void* x, int x_dtype, int64_t M, int requested) {
  if (requested == BQ_PATH_SIMT) return BQ_PATH_SIMT;
  const bool tc_ok = tc_supported(w->fmt, w->N, w->K, x_dtype, M) && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  if (requested == BQ_PATH_TENSOR) return tc_ok ? BQ_PATH_TENSOR : -1;
  const bool mma_ok = gemv_mma_supported(w->fmt, w->N, w->K, x_dtype, M) ||
                      (gemv_batch_supported(w->fmt, w->N, w->K, x_dtype, M) && (reinterpret_cast<uintptr_t>(x) & 15) == 0);
  if (requested == BQ_PATH_MMA) return mma_ok ? BQ_PATH_MMA : -1;
  if (requested != BQ_PATH_AUTO) return -1;
  if (mma_ok) return BQ_PATH_MMA;
  if (tc_ok) return BQ_PATH_TENSOR;
  return BQ_PATH_SIMT;
}

static int qlinear_impl(Weight* w, const void* x, int x_dtype, int64_t M, void* y, int y_dtype,
                        int path, cudaStream_t s) {
  if (!dt_ok(x_dtype) || !dt_ok(y_dtype)) return fail(BQ_ERR_ARG, "dtype must be BQ_DT_F32 or BQ_DT_BF16");
  if (M < 0) return fail(BQ_ERR_ARG, "M must be >= 0");
  if (M == 0 || w->N == 0) { set_last_path(BQ_PATH_AUTO); return BQ_OK; }
  if (!x || !y) return fail(BQ_ERR_ARG, "x and y must not be null");
  const int p = choose_path(w, x, x_dtype, M, path);
  if (p < 0) return fail(BQ_ERR_UNSUPPORTED, "requested kernel path does not support this shape/dtype");
  set_last_path(p);
  if (p == BQ_PATH_MMA) {
    // 3 or 4 bf16 rows: the exact-scaling GEMV needs a second column set there (4-bit: 1.5x the one-row time, int8 at 4
    // rows the same as the batched kernel or worse, measured); the batched kernel serves up to 8 rows per set
    const bool prefer_batch = M >= 3 && gemv_batch_supported(w->fmt, w->N, w->K, x_dtype, M) &&
                              (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    if (!prefer_batch && gemv_mma_supported(w->fmt, w->N, w->K, x_dtype, M))
      return launch_qlinear_mma(w->codes, w->scales, w->fmt, w->N, w->K, x, x_dtype, M, y, y_dtype, w->N, s);
    return launch_qlinear_batch(w->codes, w->scales, w->fmt, w->N, w->K, x, x_dtype, M, y, y_dtype, w->N, -1, s);
  }
  if (p == BQ_PATH_TENSOR)
    return launch_qlinear_tc(w->codes, w->scales, w->fmt, w->N, w->K, x, x_dtype, M, y, y_dtype, w->N, s);
  return launch_qlinear_simt(w->codes, w->scales, w->fmt, w->N, w->K, x, x_dtype, M, y, y_dtype, w->N, s);
}

int lm_head_local(bq_weight_t h, const void* x, int x_dtype, int64_t M, int32_t* imax, float* vmax, cudaStream_t s) {
  int rc = check_ready();
  if (rc) return rc;
  Weight* w = get_weight(h);
  if (!w) return BQ_ERR_HANDLE;
  if (w->N == 0) return fail(BQ_ERR_ARG, "lm_head needs a non-empty vocabulary");
  if ((rc = scratch_ensure(&g_logits, (size_t)M * w->N * 4, s, "bq_lm_head_sharded"))) return rc;
  if ((rc = qlinear_impl(w, x, x_dtype, M, g_logits.ptr, BQ_DT_F32, BQ_PATH_AUTO, s))) return rc;
  return launch_argmax(g_logits.ptr, BQ_DT_F32, M, w->N, imax, s, vmax);
}

}  // namespace bq

using namespace bq;

extern "C" {

int bq_version(void) { return 200; }

const char* bq_last_error(void) { return t_err.c_str(); }

int bq_init(int device) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDeviceCount");
  if (device < 0 || device >= n) return fail(BQ_ERR_ARG, "device index out of range");
  if (g_device >= 0 && g_device != device)
    return fail(BQ_ERR_STATE, "library already initialised on another device (one process per GPU)");
  BQ_CUDA(cudaSetDevice(device));
  if (g_device == device) return BQ_OK;
  cudaDeviceProp prop;
  BQ_CUDA(cudaGetDeviceProperties(&prop, device));
  if (prop.major != 10)
    return fail(BQ_ERR_UNSUPPORTED, std::string("this library is built for sm_100a only; device is ") + prop.name);
  g_sms = prop.multiProcessorCount;
  BQ_CUDA(cudaMalloc((void**)&g_status, 256));
  BQ_CUDA(cudaMemset(g_status, 0, 256));
  g_device = device;
  return BQ_OK;
}

int bq_status_poll(void) {
  int rc = check_ready();
  if (rc) return rc;
  BQ_CUDA(cudaDeviceSynchronize());
  int v = 0;
  BQ_CUDA(cudaMemcpy(&v, g_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (v != 0) {
    BQ_CUDA(cudaMemset(g_status, 0, sizeof(int)));
    if (v == BQ_ERR_TIMEOUT) { comm_mark_all_failed(); ep_mark_all_failed(); }
    return fail(v, "a kernel recorded a device-side anomaly (bounded wait expired)");
  }
  return BQ_OK;
}

int bq_weight_create(const void* codes, const void* scales, int64_t N, int64_t K, int fmt, bq_weight_t* out) {
  int rc = check_ready();
  if (rc) return rc;
  if (!out) return fail(BQ_ERR_ARG, "out must not be null");
  if ((rc = check_shape(N, K, fmt))) return rc;
  if (N > 0 && (!codes || !scales)) return fail(BQ_ERR_ARG, "codes and scales must not be null");
  Weight* w = nullptr;
  if ((rc = alloc_weight(N, K, fmt, &w))) return rc;
  cudaError_t e = cudaSuccess;
  if (w->codes_bytes) e = cudaMemcpy(w->codes, codes, w->codes_bytes, cudaMemcpyHostToDevice);
  if (e == cudaSuccess && w->scales_bytes) e = cudaMemcpy(w->scales, scales, w->scales_bytes, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cudaFree(w->codes); cudaFree(w->scales); delete w;
    return fail_cuda(e, "cudaMemcpy(weight upload)");
  }
  {
    rc = launch_device_encode(w->codes, w->codes_bytes, fmt, true, 0);
    if (rc == BQ_OK && cudaStreamSynchronize(0) != cudaSuccess) rc = fail(BQ_ERR_CUDA, "repack failed");
    if (rc) { cudaFree(w->codes); cudaFree(w->scales); delete w; return rc; }
  }
  *out = publish(w);
  return BQ_OK;
}

int bq_weight_create_device(const void* d_codes, const void* d_scales, int64_t N, int64_t K, int fmt,
                            void* stream, bq_weight_t* out) {
  int rc = check_ready();
  if (rc) return rc;
  if (!out) return fail(BQ_ERR_ARG, "out must not be null");
  if ((rc = check_shape(N, K, fmt))) return rc;
  if (N > 0 && (!d_codes || !d_scales)) return fail(BQ_ERR_ARG, "codes and scales must not be null");
  Weight* w = nullptr;
  if ((rc = alloc_weight(N, K, fmt, &w))) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = cudaSuccess;
  if (w->codes_bytes) e = cudaMemcpyAsync(w->codes, d_codes, w->codes_bytes, cudaMemcpyDeviceToDevice, s);
  if (e == cudaSuccess && w->scales_bytes)
    e = cudaMemcpyAsync(w->scales, d_scales, w->scales_bytes, cudaMemcpyDeviceToDevice, s);
  if (e == cudaSuccess && launch_device_encode(w->codes, w->codes_bytes, fmt, true, s) != BQ_OK)
    e = cudaErrorUnknown;
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    cudaFree(w->codes); cudaFree(w->scales); delete w;
    return fail_cuda(e, "cudaMemcpyAsync(weight copy)");
  }
  *out = publish(w);
  return BQ_OK;
}

int bq_weight_destroy(bq_weight_t h) {
  Weight* w = get_weight(h);
  if (!w) return BQ_ERR_HANDLE;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_weights.erase(w);
  }
  w->magic = 0;
  if (!w->view) {
    cudaFree(w->codes);
    cudaFree(w->scales);
  }
  delete w;
  return BQ_OK;
}

int bq_weight_slice_rows(bq_weight_t h, int64_t row0, int64_t nrows, bq_weight_t* out) {
  Weight* p = get_weight(h);
  if (!p) return BQ_ERR_HANDLE;
  if (!out) return fail(BQ_ERR_ARG, "out must not be null");
  if (row0 < 0 || nrows <= 0 || row0 + nrows > p->N) return fail(BQ_ERR_ARG, "row range outside the weight");
  Weight* w = new Weight();
  w->magic = WEIGHT_MAGIC;
  w->fmt = p->fmt; w->N = nrows; w->K = p->K; w->view = true;
  w->codes = p->codes + row0 * p->row_bytes();
  w->scales = p->scales + row0 * (p->K / GROUP);
  w->codes_bytes = (size_t)(nrows * p->row_bytes());
  w->scales_bytes = (size_t)(nrows * (p->K / GROUP)) * sizeof(__half);
  *out = publish(w);
  return BQ_OK;
}

int bq_weight_info(bq_weight_t h, int64_t* N, int64_t* K, int* fmt) {
  Weight* w = get_weight(h);
  if (!w) return BQ_ERR_HANDLE;
  if (N) *N = w->N;
  if (K) *K = w->K;
  if (fmt) *fmt = w->fmt;
  return BQ_OK;
}

int bq_weight_export(bq_weight_t h, void* codes_out, void* scales_out) {
  int rc = check_ready();
  if (rc) return rc;
  Weight* w = get_weight(h);
  if (!w) return BQ_ERR_HANDLE;
  if (w->N > 0 && (!codes_out || !scales_out)) return fail(BQ_ERR_ARG, "output pointers must not be null");
  if (w->codes_bytes) BQ_CUDA(cudaMemcpy(codes_out, w->codes, w->codes_bytes, cudaMemcpyDeviceToHost));
  if (w->fmt == BQ_FMT_Q8G32) {   // device bytes are code + 128
    uint32_t* p = static_cast<uint32_t*>(codes_out);
    for (size_t i = 0; i < w->codes_bytes / 4; ++i) p[i] ^= 0x80808080u;
  } else {                        // undo the device nibble order (a pure permutation inside each 32-bit word)
    uint32_t* p = static_cast<uint32_t*>(codes_out);
    for (size_t i = 0; i < w->codes_bytes / 4; ++i) {
      const uint32_t v = p[i];
      uint32_t o = 0;
      for (int j = 0; j < 8; ++j) o |= ((v >> (4 * j)) & 0xFu) << (4 * q4_elem(j));
      p[i] = o;
    }
  }
  if (w->scales_bytes) BQ_CUDA(cudaMemcpy(scales_out, w->scales, w->scales_bytes, cudaMemcpyDeviceToHost));
  return BQ_OK;
}

int bq_dequant(bq_weight_t h, void* out, int out_dtype, void* stream) {
  int rc = check_ready();
  if (rc) return rc;
  Weight* w = get_weight(h);
  if (!w) return BQ_ERR_HANDLE;
  if (!dt_ok(out_dtype)) return fail(BQ_ERR_ARG, "out_dtype must be BQ_DT_F32 or BQ_DT_BF16");
  if (w->N > 0 && !out) return fail(BQ_ERR_ARG, "out must not be null");
  return launch_dequant(w, out, out_dtype, (cudaStream_t)stream);
}

int bq_unpack_codes(bq_weight_t h, void* out_i8, void* stream) {
  int rc = check_ready();
  if (rc) return rc;
  Weight* w = get_weight(h);
  if (!w) return BQ_ERR_HANDLE;
  if (w->N > 0 && !out_i8) return fail(BQ_ERR_ARG, "out must not be null");
  return launch_unpack(w, (int8_t*)out_i8, (cudaStream_t)stream);
}

int bq_qlinear_ex(bq_weight_t h, const void* x, int x_dtype, int64_t M, void* y, int y_dtype, int path,
                  void* stream) {
  int rc = check_ready();
  if (rc) return rc;
  Weight* w = get_weight(h);
  if (!w) return BQ_ERR_HANDLE;
  return qlinear_impl(w, x, x_dtype, M, y, y_dtype, path, (cudaStream_t)stream);
}

int bq_qlinear(bq_weight_t h, const void* x, int x_dtype, int64_t M, void* y, int y_dtype, void* stream) {
  return bq_qlinear_ex(h, x, x_dtype, M, y, y_dtype, BQ_PATH_AUTO, stream);
}

int bq_qlinear_host(bq_weight_t h, const void* x_host, int x_dtype, int64_t M, void* y_host, int y_dtype) {
  int rc = check_ready();
  if (rc) return rc;
  Weight* w = get_weight(h);
  if (!w) return BQ_ERR_HANDLE;
  if (!dt_ok(x_dtype) || !dt_ok(y_dtype)) return fail(BQ_ERR_ARG, "dtype must be BQ_DT_F32 or BQ_DT_BF16");
  if (M < 0) return fail(BQ_ERR_ARG, "M must be >= 0");
  if (M == 0 || w->N == 0) return BQ_OK;
  if (!x_host || !y_host) return fail(BQ_ERR_ARG, "x and y must not be null");
  const size_t xb = (size_t)M * w->K * dt_size(x_dtype), yb = (size_t)M * w->N * dt_size(y_dtype);
  cudaStream_t s = cudaStreamPerThread;
  if ((rc = scratch_ensure(&g_stage_x, xb, s, "bq_qlinear_host"))) return rc;
  if ((rc = scratch_ensure(&g_stage_y, yb, s, "bq_qlinear_host"))) return rc;
  BQ_CUDA(cudaMemcpyAsync(g_stage_x.ptr, x_host, xb, cudaMemcpyHostToDevice, s));
  if ((rc = qlinear_impl(w, g_stage_x.ptr, x_dtype, M, g_stage_y.ptr, y_dtype, BQ_PATH_AUTO, s))) return rc;
  BQ_CUDA(cudaMemcpyAsync(y_host, g_stage_y.ptr, yb, cudaMemcpyDeviceToHost, s));
  BQ_CUDA(cudaStreamSynchronize(s));
  return BQ_OK;
}

int bq_lm_head(bq_weight_t h, const void* x, int x_dtype, int64_t M, void* logits, int logits_dtype,
               int32_t* argmax_out, void* stream) {
  int rc = check_ready();
  if (rc) return rc;
  Weight* w = get_weight(h);
  if (!w) return BQ_ERR_HANDLE;
  if (M < 0) return fail(BQ_ERR_ARG, "M must be >= 0");
  if (M == 0) return BQ_OK;
  if (w->N == 0) return fail(BQ_ERR_ARG, "lm_head needs a non-empty vocabulary");
  if (!logits && !argmax_out) return fail(BQ_ERR_ARG, "logits and argmax_out are both null");
  cudaStream_t s = (cudaStream_t)stream;
  void* lg = logits;
  int ldt = logits_dtype;
  if (!lg) {  // argmax only: logits live in the library's staging buffer
    ldt = BQ_DT_F32;
    if ((rc = scratch_ensure(&g_logits, (size_t)M * w->N * 4, s, "bq_lm_head"))) return rc;
    lg = g_logits.ptr;
  }
  if ((rc = qlinear_impl(w, x, x_dtype, M, lg, ldt, BQ_PATH_AUTO, s))) return rc;
  if (argmax_out) return launch_argmax(lg, ldt, M, w->N, argmax_out, s);
  return BQ_OK;
}

int bq_reserve(int64_t max_rows, int64_t max_K, int64_t max_N) {
  int rc = check_ready();
  if (rc) return rc;
  if (max_rows <= 0 || max_K <= 0 || max_N <= 0) return fail(BQ_ERR_ARG, "sizes must be positive");
  if ((rc = tc_reserve(max_rows, max_K, max_N))) return rc;
  if ((rc = glue_reserve(max_rows, max_N))) return rc;
  return scratch_ensure(&g_logits, (size_t)max_rows * max_N * 4, 0, "bq_reserve");
}

int bq_last_path(void) { return t_last_path; }
int64_t bq_launch_count(void) { return g_launches.load(); }

// ---- MoE expert set -------------------------------------------------------------------------
int bq_moe_create(const bq_weight_t* gate, const bq_weight_t* up, const bq_weight_t* down, int E, bq_moe_t* out) {
  int rc = check_ready();
  if (rc) return rc;
  if (!gate || !up || !down || !out || E <= 0) return fail(BQ_ERR_ARG, "bad arguments");
  std::vector<const uint8_t*> pc[3];
  std::vector<const __half*> ps[3];
  int64_t H = 0, F = 0;
  int fmt = -1;
  for (int e = 0; e < E; ++e) {
    Weight* g = get_weight(gate[e]); if (!g) return BQ_ERR_HANDLE;
    Weight* u = get_weight(up[e]);   if (!u) return BQ_ERR_HANDLE;
    Weight* d = get_weight(down[e]); if (!d) return BQ_ERR_HANDLE;
    if (e == 0) { H = g->K; F = g->N; fmt = g->fmt; }
    if (g->K != H || g->N != F || u->K != H || u->N != F || d->K != F || d->N != H || g->fmt != fmt ||
        u->fmt != fmt || d->fmt != fmt)
      return fail(BQ_ERR_ARG, "expert weights must share shapes gate/up [F,H], down [H,F] and one format");
    pc[0].push_back(g->codes); ps[0].push_back(g->scales);
    pc[1].push_back(u->codes); ps[1].push_back(u->scales);
    pc[2].push_back(d->codes); ps[2].push_back(d->scales);
  }
  Moe* m = new Moe();
  m->magic = MOE_MAGIC; m->E = E; m->H = H; m->F = F; m->fmt = fmt;
  const uint8_t*** cdst[3] = {&m->gate_codes, &m->up_codes, &m->down_codes};
  const __half*** sdst[3] = {&m->gate_scales, &m->up_scales, &m->down_scales};
  for (int i = 0; i < 3; ++i) {
    BQ_CUDA(cudaMalloc((void**)cdst[i], sizeof(void*) * E));
    BQ_CUDA(cudaMalloc((void**)sdst[i], sizeof(void*) * E));
    BQ_CUDA(cudaMemcpy((void*)*cdst[i], pc[i].data(), sizeof(void*) * E, cudaMemcpyHostToDevice));
    BQ_CUDA(cudaMemcpy((void*)*sdst[i], ps[i].data(), sizeof(void*) * E, cudaMemcpyHostToDevice));
  }
  m->tc_state = nullptr;
  if (int rc2 = moe_tc_prepare(m, pc, ps)) return rc2;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_moes.insert(m);
  }
  *out = static_cast<bq_moe_t>(reinterpret_cast<uintptr_t>(m));
  return BQ_OK;
}

int bq_moe_destroy(bq_moe_t h) {
  Moe* m = get_moe(h);
  if (!m) return BQ_ERR_HANDLE;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    g_moes.erase(m);
  }
  m->magic = 0;
  moe_tc_release(m);
  cudaFree((void*)m->gate_codes); cudaFree((void*)m->gate_scales);
  cudaFree((void*)m->up_codes);   cudaFree((void*)m->up_scales);
  cudaFree((void*)m->down_codes); cudaFree((void*)m->down_scales);
  delete m;
  return BQ_OK;
}

}  // extern "C"
