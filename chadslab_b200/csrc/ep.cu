// Expert-parallel dispatch / combine through peer memory (one process per GPU, buffers mapped with CUDA IPC): the
// all-to-all around the grouped experts written as plain stores into the owning rank's HBM.
//
// Setting: `world` ranks, E experts, El = E / world of them on each rank (rank r owns experts r*El .. r*El + El-1);
// tokens stay data-parallel.  Per MoE layer, identical on every rank (epoch e counts the layers run so far):
//   1. the rank sorts its T*k assignments by GLOBAL expert (bq_moe_permute): perm, offsets[E+1];
//   2. ep_layout_kernel: the E per-expert counts go to every rank (the receive-slot protocol of the tensor-parallel
//      sums: a word holds EP_EMPTY until its value arrives, so no flags), every rank then holds the whole count
//      matrix C[source][expert] and derives from it, without any further exchange,
//        - where in the owner's receive buffer its own rows of expert x start (rows of one local expert are
//          contiguous on the owner, sources in rank order),
//        - the row ranges of its own local experts (the `offsets` the grouped expert kernel reads), and
//        - for every (local expert, source) block of received rows the position of its first row in the source's
//          sorted order (for the way back);
//   3. ep_dispatch_kernel: every routed row x[t, :] is stored straight into the owner's receive buffer with 16-byte
//      stores (no local permuted copy); when a rank's last CTA is done it raises its flag (= e) on every rank with a
//      release store behind a system-scope fence;
//   4. ep_wait_kernel: the owner waits (bounded) until every source's flag shows e; the grouped experts then run on
//      the receive buffer;
//   5. ep_return_kernel: every output row goes back to its source's return buffer at its position in the source's
//      sorted order (fp32: the combine then adds exactly what a single GPU would add), flags as in 3;
//   6. ep_combine_kernel: waits for every rank's return flag, y[t] = sum over slots of w * row (fixed slot order),
//      and the last CTA advances the epoch on the device, so a captured CUDA graph replays.
// Buffer reuse needs no extra hand-shake: a source can only dispatch layer e+1 after its combine of layer e, which
// needs every rank's return flag of layer e, which a rank raises after its experts have consumed its receive
// buffer; the return buffer of layer e+1 is written only after the experts of layer e+1, which need every source's
// dispatch of e+1, which follows that source's combine of e.
// Every wait is bounded; on expiry the kernel records BQ_ERR_TIMEOUT, marks the object failed and returns.
// Plain ld / st on peer-mapped memory only: no multicast, no multimem.
#include <cstring>
#include <mutex>
#include <unordered_set>

#include "common.cuh"

namespace bq {

constexpr uint32_t EP_MAGIC = 0xB200E9E9u;
constexpr uint32_t EP_EMPTY = 0x80000000u;
constexpr int EP_MAX_WORLD = COMM_MAX_WORLD;
constexpr int EP_MAX_E = 1024;
constexpr int EP_WAIT_MS_DEFAULT = 5000;
// header words of a rank's shared buffer
//   [0] epoch (starts at 1)   [1] finished-CTA counter (dispatch)   [2] failed   [3] finished-CTA counter (return)
//   [4] finished-CTA counter (combine)   [16 .. 16+world) dispatch flags   [32 .. 32+world) return flags
constexpr int EP_HDR_WORDS = 64;

struct EpDev {                         // what the kernels read (device copy)
  uint8_t* base[EP_MAX_WORLD];         // every rank's shared buffer
  int32_t* priv;                       // this rank's private tables (layout results)
  uint64_t wait_ns;
  int64_t H, cap_recv, cap_send;
  int rank, world, E, El;
  // byte offsets inside a shared buffer
  int64_t off_counts, off_xrecv, off_yback;
};
// private tables (int32 indices into EpDev::priv)
//   dest_base[E]            row in the owner's receive buffer where this rank's rows of expert x start
//   loffsets[El + 1]        row ranges of this rank's local experts in its receive buffer
//   blk_start[El*world + 1] first received row of block (local expert, source); last = number of received rows
//   blk_src[El*world]       position of that block's first row in the source's sorted order
struct EpTables {
  int64_t dest_base, loffsets, blk_start, blk_src, total;
};
__host__ __device__ inline EpTables ep_tables(int E, int El, int world) {
  EpTables t;
  t.dest_base = 0;
  t.loffsets = t.dest_base + E;
  t.blk_start = t.loffsets + El + 1;
  t.blk_src = t.blk_start + (int64_t)El * world + 1;
  t.total = t.blk_src + (int64_t)El * world;
  return t;
}

struct Ep {
  uint32_t magic;
  int rank, world, E, El;
  int64_t H, cap_send, cap_recv;
  size_t bytes;
  uint8_t* local;
  void* peer[EP_MAX_WORLD];
  int32_t* priv;
  EpDev* dev;
  EpDev host;
  int wait_ms;
  bool connected, failed;
};

static std::mutex e_mu;
static std::unordered_set<void*> e_eps;

static Ep* get_ep(bq_ep_t h) {
  void* p = reinterpret_cast<void*>(static_cast<uintptr_t>(h));
  std::lock_guard<std::mutex> lk(e_mu);
  if (!p || !e_eps.count(p) || static_cast<Ep*>(p)->magic != EP_MAGIC) {
    fail(BQ_ERR_HANDLE, "invalid expert-parallel handle");
    return nullptr;
  }
  return static_cast<Ep*>(p);
}
void ep_mark_all_failed() {
  std::lock_guard<std::mutex> lk(e_mu);
  for (void* p : e_eps) static_cast<Ep*>(p)->failed = true;
}

// ---- device helpers ------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ep_ld_relaxed(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ep_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void ep_st_relaxed(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void ep_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint64_t ep_now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t* ep_hdr(const EpDev* d, int r) { return reinterpret_cast<uint32_t*>(d->base[r]); }
__device__ __noinline__ void ep_give_up(const EpDev* d, int* status) {
  atomicExch(status, (int)BQ_ERR_TIMEOUT);
  atomicExch(ep_hdr(d, d->rank) + 2, 1u);
}
__device__ __forceinline__ bool ep_failed(const EpDev* d, int* status) {
  if (*reinterpret_cast<const volatile uint32_t*>(ep_hdr(d, d->rank) + 2) == 0u) return false;
  if (threadIdx.x == 0) atomicExch(status, (int)BQ_ERR_TIMEOUT);
  return true;
}
// Bounded wait until a flag of this rank's header shows at least `want` (flags only grow).  false = gave up.
__device__ __noinline__ bool ep_wait_flag(const EpDev* d, const uint32_t* flag, uint32_t want, int* status) {
  if ((int32_t)(ep_ld_acquire(flag) - want) >= 0) return true;
  const uint64_t deadline = ep_now_ns() + d->wait_ns;
  uint32_t spins = 0;
  for (;;) {
    if ((int32_t)(ep_ld_acquire(flag) - want) >= 0) return true;
    if ((++spins & 63u) == 0 && ep_now_ns() > deadline) {
      ep_give_up(d, status);
      return false;
    }
  }
}
// All CTAs of the grid have stored their rows: the last one to get here raises this rank's flag on every rank.
// `counter`: a word of this rank's header, zero between launches; `flag_word`: index of the flag array.
__device__ __forceinline__ void ep_signal_all(const EpDev* d, int counter_word, int flag_word, uint32_t e) {
  __syncthreads();                       // every thread's stores precede thread 0's fence in causality order
  if (threadIdx.x == 0) {
    __threadfence_system();
    uint32_t* hdr = ep_hdr(d, d->rank);
    const uint32_t done = atomicAdd(hdr + counter_word, 1u);
    if (done == gridDim.x * gridDim.y - 1) {
      hdr[counter_word] = 0;
      __threadfence_system();
      for (int r = 0; r < d->world; ++r) ep_st_release(ep_hdr(d, r) + flag_word + d->rank, e);
    }
  }
}

// ---- step 2: counts to everybody, layout tables ------------------------------------------------------------
// One CTA of NT = the power of two >= E threads (at least 32); thread x owns expert x (E <= 1024).
// `matrix` != nullptr (self-test): the whole count matrix [world][E] is given, nothing is exchanged.
__global__ void __launch_bounds__(1024) ep_layout_kernel(const EpDev* __restrict__ d, const int32_t* __restrict__ offsets,
                                                          const int32_t* __restrict__ matrix, int* status) {
  __shared__ int32_t scan[1024];
  __shared__ int32_t tot[1024];
  const int x = threadIdx.x, NT = blockDim.x;
  const int world = d->world, E = d->E, El = d->El, me = d->rank;
  if (!matrix && ep_failed(d, status)) return;
  const uint32_t e = matrix ? 0u : *reinterpret_cast<const volatile uint32_t*>(ep_hdr(d, me));
  const int64_t par = (int64_t)(e & 1u) * world;
  const EpTables tb = ep_tables(E, El, world);
  int32_t* priv = d->priv;
  // deposit my count of expert x in slot [parity][me] of every rank
  if (x < E && !matrix) {
    const uint32_t c = (uint32_t)(offsets[x + 1] - offsets[x]);
    for (int r = 0; r < world; ++r) {
      uint32_t* slot = reinterpret_cast<uint32_t*>(d->base[r] + d->off_counts) + (par + me) * E;
      ep_st_relaxed(slot + x, c);
    }
  }
  // collect C[s][x] for every source s
  int32_t C[EP_MAX_WORLD];
  int32_t mine_before = 0, total = 0;
  if (matrix) {
#pragma unroll
    for (int s = 0; s < EP_MAX_WORLD; ++s) {
      C[s] = (s < world && x < E) ? matrix[(int64_t)s * E + x] : 0;
      if (s < me) mine_before += C[s];
      total += C[s];
    }
  } else {
    uint32_t* my_counts = reinterpret_cast<uint32_t*>(d->base[me] + d->off_counts);
    uint64_t deadline = 0;
#pragma unroll
    for (int s = 0; s < EP_MAX_WORLD; ++s) {
      C[s] = 0;
      if (s < world && x < E) {
        uint32_t* w = my_counts + (par + s) * E + x;
        uint32_t v = ep_ld_relaxed(w);
        if (v == EP_EMPTY) {
          if (deadline == 0) deadline = ep_now_ns() + d->wait_ns;
          uint32_t spins = 0;
          while ((v = ep_ld_relaxed(w)) == EP_EMPTY) {
            if ((++spins & 63u) == 0 && ep_now_ns() > deadline) { ep_give_up(d, status); v = 0; break; }
          }
        }
        ep_st_relaxed(w, EP_EMPTY);
        C[s] = (int32_t)v;
        if (s < me) mine_before += C[s];
        total += C[s];
      }
    }
  }
  // seg[x] = first row of expert x in its owner's receive buffer = sum of tot over the owner's experts before x
  tot[x] = x < E ? total : 0;
  scan[x] = tot[x];
  __syncthreads();
  for (int off = 1; off < NT; off <<= 1) {
    const int32_t add = x >= off ? scan[x - off] : 0;
    __syncthreads();
    scan[x] += add;
    __syncthreads();
  }
  int32_t seg = 0;
  if (x < E) {
    const int first = (x / El) * El;                       // the owner's first expert
    seg = (scan[x] - tot[x]) - (first > 0 ? scan[first - 1] : 0);
    priv[tb.dest_base + x] = seg + mine_before;
    if (x / El == me) {                                    // one of my experts: its row range and its source blocks
      const int le = x - me * El;
      priv[tb.loffsets + le] = seg;
      if (le == El - 1) priv[tb.loffsets + El] = seg + total;
      int32_t run = seg;
      for (int s = 0; s < world; ++s) {
        priv[tb.blk_start + (int64_t)le * world + s] = run;
        run += C[s];
      }
      if (le == El - 1) priv[tb.blk_start + (int64_t)El * world] = run;
    }
  }
  // blk_src[le][s] = position of expert (me*El + le) in source s's sorted order = sum over x' < x of C[s][x']
  for (int s = 0; s < world; ++s) {
    __syncthreads();
    int32_t cs = 0;
#pragma unroll
    for (int q = 0; q < EP_MAX_WORLD; ++q) if (q == s) cs = C[q];
    scan[x] = x < E ? cs : 0;
    __syncthreads();
    for (int off = 1; off < NT; off <<= 1) {
      const int32_t add = x >= off ? scan[x - off] : 0;
      __syncthreads();
      scan[x] += add;
      __syncthreads();
    }
    if (x < E && x / El == me) priv[tb.blk_src + (int64_t)(x - me * El) * world + s] = scan[x] - cs;
  }
}

// ---- step 3: rows to their owners -----------------------------------------------------------------------------
// One warp per sorted position p: expert x = idx[perm[p]], row j = p - offsets[x] of my rows for x.
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpDev* __restrict__ d, const uint4* __restrict__ x,
                                                          const int32_t* __restrict__ idx, const int32_t* __restrict__ perm,
                                                          const int32_t* __restrict__ offsets, int64_t A, int top_k,
                                                          int* status) {
  if (ep_failed(d, status)) return;
  const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(ep_hdr(d, d->rank));
  const int lane = threadIdx.x & 31;
  const int64_t row_vec = d->H / 8;                        // bf16 rows as 16-byte vectors
  const EpTables tb = ep_tables(d->E, d->El, d->world);
  for (int64_t p = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); p < A; p += (int64_t)gridDim.x * 8) {
    const int32_t a = perm[p];
    if (a < 0) continue;                                   // dropped assignment (expert id out of range)
    const int32_t ex = idx[a];
    const int64_t dst_row = (int64_t)d->priv[tb.dest_base + ex] + (p - offsets[ex]);
    if (dst_row >= d->cap_recv) {                          // would not fit the owner's receive buffer: record, skip
      if (lane == 0) atomicExch(status, (int)BQ_ERR_ARG);
      continue;
    }
    const uint4* src = x + (int64_t)(a / top_k) * row_vec;
    uint4* dst = reinterpret_cast<uint4*>(d->base[ex / d->El] + d->off_xrecv) + dst_row * row_vec;
    for (int64_t c = lane; c < row_vec; c += 32) dst[c] = src[c];
  }
  ep_signal_all(d, 1, 16, e);
}

// ---- step 4: the owner waits for every source ------------------------------------------------------------------
__global__ void __launch_bounds__(32) ep_wait_kernel(const EpDev* __restrict__ d, int flag_word, int* status) {
  if (ep_failed(d, status)) return;
  const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(ep_hdr(d, d->rank));
  if ((int)threadIdx.x < d->world) ep_wait_flag(d, ep_hdr(d, d->rank) + flag_word + threadIdx.x, e, status);
}

// ---- step 5: output rows back to their sources -------------------------------------------------------------------
__global__ void __launch_bounds__(256) ep_return_kernel(const EpDev* __restrict__ d, const uint4* __restrict__ out,
                                                        int* status) {
  if (ep_failed(d, status)) return;
  const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(ep_hdr(d, d->rank));
  const int lane = threadIdx.x & 31;
  const int64_t row_vec = d->H / 4;                        // fp32 rows as 16-byte vectors
  const EpTables tb = ep_tables(d->E, d->El, d->world);
  const int nblk = d->El * d->world;
  const int32_t* blk_start = d->priv + tb.blk_start;
  const int64_t n_recv = blk_start[nblk];
  for (int64_t i = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); i < n_recv; i += (int64_t)gridDim.x * 8) {
    int lo = 0, hi = nblk - 1;                             // last block whose first row is <= i
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (blk_start[mid] <= i) lo = mid; else hi = mid - 1;
    }
    const int s = lo % d->world;
    const int64_t p = (int64_t)d->priv[tb.blk_src + lo] + (i - blk_start[lo]);
    if (p >= d->cap_send) {
      if (lane == 0) atomicExch(status, (int)BQ_ERR_ARG);
      continue;
    }
    const uint4* src = out + i * row_vec;
    uint4* dst = reinterpret_cast<uint4*>(d->base[s] + d->off_yback) + p * row_vec;
    for (int64_t c = lane; c < row_vec; c += 32) dst[c] = src[c];
  }
  ep_signal_all(d, 3, 32, e);
}

// ---- step 6: weighted sum on the tokens' owner, epoch advance --------------------------------------------------------
template <typename YT>
__global__ void __launch_bounds__(256) ep_combine_kernel(const EpDev* __restrict__ d, const int32_t* __restrict__ inv,
                                                         const float* __restrict__ w, int64_t T, int top_k,
                                                         YT* __restrict__ y, int* status) {
  if (ep_failed(d, status)) return;
  uint32_t* hdr = ep_hdr(d, d->rank);
  const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(hdr);
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < d->world && !ep_wait_flag(d, hdr + 32 + threadIdx.x, e, status)) ok = 0;
  __syncthreads();
  const float* back = reinterpret_cast<const float*>(d->base[d->rank] + d->off_yback);
  const int64_t H = d->H, total = T * H;
  if (ok) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
      const int64_t t = i / H, c = i - t * H;
      float acc = 0.0f;
      for (int s = 0; s < top_k; ++s) {      // fixed slot order, separate multiply and add (as moe_combine_kernel)
        const int32_t p = inv[t * top_k + s];
        if (p >= 0) acc = __fadd_rn(acc, __fmul_rn(w[t * top_k + s], __ldcg(back + (int64_t)p * H + c)));
      }
      y[i] = from_float<YT>(acc);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(hdr + 4, 1u);
    if (done == gridDim.x - 1) {
      hdr[4] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(hdr) = e + 1;
    }
  }
}

__global__ void ep_fill_kernel(uint32_t* p, int64_t n, uint32_t v) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}

// ---- host side -------------------------------------------------------------------------------------------------
static int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

static cudaError_t ep_fill_local(Ep* c) {
  cudaError_t e = cudaMemset(c->local, 0, EP_HDR_WORDS * 4);
  if (e != cudaSuccess) return e;
  ep_fill_kernel<<<64, 256>>>(reinterpret_cast<uint32_t*>(c->local + c->host.off_counts), (int64_t)2 * c->world * c->E, EP_EMPTY);
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  const uint32_t one = 1;
  if ((e = cudaMemcpy(c->local, &one, sizeof(one), cudaMemcpyHostToDevice)) != cudaSuccess) return e;
  return cudaDeviceSynchronize();
}

static int ep_upload(Ep* c) {
  for (int r = 0; r < c->world; ++r) {
    uint8_t* base = r == c->rank ? c->local : static_cast<uint8_t*>(c->peer[r]);
    if (!base) return fail(BQ_ERR_STATE, "expert-parallel object is not connected to every rank");
    c->host.base[r] = base;
  }
  c->host.wait_ns = (uint64_t)c->wait_ms * 1000000ull;
  BQ_CUDA(cudaMemcpy(c->dev, &c->host, sizeof(EpDev), cudaMemcpyHostToDevice));
  return BQ_OK;
}

static int ep_usable(Ep* c) {
  if (device_id() < 0) return fail(BQ_ERR_STATE, "bq_init() has not been called");
  if (!c->connected) return fail(BQ_ERR_STATE, "expert-parallel object is not connected");
  if (c->failed) return fail(BQ_ERR_STATE, "a wait on this expert-parallel object timed out: destroy it on every rank");
  return BQ_OK;
}

}  // namespace bq

using namespace bq;

extern "C" {

int bq_ep_create(int rank, int world, int n_experts, int64_t hidden, int64_t max_send_rows, int64_t max_recv_rows,
                 bq_ep_t* out) {
  if (device_id() < 0) return fail(BQ_ERR_STATE, "bq_init() has not been called");
  if (!out) return fail(BQ_ERR_ARG, "null pointer");
  if (world < 1 || world > EP_MAX_WORLD || rank < 0 || rank >= world) return fail(BQ_ERR_ARG, "bad rank / world (world <= 8)");
  if (n_experts < world || n_experts > EP_MAX_E || n_experts % world)
    return fail(BQ_ERR_ARG, "the experts (at most 1024) must divide evenly over the ranks");
  if (hidden <= 0 || hidden % 8) return fail(BQ_ERR_ARG, "hidden must be a positive multiple of 8");
  if (max_send_rows <= 0 || max_recv_rows <= 0 || max_send_rows > ((int64_t)1 << 30) || max_recv_rows > ((int64_t)1 << 30))
    return fail(BQ_ERR_ARG, "row capacities out of range");
  Ep* c = new Ep();
  memset(c, 0, sizeof(*c));
  c->magic = EP_MAGIC;
  c->rank = rank; c->world = world; c->E = n_experts; c->El = n_experts / world;
  c->H = hidden; c->cap_send = max_send_rows; c->cap_recv = max_recv_rows;
  c->wait_ms = EP_WAIT_MS_DEFAULT;
  EpDev& h = c->host;
  h.H = hidden; h.cap_recv = max_recv_rows; h.cap_send = max_send_rows;
  h.rank = rank; h.world = world; h.E = n_experts; h.El = c->El;
  h.off_counts = align256(EP_HDR_WORDS * 4);
  h.off_xrecv = align256(h.off_counts + (int64_t)2 * world * n_experts * 4);
  h.off_yback = align256(h.off_xrecv + max_recv_rows * hidden * 2);
  c->bytes = (size_t)align256(h.off_yback + max_send_rows * hidden * 4);
  const EpTables tb = ep_tables(c->E, c->El, world);
  cudaError_t e = cudaMalloc((void**)&c->local, c->bytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&c->priv, sizeof(int32_t) * (size_t)(tb.total + 64));
  if (e == cudaSuccess) e = cudaMalloc((void**)&c->dev, sizeof(EpDev));
  if (e == cudaSuccess) e = cudaMemset(c->priv, 0, sizeof(int32_t) * (size_t)(tb.total + 64));
  if (e == cudaSuccess) { h.priv = c->priv; e = ep_fill_local(c); }
  if (e != cudaSuccess) {
    if (c->local) cudaFree(c->local);
    if (c->priv) cudaFree(c->priv);
    if (c->dev) cudaFree(c->dev);
    delete c;
    return fail_cuda(e, "cudaMalloc(expert-parallel buffers)");
  }
  if (world == 1) {
    int rc = ep_upload(c);
    if (rc) { cudaFree(c->local); cudaFree(c->priv); cudaFree(c->dev); delete c; return rc; }
    c->connected = true;
  }
  {
    std::lock_guard<std::mutex> lk(e_mu);
    e_eps.insert(c);
  }
  *out = static_cast<bq_ep_t>(reinterpret_cast<uintptr_t>(c));
  return BQ_OK;
}

int bq_ep_handle(bq_ep_t ep, void* out64) {
  Ep* c = get_ep(ep);
  if (!c) return BQ_ERR_HANDLE;
  if (!out64) return fail(BQ_ERR_ARG, "null pointer");
  cudaIpcMemHandle_t h;
  BQ_CUDA(cudaIpcGetMemHandle(&h, c->local));
  memcpy(out64, &h, sizeof(h));
  return BQ_OK;
}

int bq_ep_connect(bq_ep_t ep, const void* handles) {
  Ep* c = get_ep(ep);
  if (!c) return BQ_ERR_HANDLE;
  if (!handles) return fail(BQ_ERR_ARG, "null pointer");
  if (c->connected) return fail(BQ_ERR_STATE, "already connected");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)r * BQ_COMM_HANDLE_BYTES, sizeof(h));
    BQ_CUDA(cudaIpcOpenMemHandle(&c->peer[r], h, cudaIpcMemLazyEnablePeerAccess));
  }
  int rc = ep_upload(c);
  if (rc) return rc;
  c->connected = true;
  return BQ_OK;
}

int bq_ep_set_timeout_ms(bq_ep_t ep, int ms) {
  Ep* c = get_ep(ep);
  if (!c) return BQ_ERR_HANDLE;
  if (ms < 1 || ms > 60000) return fail(BQ_ERR_ARG, "time limit must be 1..60000 ms");
  c->wait_ms = ms;
  if (c->connected) {
    BQ_CUDA(cudaDeviceSynchronize());
    return ep_upload(c);
  }
  return BQ_OK;
}

int bq_ep_destroy(bq_ep_t ep) {
  Ep* c = get_ep(ep);
  if (!c) return BQ_ERR_HANDLE;
  {
    std::lock_guard<std::mutex> lk(e_mu);
    e_eps.erase(c);
  }
  cudaDeviceSynchronize();
  for (int r = 0; r < c->world; ++r)
    if (c->peer[r]) cudaIpcCloseMemHandle(c->peer[r]);
  cudaFree(c->local);
  cudaFree(c->priv);
  cudaFree(c->dev);
  c->magic = 0;
  delete c;
  return BQ_OK;
}

int bq_ep_dispatch(bq_ep_t ep, const void* x_bf16, const int32_t* idx, const int32_t* perm, const int32_t* offsets,
                   int64_t T, int top_k, void* stream) {
  Ep* c = get_ep(ep);
  if (!c) return BQ_ERR_HANDLE;
  int rc = ep_usable(c);
  if (rc) return rc;
  if (T < 0 || top_k <= 0) return fail(BQ_ERR_ARG, "bad sizes");
  const int64_t A = T * top_k;
  if (A > c->cap_send) return fail(BQ_ERR_ARG, "T * top_k exceeds max_send_rows of this expert-parallel object");
  if (!offsets || (A > 0 && (!x_bf16 || !idx || !perm))) return fail(BQ_ERR_ARG, "null pointer");
  if ((reinterpret_cast<uintptr_t>(x_bf16) & 15) != 0) return fail(BQ_ERR_ARG, "activations must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  int nt = 32;
  while (nt < c->E) nt <<= 1;
  ep_layout_kernel<<<1, nt, 0, s>>>(c->dev, offsets, nullptr, status_word());
  int64_t grid = (A + 7) / 8;
  if (grid > (int64_t)sm_count() * 8) grid = (int64_t)sm_count() * 8;
  if (grid < 1) grid = 1;                      // a rank without tokens still raises its flag
  ep_dispatch_kernel<<<(unsigned)grid, 256, 0, s>>>(c->dev, (const uint4*)x_bf16, idx, perm, offsets, A, top_k, status_word());
  ep_wait_kernel<<<1, 32, 0, s>>>(c->dev, 16, status_word());
  count_launch(3);
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

int bq_ep_layout_selftest(const int32_t* counts, int rank, int world, int n_experts, int32_t* tables_out, void* stream) {
  if (device_id() < 0) return fail(BQ_ERR_STATE, "bq_init() has not been called");
  if (world < 1 || world > EP_MAX_WORLD || rank < 0 || rank >= world || n_experts < world || n_experts > EP_MAX_E ||
      n_experts % world || !counts || !tables_out)
    return fail(BQ_ERR_ARG, "bad arguments");
  EpDev h;
  memset(&h, 0, sizeof(h));
  h.rank = rank; h.world = world; h.E = n_experts; h.El = n_experts / world; h.priv = tables_out;
  EpDev* dev = nullptr;
  BQ_CUDA(cudaMalloc((void**)&dev, sizeof(EpDev)));
  cudaError_t e = cudaMemcpy(dev, &h, sizeof(h), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) {
    int nt = 32;
    while (nt < n_experts) nt <<= 1;
    ep_layout_kernel<<<1, nt, 0, (cudaStream_t)stream>>>(dev, nullptr, counts, status_word());
    count_launch();
    e = cudaGetLastError();
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  cudaFree(dev);
  if (e != cudaSuccess) return fail_cuda(e, "bq_ep_layout_selftest");
  return BQ_OK;
}

int bq_ep_recv_view(bq_ep_t ep, void** xrecv_bf16, const int32_t** local_offsets, int64_t* max_rows) {
  Ep* c = get_ep(ep);
  if (!c) return BQ_ERR_HANDLE;
  const EpTables tb = ep_tables(c->E, c->El, c->world);
  if (xrecv_bf16) *xrecv_bf16 = c->local + c->host.off_xrecv;
  if (local_offsets) *local_offsets = c->priv + tb.loffsets;
  if (max_rows) *max_rows = c->cap_recv;
  return BQ_OK;
}

int bq_ep_combine(bq_ep_t ep, const float* out_rows, const int32_t* inv, const float* w, int64_t T, int top_k, void* y,
                  int y_dtype, void* stream) {
  Ep* c = get_ep(ep);
  if (!c) return BQ_ERR_HANDLE;
  int rc = ep_usable(c);
  if (rc) return rc;
  if (T < 0 || top_k <= 0) return fail(BQ_ERR_ARG, "bad sizes");
  if (y_dtype != BQ_DT_F32 && y_dtype != BQ_DT_BF16) return fail(BQ_ERR_ARG, "bad dtype");
  if (T * top_k > c->cap_send) return fail(BQ_ERR_ARG, "T * top_k exceeds max_send_rows of this expert-parallel object");
  if (!out_rows || (T > 0 && (!inv || !w || !y))) return fail(BQ_ERR_ARG, "null pointer");
  if ((reinterpret_cast<uintptr_t>(out_rows) & 15) != 0) return fail(BQ_ERR_ARG, "expert outputs must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  int64_t g1 = (c->cap_recv + 7) / 8;
  if (g1 > (int64_t)sm_count() * 8) g1 = (int64_t)sm_count() * 8;
  ep_return_kernel<<<(unsigned)g1, 256, 0, s>>>(c->dev, (const uint4*)out_rows, status_word());
  int64_t g2 = (T * c->H + 255) / 256;
  if (g2 > (int64_t)sm_count() * 16) g2 = (int64_t)sm_count() * 16;
  if (g2 < 1) g2 = 1;                          // the epoch advances on every rank, tokens or not
  if (y_dtype == BQ_DT_F32)
    ep_combine_kernel<float><<<(unsigned)g2, 256, 0, s>>>(c->dev, inv, w, T, top_k, (float*)y, status_word());
  else
    ep_combine_kernel<__nv_bfloat16><<<(unsigned)g2, 256, 0, s>>>(c->dev, inv, w, T, top_k, (__nv_bfloat16*)y, status_word());
  count_launch(2);
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

}  // extern "C"
