// Peer-memory communicator for the tensor-parallel shard boundary: a one-shot all-reduce over NVLink written as
// plain stores into the other ranks' HBM, fused with what precedes it (the row-parallel GEMV deposits its partial
// sums directly in the peers' receive slots, gemv_push.cu) and with what follows it (residual add + RMSNorm of the
// reduced row).  One process per GPU; the buffers are exchanged as CUDA IPC handles by the host code (which
// carries the 64-byte handles over its own process group).
//
// Protocol, per call (epoch e, parity p = e & 1), identical on every rank:
//   1. deposit: rank s stores its contribution into slot [p][s] of EVERY rank's buffer (its own included) with
//               16-byte system-scope stores (4-byte ones for ragged ends);
//   2. collect: every 4-byte word of a slot reads COMM_EMPTY (the bits of -0.0f; deposits never carry them) until
//               its value has arrived, so the receiver re-reads a 16-byte vector until none of its words is empty --
//               no flags and no fences, and a vector store that arrives in pieces is handled word by word.
//               The wait is bounded: after the communicator's time limit (5 s unless changed) the kernel records
//               BQ_ERR_TIMEOUT in the library's status word, marks the communicator failed and carries on;
//   3. sum:     slots [p][0..world) are added in rank order, so every rank gets bit-identical results, and the
//               thread that read a vector puts COMM_EMPTY back;
//   4. the last CTA to finish advances the epoch (device-side, so a replayed CUDA graph keeps working).
//
// Why two parities suffice, and what orders the re-emptying of a word against its next deposit.  Rank A empties a
// word of slot [p][r] inside the summing kernel of call e.  Rank r writes that word again in call e+2.  Before r can
// issue call e+2 it must have finished its own call e+1, whose sum needed A's contribution to call e+1; A deposits
// that contribution from a kernel that starts after A's summing kernel of call e has completed (same stream), and
// a completed kernel's stores have been performed at their home L2 -- here A's own memory.  r observes A's e+1 value,
// finishes its kernel, and only a later kernel of r stores to A's word again; that store reaches the same home L2
// strictly after the emptying store was performed there, so it cannot be overwritten by it.  The argument leans on
// kernel boundaries on both ranks (completion of a grid = all of its writes performed), not on release/acquire
// pairs inside the kernels; inside a kernel the only same-word sequence is load-then-store by one thread, which
// program order covers.
// A communicator that ran into a time-out stays failed: a late deposit of the abandoned call could otherwise be taken
// for a value of call e+2.  Summing calls on it record BQ_ERR_TIMEOUT again and do nothing until bq_comm_reset().
// Nothing here uses multicast or multimem: plain ld / st on peer-mapped memory only.
#include <cstring>
#include <mutex>
#include <unordered_set>

#include "common.cuh"

namespace bq {

constexpr int COMM_WAIT_MS_DEFAULT = 5000;
constexpr int COMM_HEADER_BYTES = 256;
constexpr uint32_t COMM_MAGIC = 0xB200C033u;
constexpr int AR_THREADS = 256;

struct Comm {
  uint32_t magic;
  int rank, world;
  int64_t slot_elems;
  size_t bytes;
  uint8_t* local;                       // this rank's buffer (cudaMalloc)
  void* peer[COMM_MAX_WORLD];           // mappings of the other ranks' buffers (nullptr for self / not connected)
  CommDev* dev;                         // device copy of the descriptor
  int wait_ms;
  bool connected;
  bool loopback;                        // peers are private stand-in buffers of this process (bq_comm_connect_loopback)
  bool failed;                          // a time-out was reported by bq_status_poll: unusable until bq_comm_reset
};

static std::mutex c_mu;
static std::unordered_set<void*> c_comms;

static Comm* get_comm(bq_comm_t h) {
  void* p = reinterpret_cast<void*>(static_cast<uintptr_t>(h));
  std::lock_guard<std::mutex> lk(c_mu);
  if (!p || !c_comms.count(p) || static_cast<Comm*>(p)->magic != COMM_MAGIC) {
    fail(BQ_ERR_HANDLE, "invalid communicator handle");
    return nullptr;
  }
  return static_cast<Comm*>(p);
}

// bq_status_poll saw BQ_ERR_TIMEOUT: every connected communicator of this process may be the one that gave up
void comm_mark_all_failed() {
  std::lock_guard<std::mutex> lk(c_mu);
  for (void* p : c_comms) static_cast<Comm*>(p)->failed = true;
}

static size_t comm_total_bytes(int world, int64_t slot_elems) {
  return COMM_HEADER_BYTES + (size_t)2 * world * slot_elems * sizeof(float);
}

// ---- device side ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_sys_u32(const float* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_sys_v4(const float* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_empty(float* p) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(COMM_EMPTY) : "memory");
}
__device__ __forceinline__ void st_empty_v4(float* p) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%1,%1,%1};" ::"l"(p), "r"(COMM_EMPTY) : "memory");
}
__device__ __forceinline__ uint64_t comm_now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ bool any_empty(const uint4& v) {
  return v.x == COMM_EMPTY || v.y == COMM_EMPTY || v.z == COMM_EMPTY || v.w == COMM_EMPTY;
}
// The bounded wait gave up: record it and mark the communicator failed (sticky; see the file header).
__device__ __noinline__ void comm_give_up(const CommDev* d, int* status) {
  atomicExch(status, (int)BQ_ERR_TIMEOUT);
  atomicExch(d->state + 2, 1u);
}

// Step 2 for one word whose first read found it empty: re-read until the value is there or the time is up.
// `deadline` (0 = not started) is shared by all waits of a thread, so a kernel gives up after one time limit in
// total, not one per element.
__device__ __noinline__ uint32_t comm_wait_value(const CommDev* d, const float* p, uint64_t* deadline, int* status) {
  if (*deadline == 0) *deadline = comm_now_ns() + d->wait_ns;
  uint32_t spins = 0;
  for (;;) {
    const uint32_t v = ld_sys_u32(p);
    if (v != COMM_EMPTY) return v;
    if ((++spins & 63u) == 0 && comm_now_ns() > *deadline) {
      comm_give_up(d, status);
      return 0u;
    }
  }
}
__device__ __noinline__ uint4 comm_wait_v4(const CommDev* d, const float* p, uint64_t* deadline, int* status) {
  if (*deadline == 0) *deadline = comm_now_ns() + d->wait_ns;
  uint32_t spins = 0;
  for (;;) {
    const uint4 v = ld_sys_v4(p);
    if (!any_empty(v)) return v;
    if ((++spins & 63u) == 0 && comm_now_ns() > *deadline) {
      comm_give_up(d, status);
      return make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// Steps 2 and 3 for NE single words (index idx[j], skipped when < 0) of this rank's slots: sum over the ranks in
// rank order, slots emptied.  All first reads of a rank's slot are issued together.
template <int NE>
__device__ __forceinline__ void comm_collect(const CommDev* d, int64_t par, const int64_t* idx, float* sum, uint64_t* deadline,
                                             int* status) {
  float* mine = d->data[d->rank];
  const int world = d->world;
#pragma unroll
  for (int j = 0; j < NE; ++j) sum[j] = 0.0f;
  for (int r = 0; r < world; ++r) {
    float* slot = mine + (par + r) * d->slot_elems;
    uint32_t v[NE];
#pragma unroll
    for (int j = 0; j < NE; ++j) v[j] = idx[j] >= 0 ? ld_sys_u32(slot + idx[j]) : 0u;
#pragma unroll
    for (int j = 0; j < NE; ++j) {
      if (idx[j] >= 0) {
        if (v[j] == COMM_EMPTY) v[j] = comm_wait_value(d, slot + idx[j], deadline, status);
        st_empty(slot + idx[j]);
        sum[j] = r == 0 ? __uint_as_float(v[j]) : sum[j] + __uint_as_float(v[j]);
      }
    }
  }
}
// The same for NV 16-byte vectors starting at elements i0[j] (multiples of 4, skipped when < 0): the first reads of
// EVERY rank's slot are issued before anything is waited for, so one round trip to memory covers the whole sum when
// the values are already there.  sum[4 * j .. 4 * j + 3].
template <int NV>
__device__ __forceinline__ void comm_collect_v4(const CommDev* d, int64_t par, const int64_t* i0, float* sum,
                                                uint64_t* deadline, int* status) {
  float* mine = d->data[d->rank];
  const int world = d->world;
  uint4 v[COMM_MAX_WORLD][NV];
#pragma unroll
  for (int r = 0; r < COMM_MAX_WORLD; ++r) {
    if (r < world) {
      const float* slot = mine + (par + r) * d->slot_elems;
#pragma unroll
      for (int j = 0; j < NV; ++j) v[r][j] = i0[j] >= 0 ? ld_sys_v4(slot + i0[j]) : make_uint4(0u, 0u, 0u, 0u);
    }
  }
#pragma unroll
  for (int r = 0; r < COMM_MAX_WORLD; ++r) {
    if (r < world) {
      float* slot = mine + (par + r) * d->slot_elems;
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        if (i0[j] >= 0) {
          if (any_empty(v[r][j])) v[r][j] = comm_wait_v4(d, slot + i0[j], deadline, status);
          st_empty_v4(slot + i0[j]);
          const float f0 = __uint_as_float(v[r][j].x), f1 = __uint_as_float(v[r][j].y);
          const float f2 = __uint_as_float(v[r][j].z), f3 = __uint_as_float(v[r][j].w);
          if (r == 0) { sum[4 * j] = f0; sum[4 * j + 1] = f1; sum[4 * j + 2] = f2; sum[4 * j + 3] = f3; }
          else        { sum[4 * j] += f0; sum[4 * j + 1] += f1; sum[4 * j + 2] += f2; sum[4 * j + 3] += f3; }
        }
      }
    }
  }
}

// Step 4.  Called by every thread of the CTA when its reads of the slots are done.
__device__ __forceinline__ void comm_finish(const CommDev* d, uint32_t e) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(d->state + 1, 1u);
    if (done == gridDim.x - 1) {
      d->state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(d->state) = e + 1;
    }
  }
}
// A failed communicator (an earlier call timed out) does nothing but say so again.
__device__ __forceinline__ bool comm_failed(const CommDev* d, int* status) {
  if (*reinterpret_cast<const volatile uint32_t*>(d->state + 2) == 0u) return false;
  if (threadIdx.x == 0) atomicExch(status, (int)BQ_ERR_TIMEOUT);
  return true;
}

__global__ void comm_fill_empty_kernel(uint32_t* p, int64_t n) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = COMM_EMPTY;
}

// out[i] = sum over ranks of in_r[i].  `in` == nullptr: the contributions were already deposited by the kernel
// before this one (the PUSH GEMV).  A CTA owns `chunk` consecutive elements (a multiple of 4); `vec`: in and out are
// 16-byte aligned, so whole vectors are moved.
__global__ void __launch_bounds__(AR_THREADS) allreduce_sum_kernel(const CommDev* __restrict__ d, const float* __restrict__ in,
                                                                   float* __restrict__ out, int64_t count, int64_t chunk,
                                                                   int vec, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  if (comm_failed(d, status)) return;
  const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(d->state);
  const int world = d->world;
  const int64_t lo = (int64_t)blockIdx.x * chunk;
  const int64_t hi = lo + chunk < count ? lo + chunk : count;
  const int64_t hi4 = vec ? lo + ((hi - lo) & ~(int64_t)3) : lo;      // [lo, hi4): whole vectors; [hi4, hi): single words
  const int64_t par = (int64_t)(e & 1u) * world;
  if (in) {
    const int64_t off = (par + d->rank) * d->slot_elems;
    for (int64_t i = lo + 4 * (int64_t)threadIdx.x; i < hi4; i += 4 * AR_THREADS) {
      const float4 v = *reinterpret_cast<const float4*>(in + i);
      for (int r = 0; r < world; ++r) comm_deposit4(d->data[r] + off + i, v);
    }
    for (int64_t i = hi4 + threadIdx.x; i < hi; i += AR_THREADS) {
      const float v = in[i];
      for (int r = 0; r < world; ++r) comm_deposit(d->data[r] + off + i, v);
    }
  }
  uint64_t deadline = 0;
  for (int64_t i = lo + 4 * (int64_t)threadIdx.x; i < hi4; i += 4 * AR_THREADS) {
    float s[4];
    comm_collect_v4<1>(d, par, &i, s, &deadline, status);
    *reinterpret_cast<float4*>(out + i) = make_float4(s[0], s[1], s[2], s[3]);
  }
  for (int64_t i0 = hi4 + threadIdx.x; i0 < hi; i0 += 4 * AR_THREADS) {
    int64_t idx[4];
    float s[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) idx[j] = i0 + (int64_t)j * AR_THREADS < hi ? i0 + (int64_t)j * AR_THREADS : -1;
    comm_collect<4>(d, par, idx, s, &deadline, status);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (idx[j] >= 0) out[idx[j]] = s[j];
  }
  comm_finish(d, e);
}

// One CTA per row of H elements (H a multiple of 8, at most AR_VCHUNKS * AR_THREADS * 8): delta = sum over ranks of
// the deposited rows; x <- T(x + delta) (the residual stream, stored in T); normed = T(x * rsqrt(mean(x^2) + eps) *
// gamma).  Element ownership (chunks of 8 consecutive elements per thread), arithmetic, rounding and the order of
// the sum of squares are those of add_rmsnorm_vec_kernel (glue.cu), so the two agree bit for bit.  `in` as above.
constexpr int AR_VCHUNKS = 2;
template <typename T>
__global__ void __launch_bounds__(AR_THREADS) allreduce_add_rmsnorm_kernel(const CommDev* __restrict__ d,
                                                                           const float* __restrict__ in, T* __restrict__ x,
                                                                           const float* __restrict__ gamma,
                                                                           T* __restrict__ normed, int64_t H, float eps,
                                                                           int* status) {
  pdl_launch_dependents();
  pdl_wait();
  if (comm_failed(d, status)) return;
  const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(d->state);
  const int world = d->world;
  const int64_t row0 = (int64_t)blockIdx.x * H;
  const int64_t par = (int64_t)(e & 1u) * world;
  if (in) {       // `in` is 16-byte aligned (checked by the host) and rows are multiples of 8 elements
    const int64_t off = (par + d->rank) * d->slot_elems + row0;
    for (int64_t i = 4 * (int64_t)threadIdx.x; i < H; i += 4 * AR_THREADS) {
      const float4 v = *reinterpret_cast<const float4*>(in + row0 + i);
      for (int r = 0; r < world; ++r) comm_deposit4(d->data[r] + off + i, v);
    }
  }
  T* xr = x + row0;
  T* orow = normed + row0;
  float v[AR_VCHUNKS][8], g[AR_VCHUNKS][8];
  float ss = 0.0f;
  uint64_t deadline = 0;
#pragma unroll
  for (int c = 0; c < AR_VCHUNKS; ++c) {
    const int64_t i0 = ((int64_t)threadIdx.x + c * AR_THREADS) * 8;
    if (i0 < H) {
      const int64_t idx[2] = {row0 + i0, row0 + i0 + 4};
      float s[8];
      load8<T>(xr + i0, v[c]);
      load8<float>(gamma + i0, g[c]);
      comm_collect_v4<2>(d, par, idx, s, &deadline, status);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        v[c][i] = to_float<T>(from_float<T>(v[c][i] + s[i]));
        ss += v[c][i] * v[c][i];
      }
      store8<T>(xr + i0, v[c]);
    }
  }
  __shared__ float red[AR_THREADS / 32];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.0f;
#pragma unroll
  for (int i = 0; i < AR_THREADS / 32; ++i) tot += red[i];
  const float inv = rsqrtf(tot / (float)H + eps);
#pragma unroll
  for (int c = 0; c < AR_VCHUNKS; ++c) {
    const int64_t i0 = ((int64_t)threadIdx.x + c * AR_THREADS) * 8;
    if (i0 < H) {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = v[c][i] * inv * g[c][i];
      store8<T>(orow + i0, o);
    }
  }
  comm_finish(d, e);
}

// Vocabulary-sharded greedy head: every rank holds the (maximum, global id) of its vocabulary slice per row; the
// pairs travel through the receive slots (word 2m = value, word 2m+1 = id bits) and every rank picks the largest
// value, ties to the lower id -- one launch, one thread per row.
__global__ void __launch_bounds__(AR_THREADS) argmax_exchange_kernel(const CommDev* __restrict__ d, const float* __restrict__ vmax,
                                                                     const int32_t* __restrict__ imax, int32_t id_offset,
                                                                     int64_t M, int32_t* __restrict__ ids32,
                                                                     int64_t* __restrict__ ids64, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  if (comm_failed(d, status)) return;
  const uint32_t e = *reinterpret_cast<const volatile uint32_t*>(d->state);
  const int world = d->world;
  const int64_t par = (int64_t)(e & 1u) * world;
  const int64_t off = (par + d->rank) * d->slot_elems;
  uint64_t deadline = 0;
  for (int64_t m = blockIdx.x * (int64_t)AR_THREADS + threadIdx.x; m < M; m += (int64_t)gridDim.x * AR_THREADS) {
    const float v = vmax[m];
    const uint32_t id = (uint32_t)(imax[m] + id_offset);          // < 2^31: never the "empty" pattern
    for (int r = 0; r < world; ++r) {
      comm_deposit(d->data[r] + off + 2 * m, v);
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(d->data[r] + off + 2 * m + 1), "r"(id) : "memory");
    }
    float best = -INFINITY;
    uint32_t bid = 0x7fffffffu;
    float* mine = d->data[d->rank];
    for (int r = 0; r < world; ++r) {
      float* slot = mine + (par + r) * d->slot_elems + 2 * m;
      uint32_t a = ld_sys_u32(slot), b = ld_sys_u32(slot + 1);
      if (a == COMM_EMPTY) a = comm_wait_value(d, slot, &deadline, status);
      if (b == COMM_EMPTY) b = comm_wait_value(d, slot + 1, &deadline, status);
      st_empty(slot);
      st_empty(slot + 1);
      const float rv = __uint_as_float(a);
      if (rv > best || (rv == best && b < bid)) { best = rv; bid = b; }
    }
    if (ids32) ids32[m] = (int32_t)bid;
    if (ids64) ids64[m] = (int64_t)bid;
  }
  comm_finish(d, e);
}

static int comm_ready() {
  if (device_id() < 0) return fail(BQ_ERR_STATE, "bq_init() has not been called");
  return BQ_OK;
}

static int upload_desc(Comm* c) {
  CommDev h = {};
  for (int r = 0; r < c->world; ++r) {
    uint8_t* base = r == c->rank ? c->local : static_cast<uint8_t*>(c->peer[r]);
    if (!base) return fail(BQ_ERR_STATE, "communicator is not connected to every rank");
    h.data[r] = reinterpret_cast<float*>(base + COMM_HEADER_BYTES);
  }
  h.state = reinterpret_cast<uint32_t*>(c->local);
  h.slot_elems = c->slot_elems;
  h.wait_ns = (uint64_t)c->wait_ms * 1000000ull;
  h.rank = c->rank;
  h.world = c->world;
  BQ_CUDA(cudaMemcpy(c->dev, &h, sizeof(h), cudaMemcpyHostToDevice));
  return BQ_OK;
}

// header {epoch = 1, finished-CTA counter = 0, failed = 0}, every slot word empty
static cudaError_t comm_fill_local(Comm* c) {
  cudaError_t e = cudaMemset(c->local, 0, COMM_HEADER_BYTES);
  if (e != cudaSuccess) return e;
  comm_fill_empty_kernel<<<256, 256>>>(reinterpret_cast<uint32_t*>(c->local + COMM_HEADER_BYTES),
                                       (int64_t)((c->bytes - COMM_HEADER_BYTES) / 4));
  if ((e = cudaGetLastError()) != cudaSuccess) return e;
  const uint32_t one = 1;
  if ((e = cudaMemcpy(c->local, &one, sizeof(one), cudaMemcpyHostToDevice)) != cudaSuccess) return e;
  return cudaDeviceSynchronize();
}

static int comm_usable(Comm* c) {
  if (!c->connected) return fail(BQ_ERR_STATE, "communicator is not connected");
  if (c->failed)
    return fail(BQ_ERR_STATE, "a wait on this communicator timed out: call bq_comm_reset on every rank (or destroy it)");
  return BQ_OK;
}

}  // namespace bq

using namespace bq;

extern "C" {

int bq_comm_create(int rank, int world, int64_t max_elems, bq_comm_t* out) {
  int rc = comm_ready();
  if (rc) return rc;
  if (!out) return fail(BQ_ERR_ARG, "null pointer");
  if (world < 1 || world > COMM_MAX_WORLD || rank < 0 || rank >= world) return fail(BQ_ERR_ARG, "bad rank / world (world <= 8)");
  if (max_elems <= 0 || max_elems > ((int64_t)1 << 28)) return fail(BQ_ERR_ARG, "max_elems out of range");
  Comm* c = new Comm();
  c->magic = COMM_MAGIC;
  c->rank = rank; c->world = world;
  c->slot_elems = (max_elems + 63) / 64 * 64;
  c->bytes = comm_total_bytes(world, c->slot_elems);
  c->local = nullptr; c->dev = nullptr; c->connected = false; c->loopback = false; c->failed = false;
  c->wait_ms = COMM_WAIT_MS_DEFAULT;
  for (int r = 0; r < COMM_MAX_WORLD; ++r) c->peer[r] = nullptr;
  cudaError_t e = cudaMalloc((void**)&c->local, c->bytes);
  if (e == cudaSuccess) e = cudaMalloc((void**)&c->dev, sizeof(CommDev));
  if (e == cudaSuccess) e = comm_fill_local(c);
  if (e != cudaSuccess) {
    if (c->local) cudaFree(c->local);
    if (c->dev) cudaFree(c->dev);
    delete c;
    return fail_cuda(e, "cudaMalloc(communicator)");
  }
  if (world == 1) {
    rc = upload_desc(c);
    if (rc) { cudaFree(c->local); cudaFree(c->dev); delete c; return rc; }
    c->connected = true;
  }
  {
    std::lock_guard<std::mutex> lk(c_mu);
    c_comms.insert(c);
  }
  *out = static_cast<bq_comm_t>(reinterpret_cast<uintptr_t>(c));
  return BQ_OK;
}

int bq_comm_handle(bq_comm_t comm, void* out64) {
  Comm* c = get_comm(comm);
  if (!c) return BQ_ERR_HANDLE;
  if (!out64) return fail(BQ_ERR_ARG, "null pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == BQ_COMM_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  BQ_CUDA(cudaIpcGetMemHandle(&h, c->local));
  memcpy(out64, &h, sizeof(h));
  return BQ_OK;
}

int bq_comm_connect(bq_comm_t comm, const void* handles) {
  Comm* c = get_comm(comm);
  if (!c) return BQ_ERR_HANDLE;
  if (!handles) return fail(BQ_ERR_ARG, "null pointer");
  if (c->connected) return fail(BQ_ERR_STATE, "communicator is already connected");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)r * BQ_COMM_HANDLE_BYTES, sizeof(h));
    BQ_CUDA(cudaIpcOpenMemHandle(&c->peer[r], h, cudaIpcMemLazyEnablePeerAccess));
  }
  int rc = upload_desc(c);
  if (rc) return rc;
  c->connected = true;
  return BQ_OK;
}

int bq_comm_connect_loopback(bq_comm_t comm) {
  Comm* c = get_comm(comm);
  if (!c) return BQ_ERR_HANDLE;
  if (c->connected) return fail(BQ_ERR_STATE, "communicator is already connected");
  for (int r = 0; r < c->world; ++r) {
    if (r == c->rank) continue;
    BQ_CUDA(cudaMalloc(&c->peer[r], c->bytes));
    BQ_CUDA(cudaMemset(c->peer[r], 0, c->bytes));      // stand-in for a rank that never deposits
  }
  c->loopback = true;
  int rc = upload_desc(c);
  if (rc) return rc;
  c->connected = true;
  return BQ_OK;
}

int bq_comm_set_timeout_ms(bq_comm_t comm, int ms) {
  Comm* c = get_comm(comm);
  if (!c) return BQ_ERR_HANDLE;
  if (ms < 1 || ms > 60000) return fail(BQ_ERR_ARG, "time limit must be 1..60000 ms");
  c->wait_ms = ms;
  if (c->connected) {
    BQ_CUDA(cudaDeviceSynchronize());
    return upload_desc(c);
  }
  return BQ_OK;
}

int bq_comm_reset(bq_comm_t comm) {
  Comm* c = get_comm(comm);
  if (!c) return BQ_ERR_HANDLE;
  if (!c->connected) return fail(BQ_ERR_STATE, "communicator is not connected");
  BQ_CUDA(cudaDeviceSynchronize());
  cudaError_t e = comm_fill_local(c);
  if (e != cudaSuccess) return fail_cuda(e, "bq_comm_reset");
  c->failed = false;
  return BQ_OK;
}

int bq_comm_destroy(bq_comm_t comm) {
  Comm* c = get_comm(comm);
  if (!c) return BQ_ERR_HANDLE;
  {
    std::lock_guard<std::mutex> lk(c_mu);
    c_comms.erase(c);
  }
  cudaDeviceSynchronize();
  for (int r = 0; r < c->world; ++r)
    if (c->peer[r]) {
      if (c->loopback) cudaFree(c->peer[r]);
      else cudaIpcCloseMemHandle(c->peer[r]);
    }
  cudaFree(c->local);
  cudaFree(c->dev);
  c->magic = 0;
  delete c;
  return BQ_OK;
}

int bq_allreduce(bq_comm_t comm, const float* in, float* out, int64_t count, void* stream) {
  Comm* c = get_comm(comm);
  if (!c) return BQ_ERR_HANDLE;
  int rc = comm_usable(c);
  if (rc) return rc;
  if (count < 0 || count > c->slot_elems) return fail(BQ_ERR_ARG, "count exceeds the communicator's max_elems");
  if (count == 0) return BQ_OK;
  if (!out) return fail(BQ_ERR_ARG, "null pointer");
  int64_t chunk = (count + 4 * sm_count() - 1) / (4 * sm_count());
  if (chunk < 1024) chunk = 1024;
  chunk = (chunk + 3) & ~(int64_t)3;
  const int64_t grid = (count + chunk - 1) / chunk;
  const int vec = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
  BQ_CUDA(launch_chain(allreduce_sum_kernel, dim3((unsigned)grid), dim3(AR_THREADS), 0, (cudaStream_t)stream, 1,
                       (const CommDev*)c->dev, in, out, count, chunk, vec, status_word()));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

int bq_allreduce_add_rmsnorm(bq_comm_t comm, const float* in, void* x, const float* gamma, void* normed, int64_t rows,
                             int64_t H, float eps, int dtype, void* stream) {
  Comm* c = get_comm(comm);
  if (!c) return BQ_ERR_HANDLE;
  int rc = comm_usable(c);
  if (rc) return rc;
  if (dtype != BQ_DT_F32 && dtype != BQ_DT_BF16) return fail(BQ_ERR_ARG, "dtype must be BQ_DT_F32 or BQ_DT_BF16");
  if (rows < 0 || H <= 0) return fail(BQ_ERR_ARG, "bad sizes");
  if (H > (int64_t)AR_VCHUNKS * AR_THREADS * 8 || H % 8 != 0 ||
      ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(gamma) | reinterpret_cast<uintptr_t>(normed) |
        reinterpret_cast<uintptr_t>(in)) & 15) != 0)
    return fail(BQ_ERR_UNSUPPORTED, "rows must be a multiple of 8 and at most 4096 elements, pointers 16-byte aligned");
  if (rows * H > c->slot_elems) return fail(BQ_ERR_ARG, "rows * H exceeds the communicator's max_elems");
  if (rows == 0) return BQ_OK;
  if (!x || !gamma || !normed) return fail(BQ_ERR_ARG, "null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == BQ_DT_F32)
    BQ_CUDA(launch_chain(allreduce_add_rmsnorm_kernel<float>, dim3((unsigned)rows), dim3(AR_THREADS), 0, s, 1,
                         (const CommDev*)c->dev, in, (float*)x, gamma, (float*)normed, H, eps, status_word()));
  else
    BQ_CUDA(launch_chain(allreduce_add_rmsnorm_kernel<__nv_bfloat16>, dim3((unsigned)rows), dim3(AR_THREADS), 0, s, 1,
                         (const CommDev*)c->dev, in, (__nv_bfloat16*)x, gamma, (__nv_bfloat16*)normed, H, eps, status_word()));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

int bq_qlinear_push(bq_weight_t weight, const void* x, int x_dtype, int64_t M, bq_comm_t comm, void* stream) {
  Comm* c = get_comm(comm);
  if (!c) return BQ_ERR_HANDLE;
  Weight* w = get_weight(weight);
  if (!w) return BQ_ERR_HANDLE;
  int rc = comm_usable(c);
  if (rc) return rc;
  if (x_dtype != BQ_DT_F32 && x_dtype != BQ_DT_BF16) return fail(BQ_ERR_ARG, "x dtype must be BQ_DT_F32 or BQ_DT_BF16");
  if (M <= 0 || !x) return fail(BQ_ERR_ARG, "bad arguments");
  if (M * w->N > c->slot_elems) return fail(BQ_ERR_ARG, "M * N exceeds the communicator's max_elems");
  if (!gemv_mma_supported(w->fmt, w->N, w->K, x_dtype, M))
    return fail(BQ_ERR_UNSUPPORTED, "only decode-sized calls (the tensor-core GEMV's shapes) can deposit directly");
  set_last_path(BQ_PATH_MMA);
  return launch_qlinear_mma_push(w->codes, w->scales, w->fmt, w->N, w->K, x, x_dtype, M, c->dev, (cudaStream_t)stream);
}

int bq_lm_head_sharded(bq_weight_t weight, const void* x, int x_dtype, int64_t M, int64_t vocab_offset, bq_comm_t comm,
                       int32_t* ids_out, int64_t* ids64_out, void* stream) {
  Comm* c = get_comm(comm);
  if (!c) return BQ_ERR_HANDLE;
  int rc = comm_usable(c);
  if (rc) return rc;
  if (M <= 0 || 2 * M > c->slot_elems) return fail(BQ_ERR_ARG, "2 * M exceeds the communicator's max_elems");
  if (vocab_offset < 0 || vocab_offset > 0x3fffffff) return fail(BQ_ERR_ARG, "vocab_offset out of range");
  if (!ids_out && !ids64_out) return fail(BQ_ERR_ARG, "no output");
  cudaStream_t s = (cudaStream_t)stream;
  static Scratch pairs;     // local (argmax id, maximum) per row
  if ((rc = scratch_ensure(&pairs, (size_t)M * 8 + 64, s, "bq_lm_head_sharded"))) return rc;
  int32_t* imax = (int32_t*)pairs.ptr;
  float* vmax = (float*)pairs.ptr + M;
  if ((rc = lm_head_local(weight, x, x_dtype, M, imax, vmax, s))) return rc;
  const int64_t grid = (M + AR_THREADS - 1) / AR_THREADS;
  BQ_CUDA(launch_chain(argmax_exchange_kernel, dim3((unsigned)(grid > 64 ? 64 : grid)), dim3(AR_THREADS), 0, s, 1,
                       (const CommDev*)c->dev, (const float*)vmax, (const int32_t*)imax, (int32_t)vocab_offset, M, ids_out,
                       ids64_out, status_word()));
  count_launch();
  BQ_CUDA(cudaGetLastError());
  return BQ_OK;
}

}  // extern "C"
