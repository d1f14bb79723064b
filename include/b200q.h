/*
 * b200q.h — C ABI of libb200q.so: block-quantized (group-32) weight matmuls on NVIDIA B200.
 *
 * Reference interface replaced: NONE EXISTS.  The reference checkout has no quantized
 * linear / expert-matmul / lm_head code and no FFI for one (its README, lines 1-9, lists
 * only unrelated projects; the nearest things to a plugin interface are the emulator
 * callbacks in m6502/m6502.h:20-23 and the IFileIO vtable in m++/mpp.h:20-25, neither of
 * which concerns this path).  Each entry point below therefore cites the sentence of the
 * written specification it implements instead of a reference file:line.
 *
 * Conventions
 *   - every function returns 0 (BQ_OK) or a negative BQ_ERR_* code; bq_last_error() returns
 *     a thread-local message for the last failing call on the calling thread;
 *   - no C++ exception crosses this boundary; argument errors are found on the host before
 *     anything is launched;
 *   - "device pointer" arguments are plain CUDA device addresses on the device selected by
 *     bq_init(); `stream` is a cudaStream_t passed as void* (NULL = default stream);
 *   - activations and outputs are row-major: x[M,K], y[M,N];
 *   - the host layout of a packed weight is the interface layout:
 *       Q8: codes int8[N,K],      scales fp16[N,K/32]
 *       Q4: codes uint8[N,K/2],   scales fp16[N,K/32]; byte j = element 2j in bits 0-3 and
 *           element 2j+1 in bits 4-7, each stored as (code + 8)
 *     dequantized weight = float(code) * float(scale)   (exact in fp32).
 *   - one process per GPU; a handle may be used from any thread, not concurrently.
 */
#ifndef B200Q_H
#define B200Q_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint64_t bq_weight_t;      /* opaque handle to a packed weight resident in HBM   */
typedef uint64_t bq_moe_t;         /* opaque handle to a set of MoE expert weights        */
typedef uint64_t bq_comm_t;        /* opaque handle to a peer-memory communicator         */
typedef uint64_t bq_ep_t;          /* opaque handle to an expert-parallel exchange object */
#define BQ_COMM_HANDLE_BYTES 64

enum { BQ_FMT_Q8G32 = 0, BQ_FMT_Q4G32 = 1 };
enum { BQ_DT_F32 = 0, BQ_DT_BF16 = 1 };

enum {
  BQ_OK = 0,
  BQ_ERR_ARG = -1,        /* null pointer, bad enum, K % 32 != 0, size out of range ...  */
  BQ_ERR_HANDLE = -2,     /* unknown or destroyed handle                                  */
  BQ_ERR_CUDA = -3,       /* a CUDA runtime call failed (message has the CUDA error)      */
  BQ_ERR_STATE = -4,      /* bq_init() not called, or wrong device                        */
  BQ_ERR_TIMEOUT = -5,    /* a bounded device-side wait expired (status word set)         */
  BQ_ERR_UNSUPPORTED = -6 /* valid request that this build has no kernel for              */
};

/* kernel selection for bq_qlinear_ex (bq_qlinear uses BQ_PATH_AUTO) */
enum { BQ_PATH_AUTO = 0, BQ_PATH_SIMT = 1, BQ_PATH_TENSOR = 2, BQ_PATH_MMA = 3 };

/* ---- library state ------------------------------------------------------------------ */
int bq_init(int device);                 /* select device, create context-wide state      */
const char* bq_last_error(void);
int bq_version(void);
/* Reads and clears the device status word (0 = no anomaly; else a BQ_ERR_* code that a
 * kernel recorded, e.g. BQ_ERR_TIMEOUT from a bounded mbarrier wait).  Synchronises.     */
int bq_status_poll(void);
/* Scratch owned by the library.  Several entry points keep intermediate results in buffers the library
 * allocates on demand (the fp16 copy of the activations and split-K partial tiles of the tensor-core
 * GEMM, the gate|up product of bq_qlinear_gated at large batches, logits of an argmax-only bq_lm_head,
 * partial states of split-position attention, staging of bq_qlinear_host).  Rules:
 *   - a buffer grows when a larger call arrives and the outgrown one is kept, never freed, while the
 *     library is loaded: a CUDA graph captured earlier stays valid;
 *   - a call that would have to grow a buffer while its stream is being captured returns
 *     BQ_ERR_STATE and launches nothing: run one call of the largest size, or bq_reserve, first;
 *   - the buffers are shared by all calls: order calls that use them on the device (one stream, or
 *     events between streams).
 * bq_reserve sizes the matmul scratch once for batches of up to max_rows rows on weights of up to
 * [max_N, max_K]; it must not be called during stream capture.                                      */
int bq_reserve(int64_t max_rows, int64_t max_K, int64_t max_N);

/* ---- packed weights (spec: "packed quantized weights ... int8 or 4-bit codes in groups
 *      of 32 with an fp16 scale per group"; "weight packer/loader layout on device") ---- */
/* codes/scales are HOST pointers in the interface layout, borrowed for the call only.    */
int bq_weight_create(const void* codes, const void* scales_f16, int64_t N, int64_t K,
                     int fmt, bq_weight_t* out);
/* Same, from DEVICE pointers (device-to-device copy; used for large synthetic weights).  */
int bq_weight_create_device(const void* d_codes, const void* d_scales_f16, int64_t N,
                            int64_t K, int fmt, void* stream, bq_weight_t* out);
int bq_weight_destroy(bq_weight_t w);
/* A handle to rows row0 .. row0+nrows-1 of w (e.g. one expert of a stacked [E*F, H] tensor): no copy, the
 * view shares w's memory, which must outlive it.  Every entry point takes a view like any weight.     */
int bq_weight_slice_rows(bq_weight_t w, int64_t row0, int64_t nrows, bq_weight_t* out);
int bq_weight_info(bq_weight_t w, int64_t* N, int64_t* K, int* fmt);
/* Copies the weight back to HOST memory in the interface layout (undoes any device-side
 * re-tiling; used to show the device layout is a pure permutation).                      */
int bq_weight_export(bq_weight_t w, void* codes_out, void* scales_f16_out);

/* ---- dequantize (spec: "bit-exact for code unpacking and dequantized weight values") -- */
/* out: device [N,K] of out_dtype.  F32 is exact; BF16 is round-to-nearest-even of it.    */
int bq_dequant(bq_weight_t w, void* out, int out_dtype, void* stream);
/* out: device int8[N,K] — the unpacked integer codes.                                    */
int bq_unpack_codes(bq_weight_t w, void* out_i8, void* stream);

/* Quantize on the device (spec: "weight packer/loader layout on device"): w is fp32 or bf16 [N,K] in
 * device memory; codes_out / scales_out receive the INTERFACE layout (int8[N,K] or uint8[N,K/2], and
 * fp16[N,K/32]), bit for bit what the host packer computes: scale = fp16(absmax/qmax) (qmax 127 / 7),
 * code = clip(rint(w / f32(scale)), +-qmax), zero-scale groups -> codes 0.  Feed the result to
 * bq_weight_create_device.                                                                          */
int bq_quantize(const void* w, int w_dtype, int64_t N, int64_t K, int fmt, void* codes_out,
                void* scales_out, void* stream);

/* ---- quantized linear / lm_head (spec: "multiplied against bf16/fp32 activations for
 *      every linear, MoE-expert and lm_head projection", fp32 accumulate) --------------- */
/* y[M,N] = x[M,K] . W^T.  x, y: device pointers. x_dtype/y_dtype in {F32,BF16}.          */
int bq_qlinear(bq_weight_t w, const void* x, int x_dtype, int64_t M, void* y, int y_dtype,
               void* stream);
int bq_qlinear_ex(bq_weight_t w, const void* x, int x_dtype, int64_t M, void* y,
                  int y_dtype, int path, void* stream);
/* Same with HOST buffers: copies x in, runs, copies y out, synchronises.                 */
int bq_qlinear_host(bq_weight_t w, const void* x_host, int x_dtype, int64_t M,
                    void* y_host, int y_dtype);
/* Fused gate|up projection with the gated activation applied on the way out.  `w` has 2F rows in
 * 16-row blocks: 8 gate rows followed by the 8 up rows of the same output columns (block b holds
 * columns 8b .. 8b+7; chadslab_b200.ops.interleave_gate_up builds it from the two weights).
 * out[M, F] = act(x . gate^T) * (x . up^T) in the dtype of x; act 0 = gelu (tanh), 1 = silu.
 * Decode-sized calls apply the activation in the GEMV's epilogue (one launch); larger batches run the
 * product into a scratch owned by the library (first call outside stream capture) plus a second kernel. */
int bq_qlinear_gated(bq_weight_t w, const void* x, int x_dtype, int64_t M, void* out, int act,
                     void* stream);
/* lm_head + greedy argmax: logits may be NULL (then only argmax is produced).
 * argmax_out: device int32[M]; ties resolve to the lower vocabulary index.               */
int bq_lm_head(bq_weight_t w, const void* x, int x_dtype, int64_t M, void* logits,
               int logits_dtype, int32_t* argmax_out, void* stream);
/* which kernel family the last bq_qlinear* call on this thread launched (BQ_PATH_*) and
 * how many kernels it launched                                                            */
int bq_last_path(void);
int64_t bq_launch_count(void);           /* kernels launched by this library so far       */

/* ---- decode-step glue between the quantized matmuls (the callers on either side of the path; the
 *      reference has no counterpart).  dtype = storage type of activations / KV cache (F32 or BF16);
 *      arithmetic is fp32.  `pos` is a DEVICE int64: the position being written, so a captured CUDA
 *      graph can be replayed for every token. ------------------------------------------------------ */
/* x[rows,H] += delta[rows,H] (fp32, may be NULL); out = x * rsqrt(mean(x^2) + eps) * weight[H]      */
int bq_add_rmsnorm(void* x, const float* delta, const float* weight, void* out, int64_t rows,
                   int64_t H, float eps, int dtype, void* stream);
/* qkv: fp32 [B, (Hq + 2*Hkv) * D] from a fused q|k|v projection.  Rotate-half RoPE on q and k at
 * position *pos; q -> q_out [B,Hq,D]; k, v -> caches [B,S,Hkv,D] at row *pos.                        */
int bq_rope_kv_append(const float* qkv, const int64_t* pos, void* q_out, void* k_cache, void* v_cache,
                      int64_t B, int Hq, int Hkv, int D, int64_t S, float rope_base, int dtype,
                      void* stream);
/* out[B,Hq,D] = softmax(q . K[0..*pos] / sqrt(D)) . V[0..*pos], grouped-query (Hq % Hkv == 0), D <= 256 */
int bq_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int64_t* pos,
                        void* out, int64_t B, int Hq, int Hkv, int D, int64_t S, int dtype, void* stream);
/* bq_rope_kv_append + bq_decode_attention in one launch: q and the current position's K / V are taken from
 * qkv and rotated inside the attention kernel (same roundings), the caches supply positions < *pos and
 * receive the new rows.  When the positions are split over several CTAs the first call sizes a scratch
 * buffer owned by the library: make it outside stream capture.                                            */
int bq_decode_attention_rope(const float* qkv, void* k_cache, void* v_cache, const int64_t* pos, void* out,
                             int64_t B, int Hq, int Hkv, int D, int64_t S, float rope_base, int dtype,
                             void* stream);
/* gate_up: fp32 [rows, 2F] (gate | up); out[rows,F] = act(gate) * up; act 0 = gelu(tanh), 1 = silu    */
int bq_gated_act(const float* gate_up, void* out, int64_t rows, int64_t F, int act, int dtype,
                 void* stream);

/* ---- MoE (spec: "router top-k, a token permute/gather, a grouped quantized expert GEMM
 *      and a weighted scatter-combine") ------------------------------------------------- */
/* (MoE) Expert ids outside [0, E) are legal input to bq_moe_permute: such assignments are dropped --
 * inv holds -1 for them, the sorted positions behind offsets[E] hold perm = -1, bq_moe_gather writes
 * zero rows there and bq_moe_combine skips them.                                                    */
/* softmax over E router logits (device f32[T,E]) -> top-k ids (int32[T,k], descending
 * probability, ties to the lower expert id) and weights f32[T,k]: the softmax probabilities,
 * rescaled to sum to 1 over the k selected experts when renormalise != 0.
 * Limits: E <= 1024, top_k <= 32.                                                        */
int bq_moe_route(const float* logits, int64_t T, int E, int top_k, int renormalise,
                 int32_t* idx_out, float* w_out, void* stream);
/* Router linear + bq_moe_route in one launch: router is the packed [E, H] router weight, x the token activations
 * (device bf16 [T, H]).  E <= 128 and H a multiple of 128, else BQ_ERR_UNSUPPORTED (use bq_qlinear + bq_moe_route).
 * Logits are computed like every tensor-core matmul of this library (weights rounded once to fp16).        */
int bq_moe_route_linear(bq_weight_t router, const void* x_bf16, int64_t T, int top_k, int renormalise,
                        int32_t* idx_out, float* w_out, void* stream);
/* Stable counting sort of the T*k assignments by expert.  perm int32[T*k]: sorted position
 * p holds flat assignment t*k+slot; inv int32[T*k] (may be NULL): inv[t*k+slot] = p;
 * offsets int32[E+1]: expert e owns positions offsets[e]..offsets[e+1].
 * scratch: device memory of >= bq_moe_permute_scratch_bytes(T,k,E) bytes (per-chunk
 * histograms); contents need not be initialised.  All pointers are device pointers.      */
int64_t bq_moe_permute_scratch_bytes(int64_t T, int top_k, int E);
int bq_moe_permute(const int32_t* idx, int64_t T, int top_k, int E, int32_t* perm,
                   int32_t* inv, int32_t* offsets, void* scratch, void* stream);
/* bq_moe_permute for callers that cannot allocate device memory.  No counterpart in the
 * reference: it exists for hosts that have given all free HBM to a KV-cache / arena they do
 * not control, or that sort tokens inside a section where cudaMalloc (a device-wide
 * synchronisation) is not allowed.  Same arguments and results as bq_moe_permute minus the
 * scratch pointer: the per-chunk histograms live in a fixed 512 KiB array inside the library
 * (held by every GPU that loads it, until the process exits).  Calls no cudaMalloc/cudaFree.
 *   - limit: bq_moe_permute_scratch_bytes(T, top_k, E) <= bq_moe_permute_noalloc_max_bytes()
 *     (any T*top_k when E <= 128; T*top_k <= 65536 when E = 512); larger requests return
 *     BQ_ERR_ARG and launch nothing;
 *   - the first call on a device looks up the array's device address (cudaGetSymbolAddress);
 *     make that first call before any stream capture begins;
 *   - all calls share the one array and it keeps the previous call's contents (nothing in it
 *     needs to start at zero): two calls whose kernels overlap on the GPU — different streams
 *     without an event between them — race on it.                                           */
int64_t bq_moe_permute_noalloc_max_bytes(void);
int bq_moe_permute_noalloc(const int32_t* idx, int64_t T, int top_k, int E, int32_t* perm,
                           int32_t* inv, int32_t* offsets, void* stream);
/* xp[p,:] = x[perm[p] / k, :]  (rows of H elements of `dtype`)                           */
int bq_moe_gather(const void* x, int dtype, int64_t H, const int32_t* perm, int64_t P,
                  int top_k, void* xp, void* stream);
/* Expert weight set: E experts, each gate[F,H], up[F,H], down[H,F]; arrays of E handles.
 * The set takes ownership of nothing: the handles must outlive it.                       */
int bq_moe_create(const bq_weight_t* gate, const bq_weight_t* up, const bq_weight_t* down,
                  int E, bq_moe_t* out);
int bq_moe_destroy(bq_moe_t m);
/* Grouped SwiGLU FFN over the permuted rows: for expert e and rows offsets[e]..offsets[e+1]
 *   h = silu(xp . gate_e^T) * (xp . up_e^T)  (rounded to bf16),  out = h . down_e^T.
 * xp: device bf16[P,H]; out: device f32[P,H]; hbuf: device bf16[P,F] workspace.
 * offsets: DEVICE int32[E+1] (read by the kernel; no host sync).                          */
int bq_moe_experts(bq_moe_t m, const void* xp_bf16, const int32_t* offsets, int64_t P,
                   void* hbuf_bf16, float* out, int path, void* stream);
/* Same with P only a capacity (rows the buffers hold; offsets[E] rows are in use) and rows_hint the
 * number of rows to expect, which picks the token tile; bq_moe_experts uses rows_hint = P.          */
int bq_moe_experts_ex(bq_moe_t m, const void* xp_bf16, const int32_t* offsets, int64_t P,
                      int64_t rows_hint, void* hbuf_bf16, float* out, int path, void* stream);
/* bq_moe_gather + bq_moe_experts_ex in one call: x is the TOKEN activations, device bf16 [T, H]; sorted position p
 * uses row perm[p] / top_k.  At decode sizes (about a dozen rows per expert) the expert kernel reads the token
 * rows through perm itself and xp_work is not touched; otherwise the rows are gathered into xp_work (device bf16
 * [P, H]) first.                                                                                          */
int bq_moe_experts_tokens(bq_moe_t m, const void* x_bf16, const int32_t* perm, int top_k,
                          const int32_t* offsets, int64_t P, int64_t rows_hint, void* xp_work,
                          void* hbuf_bf16, float* out, int path, void* stream);
/* y[t,:] = sum_{slot=0..k-1} w[t,slot] * out[inv[t*k+slot], :] in slot order (deterministic,
 * no atomics).  inv as produced by bq_moe_permute.  y dtype F32 or BF16.                 */
int bq_moe_combine(const float* out, const int32_t* inv, const float* w, int64_t T,
                   int top_k, int64_t H, void* y, int y_dtype, void* stream);

/* ---- tensor-parallel shard boundary: sums over the GPUs of one node through peer memory -----
 * The specification asks for "NCCL all-reduce ... only at those shard boundaries"; the host
 * mirror keeps an NCCL route (torch.distributed) and these entry points are the fused
 * alternative for decode-sized messages: one process per GPU, each owns a buffer of receive
 * slots that every other process maps through CUDA IPC; a sum is plain 4-byte stores into the
 * peers' slots (an empty slot element holds the bits of -0.0f, so a value announces itself: no
 * flags, no fences), a bounded wait for the values and an add in rank order (bit-identical on
 * every rank).  Set-up, identical on every rank:
 *   bq_comm_create(rank, world, max_elems, &c);  bq_comm_handle(c, h64);
 *   -- exchange the 64-byte handles (all-gather over any host channel), rank-major --
 *   bq_comm_connect(c, handles);  -- host barrier before the first call and before destroy --
 * world <= 8; world == 1 needs no connect.  max_elems bounds the fp32 elements of one sum.
 * All ranks must issue the same sequence of summing calls with the same sizes.  A value that
 * does not arrive within the time limit (5 s unless changed) records BQ_ERR_TIMEOUT (see
 * bq_status_poll) and the kernel returns; the results of that call are then undefined and the
 * communicator must be destroyed.  Calls are graph-capturable.  A contribution of -0.0f counts
 * as +0.0f.                                                                               */
int bq_comm_create(int rank, int world, int64_t max_elems, bq_comm_t* out);
int bq_comm_handle(bq_comm_t c, void* out_handle /* BQ_COMM_HANDLE_BYTES */);
int bq_comm_connect(bq_comm_t c, const void* handles /* world x BQ_COMM_HANDLE_BYTES */);
/* Self-test aid: instead of mapping the other ranks, give each a private stand-in buffer in
 * this process.  Nobody answers, so every summing call runs into the bounded wait: this is how
 * the time-out path (BQ_ERR_TIMEOUT from bq_status_poll, context still usable) is exercised
 * on one GPU.                                                                             */
int bq_comm_connect_loopback(bq_comm_t c);
/* Time limit of the flag wait, 1..60000 ms (synchronises the device when already connected). */
int bq_comm_set_timeout_ms(bq_comm_t c, int ms);
int bq_comm_destroy(bq_comm_t c);
/* After a time-out (bq_status_poll returned BQ_ERR_TIMEOUT) every summing call on the communicators of
 * this process returns BQ_ERR_STATE, and kernels already captured in a graph record BQ_ERR_TIMEOUT
 * again without touching the slots: a late value of the abandoned call could otherwise be taken for a
 * later one.  bq_comm_reset empties the slots and restarts the call counter; call it on EVERY rank,
 * with a host barrier before (no rank still inside a call) and after (nobody deposits into a buffer
 * that is about to be refilled).  Synchronises the device.                                          */
int bq_comm_reset(bq_comm_t c);
/* Row-parallel shard of a linear (this rank's K slice): y_partial = x . W^T, fp32, deposited
 * directly in every rank's receive slot by the GEMV's epilogue (no local y).  Decode-sized
 * calls only (the shapes of BQ_PATH_MMA), else BQ_ERR_UNSUPPORTED and nothing is launched:
 * run bq_qlinear and pass its y as `in` below.  Must be followed on the same stream by
 * exactly one of the two summing calls with in == NULL.                                   */
int bq_qlinear_push(bq_weight_t w, const void* x, int x_dtype, int64_t M, bq_comm_t c,
                    void* stream);
/* out[i] = sum over ranks of in_r[i], i < count (fp32).  in == NULL: sum what the preceding
 * bq_qlinear_push deposited (count = M * N).                                              */
int bq_allreduce(bq_comm_t c, const float* in, float* out, int64_t count, void* stream);
/* bq_add_rmsnorm with delta = the sum over ranks: x += sum; normed = rmsnorm(x) * weight.
 * H <= 4096 and a multiple of 8, 16-byte aligned pointers (else BQ_ERR_UNSUPPORTED: use
 * bq_allreduce + bq_add_rmsnorm).  in as for bq_allreduce.                                */
int bq_allreduce_add_rmsnorm(bq_comm_t c, const float* in, void* x, const float* weight,
                             void* normed, int64_t rows, int64_t H, float eps, int dtype,
                             void* stream);

/* Vocabulary-sharded greedy head (spec: "lm_head" column-sharded over the GPUs): w holds this rank's
 * vocabulary slice, whose first row is token id vocab_offset.  One call computes the local logits
 * (library scratch), the local (maximum, id) per row, exchanges the pairs through the communicator's
 * receive slots and leaves the global arg-max id (ties -> lower id, identical on every rank) in ids_out
 * (device int32[M], may be NULL) and/or ids64_out (device int64[M], may be NULL).  2*M <= max_elems.
 * Counts as one summing call of the communicator; graph-capturable.                                 */
int bq_lm_head_sharded(bq_weight_t w, const void* x, int x_dtype, int64_t M, int64_t vocab_offset,
                       bq_comm_t c, int32_t* ids_out, int64_t* ids64_out, void* stream);

/* ---- expert-parallel shard boundary (spec: "experts shard expert-parallel across the 8 GPUs ...
 *      all-to-all over NVLink only at those shard boundaries"): the two all-to-alls around the grouped
 *      experts as plain stores into the owning rank's memory.  The reference has no counterpart.
 * Ranks r = 0..world-1 each own experts r*E/world .. (r+1)*E/world - 1; tokens stay on the rank that
 * holds them.  Set-up mirrors the communicator above (create, exchange 64-byte handles, connect, host
 * barrier; world == 1 needs no connect).  max_send_rows bounds T*top_k of one call on this rank,
 * max_recv_rows the rows this rank's experts may receive in one call (safe value: the sum of T*top_k
 * over all ranks); a row that would not fit records BQ_ERR_ARG in the status word and is skipped.
 * Per MoE layer, on every rank, in this order on one stream (all ranks must make the same calls):
 *   bq_moe_route, bq_moe_permute (by GLOBAL expert id, E experts)            -- local
 *   bq_ep_dispatch    rows travel to their owners; returns once the wait for every source is queued
 *   bq_ep_recv_view   -> receive buffer (bf16 [max_recv_rows, H], rows grouped by local expert, sources
 *                        in rank order) and the DEVICE int32[E/world + 1] row ranges of the local experts
 *   bq_moe_experts_ex(local expert set, receive buffer, those row ranges, P = max_recv_rows, ...)
 *   bq_ep_combine     output rows travel back (fp32), y[t] = sum_slot w * row in slot order: bit-identical
 *                     to bq_moe_combine on one GPU given the same expert outputs.
 * Waits are bounded (5 s unless changed): on expiry BQ_ERR_TIMEOUT is recorded, the object stays failed
 * and must be destroyed.  All calls are graph-capturable; the call counter advances on the device.     */
int bq_ep_create(int rank, int world, int n_experts, int64_t hidden, int64_t max_send_rows,
                 int64_t max_recv_rows, bq_ep_t* out);
int bq_ep_handle(bq_ep_t ep, void* out_handle /* BQ_COMM_HANDLE_BYTES */);
int bq_ep_connect(bq_ep_t ep, const void* handles /* world x BQ_COMM_HANDLE_BYTES */);
int bq_ep_set_timeout_ms(bq_ep_t ep, int ms);
int bq_ep_destroy(bq_ep_t ep);
/* x: device bf16 [T, H]; idx: device int32 [T, top_k] (global expert ids); perm, offsets: from
 * bq_moe_permute(idx, T, top_k, E).                                                                 */
int bq_ep_dispatch(bq_ep_t ep, const void* x_bf16, const int32_t* idx, const int32_t* perm,
                   const int32_t* offsets, int64_t T, int top_k, void* stream);
/* Self-test aid: the row bookkeeping every rank derives from the exchanged counts, run for a GIVEN count matrix
 * (device int32 [world][E]: rows source s routes to expert x) as rank `rank` of `world`, nothing exchanged.
 * tables_out (device int32, E + (E/world + 1) + (E/world*world + 1) + E/world*world entries): dest_base[E],
 * local row ranges [E/world + 1], first received row of every (local expert, source) block [+1 = rows
 * received], position of each block's first row in its source's sorted order.  Synchronises the stream. */
int bq_ep_layout_selftest(const int32_t* counts, int rank, int world, int n_experts, int32_t* tables_out,
                          void* stream);
int bq_ep_recv_view(bq_ep_t ep, void** xrecv_bf16, const int32_t** local_offsets, int64_t* max_rows);
/* out_rows: device f32 [max_recv_rows, H], the expert outputs in receive order; inv, w: as for
 * bq_moe_combine (inv from this rank's bq_moe_permute).                                             */
int bq_ep_combine(bq_ep_t ep, const float* out_rows, const int32_t* inv, const float* w, int64_t T,
                  int top_k, void* y, int y_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200Q_H */
