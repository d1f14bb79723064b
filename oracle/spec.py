"""CPU oracle for the block-quantized matmul path (TEST INFRASTRUCTURE, not product).

Status of this oracle: PARITY UNPINNED.  The runtimes that the task statement
names as the reference for this path (numpy-gemma / reclank) are not part of the
reference checkout, which holds no quantized-matmul code, test or golden vector
(its README, lines 1-9, lists only unrelated hobby projects).  Everything below is
therefore a self-authored numpy restatement of the written specification:
"int8 or 4-bit codes in groups of 32 along K with an fp16 (absmax) scale per
group, dequantized and multiplied against bf16/fp32 activations with fp32
accumulate".  Where that text leaves a choice open the choice is a module-level
constant so it can be re-pinned in one line if the real sources appear.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module.  The product path (chadslab_b200) never does.

All functions are literal: dequantise to fp32, `np.matmul`, nothing clever.
"""
from __future__ import annotations

import numpy as np

try:  # bf16 helper type; only needed for bf16 activations / bf16 tiles
    import ml_dtypes

    bfloat16 = ml_dtypes.bfloat16
except Exception:  # pragma: no cover
    bfloat16 = None

GROUP = 32

FMT_Q8 = 0  # symmetric int8, group 32 along K, fp16 scale
FMT_Q4 = 1  # symmetric 4-bit, group 32 along K, fp16 scale, nibble = code + 8

# ---- open choices (the specification is silent; see oracle/SPEC.md) -----------------
Q8_QMAX = 127          # scale = fp16(absmax / 127), codes clipped to [-127, 127]
Q4_QMAX = 7            # scale = fp16(absmax / 7),   codes clipped to [-7, 7]
Q4_ZERO = 8            # stored nibble = code + 8  (so 1..15; 0 never produced, decodes to -8)
Q4_LOW_NIBBLE_FIRST = True   # byte j: element 2j in bits 0-3, element 2j+1 in bits 4-7
TOPK_RENORMALISE = True      # top-k router weights are rescaled to sum to 1
FP16_MAX = np.float32(65504.0)


def _check_k(K: int) -> None:
    if K <= 0 or K % GROUP != 0:
        raise ValueError(f"K={K} must be a positive multiple of {GROUP}")


def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round fp32 values to the nearest bf16 (ties to even); result stays fp32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) >> 16) << 16
    out = r.astype(np.uint32).view(np.float32)
    nan = np.isnan(a)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out.reshape(a.shape)


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> uint16 bf16 bit patterns (round to nearest even)."""
    return (bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ---------------------------------------------------------------------------------------
# S1 / S2  quantisers
# ---------------------------------------------------------------------------------------
def _group_scales(W: np.ndarray, qmax: int):
    W = np.ascontiguousarray(W, dtype=np.float32)
    if W.ndim != 2:
        raise ValueError("W must be [N, K]")
    N, K = W.shape
    _check_k(K)
    g = W.reshape(N, K // GROUP, GROUP)
    absmax = np.abs(g).max(axis=-1)
    s = np.minimum(absmax / np.float32(qmax), FP16_MAX).astype(np.float16)
    return g, s


def _codes_from(g: np.ndarray, s16: np.ndarray, qmax: int) -> np.ndarray:
    s32 = s16.astype(np.float32)
    zero = s32 == 0
    safe = np.where(zero, np.float32(1), s32)
    q = np.rint(g / safe[..., None])           # round half to even, divide by the fp16-rounded scale
    q = np.clip(q, -qmax, qmax)
    q[zero] = 0                                 # all-zero (or underflowed) group -> codes 0
    return q.astype(np.int8)


def quantize_q8_g32(W: np.ndarray):
    """W f32[N,K] -> (codes int8[N,K], scales f16[N,K/32]).  Symmetric absmax, group 32 along K."""
    g, s = _group_scales(W, Q8_QMAX)
    codes = _codes_from(g, s, Q8_QMAX).reshape(W.shape)
    return codes, s


def pack_q4(codes: np.ndarray) -> np.ndarray:
    """int8 codes in [-8,7], shape [N,K] -> uint8 [N,K/2]."""
    codes = np.asarray(codes)
    if codes.min(initial=0) < -8 or codes.max(initial=0) > 7:
        raise ValueError("4-bit codes must lie in [-8, 7]")
    nib = (codes.astype(np.int16) + Q4_ZERO).astype(np.uint8)
    a, b = nib[..., 0::2], nib[..., 1::2]
    if not Q4_LOW_NIBBLE_FIRST:
        a, b = b, a
    return (a | (b << 4)).astype(np.uint8)


def unpack_q4(packed: np.ndarray) -> np.ndarray:
    """uint8 [N,K/2] -> int8 codes [N,K] in [-8,7]."""
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    lo = (packed & 0x0F).astype(np.int8) - Q4_ZERO
    hi = (packed >> 4).astype(np.int8) - Q4_ZERO
    if not Q4_LOW_NIBBLE_FIRST:
        lo, hi = hi, lo
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.int8)
    out[..., 0::2] = lo
    out[..., 1::2] = hi
    return out


def quantize_q4_g32(W: np.ndarray):
    """W f32[N,K] -> (packed uint8[N,K/2], scales f16[N,K/32])."""
    g, s = _group_scales(W, Q4_QMAX)
    codes = _codes_from(g, s, Q4_QMAX).reshape(W.shape)
    return pack_q4(codes), s


def quantize(W: np.ndarray, fmt: int):
    if fmt == FMT_Q8:
        return quantize_q8_g32(W)
    if fmt == FMT_Q4:
        return quantize_q4_g32(W)
    raise ValueError(f"unknown format {fmt}")


# ---------------------------------------------------------------------------------------
# S3  unpack / dequantise  (bit-exact targets)
# ---------------------------------------------------------------------------------------
def codes_of(codes_or_packed: np.ndarray, fmt: int) -> np.ndarray:
    if fmt == FMT_Q8:
        return np.ascontiguousarray(codes_or_packed, dtype=np.int8)
    if fmt == FMT_Q4:
        return unpack_q4(codes_or_packed)
    raise ValueError(f"unknown format {fmt}")


def dequantize(codes_or_packed: np.ndarray, scales: np.ndarray, fmt: int) -> np.ndarray:
    """-> f32[N,K] = f32(code) * f32(scale).  The product of an <=8-bit integer and an
    fp16 value is exact in fp32, so this defines the weights bit for bit."""
    c = codes_of(codes_or_packed, fmt)
    N, K = c.shape
    _check_k(K)
    s = np.ascontiguousarray(scales, dtype=np.float16)
    if s.shape != (N, K // GROUP):
        raise ValueError(f"scales shape {s.shape} != {(N, K // GROUP)}")
    w = c.reshape(N, K // GROUP, GROUP).astype(np.float32) * s.astype(np.float32)[..., None]
    return w.reshape(N, K)


def dequantize_bf16(codes_or_packed, scales, fmt) -> np.ndarray:
    """bf16-rounded weight values (as fp32) used by the tensor-core tile path."""
    return bf16_round(dequantize(codes_or_packed, scales, fmt))


# ---------------------------------------------------------------------------------------
# S5 / S6  quantized linear and lm_head
# ---------------------------------------------------------------------------------------
def qlinear(x: np.ndarray, codes_or_packed, scales, fmt: int, *, f64: bool = False) -> np.ndarray:
    """y[M,N] = x[M,K] . dequant(W)[N,K]^T with fp32 accumulate (f64=True: float64 tie-breaker)."""
    w = dequantize(codes_or_packed, scales, fmt)
    x = np.asarray(x)
    x32 = x.astype(np.float32)
    if x32.ndim == 1:
        x32 = x32[None, :]
    if x32.shape[-1] != w.shape[1]:
        raise ValueError(f"x K={x32.shape[-1]} != weight K={w.shape[1]}")
    if f64:
        return x32.astype(np.float64) @ w.astype(np.float64).T
    return x32 @ w.T


def lm_head(x, codes_or_packed, scales, fmt, *, f64: bool = False):
    logits = qlinear(x, codes_or_packed, scales, fmt, f64=f64)
    return logits, np.argmax(logits, axis=-1).astype(np.int32)


# ---------------------------------------------------------------------------------------
# S7-S9  MoE: route, permute, experts, combine
# ---------------------------------------------------------------------------------------
def softmax(a: np.ndarray) -> np.ndarray:
    a = np.asarray(a, dtype=np.float32)
    m = a.max(axis=-1, keepdims=True)
    e = np.exp(a - m)
    return e / e.sum(axis=-1, keepdims=True)


def moe_route_from_logits(logits: np.ndarray, top_k: int):
    """softmax over experts, top-k (ties -> lower expert index), optional renormalise.
    -> (idx int32[T,k] in descending-probability order, w f32[T,k])."""
    p = softmax(logits)
    E = p.shape[-1]
    # stable argsort of -p keeps the lower index first among equal probabilities
    order = np.argsort(-p, axis=-1, kind="stable")[:, :top_k]
    w = np.take_along_axis(p, order, axis=-1)
    if TOPK_RENORMALISE:
        w = w / w.sum(axis=-1, keepdims=True)
    assert order.max(initial=0) < E
    return order.astype(np.int32), w.astype(np.float32)


def moe_route(x, router_codes, router_scales, fmt, top_k):
    return moe_route_from_logits(qlinear(x, router_codes, router_scales, fmt), top_k)


def moe_permute(idx: np.ndarray, n_experts: int):
    """Sort the T*k (token, slot) assignments by expert (stable: token-major, then slot).
    -> (perm int32[T*k] : position p holds flat assignment perm[p] = t*k + slot,
        offsets int32[E+1] : expert e owns positions offsets[e]:offsets[e+1])."""
    flat = np.asarray(idx, dtype=np.int64).reshape(-1)
    perm = np.argsort(flat, kind="stable").astype(np.int32)
    counts = np.bincount(flat, minlength=n_experts)
    offsets = np.zeros(n_experts + 1, dtype=np.int32)
    offsets[1:] = np.cumsum(counts)
    return perm, offsets


def silu(a):
    a = np.asarray(a, dtype=np.float32)
    return a / (np.float32(1) + np.exp(-a))


def gelu_tanh(a):
    a = np.asarray(a, dtype=np.float32)
    c = np.float32(0.7978845608028654)
    return np.float32(0.5) * a * (np.float32(1) + np.tanh(c * (a + np.float32(0.044715) * a * a * a)))


def moe_experts(xp: np.ndarray, offsets: np.ndarray, gate, up, down, fmt: int, *, act_bf16: bool = True):
    """Grouped SwiGLU FFN.  gate/up/down are lists (one per expert) of (codes, scales).
    xp f32[P,H] holds the permuted rows.  If act_bf16 the hidden activation is rounded to
    bf16 before the down projection (what a bf16-activation runtime feeds the next matmul)."""
    P = xp.shape[0]
    H = dequant_shape(down[0], fmt)[0]
    out = np.zeros((P, H), dtype=np.float32)
    for e in range(len(gate)):
        a, b = int(offsets[e]), int(offsets[e + 1])
        if a == b:
            continue
        xe = xp[a:b]
        g = qlinear(xe, gate[e][0], gate[e][1], fmt)
        u = qlinear(xe, up[e][0], up[e][1], fmt)
        h = silu(g) * u
        if act_bf16:
            h = bf16_round(h)
        out[a:b] = qlinear(h, down[e][0], down[e][1], fmt)
    return out


def dequant_shape(cs, fmt):
    c = cs[0]
    return (c.shape[0], c.shape[1] * (2 if fmt == FMT_Q4 else 1))


def moe_combine(out_p: np.ndarray, perm: np.ndarray, w: np.ndarray) -> np.ndarray:
    """y[t] = sum over slots (in slot order 0..k-1) of w[t,slot] * out_of(t,slot), fp32."""
    T, k = w.shape
    inv = np.empty(T * k, dtype=np.int64)
    inv[np.asarray(perm, dtype=np.int64)] = np.arange(T * k)
    y = np.zeros((T, out_p.shape[1]), dtype=np.float32)
    for s in range(k):                      # fixed slot order => deterministic sum
        y += w[:, s:s + 1] * out_p[inv[np.arange(T) * k + s]]
    return y


def moe_forward(x, router, gate, up, down, fmt, top_k, *, act_bf16=True):
    """Full MoE layer on x f32[T,H] (values already in the activation dtype)."""
    idx, w = moe_route(x, router[0], router[1], fmt, top_k)
    perm, offsets = moe_permute(idx, len(gate))
    xp = np.asarray(x, dtype=np.float32)[perm // top_k]
    out_p = moe_experts(xp, offsets, gate, up, down, fmt, act_bf16=act_bf16)
    return moe_combine(out_p, perm, w), (idx, w, perm, offsets)


def moe_dense_reference(x, router, gate, up, down, fmt, top_k, *, act_bf16=True):
    """Same layer computed the slow obvious way (every expert on every token, masked).
    Used only to check permute/combine bookkeeping in the oracle itself."""
    idx, w = moe_route(x, router[0], router[1], fmt, top_k)
    x = np.asarray(x, dtype=np.float32)
    T = x.shape[0]
    H = dequant_shape(down[0], fmt)[0]
    y = np.zeros((T, H), dtype=np.float32)
    outs = []
    for e in range(len(gate)):
        h = silu(qlinear(x, gate[e][0], gate[e][1], fmt)) * qlinear(x, up[e][0], up[e][1], fmt)
        if act_bf16:
            h = bf16_round(h)
        outs.append(qlinear(h, down[e][0], down[e][1], fmt))
    for s in range(top_k):
        for t in range(T):
            y[t] += w[t, s] * outs[int(idx[t, s])][t]
    return y


# ---------------------------------------------------------------------------------------
# S10  sharding (the sharded result must equal the unsharded one)
# ---------------------------------------------------------------------------------------
def shard(codes_or_packed, scales, fmt, axis: str, rank: int, world: int):
    """axis 'n' = column-parallel (split output rows N), 'k' = row-parallel (split K in
    multiples of 32 so no group straddles two ranks)."""
    N = codes_or_packed.shape[0]
    K = codes_or_packed.shape[1] * (2 if fmt == FMT_Q4 else 1)
    if axis == "n":
        if N % world:
            raise ValueError(f"N={N} not divisible by world={world}")
        n = N // world
        return codes_or_packed[rank * n:(rank + 1) * n], scales[rank * n:(rank + 1) * n]
    if axis == "k":
        if K % (world * GROUP):
            raise ValueError(f"K={K} not divisible by world*32={world * GROUP}")
        k = K // world
        div = 2 if fmt == FMT_Q4 else 1
        return (codes_or_packed[:, rank * k // div:(rank + 1) * k // div],
                scales[:, rank * k // GROUP:(rank + 1) * k // GROUP])
    raise ValueError("axis must be 'n' or 'k'")


# ---------------------------------------------------------------------------------------
# error measures used by every parity test
# ---------------------------------------------------------------------------------------
def rel_err(y, y_ref) -> float:
    """Tensor-normalised max error: max|y - y_ref| / max|y_ref|."""
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    d = np.abs(y - y_ref).max(initial=0.0)
    m = np.abs(y_ref).max(initial=0.0)
    return float(d / m) if m > 0 else float(d)


def rel_err_elementwise(y, y_ref) -> float:
    """max |y-y_ref| / (|y_ref| + 1e-3 * rms(y_ref))."""
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    if y_ref.size == 0:
        return 0.0
    rms = np.sqrt(np.mean(y_ref ** 2))
    return float((np.abs(y - y_ref) / (np.abs(y_ref) + 1e-3 * rms + 1e-30)).max())
