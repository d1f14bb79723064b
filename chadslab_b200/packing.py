"""Host-side weight packer: fp32 weights -> the interface layout of the packed formats.

    Q8: codes int8[N,K],    scales fp16[N,K/32]   scale = fp16(absmax/127), code = clip(rint(w/scale), +-127)
    Q4: packed uint8[N,K/2], scales fp16[N,K/32]  scale = fp16(absmax/7),   code = clip(rint(w/scale), +-7),
        nibble = code + 8, element 2j in the low nibble of byte j and 2j+1 in the high nibble.

This is one-off weight preparation (it runs once per checkpoint, before upload), not part of
the per-token path; the per-token path is CUDA only.
"""
from __future__ import annotations

import numpy as np

GROUP = 32
FMT_Q8, FMT_Q4 = 0, 1
_QMAX = {FMT_Q8: 127, FMT_Q4: 7}
_FP16_MAX = np.float32(65504.0)


def _quantize_codes(W: np.ndarray, fmt: int):
    if fmt not in _QMAX:
        raise ValueError(f"unknown format {fmt}")
    W = np.ascontiguousarray(W, dtype=np.float32)
    if W.ndim != 2:
        raise ValueError("W must be a 2-D [N, K] array")
    N, K = W.shape
    if K <= 0 or K % GROUP:
        raise ValueError(f"K={K} must be a positive multiple of {GROUP}")
    qmax = _QMAX[fmt]
    g = W.reshape(N, K // GROUP, GROUP)
    scales = np.minimum(np.abs(g).max(axis=-1) / np.float32(qmax), _FP16_MAX).astype(np.float16)
    s32 = scales.astype(np.float32)
    dead = s32 == 0
    q = np.clip(np.rint(g / np.where(dead, np.float32(1), s32)[..., None]), -qmax, qmax)
    q[dead] = 0
    return q.astype(np.int8).reshape(N, K), scales


def pack_nibbles(codes: np.ndarray) -> np.ndarray:
    nib = (codes.astype(np.int16) + 8).astype(np.uint8)
    return (nib[..., 0::2] | (nib[..., 1::2] << 4)).astype(np.uint8)


def unpack_nibbles(packed: np.ndarray) -> np.ndarray:
    packed = np.ascontiguousarray(packed, dtype=np.uint8)
    out = np.empty(packed.shape[:-1] + (packed.shape[-1] * 2,), dtype=np.int8)
    out[..., 0::2] = (packed & 0xF).astype(np.int8) - 8
    out[..., 1::2] = (packed >> 4).astype(np.int8) - 8
    return out


def quantize(W: np.ndarray, fmt: int):
    """-> (codes, scales) in the interface layout of `fmt`."""
    codes, scales = _quantize_codes(W, fmt)
    if fmt == FMT_Q4:
        codes = pack_nibbles(codes)
    return codes, scales


def codes_shape(N: int, K: int, fmt: int):
    return (N, K) if fmt == FMT_Q8 else (N, K // 2)


def codes_dtype(fmt: int):
    return np.int8 if fmt == FMT_Q8 else np.uint8


def bytes_per_weight(fmt: int) -> float:
    """Algorithmic HBM bytes per weight: codes plus one fp16 scale per 32 weights."""
    return (1.0 if fmt == FMT_Q8 else 0.5) + 2.0 / GROUP
