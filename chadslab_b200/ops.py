"""Operator surface of the quantized-matmul path.

    PackedWeight.from_float(W, fmt) / .from_arrays(codes, scales, fmt)
    QuantLinear(pw)(x) -> y          every attention / FFN projection
    LMHead(pw)(x) -> logits          .greedy(x) -> token ids
    MoEExperts(router_pw, gate_pws, up_pws, down_pws, top_k)(x) -> y
    shard(pw, axis, rank, world)     column ('n') / row ('k') parallel slices

The reference checkout has no operator surface for this path (no quantized linear, expert matmul
or lm_head exists in it), so these names are this package's own; they are identical for every
caller and the numerical contract is: dequantized weight = float(code) * float(scale) exactly,
fp32 accumulation, outputs within 1e-3 (max error / max magnitude) of an fp32 numpy evaluation.

x may be a CUDA torch tensor (device path: nothing leaves the GPU) or a host numpy array
(host path: the C ABI copies in, computes, copies out).  All compute is in libb200q.so; if the
library or a GPU is missing the calls raise — there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib, packing
from ._lib import BqError, DT_BF16, DT_F32, FMT_Q4, FMT_Q8, PATH_AUTO

GROUP = packing.GROUP


def _torch():
    import torch
    return torch


def _stream_ptr() -> int:
    return _torch().cuda.current_stream().cuda_stream


def _dt_of_torch(t) -> int:
    torch = _torch()
    if t.dtype == torch.float32:
        return DT_F32
    if t.dtype == torch.bfloat16:
        return DT_BF16
    raise TypeError(f"activations must be float32 or bfloat16, got {t.dtype}")


def _torch_dtype(dt: int):
    torch = _torch()
    return torch.float32 if dt == DT_F32 else torch.bfloat16


def _np_dt(a: np.ndarray) -> int:
    if a.dtype == np.float32:
        return DT_F32
    if a.dtype.name == "bfloat16":
        return DT_BF16
    raise TypeError(f"host activations must be float32 or ml_dtypes.bfloat16, got {a.dtype}")


class PackedWeight:
    """A block-quantized [N, K] weight: host arrays in the interface layout + a device handle."""

    def __init__(self, codes: np.ndarray, scales: np.ndarray, fmt: int, *, upload: bool = True,
                 device: Optional[int] = None):
        if fmt not in (FMT_Q8, FMT_Q4):
            raise ValueError(f"unknown format {fmt}")
        codes = np.ascontiguousarray(codes)
        scales = np.ascontiguousarray(scales)
        if codes.ndim != 2 or scales.ndim != 2:
            raise ValueError("codes and scales must be 2-D")
        N = codes.shape[0]
        K = codes.shape[1] * (2 if fmt == FMT_Q4 else 1)
        if K <= 0 or K % GROUP:
            raise ValueError(f"K={K} must be a positive multiple of {GROUP}")
        if codes.dtype != packing.codes_dtype(fmt):
            raise TypeError(f"codes dtype must be {packing.codes_dtype(fmt).__name__}")
        if scales.dtype != np.float16 or scales.shape != (N, K // GROUP):
            raise ValueError(f"scales must be float16 of shape {(N, K // GROUP)}")
        self.codes, self.scales, self.fmt, self.N, self.K = codes, scales, fmt, N, K
        self._handle = None
        self._device = device
        if upload:
            self.upload(device)

    # -- construction -------------------------------------------------------------------------
    @classmethod
    def from_float(cls, W, fmt: int, **kw) -> "PackedWeight":
        codes, scales = packing.quantize(np.asarray(W, dtype=np.float32), fmt)
        return cls(codes, scales, fmt, **kw)

    @classmethod
    def from_float_device(cls, W, fmt: int) -> "PackedWeight":
        """Quantize a CUDA tensor (fp32 or bf16 [N, K]) on the device: same codes and scales, bit for bit, as
        `from_float` computes on the host; nothing leaves the GPU."""
        torch = _torch()
        if not W.is_cuda or W.dim() != 2:
            raise BqError(_lib.ERR_ARG, "from_float_device needs a 2-D CUDA tensor")
        W = W.contiguous()
        N, K = W.shape
        if K % GROUP:
            raise ValueError(f"K={K} must be a multiple of {GROUP}")
        codes = torch.empty((N, K if fmt == FMT_Q8 else K // 2), dtype=torch.int8 if fmt == FMT_Q8 else torch.uint8,
                            device=W.device)
        scales = torch.empty((N, K // GROUP), dtype=torch.float16, device=W.device)
        _lib.check(_lib.lib().bq_quantize(W.data_ptr(), _dt_of_torch(W), N, K, fmt, codes.data_ptr(), scales.data_ptr(),
                                          _stream_ptr()))
        return cls.from_device(codes, scales, fmt)

    @classmethod
    def from_arrays(cls, codes, scales, fmt: int, **kw) -> "PackedWeight":
        return cls(codes, scales, fmt, **kw)

    @classmethod
    def from_device(cls, d_codes, d_scales, fmt: int) -> "PackedWeight":
        """Wrap device-resident torch tensors (codes int8/uint8 [N,K or K/2], scales fp16)."""
        torch = _torch()
        self = cls.__new__(cls)
        N = d_codes.shape[0]
        K = d_codes.shape[1] * (2 if fmt == FMT_Q4 else 1)
        assert d_scales.dtype == torch.float16 and tuple(d_scales.shape) == (N, K // GROUP)
        assert d_codes.is_contiguous() and d_scales.is_contiguous()
        self.codes = self.scales = None
        self.fmt, self.N, self.K = fmt, N, K
        lib = _lib.init(d_codes.device.index or 0)
        h = C.c_uint64(0)
        _lib.check(lib.bq_weight_create_device(d_codes.data_ptr(), d_scales.data_ptr(), N, K, fmt,
                                               _stream_ptr(), C.byref(h)))
        self._handle = h.value
        self._device = d_codes.device.index or 0
        return self

    def slice_rows(self, row0: int, nrows: int) -> "PackedWeight":
        """Rows row0 .. row0+nrows-1 as a weight of their own (a view: no copy; keeps this weight alive)."""
        view = PackedWeight.__new__(PackedWeight)
        view.codes = None if self.codes is None else self.codes[row0:row0 + nrows]
        view.scales = None if self.scales is None else self.scales[row0:row0 + nrows]
        view.fmt, view.N, view.K = self.fmt, int(nrows), self.K
        h = C.c_uint64(0)
        _lib.check(_lib.lib().bq_weight_slice_rows(self.handle, int(row0), int(nrows), C.byref(h)))
        view._handle, view._device, view._parent = h.value, self._device, self
        return view

    def upload(self, device: Optional[int] = None) -> "PackedWeight":
        if self._handle is not None:
            return self
        if device is None:
            device = _torch().cuda.current_device() if _torch().cuda.is_available() else 0
        lib = _lib.init(device)
        h = C.c_uint64(0)
        _lib.check(lib.bq_weight_create(self.codes.ctypes.data, self.scales.ctypes.data, self.N, self.K,
                                        self.fmt, C.byref(h)))
        self._handle, self._device = h.value, device
        return self

    @property
    def handle(self) -> int:
        if self._handle is None:
            self.upload(self._device)
        return self._handle

    def close(self) -> None:
        if self._handle is not None:
            try:
                _lib.load().bq_weight_destroy(self._handle)
            finally:
                self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # -- queries ---------------------------------------------------------------------------------
    @property
    def nbytes(self) -> int:
        """Algorithmic bytes of the packed weight (codes + scales)."""
        return int(self.N * self.K * packing.bytes_per_weight(self.fmt))

    def export(self):
        """Read the weight back from the device in the interface layout."""
        codes = np.empty(packing.codes_shape(self.N, self.K, self.fmt), dtype=packing.codes_dtype(self.fmt))
        scales = np.empty((self.N, self.K // GROUP), dtype=np.float16)
        _lib.check(_lib.lib().bq_weight_export(self.handle, codes.ctypes.data, scales.ctypes.data))
        return codes, scales

    def dequantize(self, dtype=None):
        """-> CUDA tensor [N,K]; float32 (exact) or bfloat16 (round-to-nearest-even of it)."""
        torch = _torch()
        dtype = dtype or torch.float32
        out = torch.empty((self.N, self.K), dtype=dtype, device=f"cuda:{self._device or 0}")
        _lib.check(_lib.lib().bq_dequant(self.handle, out.data_ptr(), _dt_of_torch(out), _stream_ptr()))
        return out

    def unpack(self):
        """-> CUDA int8 tensor [N,K] of integer codes."""
        torch = _torch()
        h = self.handle
        out = torch.empty((self.N, self.K), dtype=torch.int8, device=f"cuda:{self._device or 0}")
        _lib.check(_lib.lib().bq_unpack_codes(h, out.data_ptr(), _stream_ptr()))
        return out


def shard(pw: PackedWeight, axis: str, rank: int, world: int, **kw) -> PackedWeight:
    """Column-parallel ('n': split output rows) or row-parallel ('k': split K in multiples of 32,
    so no quantization group straddles two ranks) slice of a packed weight."""
    if pw.codes is None:
        raise ValueError("shard() needs the host arrays of the weight")
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    if axis == "n":
        if pw.N % world:
            raise ValueError(f"N={pw.N} is not divisible by world={world}")
        n = pw.N // world
        return PackedWeight(pw.codes[rank * n:(rank + 1) * n], pw.scales[rank * n:(rank + 1) * n], pw.fmt, **kw)
    if axis == "k":
        if pw.K % (world * GROUP):
            raise ValueError(f"K={pw.K} is not divisible by world*32={world * GROUP}")
        k = pw.K // world
        div = 2 if pw.fmt == FMT_Q4 else 1
        return PackedWeight(pw.codes[:, rank * k // div:(rank + 1) * k // div],
                            pw.scales[:, rank * k // GROUP:(rank + 1) * k // GROUP], pw.fmt, **kw)
    raise ValueError("axis must be 'n' or 'k'")


def interleave_gate_up(gate: PackedWeight, up: PackedWeight, **kw) -> PackedWeight:
    """Fused gate|up weight for `QuantLinear.gated`: 2F rows in 16-row blocks, 8 gate rows followed by the 8 up
    rows of the same output columns (a row permutation of the concatenated weights)."""
    if gate.codes is None or up.codes is None:
        raise ValueError("interleave_gate_up() needs the host arrays of both weights")
    if (gate.N, gate.K, gate.fmt) != (up.N, up.K, up.fmt) or gate.N % 8:
        raise ValueError("gate and up must have the same shape and format, with a multiple of 8 rows")
    F = gate.N

    def mix(a, b):
        return np.stack([a.reshape(F // 8, 8, -1), b.reshape(F // 8, 8, -1)], axis=1).reshape(2 * F, -1)
    return PackedWeight(mix(gate.codes, up.codes), mix(gate.scales, up.scales), gate.fmt, **kw)


def split_gate_up(gu):
    """[..., 2F] output of a plain product with an interleaved gate|up weight -> (gate [..., F], up [..., F])."""
    F = gu.shape[-1] // 2
    g4 = gu.reshape(*gu.shape[:-1], F // 8, 2, 8)
    return g4[..., 0, :].reshape(*gu.shape[:-1], F), g4[..., 1, :].reshape(*gu.shape[:-1], F)


class QuantLinear:
    """y = x . dequant(W)^T for a packed weight; fp32 accumulate."""

    def __init__(self, pw: PackedWeight, out_dtype=None, path: int = PATH_AUTO):
        self.pw = pw
        self.out_dtype = out_dtype
        self.path = path

    @property
    def in_features(self) -> int:
        return self.pw.K

    @property
    def out_features(self) -> int:
        return self.pw.N

    def __call__(self, x, out=None):
        if isinstance(x, np.ndarray):
            return self._host(x)
        torch = _torch()
        if not x.is_cuda:
            raise BqError(_lib.ERR_ARG, "activations must be a CUDA tensor (or a host numpy array)")
        lead = x.shape[:-1]
        if x.shape[-1] != self.pw.K:
            raise ValueError(f"x has K={x.shape[-1]}, weight has K={self.pw.K}")
        x2 = x.reshape(-1, self.pw.K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        odt = self.out_dtype or torch.float32
        if out is None:
            out = torch.empty((M, self.pw.N), dtype=odt, device=x.device)
        _lib.check(_lib.lib().bq_qlinear_ex(self.pw.handle, x2.data_ptr(), _dt_of_torch(x2), M, out.data_ptr(),
                                            _dt_of_torch(out), self.path, _stream_ptr()))
        return out.reshape(*lead, self.pw.N)

    def gated(self, x, act: int = 0, out=None):
        """For a weight built by `interleave_gate_up`: act(x . gate^T) * (x . up^T) in the dtype of x
        (act 0 = gelu-tanh, 1 = silu); decode-sized calls are one launch."""
        torch = _torch()
        x2 = x.reshape(-1, self.pw.K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        if out is None:
            out = torch.empty((M, self.pw.N // 2), dtype=x2.dtype, device=x.device)
        _lib.check(_lib.lib().bq_qlinear_gated(self.pw.handle, x2.data_ptr(), _dt_of_torch(x2), M, out.data_ptr(), int(act),
                                               _stream_ptr()))
        return out.reshape(*x.shape[:-1], self.pw.N // 2)

    def _host(self, x: np.ndarray) -> np.ndarray:
        x2 = np.ascontiguousarray(x).reshape(-1, self.pw.K)
        y = np.empty((x2.shape[0], self.pw.N), dtype=np.float32)
        _lib.check(_lib.lib().bq_qlinear_host(self.pw.handle, x2.ctypes.data, _np_dt(x2), x2.shape[0],
                                              y.ctypes.data, DT_F32))
        return y.reshape(*x.shape[:-1], self.pw.N)


class PeerComm:
    """Sums over the GPUs of one node through peer-mapped memory (one process per GPU): the fused alternative
    to an NCCL all-reduce for decode-sized messages.  `group` is the torch.distributed process group that
    carries the 64-byte IPC handles at set-up (any backend); it is not used afterwards.  Every rank must issue
    the same sequence of summing calls.  `max_elems` bounds the fp32 elements of one sum."""

    def __init__(self, max_elems: int, group=None, rank: int = 0, world: int = 1):
        import ctypes as C
        self.group, self.max_elems = group, int(max_elems)
        if world > 1 or group is not None:
            import torch.distributed as dist
            rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.rank, self.world = rank, world
        lib = _lib.lib()
        h = C.c_uint64(0)
        _lib.check(lib.bq_comm_create(rank, world, self.max_elems, C.byref(h)))
        self.handle = h.value
        if world > 1:
            buf = C.create_string_buffer(64)
            _lib.check(lib.bq_comm_handle(self.handle, buf))
            handles = [None] * world
            dist.all_gather_object(handles, buf.raw, group=group)
            _lib.check(lib.bq_comm_connect(self.handle, b"".join(handles)))
            dist.barrier(group)           # nobody deposits before every buffer is zeroed and mapped

    def close(self):
        if self.handle:
            if self.world > 1:
                import torch.distributed as dist
                _torch().cuda.synchronize()
                dist.barrier(self.group)  # nobody frees while a peer may still store into the buffer
            _lib.check(_lib.lib().bq_comm_destroy(self.handle))
            self.handle = 0

    def reset(self):
        """After a time-out: empty the receive slots and restart the call counter, on every rank together."""
        if self.world > 1:
            import torch.distributed as dist
            _torch().cuda.synchronize()
            dist.barrier(self.group)      # no rank is still inside a call
        _lib.check(_lib.lib().bq_comm_reset(self.handle))
        if self.world > 1:
            dist.barrier(self.group)      # nobody deposits into a buffer that is still being refilled

    def greedy_head(self, head: "QuantLinear", x, vocab_offset: int, out=None):
        """Vocabulary-sharded lm_head + greedy arg-max: `head` holds this rank's vocabulary slice starting at token
        id `vocab_offset`; returns the global ids (int64 [M], ties -> lower id, identical on every rank).  The
        per-rank (maximum, id) pairs travel through the receive slots inside one kernel."""
        torch = _torch()
        x2 = x.reshape(-1, head.pw.K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        M = x2.shape[0]
        if out is None:
            out = torch.empty((M,), dtype=torch.int64, device=x.device)
        _lib.check(_lib.lib().bq_lm_head_sharded(head.pw.handle, x2.data_ptr(), _dt_of_torch(x2), M, int(vocab_offset),
                                                 self.handle, None, out.data_ptr(), _stream_ptr()))
        return out

    def push_linear(self, linear: "QuantLinear", x):
        """Row-parallel partial product of `linear` on this rank's K slice.  Returns None when the GEMV deposited
        its partial sums directly in the peers' receive slots, else the local fp32 partial y (to be passed as
        `inp` to the summing call)."""
        x2 = x.reshape(-1, linear.pw.K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rc = _lib.lib().bq_qlinear_push(linear.pw.handle, x2.data_ptr(), _dt_of_torch(x2), x2.shape[0], self.handle,
                                        _stream_ptr())
        if rc == _lib.ERR_UNSUPPORTED:
            return QuantLinear(linear.pw)(x2)
        _lib.check(rc)
        return None

    def all_reduce(self, inp, count: int = 0, out=None):
        """Sum of `inp` (fp32, CUDA) over the ranks; inp None sums what push_linear deposited (count elements)."""
        torch = _torch()
        n = inp.numel() if inp is not None else int(count)
        if out is None:
            out = torch.empty(n, dtype=torch.float32, device="cuda") if inp is None else torch.empty_like(inp)
        _lib.check(_lib.lib().bq_allreduce(self.handle, inp.data_ptr() if inp is not None else None, out.data_ptr(), n,
                                           _stream_ptr()))
        return out

    def add_rmsnorm(self, inp, x, weight, normed, eps: float):
        """x[rows, H] += sum over ranks (of `inp`, or of the deposited partial sums when inp is None);
        normed = rmsnorm(x) * weight.  In place on x and normed."""
        rows, H = x.shape
        lib = _lib.lib()
        rc = lib.bq_allreduce_add_rmsnorm(self.handle, inp.data_ptr() if inp is not None else None, x.data_ptr(),
                                          weight.data_ptr(), normed.data_ptr(), rows, H, float(eps), _dt_of_torch(x),
                                          _stream_ptr())
        if rc == _lib.ERR_UNSUPPORTED:         # long or unaligned rows: the sum, then the single-GPU kernel
            delta = self.all_reduce(inp, count=rows * H)
            rc = lib.bq_add_rmsnorm(x.data_ptr(), delta.data_ptr(), weight.data_ptr(), normed.data_ptr(), rows, H,
                                    float(eps), _dt_of_torch(x), _stream_ptr())
        _lib.check(rc)


class PeerEP:
    """Expert-parallel exchange through peer-mapped memory (one process per GPU): routed rows are stored straight
    into the owning rank's receive buffer and the expert outputs straight back, with no host involvement per layer.
    `group` carries the 64-byte IPC handles at set-up only.  max_send_rows bounds T * top_k of one call on this rank,
    max_recv_rows the rows this rank's experts may receive (default: world * max_send_rows, which always fits)."""

    def __init__(self, n_experts: int, hidden: int, max_send_rows: int, max_recv_rows: int = 0, group=None, rank: int = 0,
                 world: int = 1):
        torch = _torch()
        if world > 1 or group is not None:
            import torch.distributed as dist
            rank, world = dist.get_rank(group), dist.get_world_size(group)
        self.group, self.rank, self.world = group, rank, world
        self.E, self.H = int(n_experts), int(hidden)
        self.max_send, self.max_recv = int(max_send_rows), int(max_recv_rows or world * max_send_rows)
        lib = _lib.lib()
        h = C.c_uint64(0)
        _lib.check(lib.bq_ep_create(rank, world, self.E, self.H, self.max_send, self.max_recv, C.byref(h)))
        self.handle = h.value
        if world > 1:
            buf = C.create_string_buffer(64)
            _lib.check(lib.bq_ep_handle(self.handle, buf))
            handles = [None] * world
            dist.all_gather_object(handles, buf.raw, group=group)
            _lib.check(lib.bq_ep_connect(self.handle, b"".join(handles)))
            dist.barrier(group)
        xr, lo, cap = C.c_void_p(0), C.c_void_p(0), C.c_int64(0)
        _lib.check(lib.bq_ep_recv_view(self.handle, C.byref(xr), C.byref(lo), C.byref(cap)))
        self.xrecv_ptr, self.loffsets_ptr = xr.value, lo.value
        dev = torch.device("cuda", torch.cuda.current_device())
        # expert outputs in receive order (fp32) live here between the grouped experts and the way back
        self.out_rows = torch.empty((self.max_recv, self.H), dtype=torch.float32, device=dev)

    def close(self):
        if getattr(self, "handle", 0):
            if self.world > 1:
                import torch.distributed as dist
                _torch().cuda.synchronize()
                dist.barrier(self.group)
            _lib.check(_lib.lib().bq_ep_destroy(self.handle))
            self.handle = 0

    def dispatch(self, xb, idx, perm, offsets):
        T, k = idx.shape
        _lib.check(_lib.lib().bq_ep_dispatch(self.handle, xb.data_ptr(), idx.data_ptr(), perm.data_ptr(), offsets.data_ptr(),
                                             T, k, _stream_ptr()))

    def combine(self, inv, w, out_dtype=None):
        torch = _torch()
        T, k = w.shape
        y = torch.empty((T, self.H), dtype=out_dtype or torch.float32, device=w.device)
        _lib.check(_lib.lib().bq_ep_combine(self.handle, self.out_rows.data_ptr(), inv.data_ptr(), w.data_ptr(), T, k,
                                            y.data_ptr(), _dt_of_torch(y), _stream_ptr()))
        return y


class LMHead(QuantLinear):
    """Vocabulary projection; `greedy` returns argmax token ids (ties -> lower id)."""

    def greedy(self, x, return_logits: bool = False):
        torch = _torch()
        x2 = x.reshape(-1, self.pw.K).contiguous()
        M = x2.shape[0]
        ids = torch.empty((M,), dtype=torch.int32, device=x.device)
        logits = torch.empty((M, self.pw.N), dtype=torch.float32, device=x.device) if return_logits else None
        _lib.check(_lib.lib().bq_lm_head(self.pw.handle, x2.data_ptr(), _dt_of_torch(x2), M,
                                         logits.data_ptr() if return_logits else None, DT_F32,
                                         ids.data_ptr(), _stream_ptr()))
        return (ids, logits) if return_logits else ids


def moe_route(logits, top_k: int, renormalise: bool = True):
    torch = _torch()
    logits = logits.contiguous().float()
    T, E = logits.shape
    idx = torch.empty((T, top_k), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
    _lib.check(_lib.lib().bq_moe_route(logits.data_ptr(), T, E, top_k, int(renormalise), idx.data_ptr(),
                                       w.data_ptr(), _stream_ptr()))
    return idx, w


def moe_route_linear(router: "QuantLinear", xb, top_k: int, renormalise: bool = True):
    """Router logits + softmax + top-k for bf16 tokens xb[T,H]: one launch when the router has at most 128 experts
    (bq_moe_route_linear), else the router matmul followed by bq_moe_route."""
    torch = _torch()
    pw = router.pw
    xb = xb.contiguous()
    T = xb.shape[0]
    if xb.dtype == torch.bfloat16 and pw.N <= 128 and pw.K % 128 == 0 and top_k <= min(32, pw.N):
        idx = torch.empty((T, top_k), dtype=torch.int32, device=xb.device)
        w = torch.empty((T, top_k), dtype=torch.float32, device=xb.device)
        rc = _lib.lib().bq_moe_route_linear(pw.handle, xb.data_ptr(), T, top_k, int(renormalise), idx.data_ptr(), w.data_ptr(),
                                            _stream_ptr())
        if rc != _lib.ERR_UNSUPPORTED:
            _lib.check(rc)
            return idx, w
    return moe_route(router(xb), top_k, renormalise)


def moe_permute(idx, n_experts: int):
    torch = _torch()
    idx = idx.contiguous()
    T, k = idx.shape
    A = T * k
    lib = _lib.lib()
    perm = torch.empty((A,), dtype=torch.int32, device=idx.device)
    inv = torch.empty((A,), dtype=torch.int32, device=idx.device)
    offsets = torch.empty((n_experts + 1,), dtype=torch.int32, device=idx.device)
    sb = max(int(lib.bq_moe_permute_scratch_bytes(T, k, n_experts)), 16)
    scratch = torch.empty((sb,), dtype=torch.uint8, device=idx.device)
    _lib.check(lib.bq_moe_permute(idx.data_ptr(), T, k, n_experts, perm.data_ptr(), inv.data_ptr(),
                                  offsets.data_ptr(), scratch.data_ptr(), _stream_ptr()))
    return perm, inv, offsets


def moe_gather(x, perm, top_k: int):
    torch = _torch()
    x = x.contiguous()
    P = perm.numel()
    xp = torch.empty((P, x.shape[1]), dtype=x.dtype, device=x.device)
    _lib.check(_lib.lib().bq_moe_gather(x.data_ptr(), _dt_of_torch(x), x.shape[1], perm.data_ptr(), P, top_k,
                                        xp.data_ptr(), _stream_ptr()))
    return xp


def moe_combine(out_p, inv, w, out_dtype=None):
    torch = _torch()
    T, k = w.shape
    H = out_p.shape[1]
    y = torch.empty((T, H), dtype=out_dtype or torch.float32, device=out_p.device)
    _lib.check(_lib.lib().bq_moe_combine(out_p.data_ptr(), inv.data_ptr(), w.data_ptr(), T, k, H, y.data_ptr(),
                                         _dt_of_torch(y), _stream_ptr()))
    return y


class MoEExperts:
    """Sparse MoE layer: router linear -> softmax/top-k -> permute -> grouped SwiGLU experts ->
    weighted combine.  Activations are bf16 between the matmuls, accumulation is fp32."""

    def __init__(self, router_pw: Optional[PackedWeight], gate_pws: Sequence[PackedWeight], up_pws: Sequence[PackedWeight],
                 down_pws: Sequence[PackedWeight], top_k: int, renormalise: bool = True, path: int = PATH_AUTO):
        E = len(gate_pws)
        if not (len(up_pws) == len(down_pws) == E) or E == 0:
            raise ValueError("gate/up/down must hold one weight per expert")
        # router_pw None: only this rank's experts (expert parallel: routing happens over all ranks' experts elsewhere)
        if router_pw is not None and router_pw.N != E:
            raise ValueError("router must have one output row per expert")
        self.router = QuantLinear(router_pw) if router_pw is not None else None
        self.gate, self.up, self.down = list(gate_pws), list(up_pws), list(down_pws)
        self.E, self.top_k, self.renormalise, self.path = E, top_k, renormalise, path
        self.H, self.F = gate_pws[0].K, gate_pws[0].N
        arr = lambda pws: (C.c_uint64 * E)(*[p.handle for p in pws])
        h = C.c_uint64(0)
        _lib.check(_lib.lib().bq_moe_create(arr(self.gate), arr(self.up), arr(self.down), E, C.byref(h)))
        self._handle = h.value

    def close(self):
        if getattr(self, "_handle", None):
            _lib.load().bq_moe_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def experts(self, xp, offsets, return_h: bool = False):
        """Grouped SwiGLU FFN on permuted bf16 rows xp[P,H] -> f32[P,H] (and the bf16 hidden h[P,F])."""
        torch = _torch()
        P = xp.shape[0]
        hbuf = torch.empty((P, self.F), dtype=torch.bfloat16, device=xp.device)
        out = torch.empty((P, self.H), dtype=torch.float32, device=xp.device)
        _lib.check(_lib.lib().bq_moe_experts(self._handle, xp.data_ptr(), offsets.data_ptr(), P, hbuf.data_ptr(),
                                             out.data_ptr(), self.path, _stream_ptr()))
        return (out, hbuf) if return_h else out

    def experts_tokens(self, xb, perm, offsets):
        """Grouped SwiGLU FFN on the TOKEN rows xb[T,H] (bf16) of a routed batch: sorted position p uses row
        perm[p] // top_k.  -> f32 [T*k, H] in sorted order.  No gathered copy is made at decode sizes."""
        torch = _torch()
        P = perm.numel()
        hbuf = torch.empty((P, self.F), dtype=torch.bfloat16, device=xb.device)
        out = torch.empty((P, self.H), dtype=torch.float32, device=xb.device)
        work = torch.empty((P, self.H), dtype=torch.bfloat16, device=xb.device)
        _lib.check(_lib.lib().bq_moe_experts_tokens(self._handle, xb.data_ptr(), perm.data_ptr(), self.top_k, offsets.data_ptr(), P,
                                                    P, work.data_ptr(), hbuf.data_ptr(), out.data_ptr(), self.path, _stream_ptr()))
        return out

    def experts_received(self, ep: "PeerEP", rows_hint: int):
        """Grouped SwiGLU FFN of this rank's experts on the rows `ep.dispatch` delivered: reads the receive buffer and
        the device-side row ranges of the exchange object, writes `ep.out_rows`.  `rows_hint`: rows to expect (picks
        the token tile; the actual count is only known on the device)."""
        torch = _torch()
        if getattr(self, "_hrecv", None) is None or self._hrecv.shape[0] < ep.max_recv:
            self._hrecv = torch.empty((ep.max_recv, self.F), dtype=torch.bfloat16, device=ep.out_rows.device)
        _lib.check(_lib.lib().bq_moe_experts_ex(self._handle, ep.xrecv_ptr, ep.loffsets_ptr, ep.max_recv,
                                                min(int(rows_hint), ep.max_recv), self._hrecv.data_ptr(),
                                                ep.out_rows.data_ptr(), self.path, _stream_ptr()))

    def __call__(self, x, return_aux: bool = False):
        torch = _torch()
        x = x.reshape(-1, self.H)
        xb = x if x.dtype == torch.bfloat16 else x.to(torch.bfloat16)
        idx, w = moe_route_linear(self.router, xb, self.top_k, self.renormalise)
        perm, inv, offsets = moe_permute(idx, self.E)
        out_p = self.experts_tokens(xb.contiguous(), perm, offsets)
        y = moe_combine(out_p, inv, w)
        return (y, (idx, w, perm, inv, offsets)) if return_aux else y
