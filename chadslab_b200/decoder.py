"""Decoder drivers around the quantized-matmul path (the caller side of the path).

`QuantDecoder` (Gemma-shaped, dense GeGLU FFN): every projection (q/k/v/o, gate/up/down, lm_head) is a
`QuantLinear` on packed weights.  With `world > 1` the projections are tensor-parallel (`parallel.py`): q/k/v and
gate/up column-sharded, o and down row-sharded with a sum over the ranks, the head vocabulary-sharded.
`MoEDecoder` (sparse-MoE FFN in every layer): attention and router replicated, sequences data-parallel over the
ranks, experts expert-parallel (E / world per rank) with the device-side exchange of `ops.PeerEP`.
Prefill runs the glue between the matmuls in PyTorch; the decode step (`_step_static`) runs the library's glue
kernels and is captured in a CUDA graph.
Architecture choices the specification leaves open: norm weights multiply the normalised value directly, eps 1e-6,
no embedding scaling, no logit soft-capping, rotate-half RoPE with base 10000, untied embedding table.
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass

import numpy as np
import torch
import torch.nn.functional as F

from . import parallel
from .ops import LMHead, PackedWeight, QuantLinear, interleave_gate_up, shard, split_gate_up
from .synth import make_device_weight


@dataclass
class DecoderConfig:
    layers: int
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    ffn: int
    vocab: int
    fmt: int = 0
    rope_base: float = 10000.0
    eps: float = 1e-6
    n_experts: int = 0          # > 0: every layer's FFN is a sparse MoE (SwiGLU experts of width moe_ffn, routed top_k)
    top_k: int = 0
    moe_ffn: int = 0

    def as_dict(self):
        return dict(self.__dict__)


GEMMA_2B_SHAPE = DecoderConfig(18, 2048, 8, 1, 256, 16384, 256000, fmt=0)
GEMMA_7B_SHAPE = DecoderConfig(28, 3072, 16, 16, 256, 24576, 256000, fmt=1)
# sparse-MoE decoder: 48 layers, hidden 2048, 32 query / 4 KV heads of 128, 128 experts of SwiGLU 768, top-8, 4-bit.
# The vocabulary size is not part of the written shape; 32000 is this package's choice.
MOE_SHAPE = DecoderConfig(48, 2048, 32, 4, 128, 0, 32000, fmt=1, n_experts=128, top_k=8, moe_ffn=768)


def _rope(x, pos, base):
    """x [B, T, heads, d], pos [T]."""
    d = x.shape[-1]
    inv = 1.0 / (base ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = pos.float()[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    xf = x.float()
    x1, x2 = xf[..., : d // 2], xf[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class QuantDecoder:
    def __init__(self, cfg: DecoderConfig, lin: dict, embed, norms: dict, act_dtype=torch.bfloat16, rank: int = 0,
                 world: int = 1, max_seq: int = 4096, max_batch: int = 1, comm=None):
        self.cfg, self.lin, self.embed, self.norms = cfg, lin, embed, norms
        # ops.PeerComm (optional, world > 1): the static decode step then sums the row-parallel partial products
        # through peer memory (GEMV deposits -> fused sum + residual add + RMSNorm) instead of NCCL all-reduces
        self.comm = comm
        self.act_dtype, self.rank, self.world = act_dtype, rank, world
        self.kv_sharded = cfg.n_kv_heads % world == 0 and cfg.n_kv_heads >= world
        self.h_local = cfg.n_heads // world
        self.kv_local = cfg.n_kv_heads // world if self.kv_sharded else cfg.n_kv_heads
        self.ffn_local = cfg.ffn // world
        dev = embed.device
        self.k_cache = [torch.zeros((max_batch, max_seq, self.kv_local, cfg.head_dim), dtype=act_dtype, device=dev)
                        for _ in range(cfg.layers)]
        self.v_cache = [torch.zeros_like(self.k_cache[0]) for _ in range(cfg.layers)]
        self.pos = 0

    # ---- construction -------------------------------------------------------------------------------
    @staticmethod
    def _wrap(cfg, get, rank, world):
        """get(name, axis) -> PackedWeight shard.  Builds the (possibly tensor-parallel) projection objects."""
        lin = {}
        kv_sharded = cfg.n_kv_heads % world == 0 and cfg.n_kv_heads >= world
        kv_axis = "n" if kv_sharded else None
        for l in range(cfg.layers):
            # q|k|v and gate|up are each one packed weight (rows concatenated): one launch instead of three / two
            lin[f"l{l}.qkv"] = QuantLinear(get([f"l{l}.q", f"l{l}.k", f"l{l}.v"], ["n", kv_axis, kv_axis]))
            # gate|up rows interleaved in blocks of 8 (ops.interleave_gate_up): the decode GEMV applies the gated
            # activation in its epilogue
            lin[f"l{l}.gate_up"] = QuantLinear(get([f"l{l}.gate", f"l{l}.up"], ["n", "n"], True))
            o, d = QuantLinear(get(f"l{l}.o", "k")), QuantLinear(get(f"l{l}.down", "k"))
            lin[f"l{l}.o"] = parallel.RowParallelLinear(o) if world > 1 else o
            lin[f"l{l}.down"] = parallel.RowParallelLinear(d) if world > 1 else d
        head = LMHead(get("lm_head", "n"))
        lin["lm_head"] = head
        return lin

    @classmethod
    def from_numpy(cls, cfg: DecoderConfig, w: dict, act_dtype=torch.float32, rank=0, world=1, **kw):
        """w: name -> (codes, scales) for projections, arrays for 'embed', norms (as oracle.model.random_weights)."""
        def get_one(name, axis, upload):
            pw = PackedWeight(w[name][0], w[name][1], cfg.fmt, upload=upload and (world == 1 or axis is None))
            return pw if (world == 1 or axis is None) else shard(pw, axis, rank, world, upload=upload)

        def get(name, axis, blocked=False):
            if isinstance(name, str):
                return get_one(name, axis, True)
            parts = [get_one(n_, a_, False) for n_, a_ in zip(name, axis)]
            if blocked:
                return interleave_gate_up(parts[0], parts[1])
            return PackedWeight(np.concatenate([p_.codes for p_ in parts], 0), np.concatenate([p_.scales for p_ in parts], 0),
                                cfg.fmt)
        lin = cls._wrap(cfg, get, rank, world)
        dev = torch.device("cuda", torch.cuda.current_device())
        embed = torch.from_numpy(w["embed"]).to(dev)
        norms = {k: torch.from_numpy(v).to(dev) for k, v in w.items() if "norm" in k}
        return cls(cfg, lin, embed, norms, act_dtype, rank, world, **kw)

    @classmethod
    def random(cls, cfg: DecoderConfig, seed=0, act_dtype=torch.bfloat16, rank=0, world=1, **kw):
        """Random-init N(0,0.02) packed weights generated on the device, shard by shard (synthetic benchmark
        weights: each shard has its own seed, so a sharded model is not a slice of the unsharded one)."""
        shapes = {"q": (cfg.n_heads * cfg.head_dim, cfg.hidden), "k": (cfg.n_kv_heads * cfg.head_dim, cfg.hidden),
                  "v": (cfg.n_kv_heads * cfg.head_dim, cfg.hidden), "o": (cfg.hidden, cfg.n_heads * cfg.head_dim),
                  "gate": (cfg.ffn, cfg.hidden), "up": (cfg.ffn, cfg.hidden), "down": (cfg.hidden, cfg.ffn),
                  "lm_head": (cfg.vocab, cfg.hidden)}

        def get(name, axis, blocked=False):          # random rows: the interleaved layout needs no permutation
            names, axes = ([name], [axis]) if isinstance(name, str) else (name, axis)
            N, K = 0, shapes[names[0].split(".")[-1]][1]
            for n_, a_ in zip(names, axes):
                N += shapes[n_.split(".")[-1]][0] // (world if (world > 1 and a_ == "n") else 1)
            if world > 1 and axes[0] == "k":
                K //= world
            name, axis = "+".join(names), axes[0]
            gen = torch.Generator(device="cuda").manual_seed(zlib.crc32(f"{seed}:{name}:{rank if axis else 0}".encode()))
            codes, scales = make_device_weight(torch, N, K, cfg.fmt, gen)
            return PackedWeight.from_device(codes, scales, cfg.fmt)
        lin = cls._wrap(cfg, get, rank, world)
        dev = torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device="cuda").manual_seed(seed)
        embed = torch.randn((cfg.vocab, cfg.hidden), device=dev, generator=g, dtype=torch.float32).to(act_dtype)
        norms = {f"l{l}.norm{i}": torch.ones(cfg.hidden, device=dev) for l in range(cfg.layers) for i in (1, 2)}
        norms["norm_f"] = torch.ones(cfg.hidden, device=dev)
        return cls(cfg, lin, embed, norms, act_dtype, rank, world, **kw)

    # ---- forward ---------------------------------------------------------------------------------------
    def reset(self):
        self.pos = 0

    def hidden_states(self, tokens):
        """tokens int64 [B, T] -> final normalised hidden states [B, T, hidden]; appends to the KV cache."""
        c = self.cfg
        B, T = tokens.shape
        if self.pos + T > self.k_cache[0].shape[1] or B > self.k_cache[0].shape[0]:
            raise ValueError(f"KV cache holds {self.k_cache[0].shape[1]} positions x {self.k_cache[0].shape[0]} sequences; "
                             f"asked for positions {self.pos}..{self.pos + T - 1} of {B} sequences")
        M = B * T
        x = self.embed[tokens].to(self.act_dtype).reshape(M, c.hidden).contiguous()      # residual stream
        h = torch.empty_like(x)
        pos = torch.arange(self.pos, self.pos + T, device=x.device)
        S = self.pos + T
        nq, nkv = self.h_local * c.head_dim, self.kv_local * c.head_dim
        rep = self.h_local // self.kv_local
        delta = None
        for l in range(c.layers):
            self._add_norm(x, delta, self.norms[f"l{l}.norm1"], h)                        # x += delta; h = rmsnorm(x) * w
            qkv = self.lin[f"l{l}.qkv"](h, out=torch.empty((M, nq + 2 * nkv), dtype=self.act_dtype, device=x.device))
            q = qkv[:, :nq].reshape(B, T, self.h_local, c.head_dim)
            k = qkv[:, nq:nq + nkv].reshape(B, T, self.kv_local, c.head_dim)
            v = qkv[:, nq + nkv:].reshape(B, T, self.kv_local, c.head_dim)
            q, k = _rope(q, pos, c.rope_base), _rope(k, pos, c.rope_base)
            self.k_cache[l][:B, self.pos:S] = k
            self.v_cache[l][:B, self.pos:S] = v
            kk, vv = self.k_cache[l][:B, :S], self.v_cache[l][:B, :S]
            if rep > 1:
                kk, vv = kk.repeat_interleave(rep, dim=2), vv.repeat_interleave(rep, dim=2)
            if self.pos == 0 and T > 1:      # no earlier context: plain causal attention (lets PyTorch pick a fused kernel)
                o = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=True)
            else:
                mask = (torch.arange(S, device=x.device)[None, :] <= pos[:, None])      # [T, S]
                o = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), attn_mask=mask)
            o = o.transpose(1, 2).reshape(M, self.h_local * c.head_dim)
            delta = self.lin[f"l{l}.o"](o.contiguous())                                   # fp32 (summed over the ranks when sharded)
            self._add_norm(x, delta, self.norms[f"l{l}.norm2"], h)
            a = self.lin[f"l{l}.gate_up"].gated(h, 0)                                     # GeGLU applied inside the matmul kernel
            delta = self.lin[f"l{l}.down"](a)
        self._add_norm(x, delta, self.norms["norm_f"], h)
        self.pos = S
        return h.reshape(B, T, c.hidden)

    def _add_norm(self, x, delta, gamma, out):
        """x[rows, hidden] += delta (fp32, may be None); out = rmsnorm(x) * gamma -- the library's kernel."""
        from . import _lib
        from .ops import _dt_of_torch, _stream_ptr
        _lib.check(_lib.lib().bq_add_rmsnorm(x.data_ptr(), delta.data_ptr() if delta is not None else None, gamma.data_ptr(),
                                             out.data_ptr(), x.shape[0], x.shape[1], self.cfg.eps, _dt_of_torch(x), _stream_ptr()))

    def logits(self, tokens):
        h = self.hidden_states(tokens)
        B, T, _ = h.shape
        lg = self.lin["lm_head"](h.reshape(B * T, -1))
        if self.world > 1:
            parts = [torch.empty_like(lg) for _ in range(self.world)]
            torch.distributed.all_gather(parts, lg.contiguous())
            lg = torch.cat(parts, dim=-1)
        return lg.reshape(B, T, -1)

    def next_tokens(self, tokens):
        """Greedy next token for every sequence: tokens [B, T] -> ids [B] (only the last position is projected)."""
        h = self.hidden_states(tokens)[:, -1].contiguous()
        head = self.lin["lm_head"]
        if self.world > 1:
            return parallel.VocabParallelHead(head, self.cfg.vocab // self.world).greedy(h)
        return head.greedy(h).long()

    def generate(self, prompt, n_new):
        """prompt int64 [B, T] -> generated ids [B, n_new] (greedy)."""
        tok = self.next_tokens(prompt)
        out = []
        for _ in range(n_new):
            out.append(tok)
            tok = self.next_tokens(tok[:, None])
        return torch.stack(out, dim=1)

    # ---- static-shape decode step (capturable in a CUDA graph) -----------------------------------------
    def _step_static(self, tokens, pos_t):
        """One greedy decode step with every shape fixed: `tokens` int64 [B] and `pos_t` int64 [1] live on the
        device and are updated in place (tokens <- next ids, pos_t += 1).  Between the quantized matmuls the step
        runs the library's glue kernels (residual add + RMSNorm, RoPE + KV append + single-query attention, gated
        activation), all of which read the position from device memory, so the step is graph-capturable."""
        from . import _lib
        from .ops import _dt_of_torch, _stream_ptr
        c, lib, st = self.cfg, _lib.lib(), _stream_ptr()
        B = tokens.shape[0]
        dt = _dt_of_torch(self.k_cache[0])
        dev = tokens.device
        x = self.embed[tokens].to(self.act_dtype).contiguous()                    # residual stream [B, hidden]
        h = torch.empty_like(x)
        S = self.k_cache[0].shape[1]
        att = torch.empty((B, self.h_local, c.head_dim), dtype=self.act_dtype, device=dev)
        act = torch.empty((B, self.ffn_local), dtype=self.act_dtype, device=dev)
        comm = self.comm if self.world > 1 else None
        PUSHED = object()                  # the partial sums sit in the communicator's receive slots

        def row_parallel(name, inp):
            if comm is None:
                return self.lin[name](inp)                   # fp32 (all-reduced by NCCL when sharded)
            y = comm.push_linear(self.lin[name].linear, inp)
            return PUSHED if y is None else y

        def add_norm(delta, gamma):
            if comm is None or delta is None:
                _lib.check(lib.bq_add_rmsnorm(x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                              gamma.data_ptr(), h.data_ptr(), B, c.hidden, c.eps, dt, st))
            else:
                comm.add_rmsnorm(None if delta is PUSHED else delta, x, gamma, h, c.eps)

        delta = None
        for l in range(c.layers):
            add_norm(delta, self.norms[f"l{l}.norm1"])
            qkv = self.lin[f"l{l}.qkv"](h)                                        # fp32 [B, (Hq + 2 Hkv) D]
            # RoPE, KV append and single-query attention in one launch
            _lib.check(lib.bq_decode_attention_rope(qkv.data_ptr(), self.k_cache[l].data_ptr(), self.v_cache[l].data_ptr(),
                                                    pos_t.data_ptr(), att.data_ptr(), B, self.h_local, self.kv_local,
                                                    c.head_dim, S, c.rope_base, dt, st))
            delta = row_parallel(f"l{l}.o", att.reshape(B, -1))
            add_norm(delta, self.norms[f"l{l}.norm2"])
            self.lin[f"l{l}.gate_up"].gated(h, 0, out=act)                         # GeGLU in the GEMV's epilogue
            delta = row_parallel(f"l{l}.down", act)
        add_norm(delta, self.norms["norm_f"])
        head = self.lin["lm_head"]
        if self.world > 1:
            ids = parallel.VocabParallelHead(head, c.vocab // self.world, comm=comm).greedy(h)
        else:
            ids = head.greedy(h).long()
        tokens.copy_(ids)
        pos_t.add_(1)

    def _check_graph_room(self, batch: int, start_pos: int):
        S, Bmax = self.k_cache[0].shape[1], self.k_cache[0].shape[0]
        if batch > Bmax or start_pos + 2 > S:
            raise ValueError(f"KV cache holds {S} positions x {Bmax} sequences: no room to capture a step at position "
                             f"{start_pos} for {batch} sequences")

    def make_graph_stepper(self, batch: int, first_tokens, start_pos: int, host_in=None, host_out=None):
        """Capture `_step_static` in a CUDA graph.  Returns (step, tokens): calling step() advances every sequence
        by one token; `tokens` (int64 [B], device) then holds the ids just generated.  host_in / host_out (pinned int64
        [B] host tensors): the graph then starts with the copy of the ids to decode from host_in and ends with the copy
        of the new ids to host_out, so that a step driven from host buffers is still a single graph launch (a copy
        issued next to the launch on the same stream costs ~0.4 ms of start-up per step, measured)."""
        dev = self.embed.device
        self._check_graph_room(batch, start_pos)
        tokens = first_tokens.to(dev).long().clone()
        pos_t = torch.tensor([start_pos], device=dev, dtype=torch.int64)
        # the two trial steps below (warm-up, capture) write cache positions start_pos and start_pos + 1 only
        sl = (slice(0, batch), slice(start_pos, start_pos + 2))
        keep = (tokens.clone(), pos_t.clone(), [k[sl].clone() for k in self.k_cache], [v[sl].clone() for v in self.v_cache])
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        if (host_in is not None and not host_in.is_pinned()) or (host_out is not None and not host_out.is_pinned()):
            raise ValueError("host_in / host_out must be pinned host tensors")

        def body():
            if host_in is not None:
                tokens.copy_(host_in, non_blocking=True)
            self._step_static(tokens, pos_t)
            if host_out is not None:
                host_out.copy_(tokens, non_blocking=True)
        with torch.cuda.stream(side):                      # warm-up outside capture (sizes library scratch)
            body()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            body()
        # restore the state the two trial steps consumed
        tokens.copy_(keep[0]); pos_t.copy_(keep[1])
        for dst, src in zip(self.k_cache, keep[2]):
            dst[sl].copy_(src)
        for dst, src in zip(self.v_cache, keep[3]):
            dst[sl].copy_(src)
        self.pos = start_pos

        S = self.k_cache[0].shape[1]

        def step():
            if self.pos >= S:
                raise ValueError(f"KV cache is full ({S} positions): the next token has no row to be written to")
            graph.replay()
            self.pos += 1
        return step, tokens

    def linear_bytes_per_token(self) -> float:
        """Algorithmic packed-weight bytes every decoded token streams on this rank (codes + scales)."""
        tot = 0
        for name, l in self.lin.items():
            q = l.linear if isinstance(l, parallel.RowParallelLinear) else l
            tot += q.pw.nbytes
        return float(tot)


class MoEDecoder(QuantDecoder):
    """Sparse-MoE decoder: GQA attention as in QuantDecoder, every FFN a routed top-k mixture of SwiGLU experts.

    Parallel layout (`world > 1`): attention, router, norms, embedding and head are replicated; each rank decodes
    its own sequences (data parallel) and holds n_experts / world experts; routed rows travel to the owning rank
    and back through `ops.PeerEP` (device-side stores into peer memory, no host step per layer)."""

    def __init__(self, cfg: DecoderConfig, lin: dict, moe: list, embed, norms: dict, act_dtype=torch.bfloat16, rank: int = 0,
                 world: int = 1, max_seq: int = 4096, max_batch: int = 1, ep=None, keep=None):
        self.cfg, self.lin, self.moe, self.embed, self.norms = cfg, lin, moe, embed, norms
        self.comm, self.ep, self._keep = None, ep, keep
        self.act_dtype, self.rank, self.world = act_dtype, rank, world
        self.h_local, self.kv_local, self.kv_sharded = cfg.n_heads, cfg.n_kv_heads, False
        dev = embed.device
        self.k_cache = [torch.zeros((max_batch, max_seq, cfg.n_kv_heads, cfg.head_dim), dtype=act_dtype, device=dev)
                        for _ in range(cfg.layers)]
        self.v_cache = [torch.zeros_like(self.k_cache[0]) for _ in range(cfg.layers)]
        self.pos = 0
        if world > 1:
            if ep is None:
                raise ValueError("expert parallel needs an ops.PeerEP exchange object")
            self.ffn = [parallel.ExpertParallelMoE(self.lin[f"l{l}.router"], None, cfg.n_experts, cfg.top_k, ep=ep,
                                                   local_moe=moe[l], act_dtype=torch.bfloat16) for l in range(cfg.layers)]
        else:
            self.ffn = moe

    # ---- construction -------------------------------------------------------------------------------
    @classmethod
    def _assemble(cls, cfg, get, get_experts, rank, world):
        """get(name) -> PackedWeight (replicated); get_experts(layer, which) -> list of this rank's expert weights."""
        from .ops import MoEExperts
        lin, moe = {}, []
        for l in range(cfg.layers):
            lin[f"l{l}.qkv"] = QuantLinear(get([f"l{l}.q", f"l{l}.k", f"l{l}.v"]))
            lin[f"l{l}.o"] = QuantLinear(get(f"l{l}.o"))
            router = get(f"l{l}.router")
            lin[f"l{l}.router"] = QuantLinear(router)
            g, u, d = (get_experts(l, w_) for w_ in ("gate", "up", "down"))
            moe.append(MoEExperts(router if world == 1 else None, g, u, d, cfg.top_k))
        lin["lm_head"] = LMHead(get("lm_head"))
        return lin, moe

    @classmethod
    def from_numpy(cls, cfg: DecoderConfig, w: dict, act_dtype=torch.float32, rank=0, world=1, **kw):
        """w: name -> (codes, scales) as built by the test oracle's random weights ('l{l}.router', 'l{l}.e{e}.gate', ...)."""
        def get(name):
            if isinstance(name, str):
                return PackedWeight(w[name][0], w[name][1], cfg.fmt)
            return PackedWeight(np.concatenate([w[n_][0] for n_ in name], 0), np.concatenate([w[n_][1] for n_ in name], 0), cfg.fmt)

        def get_experts(l, which):
            ids = parallel.shard_experts(list(range(cfg.n_experts)), rank, world)
            return [PackedWeight(*w[f"l{l}.e{e}.{which}"], cfg.fmt) for e in ids]
        lin, moe = cls._assemble(cfg, get, get_experts, rank, world)
        dev = torch.device("cuda", torch.cuda.current_device())
        embed = torch.from_numpy(w["embed"]).to(dev)
        norms = {k: torch.from_numpy(v).to(dev) for k, v in w.items() if "norm" in k}
        return cls(cfg, lin, moe, embed, norms, act_dtype, rank, world, **kw)

    @classmethod
    def random(cls, cfg: DecoderConfig, seed=0, act_dtype=torch.bfloat16, rank=0, world=1, **kw):
        """Random-init N(0, 0.02) packed weights generated on the device.  Every tensor is seeded by its name (experts by
        their global id), so replicated tensors agree on every rank and the expert-parallel model is a slice of the
        single-GPU one.  The experts of a layer live in one stacked tensor per projection; each expert is a row view."""
        D, Hd, Fm = cfg.head_dim, cfg.hidden, cfg.moe_ffn
        shapes = {"q": (cfg.n_heads * D, Hd), "k": (cfg.n_kv_heads * D, Hd), "v": (cfg.n_kv_heads * D, Hd),
                  "o": (Hd, cfg.n_heads * D), "router": (cfg.n_experts, Hd), "lm_head": (cfg.vocab, Hd),
                  "gate": (Fm, Hd), "up": (Fm, Hd), "down": (Hd, Fm)}
        keep = []

        def gen(name, N, K):
            g = torch.Generator(device="cuda").manual_seed(zlib.crc32(f"{seed}:{name}".encode()))
            return make_device_weight(torch, N, K, cfg.fmt, g)

        def get(name):
            names = [name] if isinstance(name, str) else name
            parts = [gen(n_, *shapes[n_.split(".")[-1]]) for n_ in names]
            return PackedWeight.from_device(torch.cat([p_[0] for p_ in parts], 0), torch.cat([p_[1] for p_ in parts], 0), cfg.fmt)

        def get_experts(l, which):
            ids = parallel.shard_experts(list(range(cfg.n_experts)), rank, world)
            N, K = shapes[which]
            parts = [gen(f"l{l}.e{e}.{which}", N, K) for e in ids]
            stack = PackedWeight.from_device(torch.cat([p_[0] for p_ in parts], 0), torch.cat([p_[1] for p_ in parts], 0), cfg.fmt)
            keep.append(stack)
            return [stack.slice_rows(i * N, N) for i in range(len(ids))]
        lin, moe = cls._assemble(cfg, get, get_experts, rank, world)
        dev = torch.device("cuda", torch.cuda.current_device())
        g = torch.Generator(device="cuda").manual_seed(seed)
        embed = torch.randn((cfg.vocab, cfg.hidden), device=dev, generator=g, dtype=torch.float32).to(act_dtype)
        norms = {f"l{l}.norm{i}": torch.ones(cfg.hidden, device=dev) for l in range(cfg.layers) for i in (1, 2)}
        norms["norm_f"] = torch.ones(cfg.hidden, device=dev)
        return cls(cfg, lin, moe, embed, norms, act_dtype, rank, world, keep=keep, **kw)

    # ---- forward ---------------------------------------------------------------------------------------
    def hidden_states(self, tokens, b0: int = 0, advance: bool = True):
        """tokens int64 [B, T] (this rank's sequences b0 .. b0+B-1) -> final normalised hidden states [B, T, hidden];
        appends to the KV cache rows of those sequences.  `advance=False` leaves the position counter alone (prefill in
        chunks of sequences: every chunk starts at the same position)."""
        c = self.cfg
        B, T = tokens.shape
        S = self.pos + T
        if S > self.k_cache[0].shape[1] or b0 + B > self.k_cache[0].shape[0]:
            raise ValueError(f"KV cache holds {self.k_cache[0].shape[1]} positions x {self.k_cache[0].shape[0]} sequences; "
                             f"asked for positions up to {S - 1} of sequences {b0}..{b0 + B - 1}")
        M = B * T
        x = self.embed[tokens].to(self.act_dtype).reshape(M, c.hidden).contiguous()
        h = torch.empty_like(x)
        pos = torch.arange(self.pos, S, device=x.device)
        nq, nkv = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
        rep = c.n_heads // c.n_kv_heads
        delta = None
        for l in range(c.layers):
            self._add_norm(x, delta, self.norms[f"l{l}.norm1"], h)
            qkv = self.lin[f"l{l}.qkv"](h, out=torch.empty((M, nq + 2 * nkv), dtype=self.act_dtype, device=x.device))
            q = qkv[:, :nq].reshape(B, T, c.n_heads, c.head_dim)
            k = qkv[:, nq:nq + nkv].reshape(B, T, c.n_kv_heads, c.head_dim)
            v = qkv[:, nq + nkv:].reshape(B, T, c.n_kv_heads, c.head_dim)
            q, k = _rope(q, pos, c.rope_base), _rope(k, pos, c.rope_base)
            self.k_cache[l][b0:b0 + B, self.pos:S] = k
            self.v_cache[l][b0:b0 + B, self.pos:S] = v
            kk, vv = self.k_cache[l][b0:b0 + B, :S], self.v_cache[l][b0:b0 + B, :S]
            if rep > 1:
                kk, vv = kk.repeat_interleave(rep, dim=2), vv.repeat_interleave(rep, dim=2)
            if self.pos == 0 and T > 1:
                o = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), is_causal=True)
            else:
                mask = (torch.arange(S, device=x.device)[None, :] <= pos[:, None])
                o = F.scaled_dot_product_attention(q.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), attn_mask=mask)
            o = o.transpose(1, 2).reshape(M, nq)
            delta = self.lin[f"l{l}.o"](o.contiguous())
            self._add_norm(x, delta, self.norms[f"l{l}.norm2"], h)
            delta = self.ffn[l](h)                                                        # fp32 [M, hidden]
        self._add_norm(x, delta, self.norms["norm_f"], h)
        if advance:
            self.pos = S
        return h.reshape(B, T, c.hidden)

    def logits(self, tokens):
        h = self.hidden_states(tokens)
        B, T, _ = h.shape
        return self.lin["lm_head"](h.reshape(B * T, -1)).reshape(B, T, -1)

    def next_tokens(self, tokens):
        h = self.hidden_states(tokens)[:, -1].contiguous()
        return self.lin["lm_head"].greedy(h).long()

    def prefill(self, tokens, chunk_seqs: int):
        """Prefill this rank's sequences (tokens int64 [B, T]) in chunks of `chunk_seqs` sequences, which bounds the
        activation and exchange buffers; returns the first generated token of every sequence.  Under expert
        parallelism every rank must run the same number of chunks."""
        B, T = tokens.shape
        out = []
        for b0 in range(0, B, chunk_seqs):
            h = self.hidden_states(tokens[b0:b0 + chunk_seqs], b0=b0, advance=False)[:, -1].contiguous()
            out.append(self.lin["lm_head"].greedy(h).long())
        self.pos += T
        return torch.cat(out)

    def _step_static(self, tokens, pos_t):
        """One greedy decode step of this rank's sequences, every shape fixed (graph-capturable): library glue kernels
        between the quantized matmuls, the MoE FFN through the device-side kernels (and exchange, when expert parallel)."""
        from . import _lib
        from .ops import _dt_of_torch, _stream_ptr
        c, lib, st = self.cfg, _lib.lib(), _stream_ptr()
        B = tokens.shape[0]
        dt = _dt_of_torch(self.k_cache[0])
        dev = tokens.device
        x = self.embed[tokens].to(self.act_dtype).contiguous()
        h = torch.empty_like(x)
        S = self.k_cache[0].shape[1]
        att = torch.empty((B, c.n_heads, c.head_dim), dtype=self.act_dtype, device=dev)

        def add_norm(delta, gamma):
            _lib.check(lib.bq_add_rmsnorm(x.data_ptr(), delta.data_ptr() if delta is not None else None, gamma.data_ptr(),
                                          h.data_ptr(), B, c.hidden, c.eps, dt, st))
        delta = None
        for l in range(c.layers):
            add_norm(delta, self.norms[f"l{l}.norm1"])
            qkv = self.lin[f"l{l}.qkv"](h)
            _lib.check(lib.bq_decode_attention_rope(qkv.data_ptr(), self.k_cache[l].data_ptr(), self.v_cache[l].data_ptr(),
                                                    pos_t.data_ptr(), att.data_ptr(), B, c.n_heads, c.n_kv_heads,
                                                    c.head_dim, S, c.rope_base, dt, st))
            delta = self.lin[f"l{l}.o"](att.reshape(B, -1))
            add_norm(delta, self.norms[f"l{l}.norm2"])
            delta = self.ffn[l](h)
        add_norm(delta, self.norms["norm_f"])
        tokens.copy_(self.lin["lm_head"].greedy(h).long())
        pos_t.add_(1)

    def weight_bytes(self) -> float:
        """Algorithmic packed-weight bytes resident on this rank (codes + scales): what a decode step that touches
        every expert streams."""
        tot = sum(l.pw.nbytes for l in self.lin.values())
        for m in self.moe:
            tot += sum(p.nbytes for ws in (m.gate, m.up, m.down) for p in ws)
        return float(tot)
