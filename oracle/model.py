"""numpy decoder used as the end-to-end oracle (TEST INFRASTRUCTURE; self-authored, parity unpinned — the
reference checkout has no LLM runtime).  Gemma-shaped block: RMSNorm -> q/k/v -> RoPE -> causal GQA attention
with a KV cache -> o -> residual -> RMSNorm -> GeGLU FFN -> residual; final RMSNorm -> lm_head -> argmax.
Open choices (the specification is silent): RMSNorm weight multiplies directly (initialised to 1), eps 1e-6,
no embedding scaling, no logit soft-capping, rotate-half RoPE with base 10000, untied fp32 embedding table.
A config with `n_experts` > 0 replaces the dense FFN of every layer by the sparse-MoE FFN of spec.moe_forward
(router -> softmax -> top-k -> SwiGLU experts -> weighted combine); the MoE block sees its input rounded to bf16
(`moe_in_bf16`, the activation type the specification names for the quantized matmuls) and rounds the hidden
activation to bf16 between the expert matmuls, as spec.moe_experts does."""
from __future__ import annotations

import numpy as np

from . import spec


def rmsnorm(x, w, eps=1e-6):
    x = x.astype(np.float32)
    return (x / np.sqrt((x * x).mean(-1, keepdims=True) + np.float32(eps))) * w


def rope(x, pos, base=10000.0):
    """x [T, heads, d]; rotate-half convention; pos [T]."""
    d = x.shape[-1]
    inv = (1.0 / (base ** (np.arange(0, d, 2, dtype=np.float32) / d))).astype(np.float32)
    ang = pos.astype(np.float32)[:, None] * inv[None, :]
    cos, sin = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return np.concatenate([x1 * cos - x2 * sin, x2 * cos + x1 * sin], axis=-1).astype(np.float32)


class OracleDecoder:
    def __init__(self, cfg: dict, weights: dict):
        self.c, self.w = cfg, weights
        self.kc = [np.zeros((0, cfg["n_kv_heads"], cfg["head_dim"]), np.float32) for _ in range(cfg["layers"])]
        self.vc = [np.zeros((0, cfg["n_kv_heads"], cfg["head_dim"]), np.float32) for _ in range(cfg["layers"])]
        self.pos = 0

    def _lin(self, name, x):
        codes, scales = self.w[name]
        return spec.qlinear(x, codes, scales, self.c["fmt"])

    def forward(self, tokens):
        c = self.c
        T = len(tokens)
        x = self.w["embed"][np.asarray(tokens)].astype(np.float32)
        pos = np.arange(self.pos, self.pos + T)
        H, KV, D = c["n_heads"], c["n_kv_heads"], c["head_dim"]
        for l in range(c["layers"]):
            h = rmsnorm(x, self.w[f"l{l}.norm1"])
            q = rope(self._lin(f"l{l}.q", h).reshape(T, H, D), pos)
            k = rope(self._lin(f"l{l}.k", h).reshape(T, KV, D), pos)
            v = self._lin(f"l{l}.v", h).reshape(T, KV, D)
            self.kc[l] = np.concatenate([self.kc[l], k], 0)
            self.vc[l] = np.concatenate([self.vc[l], v], 0)
            S = self.kc[l].shape[0]
            rep = H // KV
            kk = np.repeat(self.kc[l], rep, axis=1)          # [S, H, D]
            vv = np.repeat(self.vc[l], rep, axis=1)
            att = np.einsum("thd,shd->hts", q, kk) / np.sqrt(np.float32(D))
            mask = np.arange(S)[None, :] > pos[:, None]
            att = np.where(mask[None], -np.inf, att)
            p = spec.softmax(att)
            o = np.einsum("hts,shd->thd", p, vv).reshape(T, H * D).astype(np.float32)
            x = x + self._lin(f"l{l}.o", o)
            h = rmsnorm(x, self.w[f"l{l}.norm2"])
            if c.get("n_experts", 0):
                E = c["n_experts"]
                if c.get("moe_in_bf16", True):
                    h = spec.bf16_round(h)
                y, _ = spec.moe_forward(h, self.w[f"l{l}.router"], [self.w[f"l{l}.e{e}.gate"] for e in range(E)],
                                        [self.w[f"l{l}.e{e}.up"] for e in range(E)],
                                        [self.w[f"l{l}.e{e}.down"] for e in range(E)], c["fmt"], c["top_k"])
                x = x + y
                continue
            a = spec.gelu_tanh(self._lin(f"l{l}.gate", h)) * self._lin(f"l{l}.up", h)
            x = x + self._lin(f"l{l}.down", a)
        self.pos += T
        return self._lin("lm_head", rmsnorm(x, self.w["norm_f"]))

    def generate(self, prompt, n_new):
        logits = self.forward(prompt)
        out, all_logits = [], [logits[-1]]
        tok = int(np.argmax(logits[-1]))
        for _ in range(n_new):
            out.append(tok)
            logits = self.forward([tok])
            all_logits.append(logits[-1])
            tok = int(np.argmax(logits[-1]))
        return out, np.stack(all_logits)


def random_weights(cfg: dict, seed: int = 0):
    """Seeded N(0, 0.02) weights, quantized with the oracle's packer."""
    rng = np.random.default_rng(seed)
    c = cfg
    Hd, H, KV, D, F, V = c["hidden"], c["n_heads"], c["n_kv_heads"], c["head_dim"], c["ffn"], c["vocab"]
    q = lambda n, k: spec.quantize(rng.normal(0, 0.02, (n, k)).astype(np.float32), c["fmt"])
    w = {"embed": rng.normal(0, 0.02, (V, Hd)).astype(np.float32) * 50, "norm_f": np.ones(Hd, np.float32),
         "lm_head": q(V, Hd)}
    for l in range(c["layers"]):
        w[f"l{l}.norm1"] = np.ones(Hd, np.float32)
        w[f"l{l}.norm2"] = np.ones(Hd, np.float32)
        w[f"l{l}.q"], w[f"l{l}.k"], w[f"l{l}.v"] = q(H * D, Hd), q(KV * D, Hd), q(KV * D, Hd)
        w[f"l{l}.o"] = q(Hd, H * D)
        if c.get("n_experts", 0):
            Fm = c["moe_ffn"]
            w[f"l{l}.router"] = spec.quantize(rng.normal(0, 0.3, (c["n_experts"], Hd)).astype(np.float32), c["fmt"])
            for e in range(c["n_experts"]):
                w[f"l{l}.e{e}.gate"], w[f"l{l}.e{e}.up"], w[f"l{l}.e{e}.down"] = q(Fm, Hd), q(Fm, Hd), q(Hd, Fm)
        else:
            w[f"l{l}.gate"], w[f"l{l}.up"], w[f"l{l}.down"] = q(F, Hd), q(F, Hd), q(Hd, F)
    return w
