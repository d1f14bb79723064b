#!/usr/bin/env python
"""Benchmark of the block-quantized matmul hot path, end to end.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--extras 0|1]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...      (N > 1)

Headline (every N): greedy decode tokens/s of the Gemma-7B-shaped decoder of configs[2] — 28 layers, hidden 3072,
16 heads of 256, GeGLU 24576, vocabulary 256000, every linear 4-bit group-32, bf16 activations, a 2048-position
context, batch HEADLINE_BATCH — tensor-parallel over the N GPUs of the run (column / row sharded linears, sums
through the peer-memory communicator, vocabulary-sharded head).  One "step" is one decode step of the whole batch;
the K timed steps are K replays of the captured CUDA graph between two events (device-resident inputs), `e2e` is
the same step driven from host buffers: token ids copied in from pinned memory and the new ids copied back out
every step.  Strong scaling: the work per step is fixed, N GPUs share it.  Weights are random-init (seeded,
N(0, 0.02), quantized with the format's rule) and the context is synthetic (random K/V in the cache).

`roofline` is the kernel with the largest share of the step (decode attention at this batch: K and V rows are its
algorithmic bytes), `roofline_quantized_matmul` the largest quantized-matmul launch of the step (the lm_head on this
rank's vocabulary slice); both are timed alone with CUDA events, L2 flushed between launches.  `extras` holds what else the configs name:
the standalone sweep of configs[1] (with per-problem and aggregate fractions of the HBM peak), the Gemma-2B-shaped
decoder of configs[0], all three batch sizes of configs[2], one sparse-MoE layer and the whole sparse-MoE decoder of
configs[3], the long prefill of configs[4], and `parity`: a small same-weights decoder and MoE layer sharded over
the N ranks of this run and compared with the numpy oracle (the oracle is only ever the checker).

`--impl reference`: the reference checkout has no code for this path, so the CPU arm times the self-authored numpy
oracle on the host cores on a bounded sample of the same decode step (stated in `cpu_baseline.sample`).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

HEADLINE_BATCH = 64
HEADLINE_CTX = 2048
SHAPES = [(2048, 2048), (16384, 2048), (2048, 16384), (256000, 2048)]
FMT_NAMES = {0: "int8_g32", 1: "q4_g32"}
L2_BYTES = 126 * 1024 * 1024

from chadslab_b200.synth import algorithmic_bytes, make_device_weight  # noqa: E402


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# clocks sampling (nvidia-smi in the background during the timed region)
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.gpu_index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            f = [s.strip() for s in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------------
# CPU arm: the numpy oracle on a bounded sample of the headline decode step
# ------------------------------------------------------------------------------------------------
def cpu_decode_sample(steps: int, warmup: int, batch: int = HEADLINE_BATCH, ctx: int = HEADLINE_CTX):
    """One decoder layer of the Gemma-7B shape (q4-g32, fp32 activations, a `ctx`-position KV cache for `batch`
    sequences) plus 32000 rows of the head, timed with the numpy oracle's own functions; a full step is 28 such
    layers and 8 such head slices, so step time = 28 t_layer + 8 t_head (extrapolated, stated in `sample`)."""
    from oracle import model as omodel
    from oracle import spec
    from threadpoolctl import threadpool_info
    from chadslab_b200.decoder import GEMMA_7B_SHAPE as c
    rng = np.random.default_rng(0)
    fmt, Hd, D, Hq, Hkv, Fd = c.fmt, c.hidden, c.head_dim, c.n_heads, c.n_kv_heads, c.ffn

    def q(n, k):       # N(0, 0.02) weights; one 512-row block of random values tiled over the rows keeps set-up short
        blk = rng.normal(0, 0.02, (min(n, 512), k)).astype(np.float32)
        return spec.quantize(np.tile(blk, ((n + 511) // 512, 1))[:n], fmt)
    w = {"q": q(Hq * D, Hd), "k": q(Hkv * D, Hd), "v": q(Hkv * D, Hd), "o": q(Hd, Hq * D), "gate": q(Fd, Hd), "up": q(Fd, Hd),
         "down": q(Hd, Fd), "head": q(32000, Hd)}
    kc = np.tile(rng.normal(0, 1, (1, 64, Hkv, D)).astype(np.float32), (batch, (ctx + 1 + 63) // 64, 1, 1))[:, :ctx + 1]
    vc = kc[:, ::-1].copy()
    x = rng.normal(0, 1, (batch, Hd)).astype(np.float32)
    g1 = np.ones(Hd, np.float32)
    pos = np.full((1,), ctx)

    def lin(name, a):
        return spec.qlinear(a, w[name][0], w[name][1], fmt)

    def layer(x):
        h = omodel.rmsnorm(x, g1)
        qh = np.stack([omodel.rope(r[None], pos)[0] for r in lin("q", h).reshape(batch, Hq, D)])
        kh = np.stack([omodel.rope(r[None], pos)[0] for r in lin("k", h).reshape(batch, Hkv, D)])
        kc[:, ctx], vc[:, ctx] = kh, lin("v", h).reshape(batch, Hkv, D)
        rep = Hq // Hkv
        att = np.einsum("bhd,bshd->bhs", qh, np.repeat(kc, rep, axis=2) if rep > 1 else kc) / np.sqrt(np.float32(D))
        p = spec.softmax(att)
        o = np.einsum("bhs,bshd->bhd", p, np.repeat(vc, rep, axis=2) if rep > 1 else vc).reshape(batch, Hq * D)
        x = x + lin("o", o.astype(np.float32))
        h = omodel.rmsnorm(x, g1)
        return x + lin("down", spec.gelu_tanh(lin("gate", h)) * lin("up", h))

    def head(x):
        return np.argmax(lin("head", omodel.rmsnorm(x, g1)), axis=-1)

    tl, th = [], []
    for i in range(max(1, warmup) + steps):
        t0 = time.perf_counter()
        y = layer(x)
        t1 = time.perf_counter()
        head(y)
        t2 = time.perf_counter()
        if i >= max(1, warmup):
            tl.append(t1 - t0); th.append(t2 - t1)
    step_s = c.layers * statistics.mean(tl) + (c.vocab / 32000.0) * statistics.mean(th)
    threads = max([i.get("num_threads", 1) for i in threadpool_info() if i.get("user_api") == "blas"] or [1])
    return {"value": batch / step_s, "unit": "tokens/s", "cores": int(threads), "kind": "port",
            "sample": "numpy oracle (dequantize to fp32 + np.matmul, fp32 activations): ONE layer of the Gemma-7B shape "
                      f"(q4-g32, batch {batch}, {ctx}-position context) and 32000 of the 256000 head rows, timed "
                      f"{steps}x; step = 28 x layer + 8 x head slice (extrapolated); host cores={os.cpu_count() or 0}, "
                      f"affinity={len(os.sched_getaffinity(0))}",
            "ms_per_step": step_s * 1e3, "layer_ms": statistics.mean(tl) * 1e3, "head_slice_ms": statistics.mean(th) * 1e3}


def headline_config(world: int):
    return {"workload": f"configs[2]: Gemma-7B-shaped decoder (28 layers, hidden 3072, 16 heads x 256, GeGLU 24576, vocab 256000), "
                        f"all linears q4-g32, bf16 activations, greedy decode at batch {HEADLINE_BATCH} behind a "
                        f"{HEADLINE_CTX}-position context (synthetic K/V)",
            "batch": HEADLINE_BATCH, "context": HEADLINE_CTX, "parallelism": f"tp{world}" if world > 1 else "single GPU",
            "l2": "one step streams this rank's packed weights and KV cache, several times the 126 MB L2",
            "launch": "the K timed steps are K replays of one captured CUDA graph"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # a sample step (one layer + a head slice) takes 1.5-3 s on 8-16 host cores: the requested counts are honoured up to
    # 40 + 5 samples, which keeps the whole run within a few minutes
    steps, warmup = max(1, min(args.steps, 40)), max(1, min(args.warmup, 5))
    cb = cpu_decode_sample(steps, warmup)
    line = {"impl": "reference", "metric": "decode_tokens_per_s", "value": cb["value"], "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": cb["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": dict(headline_config(1), note="the reference checkout has no implementation of this path; this arm times "
                                                   "the self-authored numpy oracle on the host cores on a bounded sample"),
            "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# extras
# ------------------------------------------------------------------------------------------------
def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def run_sweep(torch, cb, lib, seed, reps=20):
    """configs[1]: the standalone quantized matmul sweep.  M = 1 for all 8 (shape, format) problems as one CUDA graph
    (weights rotate over distinct copies so that more than 2 x L2 is touched between reuses), then M = 8 ... 4096."""
    from chadslab_b200 import _lib
    peaks = load_peaks()
    gen = torch.Generator(device="cuda").manual_seed(seed)
    stream = torch.cuda.current_stream().cuda_stream
    problems = []
    for (N, K) in SHAPES:
        for fmt in (0, 1):
            wbytes = algorithmic_bytes(N, K, fmt, 0)
            copies = 1 if wbytes > 2 * L2_BYTES else int(np.ceil(2 * L2_BYTES / wbytes))
            base = make_device_weight(torch, N, K, fmt, gen)
            pws = [cb.PackedWeight.from_device(base[0].roll(c, 0).contiguous() if c else base[0],
                                               base[1].roll(c, 0).contiguous() if c else base[1], fmt) for c in range(copies)]
            x = torch.randn((1, K), device="cuda", generator=gen).to(torch.bfloat16)
            y = torch.empty((1, N), dtype=torch.float32, device="cuda")
            problems.append({"N": N, "K": K, "fmt": fmt, "pws": pws, "x": x, "y": y, "i": 0, "bytes": algorithmic_bytes(N, K, fmt, 1)})
            del base

    def launch(p, s):
        pw = p["pws"][p["i"] % len(p["pws"])]
        p["i"] += 1
        _lib.check(lib.bq_qlinear(pw.handle, p["x"].data_ptr(), cb.DT_BF16, 1, p["y"].data_ptr(), cb.DT_F32, s))
    for _ in range(3):
        for p in problems:
            launch(p, stream)
    torch.cuda.synchronize()
    graph, cap = torch.cuda.CUDAGraph(), torch.cuda.Stream()
    cap.wait_stream(torch.cuda.current_stream())
    with torch.cuda.graph(graph, stream=cap):
        cs = torch.cuda.current_stream().cuda_stream
        for _ in range(reps):
            for p in problems:
                launch(p, cs)
    graph.replay()
    torch.cuda.synchronize()
    a, b = _events(torch)
    a.record()
    graph.replay()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / reps
    step_bytes = sum(p["bytes"] for p in problems)
    out = {"workload": "configs[1], M = 1: 8 (shape, format) problems per pass, bf16 x, fp32 y; one CUDA-graph replay of "
                       f"{reps} passes between two events", "ms_per_pass": round(ms, 4), "gbs": round(step_bytes / ms / 1e6, 1),
           "aggregate_frac": round(step_bytes / ms / 1e6 / peaks["hbm_gbs"], 4), "problems": [], "batch_sweep": []}
    for p in problems:
        for _ in range(3):
            launch(p, stream)
        a, b = _events(torch)
        a.record()
        for _ in range(reps):
            launch(p, stream)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / reps
        out["problems"].append({"N": p["N"], "K": p["K"], "fmt": FMT_NAMES[p["fmt"]], "M": 1, "us": round(us, 2),
                                "gbs": round(p["bytes"] / us / 1e3, 1), "frac": round(p["bytes"] / us / 1e3 / peaks["hbm_gbs"], 3),
                                "copies": len(p["pws"])})
    for p in problems:
        if p["N"] < 16384:
            continue
        pw = p["pws"][0]
        for M in (8, 64, 512, 4096):
            x = torch.randn((M, p["K"]), device="cuda").to(torch.bfloat16)
            y = torch.empty((M, p["N"]), dtype=torch.float32, device="cuda")
            call = lambda: _lib.check(lib.bq_qlinear(pw.handle, x.data_ptr(), cb.DT_BF16, M, y.data_ptr(), cb.DT_F32, stream))
            call()
            a, b = _events(torch)
            a.record()
            for _ in range(3):
                call()
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / 3
            tf = 2.0 * M * p["N"] * p["K"] / us / 1e6
            gbs = algorithmic_bytes(p["N"], p["K"], p["fmt"], M) / us / 1e3
            out["batch_sweep"].append({"N": p["N"], "K": p["K"], "fmt": FMT_NAMES[p["fmt"]], "M": M, "us": round(us, 1),
                                       "gbs": round(gbs, 1), "tflops": round(tf, 1),
                                       "frac": round(tf / peaks["bf16_tflops"], 3) if M >= 512 else round(gbs / peaks["hbm_gbs"], 3),
                                       "of": "bf16 burst peak" if M >= 512 else "HBM peak"})
            del x, y
    for p in problems:
        for pw in p["pws"]:
            pw.close()
    torch.cuda.empty_cache()
    return out


def run_gemma2b(torch, cb):
    """configs[0] on the GPU: Gemma-2B-shaped int8-g32 decoder, 128-token prefill then 32 greedy tokens at batch 1
    (CUDA-graph replays), fp32 activations as the config says and bf16 for comparison."""
    from chadslab_b200.decoder import GEMMA_2B_SHAPE, QuantDecoder
    peaks = load_peaks()
    out = {}
    for name, adt in (("fp32_activations", torch.float32), ("bf16_activations", torch.bfloat16)):
        try:
            dec = QuantDecoder.random(GEMMA_2B_SHAPE, seed=0, act_dtype=adt, max_seq=192, max_batch=1)
            g = torch.Generator(device="cuda").manual_seed(0)
            prompt = torch.randint(0, GEMMA_2B_SHAPE.vocab, (1, 128), device="cuda", generator=g)
            dec.next_tokens(prompt)                       # untimed pass: sizes the library's scratch
            dec.reset()
            torch.cuda.synchronize()
            a, b = _events(torch)
            a.record()
            first = dec.next_tokens(prompt)
            b.record()
            torch.cuda.synchronize()
            prefill_ms = a.elapsed_time(b)
            step, tokens = dec.make_graph_stepper(1, first, start_pos=dec.pos)
            for _ in range(3):
                step()
            a, b = _events(torch)
            a.record()
            for _ in range(32):
                step()
            b.record()
            torch.cuda.synchronize()
            ms_tok = a.elapsed_time(b) / 32
            bpt = dec.linear_bytes_per_token()
            out[name] = {"tokens_per_s": round(1e3 / ms_tok, 1), "ms_per_token": round(ms_tok, 4),
                         "prefill_128_tokens_ms": round(prefill_ms, 2),
                         "frac_of_hbm_ceiling": round(bpt / ms_tok / 1e6 / peaks["hbm_gbs"], 4),
                         "linear_GB_per_token": round(bpt / 1e9, 3)}
            del step, dec
        except Exception as e:
            out[name] = {"error": repr(e)[:300]}
        torch.cuda.empty_cache()
    out["model"] = "configs[0]: gemma-2b-shape int8-g32, batch 1, random-init, 128-token prefill then 32 greedy tokens (graph replays)"
    return out


def parity_check(torch, dist, cb, rank, world):
    """Same-weights correctness of the sharded paths of THIS run (not timed): a small decoder and a small MoE layer
    are built from the oracle's seeded weights, sharded over the `world` ranks, run through the peer-memory
    communicator / exchange, and compared with the numpy oracle."""
    from oracle import model as omodel
    from oracle import spec
    from chadslab_b200 import _lib, parallel
    from chadslab_b200.decoder import DecoderConfig, MoEDecoder, QuantDecoder
    out = {"world": world}
    try:
        cfg = dict(layers=2, hidden=512, n_heads=16, n_kv_heads=8, head_dim=64, ffn=2048, vocab=2048, fmt=1)
        w = omodel.random_weights(cfg, seed=21)
        prompt = np.random.default_rng(5).integers(0, cfg["vocab"], (1, 6))
        ref_tokens, ref_logits = omodel.OracleDecoder(cfg, w).generate(list(prompt[0]), 4)
        comm = cb.PeerComm(max_elems=4 * 4096, group=dist.group.WORLD if world > 1 else None)
        dec = QuantDecoder.from_numpy(DecoderConfig(**cfg), w, act_dtype=torch.float32, rank=rank, world=world, max_seq=32,
                                      comm=comm if world > 1 else None)
        pt = torch.from_numpy(prompt).cuda()
        lg = dec.logits(pt)[0, -1].cpu().numpy()
        out["tp_logits_rel_err"] = float(spec.rel_err(lg, ref_logits[0]))
        dec.reset()
        first = dec.next_tokens(pt)
        step, tokens = dec.make_graph_stepper(1, first, start_pos=dec.pos)       # the captured step: peer-memory sums
        got = [int(first[0])]
        for _ in range(3):
            step()
            got.append(int(tokens[0]))
        out["tp_tokens_equal"] = got == ref_tokens
        out["tp_tokens"] = {"got": got, "oracle": ref_tokens}
        del step, dec
        comm.close()
    except Exception as e:
        out["tp_error"] = repr(e)[:300]
    try:
        rng = np.random.default_rng(2)
        E, H, Fd, k, fmt = 16, 256, 256, 4, 1
        q = lambda W: spec.quantize(W.astype(np.float32), fmt)
        router = q(rng.normal(0, 0.5, (E, H)))
        gate = [q(rng.normal(0, 0.05, (Fd, H))) for _ in range(E)]
        up = [q(rng.normal(0, 0.05, (Fd, H))) for _ in range(E)]
        down = [q(rng.normal(0, 0.05, (H, Fd))) for _ in range(E)]
        xs = [spec.bf16_round(rng.normal(0, 1, (5 + 3 * r, H)).astype(np.float32)) for r in range(world)]   # ragged
        x = xs[rank]
        mk = lambda cs: cb.PackedWeight.from_arrays(cs[0], cs[1], fmt)
        lg_, lu_, ld_ = (parallel.shard_experts(w_, rank, world) for w_ in (gate, up, down))
        ep = cb.PeerEP(E, H, max_send_rows=64 * k, group=dist.group.WORLD if world > 1 else None)
        local = cb.MoEExperts(None, [mk(g) for g in lg_], [mk(u) for u in lu_], [mk(d) for d in ld_], top_k=k)
        layer = parallel.ExpertParallelMoE(cb.QuantLinear(mk(router)), None, E, k, ep=ep, local_moe=local)
        y = layer(torch.from_numpy(x).cuda().to(torch.bfloat16)).cpu().numpy()
        ref, _ = spec.moe_forward(x, router, gate, up, down, fmt, k)
        err = torch.tensor([spec.rel_err(y, ref)], device="cuda")
        if world > 1:
            dist.all_reduce(err, op=dist.ReduceOp.MAX)
        out["ep_layer_rel_err"] = float(err[0])
        ep.close()
        # sparse-MoE decoder, expert parallel, each rank its own sequence, graph decode vs the oracle's tokens
        mcfg = dict(layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=0, vocab=1024, fmt=1, n_experts=16, top_k=2,
                    moe_ffn=256)
        mw = omodel.random_weights(mcfg, seed=12)
        prompts = np.random.default_rng(9).integers(0, mcfg["vocab"], (world, 6))
        ref_tokens, ref_logits = omodel.OracleDecoder(mcfg, mw).generate(list(prompts[rank]), 3)
        ep2 = cb.PeerEP(mcfg["n_experts"], mcfg["hidden"], max_send_rows=6 * mcfg["top_k"],
                        group=dist.group.WORLD if world > 1 else None) if world > 1 else None
        mdec = MoEDecoder.from_numpy(DecoderConfig(**mcfg), mw, act_dtype=torch.float32, rank=rank, world=world, max_seq=32, ep=ep2)
        pt = torch.from_numpy(prompts[rank])[None].cuda()
        lg = mdec.logits(pt)[0, -1].cpu().numpy()
        mdec.reset()
        first = mdec.next_tokens(pt)
        step, tokens = mdec.make_graph_stepper(1, first, start_pos=mdec.pos)
        got = [int(first[0])]
        for _ in range(2):
            step()
            got.append(int(tokens[0]))
        res = torch.tensor([spec.rel_err(lg, ref_logits[0]), 0.0 if got == ref_tokens else 1.0], device="cuda")
        if world > 1:
            dist.all_reduce(res, op=dist.ReduceOp.MAX)
        out["moe_decoder_logits_rel_err"] = float(res[0])
        out["moe_decoder_tokens_equal"] = bool(res[1] == 0)
        del step, mdec
        if ep2 is not None:
            ep2.close()
    except Exception as e:
        out["ep_error"] = repr(e)[:300]
    out["status"] = int(_lib.lib().bq_status_poll())
    out["tolerances"] = "logits <= 1e-3 (dense), <= 2e-3 (MoE decoder), MoE layer <= 4e-3 (bf16 hidden activation between the expert matmuls)"
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist
    import chadslab_b200 as cb
    from chadslab_b200 import _lib, decode_bench, moe_bench

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = _lib.init(local)
    peaks = load_peaks()
    steps, warmup = args.steps, max(3, args.warmup)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    batches = (1, 16, HEADLINE_BATCH) if args.extras else (HEADLINE_BATCH,)
    head = decode_bench.run(torch, dist, rank, world, "gemma7b", batches, HEADLINE_CTX, steps, warmup=warmup,
                            headline_batch=HEADLINE_BATCH)
    clocks = sampler.stop() if rank == 0 else None
    hb = head.get("headline") or {}

    extras = {}
    if args.extras:
        extras["parity"] = parity_check(torch, dist, cb, rank, world)
        if world > 1:
            # the same step on ONE GPU, measured in this run by rank 0 alone (the others wait): the basis of the speed-up
            one = None
            if rank == 0:
                one = decode_bench.run(torch, dist, 0, 1, "gemma7b", batches, HEADLINE_CTX, max(4, steps // 2), warmup=3)
            dist.barrier()
            if rank == 0:
                extras["one_gpu_same_run"] = {"batches": one.get("batches"), "error": one.get("error")}
                by_b = {b["batch"]: b["ms_per_step"] for b in one.get("batches", [])}
                extras["speedup_vs_one_gpu"] = {str(b["batch"]): round(by_b[b["batch"]] / b["ms_per_step"], 3)
                                                for b in head.get("batches", []) if b["batch"] in by_b}
        try:
            extras["moe_layer"] = moe_bench.run(torch, dist, rank, world, tokens=(256, 4096), reps=5)
        except Exception as e:
            extras["moe_layer"] = {"error": repr(e)[:300]}
        try:
            extras["moe_decoder"] = moe_bench.run_decoder(torch, dist, rank, world)
        except Exception as e:
            extras["moe_decoder"] = {"error": repr(e)[:300]}
        try:
            extras["prefill"] = decode_bench.run_prefill(torch, dist, rank, world, "gemma7b", 0, 8, 4096, reps=2)
        except Exception as e:
            extras["prefill"] = {"error": repr(e)[:300]}
        if world == 1:
            try:
                extras["sweep"] = run_sweep(torch, cb, lib, seed=0, reps=max(5, steps))
            except Exception as e:
                extras["sweep"] = {"error": repr(e)[:300]}
            extras["gemma2b_decode"] = run_gemma2b(torch, cb)
    if rank == 0:
        ms = hb.get("ms_per_step")
        value = HEADLINE_BATCH * 1e3 / ms if ms else None
        e2e_ms = hb.get("e2e_ms_per_step")
        line = {
            "metric": "decode_tokens_per_s", "value": round(value, 1) if value else None, "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warmup, "ms_per_step": round(ms, 4) if ms else None, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": headline_config(world),
            "roofline": hb.get("roofline"),
            "roofline_quantized_matmul": hb.get("roofline_quantized_matmul"),
            "e2e": {"value": round(HEADLINE_BATCH * 1e3 / e2e_ms, 1) if e2e_ms else None, "unit": "tokens/s",
                    "h2d_bytes_per_step": HEADLINE_BATCH * 8, "d2h_bytes_per_step": HEADLINE_BATCH * 8,
                    "how": "every step: ONE graph launch that holds the copy of the token ids from pinned host memory, the "
                           "step's kernels and the copy of the new ids back to pinned host memory; stream synchronised, "
                           "wall clock over the steps"},
            "gpu_launches": int(hb.get("launches_per_step", 0)) * steps, "clocks": clocks,
            "step": {"launches_per_step": hb.get("launches_per_step"), "stream_GB_per_step_per_gpu": hb.get("stream_GB_per_step_per_gpu"),
                     "frac_of_hbm_peak": hb.get("frac_of_hbm_peak"), "peak_gbs": peaks["hbm_gbs"], "peak_source": peaks["source"]},
            "tp_decode": {k: head.get(k) for k in ("model", "tensor_parallel", "context", "exchange", "timing", "batches", "status",
                                                   "error") if k in head},
        }
        if world == 1 and args.cpu:
            try:
                cpu = cpu_decode_sample(1, 1)
                line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
            except Exception as e:
                line["cpu_baseline"] = {"error": repr(e)[:300]}
        if extras:
            line["extras"] = extras
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_one_qlinear(args):
    """`--only qlinear`: one weight shape, the given batch sizes and kernel path, CUDA-event timing per launch (the small,
    single-kernel case the ncu summaries under profiles/ are captured on).  One JSON line per (format, M)."""
    import torch
    import chadslab_b200 as cb
    from chadslab_b200 import _lib
    torch.cuda.set_device(0)
    lib = _lib.init(0)
    paths = {"auto": 0, "simt": 1, "tensor": 2, "mma": 3}
    gen = torch.Generator(device="cuda").manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for fname in args.fmt.split(","):
        fmt = {"int8": 0, "q4": 1}[fname]
        codes, scales = make_device_weight(torch, args.n, args.k, fmt, gen)
        pws = [cb.PackedWeight.from_device(codes.roll(c, 0).contiguous() if c else codes,
                                           scales.roll(c, 0).contiguous() if c else scales, fmt) for c in range(args.copies)]
        del codes, scales
        for M in [int(v) for v in args.m.split(",")]:
            x = torch.randn((M, args.k), device="cuda", generator=gen).to(torch.bfloat16)
            y = torch.empty((M, args.n), dtype=torch.float32, device="cuda")
            call = lambda i: _lib.check(lib.bq_qlinear_ex(pws[i % len(pws)].handle, x.data_ptr(), cb.DT_BF16, M, y.data_ptr(),
                                                          cb.DT_F32, paths[args.path], stream))
            for i in range(3):
                call(i)
            a, b = _events(torch)
            a.record()
            for i in range(args.reps):
                call(i)
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / args.reps
            print(json.dumps({"N": args.n, "K": args.k, "fmt": fname, "M": M,
                              "path": {0: "none", 1: "simt", 2: "tensor", 3: "mma"}[lib.bq_last_path()], "us": round(us, 2),
                              "GBps": round(algorithmic_bytes(args.n, args.k, fmt, M) / us / 1e3, 1),
                              "TFLOPs": round(2.0 * M * args.n * args.k / us / 1e6, 2)}), flush=True)
        for p in pws:
            p.close()
    _lib.check(lib.bq_status_poll())


def run_one_attention(args):
    """`--only attention`: the decode-attention kernel alone (RoPE + KV append + single-query attention) on a synthetic
    cache: `--batch` sequences, `--heads` query / `--kv-heads` KV heads of `--head-dim`, `--ctx` positions, bf16."""
    import torch
    from chadslab_b200 import _lib
    torch.cuda.set_device(0)
    lib = _lib.init(0)
    B, Hq, Hkv, D, ctx = args.batch, args.heads, args.kv_heads, args.head_dim, args.ctx
    S = ctx + 8
    g = torch.Generator(device="cuda").manual_seed(0)
    kc = torch.randn((B, S, Hkv, D), device="cuda", generator=g).to(torch.bfloat16)
    vc = torch.randn((B, S, Hkv, D), device="cuda", generator=g).to(torch.bfloat16)
    qkv = torch.randn((B, (Hq + 2 * Hkv) * D), device="cuda", generator=g)
    out = torch.empty((B, Hq, D), dtype=torch.bfloat16, device="cuda")
    pos = torch.tensor([ctx], device="cuda", dtype=torch.int64)
    st = torch.cuda.current_stream().cuda_stream
    call = lambda: _lib.check(lib.bq_decode_attention_rope(qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(),
                                                           out.data_ptr(), B, Hq, Hkv, D, S, 10000.0, 1, st))
    flush = torch.empty((256 << 20,), dtype=torch.uint8, device="cuda")
    call()
    times = []
    for _ in range(args.reps):
        flush.zero_()
        a, b = _events(torch)
        a.record()
        call()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3)
    us = sorted(times)[len(times) // 2]
    nbytes = 2.0 * B * (ctx + 1) * Hkv * D * 2
    print(json.dumps({"kernel": "decode attention", "batch": B, "heads": Hq, "kv_heads": Hkv, "head_dim": D, "ctx": ctx,
                      "us": round(us, 2), "kv_bytes": int(nbytes), "GBps": round(nbytes / us / 1e3, 1)}))
    _lib.check(lib.bq_status_poll())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--extras", type=int, default=1, help="also run the other configs, the parity check and the sweep")
    ap.add_argument("--cpu", type=int, default=1, help="N = 1: also time the numpy oracle sample (cpu_baseline)")
    ap.add_argument("--only", default="", choices=["", "qlinear", "attention"],
                    help="qlinear / attention: time one kernel on one shape instead of the benchmark")
    ap.add_argument("--batch", type=int, default=16)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=16)
    ap.add_argument("--head-dim", type=int, default=256)
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--n", type=int, default=65536)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--fmt", default="int8,q4")
    ap.add_argument("--m", default="1")
    ap.add_argument("--path", default="auto", choices=["auto", "simt", "tensor", "mma"])
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--copies", type=int, default=1)
    args = ap.parse_args()
    if args.only == "qlinear":
        run_one_qlinear(args)
    elif args.only == "attention":
        run_one_attention(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
