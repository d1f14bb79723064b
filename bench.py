#!/usr/bin/env python
"""Benchmark of the block-quantized matmul hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (configs[1] of BASELINE.json, decode-shaped part): the standalone quantized matmul sweep
at M = 1 — W[N,K] ~ N(0, 0.02) quantized to int8-g32 and 4-bit-g32, x[1,K] ~ N(0,1) in bf16, for
(N,K) in {(2048,2048), (16384,2048), (2048,16384), (256000,2048)}.  One "step" is one pass over
all 8 (shape, format) problems.  Metric: quantized GEMV HBM GB/s = algorithmic bytes (codes +
fp16 scales + activations + fp32 outputs) / device time.  Small shapes rotate over enough distinct
weight copies that the bytes touched between two uses of a copy exceed the 126 MB L2.

Lines printed: one JSON object on rank 0.
Multi-GPU (torchrun): every rank runs the same sweep on its own GPU with its own weights (the
sweep has no cross-GPU dependency: weak scaling, no collective on the data path); value is the
sum of bytes over ranks / max time over ranks.
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

SHAPES = [(2048, 2048), (16384, 2048), (2048, 16384), (256000, 2048)]
FMT_NAMES = {0: "int8_g32", 1: "q4_g32"}
L2_BYTES = 126 * 1024 * 1024
DOMINANT = (256000, 2048, 0)      # the launch with the most bytes: int8 lm_head-shaped GEMV
NCU_TRAFFIC_RATIO = 146.4 / 142.7   # measured DRAM traffic / algorithmic bytes (profiles/qgemv_mma_65536x2048.md)


from chadslab_b200.synth import algorithmic_bytes, make_device_weight  # noqa: E402


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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
# synthetic data
# ------------------------------------------------------------------------------------------------
def build_problems(torch, cb, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    problems = []
    for (N, K) in SHAPES:
        for fmt in (0, 1):
            wbytes = algorithmic_bytes(N, K, fmt, 0)
            copies = 1 if wbytes > 2 * L2_BYTES else int(np.ceil(2 * L2_BYTES / wbytes))
            base = make_device_weight(torch, N, K, fmt, gen)
            pws = []
            for c in range(copies):
                if c:   # distinct memory, rolled rows (cheap) so contents differ as well
                    codes, scales = base[0].roll(c, 0).contiguous(), base[1].roll(c, 0).contiguous()
                else:
                    codes, scales = base
                pws.append(cb.PackedWeight.from_device(codes, scales, fmt))
            x = torch.randn((1, K), device="cuda", generator=gen).to(torch.bfloat16)
            y = torch.empty((1, N), dtype=torch.float32, device="cuda")
            problems.append({"N": N, "K": K, "fmt": fmt, "pws": pws, "x": x, "y": y, "i": 0,
                             "bytes": algorithmic_bytes(N, K, fmt, 1)})
            del base
    return problems


# ------------------------------------------------------------------------------------------------
# CPU arm (oracle port of the path; the reference checkout has no code for it)
# ------------------------------------------------------------------------------------------------
def cpu_sample(steps: int, warmup: int):
    """The numpy oracle on a bounded sample of the sweep: every shape/format at M=1, the 256000-row
    shape cut to its first 32000 rows.  Weights are dequantized per call (as the GPU kernel does)."""
    from oracle import spec
    from threadpoolctl import threadpool_info
    rng = np.random.default_rng(0)
    probs = []
    for (N, K) in SHAPES:
        n = min(N, 32000)
        W = rng.normal(0, 0.02, (n, K)).astype(np.float32)
        for fmt in (0, 1):
            codes, scales = spec.quantize(W, fmt)
            x = spec.bf16_round(rng.normal(0, 1, (1, K)).astype(np.float32))
            probs.append((codes, scales, fmt, x, algorithmic_bytes(n, K, fmt, 1)))
    total = sum(p[4] for p in probs)

    def one_pass():
        for codes, scales, fmt, x, _ in probs:
            spec.qlinear(x, codes, scales, fmt)

    for _ in range(max(1, warmup)):
        one_pass()
    t0 = time.perf_counter()
    for _ in range(steps):
        one_pass()
    dt = (time.perf_counter() - t0) / steps
    threads = max([i.get("num_threads", 1) for i in threadpool_info() if i.get("user_api") == "blas"] or [1])
    return {"value": total / dt / 1e9, "unit": "GB/s", "cores": int(threads), "kind": "port",
            "sample": "numpy oracle (dequantize to fp32 + np.matmul), M=1, all 8 problems of the sweep with the "
                      "256000-row shape cut to 32000 rows; host cores=%d, affinity=%d" % (
                          os.cpu_count() or 0, len(os.sched_getaffinity(0))),
            "ms_per_pass": dt * 1e3}


# ------------------------------------------------------------------------------------------------
# extras (reported beside the headline, N=1 only): the rest of configs[1] and a decode loop
# ------------------------------------------------------------------------------------------------
def run_extras(torch, cb, lib, problems):
    from chadslab_b200 import _lib
    from chadslab_b200.decoder import GEMMA_2B_SHAPE, QuantDecoder
    stream = torch.cuda.current_stream().cuda_stream
    out = {"batch_sweep": [], "note": "batch_sweep: same weights as the headline, bf16 activations, CUDA events, "
                                      "3 launches each after 1 warm-up; decode: Gemma-2B-shaped decoder, int8-g32, "
                                      "batch 1, random-init, 128-token prefill then 32 greedy tokens replayed from a "
                                      "CUDA graph"}
    for p in problems:
        if p["N"] < 16384:
            continue
        pw = p["pws"][0]
        for M in (8, 64, 512, 4096):
            x = torch.randn((M, p["K"]), device="cuda").to(torch.bfloat16)
            y = torch.empty((M, p["N"]), dtype=torch.float32, device="cuda")
            call = lambda: _lib.check(lib.bq_qlinear(pw.handle, x.data_ptr(), cb.DT_BF16, M, y.data_ptr(), cb.DT_F32, stream))
            call()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(3):
                call()
            b.record()
            torch.cuda.synchronize()
            us = a.elapsed_time(b) * 1e3 / 3
            out["batch_sweep"].append({"N": p["N"], "K": p["K"], "fmt": FMT_NAMES[p["fmt"]], "M": M, "us": round(us, 1),
                                       "gbs": round(algorithmic_bytes(p["N"], p["K"], p["fmt"], M) / us / 1e3, 1),
                                       "tflops": round(2.0 * M * p["N"] * p["K"] / us / 1e6, 1)})
            del x, y
    for p in problems:
        for pw in p["pws"]:
            pw.close()
    torch.cuda.empty_cache()
    try:
        dec = QuantDecoder.random(GEMMA_2B_SHAPE, seed=0, act_dtype=torch.bfloat16, max_seq=192, max_batch=1)
        g = torch.Generator(device="cuda").manual_seed(0)
        prompt = torch.randint(0, GEMMA_2B_SHAPE.vocab, (1, 128), device="cuda", generator=g)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        first = dec.next_tokens(prompt)
        torch.cuda.synchronize()
        prefill_s = time.perf_counter() - t0
        step, tokens = dec.make_graph_stepper(1, first, start_pos=dec.pos)
        for _ in range(3):
            step()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(32):
            step()
        b.record()
        torch.cuda.synchronize()
        ms_tok = a.elapsed_time(b) / 32
        bpt = dec.linear_bytes_per_token()
        peak, _ = load_peaks()
        out["decode"] = {"model": "gemma-2b-shape int8-g32, bf16 activations, batch 1", "tokens_per_s": round(1e3 / ms_tok, 1),
                         "ms_per_token": round(ms_tok, 4), "linear_GB_per_token": round(bpt / 1e9, 3),
                         "linear_stream_gbs": round(bpt / ms_tok / 1e6, 1),
                         "frac_of_hbm_ceiling": round(bpt / ms_tok / 1e6 / peak, 4),
                         "prefill_128_tokens_s": round(prefill_s, 4)}
    except Exception as e:  # extras never break the headline line
        out["decode"] = {"error": repr(e)[:300]}
    return out


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = min(args.steps, 5)
    cb = cpu_sample(steps, min(args.warmup, 1))
    line = {"impl": "reference", "metric": "quantized_gemv_hbm_gbs", "value": cb["value"], "unit": "GB/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": cb["ms_per_pass"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "configs[1] quantized matmul sweep, M=1 (bounded CPU sample)",
                       "note": "the reference checkout has no implementation of this path; this arm times the "
                               "self-authored numpy oracle on the host cores"},
            "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist
    import chadslab_b200 as cb
    from chadslab_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = _lib.init(local)
    problems = build_problems(torch, cb, seed=rank)
    stream = torch.cuda.current_stream().cuda_stream
    step_bytes = sum(p["bytes"] for p in problems)

    def launch(p):
        pw = p["pws"][p["i"] % len(p["pws"])]
        p["i"] += 1
        _lib.check(lib.bq_qlinear(pw.handle, p["x"].data_ptr(), cb.DT_BF16, 1, p["y"].data_ptr(), cb.DT_F32, stream))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    dom = [p for p in problems if (p["N"], p["K"], p["fmt"]) == DOMINANT][0]
    for _ in range(max(3, args.warmup)):
        for p in problems:
            launch(p)
    barrier()

    # ---- the K steps as one CUDA graph (what a decode loop replays); copies rotate inside it -------
    launches0 = lib.bq_launch_count()
    graph = torch.cuda.CUDAGraph()
    cap_stream = torch.cuda.Stream()
    cap_stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.graph(graph, stream=cap_stream):
        cs = torch.cuda.current_stream().cuda_stream
        for s in range(args.steps):
            for p in problems:
                pw = p["pws"][p["i"] % len(p["pws"])]
                p["i"] += 1
                _lib.check(lib.bq_qlinear(pw.handle, p["x"].data_ptr(), cb.DT_BF16, 1, p["y"].data_ptr(), cb.DT_F32, cs))
    launches = lib.bq_launch_count() - launches0          # kernels of ours inside one replay = the timed region
    graph.replay()                                          # one untimed replay (graph upload)
    barrier()

    # ---- timed region: device-resident inputs, exactly K steps = one replay ---------------------------
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    graph.replay()
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)

    # ---- the same K steps launched eagerly, with events around the dominant kernel (roofline) ----------
    dom_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    eg0, eg1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    eg0.record()
    for s in range(args.steps):
        for p in problems:
            if p is dom:
                dom_ev[s][0].record()
                launch(p)
                dom_ev[s][1].record()
            else:
                launch(p)
    eg1.record()
    barrier()
    ms_eager = eg0.elapsed_time(eg1)
    dom_ms = statistics.mean(a.elapsed_time(b) for a, b in dom_ev)

    # ---- per-problem timings (reported in "detail"; not the headline) ----------------------------
    detail = []
    for p in problems:
        reps = max(args.steps, 20)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            launch(p)
        a.record()
        for _ in range(reps):
            launch(p)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) * 1e3 / reps
        detail.append({"N": p["N"], "K": p["K"], "fmt": FMT_NAMES[p["fmt"]], "M": 1, "us": round(us, 2),
                       "gbs": round(p["bytes"] / us / 1e3, 1), "copies": len(p["pws"])})

    # ---- end to end: host buffers through the C ABI (H2D of x and D2H of y inside the timing) ----
    hx = [torch.randn((1, p["K"])).to(torch.bfloat16).pin_memory() for p in problems]
    hy = [torch.empty((1, p["N"]), dtype=torch.float32).pin_memory() for p in problems]

    def e2e_pass():
        for p, x, y in zip(problems, hx, hy):
            pw = p["pws"][p["i"] % len(p["pws"])]
            p["i"] += 1
            _lib.check(lib.bq_qlinear_host(pw.handle, x.data_ptr(), cb.DT_BF16, 1, y.data_ptr(), cb.DT_F32))

    for _ in range(3):
        e2e_pass()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        e2e_pass()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms_total, e2e_s * 1e3], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms = float(t[0]), float(t[1])

    tp_decode = None
    moe_layer = None
    if args.extras:      # configs[2]: Gemma-7B-shaped decoder, 4-bit g32, tensor-parallel over all ranks of the run
        from chadslab_b200 import decode_bench
        tp_decode = decode_bench.run(torch, dist, rank, world, "gemma7b", (1, 16, 64), 2048, 16)
        try:             # configs[3]: one sparse-MoE layer (128 experts, top-8, q4), expert-parallel over the ranks
            from chadslab_b200 import moe_bench
            moe_layer = moe_bench.run(torch, dist, rank, world, tokens=(256, 4096), reps=5)
        except Exception as e:  # extras never break the headline line
            moe_layer = {"error": repr(e)[:300]}
    if rank == 0:
        peak, peak_src = load_peaks()
        value = world * step_bytes * args.steps / (ms_total * 1e-3) / 1e9
        e2e_value = world * step_bytes * args.steps / (e2e_ms * 1e-3) / 1e9
        achieved = dom["bytes"] / (dom_ms * 1e-3) / 1e9
        cpu = cpu_sample(2, 1) if world == 1 else None
        extras = None
        if world == 1 and args.extras:
            del hx, hy
            for p in problems:           # keep only what the extras reuse
                for pw in p["pws"][1:]:
                    pw.close()
                p["pws"] = p["pws"][:1]
            torch.cuda.empty_cache()
            extras = run_extras(torch, cb, lib, problems)
        line = {
            "metric": "quantized_gemv_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms_total / args.steps, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "configs[1] quantized matmul sweep, decode-shaped M=1: (N,K) in "
                                   "{(2048,2048),(16384,2048),(2048,16384),(256000,2048)} x {int8-g32, q4-g32}, "
                                   "x bf16 N(0,1), W N(0,0.02)",
                       "l2": "weights rotate over distinct copies so > 2x L2 (126 MB) is touched between reuses; "
                             "the 256000-row weights exceed L2 by themselves",
                       "launch": "the K timed steps are one CUDA-graph replay; roofline.achieved is the same kernel timed "
                                 "with events in an eager pass of the same step sequence",
                       "bytes_per_step_per_gpu": int(step_bytes), "parallelism": f"independent sweep per GPU x{world}"},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4), "traffic": int(NCU_TRAFFIC_RATIO * dom["bytes"]),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of the same kernel on a 65536-row "
                                           "case (146.4 MB for 142.7 MB algorithmic), scaled by rows to this launch",
                         "peak_source": peak_src,
                         "kernel": "qgemv int8-g32 (256000,2048) M=1", "frac_of_nominal_8TBs": round(achieved / 8000, 4),
                         "launch_us": round(dom_ms * 1e3, 2)},
            "e2e": {"value": round(e2e_value, 1), "unit": "GB/s",
                    "h2d_bytes_per_step": int(sum(p["K"] * 2 for p in problems)),
                    "d2h_bytes_per_step": int(sum(p["N"] * 4 for p in problems))},
            "gpu_launches": int(launches), "clocks": clocks, "detail": detail,
            "eager_ms_per_step": round(ms_eager / args.steps, 4),
        }
        if cpu:
            line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
        if extras:
            line["extras"] = extras
        if tp_decode:
            line.setdefault("extras", {})["tp_decode"] = tp_decode
        if moe_layer:
            line.setdefault("extras", {})["moe_layer"] = moe_layer
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--extras", type=int, default=1, help="also report the batch sweep and decode tokens/s (N=1 only)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
