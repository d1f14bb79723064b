"""Decode-step throughput of a Gemma-shaped decoder with random-init packed weights.

    python -m chadslab_b200.decode_bench --shape gemma7b --batch 1,16,64 --ctx 2048 --steps 16
    torchrun --nproc-per-node N ... -m chadslab_b200.decode_bench ...     (tensor parallel over the N ranks)

The context is synthetic: `ctx` positions of random K/V are placed in the cache instead of running a prefill.
Each batch size is captured as one CUDA graph per step and replayed; `--eager 1` launches the kernels directly
(what a profiler wants).  `--prefill 8x4096 --fmt int8` times a prefill pass of 8 sequences of 4096 tokens instead
(tcgen05 dequant-GEMM path).  Prints one JSON object on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one decode_attention_kernel launch under ncu, and the K/V
# bytes that launch streams: batch 32, 16 query / 16 KV heads x 256, 2048 positions, bf16 cache (the 8-positions-per-trip
# variant the headline step runs).
NCU_ATT_TRAFFIC_MB = 1081.77
NCU_ATT_ALGORITHMIC_MB = 1074.27


def _flush_l2(torch, buf):
    buf.zero_()


def _headline(torch, dist, rank, world, dec, cfg, B, ctx, step, tokens, steps, ms, launches, bpt, kv_bytes):
    """For the batch the benchmark quotes: the same step driven from host buffers (token ids in from pinned memory, new
    ids out, every step) and the largest quantized-matmul launch of the step -- the head on this rank's vocabulary
    slice -- timed alone with events, L2 flushed between launches."""
    import json
    import os
    from chadslab_b200 import _lib
    from chadslab_b200.synth import algorithmic_bytes
    lib = _lib.lib()
    h_in = torch.randint(0, cfg.vocab, (B,), dtype=torch.int64).pin_memory()
    h_out = torch.empty((B,), dtype=torch.int64).pin_memory()

    # one graph launch per step: copy of the ids from pinned host memory, the step, copy of the new ids back
    dec.pos = ctx
    step_h, _ = dec.make_graph_stepper(B, h_in.to("cuda"), start_pos=ctx, host_in=h_in, host_out=h_out)

    def e2e_step():
        step_h()
        torch.cuda.current_stream().synchronize()
    for _ in range(3):
        e2e_step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    import time
    t0 = time.perf_counter()
    for _ in range(steps):
        e2e_step()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / steps
    t = torch.tensor([e2e_ms], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t[0])
    # the head launch alone
    head = dec.lin["lm_head"]
    pw = head.pw
    x = torch.randn((B, pw.K), device="cuda").to(torch.bfloat16)
    y = torch.empty((B, pw.N), dtype=torch.float32, device="cuda")
    flush = torch.empty((256 << 20,), dtype=torch.uint8, device="cuda")
    st = torch.cuda.current_stream().cuda_stream
    call = lambda: _lib.check(lib.bq_qlinear(pw.handle, x.data_ptr(), 1, B, y.data_ptr(), 0, st))
    call()
    n0 = lib.bq_launch_count()
    call()
    head_launches = lib.bq_launch_count() - n0
    times = []
    for _ in range(8):
        _flush_l2(torch, flush)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        call()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    us = sorted(times)[len(times) // 2] * 1e3
    abytes = algorithmic_bytes(pw.N, pw.K, pw.fmt, B)
    peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peak, src = (float(json.load(open(peaks_path))["hbm_gbs"]), "measured") if os.path.exists(peaks_path) else (6650.0, "fallback")
    ach = abytes / us / 1e3
    quant = {"bound": "hbm", "achieved": round(ach, 1), "peak": peak, "unit": "GB/s", "frac": round(ach / peak, 4),
             "traffic": None, "traffic_source": "not captured in this run",
             "peak_source": src, "kernel": f"lm_head {'int8' if pw.fmt == 0 else 'q4'}-g32 ({pw.N},{pw.K}) M={B}: the largest "
                                           f"quantized-matmul launch of the step ({head_launches} kernel"
                                           f"{'s' if head_launches != 1 else ''}: activation pre-pass + GEMM when M > 16)",
             "algorithmic_bytes": int(abytes), "launch_us": round(us, 2), "share_of_step": round(us / (ms * 1e3), 4),
             "frac_of_nominal_8TBs": round(ach / 8000, 4)}
    # decode attention of one layer alone (RoPE + KV append + single-query attention over the ctx-position cache)
    c = cfg
    kc, vc = dec.k_cache[0], dec.v_cache[0]
    S = kc.shape[1]
    qkv = torch.randn((B, (dec.h_local + 2 * dec.kv_local) * c.head_dim), device="cuda")
    att = torch.empty((B, dec.h_local, c.head_dim), dtype=kc.dtype, device="cuda")
    pos_t = torch.tensor([ctx], device="cuda", dtype=torch.int64)
    acall = lambda: _lib.check(lib.bq_decode_attention_rope(qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos_t.data_ptr(),
                                                            att.data_ptr(), B, dec.h_local, dec.kv_local, c.head_dim, S,
                                                            c.rope_base, 1 if kc.dtype == torch.bfloat16 else 0, st))
    acall()
    times = []
    for _ in range(8):
        _flush_l2(torch, flush)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        acall()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    aus = sorted(times)[len(times) // 2] * 1e3
    att_bytes = 2.0 * B * (ctx + 1) * dec.kv_local * c.head_dim * kc.element_size() + B * dec.h_local * c.head_dim * (4 + kc.element_size())
    aach = att_bytes / aus / 1e3
    attn = {"bound": "hbm", "achieved": round(aach, 1), "peak": peak, "unit": "GB/s", "frac": round(aach / peak, 4),
            "traffic": int(att_bytes * NCU_ATT_TRAFFIC_MB / NCU_ATT_ALGORITHMIC_MB),
            "traffic_source": (f"scaled, not re-measured in this run: one ncu capture of this kernel at batch 32 (16 heads x 256, 2048 positions) "
                               f"read + wrote {NCU_ATT_TRAFFIC_MB} MB of DRAM for {NCU_ATT_ALGORITHMIC_MB} MB of K/V rows; the traffic is "
                               "proportional to the rows streamed"),
            "peak_source": src, "kernel": f"decode attention of one layer: batch {B}, {dec.h_local} query / {dec.kv_local} KV heads x "
                                          f"{c.head_dim}, {ctx}-position cache ({'bf16' if kc.element_size() == 2 else 'fp32'}): K and V "
                                          "rows are the algorithmic bytes",
            "algorithmic_bytes": int(att_bytes), "launch_us": round(aus, 2),
            "share_of_step": round(aus * c.layers / (ms * 1e3), 4), "frac_of_nominal_8TBs": round(aach / 8000, 4)}
    del flush, x, y, qkv, att
    dominant, other = (attn, quant) if aus * c.layers >= us else (quant, attn)
    return {"ms_per_step": ms, "e2e_ms_per_step": e2e_ms, "launches_per_step": int(launches),
            "stream_GB_per_step_per_gpu": round((bpt + B * kv_bytes) / 1e9, 3),
            "frac_of_hbm_peak": round((bpt + B * kv_bytes) / ms / 1e6 / peak, 4),
            "roofline": dominant, "roofline_quantized_matmul" if dominant is attn else "roofline_attention": other}


def run(torch, dist, rank: int, world: int, shape: str = "gemma7b", batches=(1, 16, 64), ctx: int = 2048, steps: int = 16,
        eager: bool = False, warmup: int = 3, headline_batch=None):
    """Runs on every rank; returns the report (complete on rank 0).  `headline_batch`: also measure that batch end to
    end from host buffers and time its largest quantized-matmul launch alone (`headline` in the report)."""
    import chadslab_b200 as cb
    from chadslab_b200 import _lib
    from chadslab_b200.decoder import GEMMA_2B_SHAPE, GEMMA_7B_SHAPE, QuantDecoder
    cfg = {"gemma2b": GEMMA_2B_SHAPE, "gemma7b": GEMMA_7B_SHAPE}[shape]
    fmt = "int8-g32" if cfg.fmt == 0 else "q4-g32"
    out = {"model": f"{shape}-shape {fmt}, bf16 activations, random-init", "tensor_parallel": world,
           "context": f"{ctx} positions of synthetic (random) K/V in the cache instead of a prefill pass",
           "exchange": "peer-memory communicator (GEMV deposits + fused sum/add/RMSNorm)" if world > 1 else "none",
           "timing": (f"{steps} eager steps" if eager else f"{steps} CUDA-graph replays") + f" after {warmup}, CUDA events, max over ranks",
           "batches": []}
    comm = None
    try:
        max_b = max(batches)
        if world > 1:
            comm = cb.PeerComm(max_elems=max(max_b * cfg.hidden, 4096), group=dist.group.WORLD)
            _lib.check(_lib.lib().bq_comm_set_timeout_ms(comm.handle, 1000))   # a benchmark should fail fast
        spare = warmup + 2 * steps + 16            # cache rows behind the context: every step of a batch size writes one
        dec = QuantDecoder.random(cfg, seed=0, act_dtype=torch.bfloat16, rank=rank, world=world, max_seq=ctx + spare,
                                  max_batch=max_b, comm=comm)
        for kc, vc in zip(dec.k_cache, dec.v_cache):
            kc.normal_()
            vc.normal_()
        bpt = dec.linear_bytes_per_token()
        kv_bytes = sum(k[:1, :ctx].numel() * k.element_size() for k in dec.k_cache) * 2      # K + V, per sequence
        for B in batches:
            g = torch.Generator(device="cuda").manual_seed(B)
            first = torch.randint(0, cfg.vocab, (B,), device="cuda", generator=g)
            dec.pos = ctx
            if eager:
                tokens = first.clone()
                pos_t = torch.tensor([ctx], device="cuda", dtype=torch.int64)

                def step():
                    dec._step_static(tokens, pos_t)
                    pos_t.fill_(ctx)                     # stay at the same position
            else:
                n0 = _lib.lib().bq_launch_count()
                step, tokens = dec.make_graph_stepper(B, first, start_pos=ctx)
                launches = (_lib.lib().bq_launch_count() - n0) // 2       # warm-up step + captured step
            step()
            torch.cuda.synchronize()
            st = int(_lib.lib().bq_status_poll())
            if st != 0:                      # e.g. a peer that never delivered: do not time the remaining steps
                raise RuntimeError(f"device status {st} after the first step at batch {B}")
            for _ in range(max(0, warmup - 1)):
                step()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            a.record()
            for _ in range(steps):
                step()
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b) / steps], device="cuda")
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
            out["batches"].append({"batch": B, "ms_per_step": round(ms, 4), "tokens_per_s": round(B * 1e3 / ms, 1),
                                   "stream_gbs_per_gpu": round((bpt + B * kv_bytes) / ms / 1e6, 1)})
            if headline_batch == B and not eager:
                out["headline"] = _headline(torch, dist, rank, world, dec, cfg, B, ctx, step, tokens, steps, ms, launches, bpt,
                                            kv_bytes)
            del step
        out["linear_GB_per_step_per_gpu"] = round(bpt / 1e9, 3)
        out["kv_GB_per_sequence_per_gpu"] = round(kv_bytes / 1e9, 3)
        out["status"] = int(_lib.lib().bq_status_poll())
        del dec
    except Exception as e:  # the caller decides what a failure means
        out["error"] = repr(e)[:300]
    if comm is not None:
        try:
            comm.close()
        except Exception as e:
            out["close_error"] = repr(e)[:200]
    torch.cuda.empty_cache()
    return out


def run_prefill(torch, dist, rank: int, world: int, shape: str = "gemma7b", fmt: int = 0, B: int = 8, T: int = 4096,
                reps: int = 2):
    """Prefill of B sequences of T random token ids through the eager path (tcgen05 dequant-GEMM for every linear,
    PyTorch attention and glue, NCCL all-reduce after the row-parallel linears).  Runs on every rank."""
    import dataclasses
    from chadslab_b200 import _lib
    from chadslab_b200.decoder import GEMMA_2B_SHAPE, GEMMA_7B_SHAPE, QuantDecoder
    cfg = dataclasses.replace({"gemma2b": GEMMA_2B_SHAPE, "gemma7b": GEMMA_7B_SHAPE}[shape], fmt=fmt)
    out = {"model": f"{shape}-shape {'int8' if fmt == 0 else 'q4'}-g32, bf16 activations, random-init",
           "tensor_parallel": world, "batch": B, "seq_len": T,
           "timing": f"{reps} passes after 1, CUDA events, max over ranks; last position projected by the head"}
    try:
        dec = QuantDecoder.random(cfg, seed=0, act_dtype=torch.bfloat16, rank=rank, world=world, max_seq=T, max_batch=B)
        g = torch.Generator(device="cuda").manual_seed(0)
        tokens = torch.randint(0, cfg.vocab, (B, T), device="cuda", generator=g)
        lin_weights = sum((l.linear if hasattr(l, "linear") else l).pw.N * (l.linear if hasattr(l, "linear") else l).pw.K
                          for n, l in dec.lin.items() if n != "lm_head")
        times = []
        for i in range(reps + 1):
            dec.reset()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            a.record()
            dec.next_tokens(tokens)
            b.record()
            torch.cuda.synchronize()
            if i:
                times.append(a.elapsed_time(b))
        t = torch.tensor([sum(times) / len(times)], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        out.update({"ms": round(ms, 2), "tokens_per_s": round(B * T / ms * 1e3, 1),
                    "linear_tflops_per_gpu": round(2.0 * B * T * lin_weights / ms / 1e9, 1),
                    "status": int(_lib.lib().bq_status_poll())})
        del dec
    except Exception as e:
        out["error"] = repr(e)[:300]
    torch.cuda.empty_cache()
    return out


def main():
    import torch
    import torch.distributed as dist
    from chadslab_b200 import _lib
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="gemma7b", choices=["gemma2b", "gemma7b"])
    ap.add_argument("--batch", default="1,16,64")
    ap.add_argument("--ctx", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=16)
    ap.add_argument("--eager", type=int, default=0)
    ap.add_argument("--prefill", default="", help="BxT: time a prefill pass instead (e.g. 8x4096)")
    ap.add_argument("--fmt", default="", choices=["", "int8", "q4"], help="prefill: weight format (default: the shape's)")
    args = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _lib.init(local)
    if args.prefill:
        B, T = (int(v) for v in args.prefill.lower().split("x"))
        fmt = {"": 0 if args.shape == "gemma2b" else 1, "int8": 0, "q4": 1}[args.fmt]
        rep = run_prefill(torch, dist, rank, world, args.shape, fmt, B, T)
    else:
        rep = run(torch, dist, rank, world, args.shape, tuple(int(b) for b in args.batch.split(",")), args.ctx, args.steps,
                  bool(args.eager))
    if rank == 0:
        print(json.dumps(rep))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
