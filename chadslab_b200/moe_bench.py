"""Throughput of one sparse-MoE FFN layer: router -> top-k -> permute -> gather -> grouped SwiGLU experts -> combine.

    python -m chadslab_b200.moe_bench --tokens 256,4096,32768 [--experts 128 --hidden 2048 --ffn 768 --top-k 8 --fmt q4]
    torchrun --nproc-per-node N ... -m chadslab_b200.moe_bench ...   (expert parallel: E/N experts and tokens/N per rank)

Random-init packed weights generated on the device; router logits come from x . Wr^T with x ~ N(0,1).  Per token
count: microseconds of the whole layer (replays of one captured CUDA graph, as a decode step runs it; the eager figure
beside it includes the host time between launches) and of its stages (CUDA events, `--reps` launches after 2), the expert
weight bytes one pass streams (every expert that received a token), the resulting GB/s, and TFLOP/s of the expert
matmuls.  Prints one JSON object on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os


def _timed(torch, fn, reps):
    for _ in range(2):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) * 1e3 / reps


def _timed_graph(torch, fn, reps):
    """The same launches captured once and replayed (how a decode step runs them): no host time between kernels."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            fn()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        keep = fn()
    for _ in range(2):
        graph.replay()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        graph.replay()
    b.record()
    torch.cuda.synchronize()
    del keep, graph
    return a.elapsed_time(b) * 1e3 / reps


def run(torch, dist, rank, world, tokens=(256,), E=128, H=2048, F=768, top_k=8, fmt=1, reps=10):
    import chadslab_b200 as cb
    from chadslab_b200 import ops, parallel
    from chadslab_b200.synth import make_device_weight
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)

    def mk(n, k):
        codes, scales = make_device_weight(torch, n, k, fmt, gen)
        return cb.PackedWeight.from_device(codes, scales, fmt)
    E_loc = E // world
    gate, up, down = [mk(F, H) for _ in range(E_loc)], [mk(F, H) for _ in range(E_loc)], [mk(H, F) for _ in range(E_loc)]
    gr = torch.Generator(device="cuda").manual_seed(99)            # the router is replicated: same seed on every rank
    rc, rs = make_device_weight(torch, E, H, fmt, gr)
    router = cb.PackedWeight.from_device(rc, rs, fmt)
    bytes_per_expert = sum(p.nbytes for p in (gate[0], up[0], down[0]))
    out = {"layer": f"{E} experts, hidden {H}, SwiGLU ffn {F}, top-{top_k}, {'int8' if fmt == 0 else 'q4'}-g32",
           "expert_parallel": world, "expert_MB": round(bytes_per_expert / 1e6, 3), "cases": []}
    ep = None
    if world == 1:
        moe = cb.MoEExperts(router, gate, up, down, top_k)
        layer = moe
    else:                      # both exchanges on the device: rows stored straight into the owning rank's memory
        local = cb.MoEExperts(None, gate, up, down, top_k=top_k)
        ep = cb.PeerEP(E, H, max_send_rows=max(tokens) // world * top_k, group=dist.group.WORLD)
        layer = parallel.ExpertParallelMoE(cb.QuantLinear(router), None, E, top_k, ep=ep, local_moe=local)
        out["exchange"] = "peer-memory stores (ops.PeerEP): counts, rows and outputs travel without a collective call or a host step"
    for T in tokens:
        T_loc = T // world
        x = torch.randn((T_loc, H), device="cuda", generator=gen).to(torch.bfloat16)
        eager_us = _timed(torch, lambda: layer(x), reps)
        us = _timed_graph(torch, lambda: layer(x), reps)            # the headline figure: one captured layer, replayed
        case = {"tokens": T, "tokens_per_rank": T_loc, "layer_us": round(us, 1), "layer_us_eager": round(eager_us, 1)}
        if world == 1:
            logits = moe.router(x)
            idx, w = ops.moe_route(logits, top_k)
            perm, inv, offsets = ops.moe_permute(idx, E)
            xp = ops.moe_gather(x, perm, top_k)
            outp = moe.experts(xp, offsets)
            case["stages_us"] = {
                "router": round(_timed(torch, lambda: moe.router(x), reps), 1),
                "route": round(_timed(torch, lambda: ops.moe_route(logits, top_k), reps), 1),
                "permute": round(_timed(torch, lambda: ops.moe_permute(idx, E), reps), 1),
                "gather": round(_timed(torch, lambda: ops.moe_gather(x, perm, top_k), reps), 1),
                "experts": round(_timed(torch, lambda: moe.experts(xp, offsets), reps), 1),
                "combine": round(_timed(torch, lambda: ops.moe_combine(outp, inv, w), reps), 1)}
            touched = int((offsets[1:] > offsets[:-1]).sum().item())
            case["experts_touched"] = touched
            wbytes = touched * bytes_per_expert
            case["expert_weight_gbs"] = round(wbytes / case["stages_us"]["experts"] / 1e3, 1)
            case["expert_tflops"] = round(2.0 * T * top_k * 3 * H * F / case["stages_us"]["experts"] / 1e6, 1)
        t = torch.tensor([us, eager_us], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            case["layer_us"], case["layer_us_eager"] = round(float(t[0]), 1), round(float(t[1]), 1)
        case["tokens_per_s_per_layer"] = round(T / float(t[0]) * 1e6, 1)
        out["cases"].append(case)
        del x
    out["status"] = int(cb._lib.lib().bq_status_poll())
    if ep is not None:
        ep.close()
    return out


def run_decoder(torch, dist, rank, world, batch: int = 256, prompt_len: int = 512, steps: int = 8, chunk_seqs: int = 16,
                cfg=None, eager: bool = False):
    """The whole sparse-MoE decoder (48 layers, hidden 2048, 32 query / 4 KV heads of 128, 128 experts of SwiGLU 768,
    top-8, every weight 4-bit group-32, random-init): prefill of `batch` random sequences of `prompt_len` tokens in
    chunks of sequences, then greedy decode of the whole batch as replays of one captured CUDA graph.  With `world`
    ranks the sequences are data-parallel (batch / world per rank), attention is replicated and the experts are
    expert-parallel through the device-side exchange.  Times are CUDA events, max over ranks."""
    import chadslab_b200 as cb
    from chadslab_b200 import _lib
    from chadslab_b200.decoder import MOE_SHAPE, MoEDecoder
    cfg = cfg or MOE_SHAPE
    B_loc = batch // world
    out = {"model": f"sparse-MoE decoder: {cfg.layers} layers, hidden {cfg.hidden}, {cfg.n_heads}/{cfg.n_kv_heads} heads x "
                    f"{cfg.head_dim}, {cfg.n_experts} experts x SwiGLU {cfg.moe_ffn}, top-{cfg.top_k}, q4-g32, vocab {cfg.vocab}",
           "expert_parallel": world, "batch": batch, "sequences_per_rank": B_loc, "prompt_len": prompt_len}
    ep = None
    try:
        chunk = min(chunk_seqs, B_loc)
        if world > 1:
            send = max(chunk * prompt_len, B_loc) * cfg.top_k
            # receive capacity: twice the balanced share (random routing stays within a few percent of it); a row that
            # would not fit is skipped and recorded in the status word, which this report prints
            ep = cb.PeerEP(cfg.n_experts, cfg.hidden, max_send_rows=send, max_recv_rows=2 * send, group=dist.group.WORLD)
        dec = MoEDecoder.random(cfg, seed=0, act_dtype=torch.bfloat16, rank=rank, world=world, max_seq=prompt_len + steps + 8,
                                max_batch=B_loc, ep=ep)
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        tokens = torch.randint(0, cfg.vocab, (B_loc, prompt_len), device="cuda", generator=g)
        dec.prefill(tokens[:chunk], chunk)                # untimed pass over one chunk: sizes the library's scratch
        dec.reset()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        first = dec.prefill(tokens, chunk)
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        pre_ms = float(t[0])
        if eager:                      # launches the step's kernels directly (what a profiler wants)
            toks = first.clone()
            pos_t = torch.tensor([dec.pos], device="cuda", dtype=torch.int64)
            p0 = dec.pos

            def step():
                dec._step_static(toks, pos_t)
                pos_t.fill_(p0)
        else:
            step, toks = dec.make_graph_stepper(B_loc, first, start_pos=dec.pos)
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / steps], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        wb = dec.weight_bytes()
        kvb = sum(k[:, :prompt_len].numel() * k.element_size() for k in dec.k_cache) * 2
        out.update({"prefill_ms": round(pre_ms, 1), "prefill_tokens_per_s": round(batch * prompt_len / pre_ms * 1e3, 1),
                    "prefill_chunk_sequences": chunk,
                    "decode_ms_per_step": round(ms, 4), "decode_tokens_per_s": round(batch * 1e3 / ms, 1),
                    "weight_GB_per_gpu": round(wb / 1e9, 3), "kv_GB_per_gpu": round(kvb / 1e9, 3),
                    "floor_ms_weights_plus_kv_at_measured_hbm": round((wb + kvb) / 6545e6, 3),
                    "status": int(_lib.lib().bq_status_poll())})
        del step, dec
    except Exception as e:
        out["error"] = repr(e)[:300]
    if ep is not None:
        try:
            ep.close()
        except Exception as e:
            out["close_error"] = repr(e)[:200]
    torch.cuda.empty_cache()
    return out


def main():
    import torch
    import torch.distributed as dist
    from chadslab_b200 import _lib
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="256,4096,32768")
    ap.add_argument("--experts", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=768)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--fmt", default="q4", choices=["int8", "q4"])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--decoder", type=int, default=0, help="1: time the whole sparse-MoE decoder (prefill + decode) instead")
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--layers", type=int, default=0, help="decoder: use this many layers instead of the shape's 48")
    ap.add_argument("--eager", type=int, default=0, help="decoder: launch the decode step's kernels directly")
    ap.add_argument("--steps", type=int, default=8)
    a = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _lib.init(local)
    if a.decoder:
        import dataclasses
        from chadslab_b200.decoder import MOE_SHAPE
        cfg = dataclasses.replace(MOE_SHAPE, layers=a.layers) if a.layers else MOE_SHAPE
        rep = run_decoder(torch, dist, rank, world, batch=a.batch, prompt_len=a.prompt, steps=a.steps, cfg=cfg, eager=bool(a.eager))
    else:
        rep = run(torch, dist, rank, world, tuple(int(t) for t in a.tokens.split(",")), a.experts, a.hidden, a.ffn, a.top_k,
                  0 if a.fmt == "int8" else 1, a.reps)
    if rank == 0:
        print(json.dumps(rep))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
