"""Throughput of one sparse-MoE FFN layer: router -> top-k -> permute -> gather -> grouped SwiGLU experts -> combine.

    python -m chadslab_b200.moe_bench --tokens 256,4096,32768 [--experts 128 --hidden 2048 --ffn 768 --top-k 8 --fmt q4]
    torchrun --nproc-per-node N ... -m chadslab_b200.moe_bench ...   (expert parallel: E/N experts and tokens/N per rank)

Random-init packed weights generated on the device; router logits come from x . Wr^T with x ~ N(0,1).  Per token
count: microseconds of the whole layer and of its stages (CUDA events, `--reps` launches after 2), the expert
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
    if world == 1:
        moe = cb.MoEExperts(router, gate, up, down, top_k)
        layer = moe
    else:
        local = cb.MoEExperts(mk(E_loc, H), gate, up, down, top_k=1)       # only its grouped-expert kernel is used
        layer = parallel.ExpertParallelMoE(cb.QuantLinear(router), local.experts, E, top_k)
    for T in tokens:
        T_loc = T // world
        x = torch.randn((T_loc, H), device="cuda", generator=gen).to(torch.bfloat16)
        us = _timed(torch, lambda: layer(x), reps)
        case = {"tokens": T, "tokens_per_rank": T_loc, "layer_us": round(us, 1)}
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
        t = torch.tensor([us], device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            case["layer_us"] = round(float(t[0]), 1)
        case["tokens_per_s_per_layer"] = round(T / float(t[0]) * 1e6, 1)
        out["cases"].append(case)
        del x
    out["status"] = int(cb._lib.lib().bq_status_poll())
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
    a = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    _lib.init(local)
    rep = run(torch, dist, rank, world, tuple(int(t) for t in a.tokens.split(",")), a.experts, a.hidden, a.ffn, a.top_k,
              0 if a.fmt == "int8" else 1, a.reps)
    if rank == 0:
        print(json.dumps(rep))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
