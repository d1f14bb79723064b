"""Launched by tests/test_gpu_decoder.py under torchrun on 2 GPUs: the tensor-parallel decoder and the
expert-parallel MoE layer must reproduce the oracle (same seeded weights on every rank)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
from oracle import model as omodel  # noqa: E402
from oracle import spec  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import chadslab_b200 as cb
    from chadslab_b200 import parallel
    from chadslab_b200.decoder import DecoderConfig, QuantDecoder
    # ---- tensor-parallel decoder (2 KV heads so K/V shard too) ----
    for fmt in (0, 1):
        cfg = dict(layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=1024, fmt=fmt)
        w = omodel.random_weights(cfg, seed=5)
        prompt = np.random.default_rng(1).integers(0, cfg["vocab"], 6)
        ref_tokens, ref_logits = omodel.OracleDecoder(cfg, w).generate(list(prompt), 3)
        dec = QuantDecoder.from_numpy(DecoderConfig(**cfg), w, act_dtype=torch.float32, rank=rank, world=world, max_seq=32)
        pt = torch.from_numpy(prompt)[None].cuda()
        lg = dec.logits(pt)[0, -1].cpu().numpy()
        assert spec.rel_err(lg, ref_logits[0]) <= 1e-3, spec.rel_err(lg, ref_logits[0])
        dec.reset()
        out = dec.generate(pt, 3)[0].cpu().numpy().tolist()
        assert out == ref_tokens, (out, ref_tokens)
    # ---- peer-memory communicator: sums through NVLink stores + flags instead of NCCL ----
    comm = cb.PeerComm(max_elems=4 * 4096, group=dist.group.WORLD)
    g = torch.Generator(device="cuda").manual_seed(100 + rank)
    for n in (1, 256, 3072, 12288):                                   # several sizes, both parities, chunked
        for _ in range(3):
            v = torch.randn(n, device="cuda", generator=g)
            want = v.clone()
            dist.all_reduce(want)
            got = comm.all_reduce(v)
            assert torch.equal(got, want), n                          # fp32 a + b is commutative: bit-identical at world 2
    # row-parallel linear: GEMV deposits in both ranks' slots, fused sum + residual add + RMSNorm follows
    rngc = np.random.default_rng(11)
    Wf = rngc.normal(0, 0.02, (3072, 4096)).astype(np.float32)
    for fmt in (0, 1):
        codes, scales = spec.quantize(Wf, fmt)
        full = cb.PackedWeight.from_arrays(codes, scales, fmt, upload=False)
        lin = cb.QuantLinear(cb.shard(full, "k", rank, world))
        xfull = spec.bf16_round(rngc.normal(0, 1, (2, 4096)).astype(np.float32))
        ksl = slice(rank * 4096 // world, (rank + 1) * 4096 // world)
        xloc = torch.from_numpy(np.ascontiguousarray(xfull[:, ksl])).cuda().to(torch.bfloat16)
        assert comm.push_linear(lin, xloc) is None
        y = comm.all_reduce(None, count=2 * 3072).reshape(2, 3072).cpu().numpy()
        ref = xfull.astype(np.float64) @ spec.dequantize(codes, scales, fmt).astype(np.float64).T
        assert spec.rel_err(y, ref) <= 1e-3, spec.rel_err(y, ref)
        res = torch.from_numpy(rngc.normal(0, 1, (2, 3072)).astype(np.float32)).cuda()
        gamma = torch.from_numpy(rngc.uniform(0.5, 1.5, 3072).astype(np.float32)).cuda()
        normed, res0 = torch.empty_like(res), res.cpu().numpy()
        assert comm.push_linear(lin, xloc) is None
        comm.add_rmsnorm(None, res, gamma, normed, 1e-6)
        xr = res.cpu().numpy()
        assert np.array_equal(xr, res0 + y)                           # same sum, same order, one fp32 add
        nref = xr * (1.0 / np.sqrt((xr.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6)) * gamma.cpu().numpy()
        assert spec.rel_err(normed.cpu().numpy(), nref) <= 1e-5
        both = [torch.empty_like(normed) for _ in range(world)]
        dist.all_gather(both, normed)
        assert all(torch.equal(both[0], b) for b in both)             # fixed summing order: identical on every rank
    # CUDA-graph decode of the tensor-parallel decoder through the communicator == the eager NCCL route
    for adt in (torch.float32, torch.bfloat16):
        cfg = dict(layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=512, vocab=1024, fmt=1)
        w = omodel.random_weights(cfg, seed=8)
        prompt = torch.from_numpy(np.random.default_rng(3).integers(0, cfg["vocab"], (2, 5))).cuda()
        dec = QuantDecoder.from_numpy(DecoderConfig(**cfg), w, act_dtype=adt, rank=rank, world=world, max_seq=32,
                                      max_batch=2, comm=comm)
        eager = dec.generate(prompt, 6).cpu().numpy()
        dec.reset()
        first = dec.next_tokens(prompt)
        step, tokens = dec.make_graph_stepper(2, first, start_pos=dec.pos)
        got = [first.cpu().numpy()]
        for _ in range(5):
            step()
            got.append(tokens.cpu().numpy().copy())
        got = np.stack(got, axis=1)
        if adt == torch.float32:
            assert np.array_equal(got, eager), (got, eager)
        else:                               # bf16 residual stream: a different summing order may flip a late token
            assert np.array_equal(got[:, :2], eager[:, :2]), (got, eager)
    assert cb._lib.lib().bq_status_poll() == 0
    comm.close()
    # ---- expert-parallel MoE layer ----
    rng = np.random.default_rng(2)
    E, H, Fd, k, fmt = 8, 256, 256, 2, 1
    q = lambda W: spec.quantize(W.astype(np.float32), fmt)
    router = q(rng.normal(0, 0.5, (E, H)))
    gate = [q(rng.normal(0, 0.05, (Fd, H))) for _ in range(E)]
    up = [q(rng.normal(0, 0.05, (Fd, H))) for _ in range(E)]
    down = [q(rng.normal(0, 0.05, (H, Fd))) for _ in range(E)]
    xs = [spec.bf16_round(rng.normal(0, 1, (t, H)).astype(np.float32)) for t in (9, 20)]
    x = xs[rank]
    mk = lambda cs: cb.PackedWeight.from_arrays(cs[0], cs[1], fmt)
    lg_, lu_, ld_ = (parallel.shard_experts(w_, rank, world) for w_ in (gate, up, down))
    local_moe = cb.MoEExperts(mk(q(rng.normal(0, 0.5, (E // world, H)))), [mk(g) for g in lg_], [mk(u) for u in lu_],
                              [mk(d) for d in ld_], top_k=1)            # only its grouped-expert kernel is used
    layer = parallel.ExpertParallelMoE(cb.QuantLinear(mk(router)), local_moe.experts, E, k)
    y = layer(torch.from_numpy(x).cuda().to(torch.bfloat16)).cpu().numpy()
    ref, _ = spec.moe_forward(x, router, gate, up, down, fmt, k)
    err = spec.rel_err(y, ref)
    assert err <= 4e-3, err      # layer-level bound (bf16 hidden activation between the expert matmuls)
    # the same layer with both exchanges on the device (peer-memory stores, no collective call, no host step):
    # bit-identical to the route through the process group, eagerly and from a replayed CUDA graph.  (The router is
    # passed as a plain callable here so that both routes compute the routing weights with the same two kernels; with
    # a QuantLinear the device route fuses router matmul + softmax + top-k into one launch, checked below.)
    ep = cb.PeerEP(E, H, max_send_rows=64, group=dist.group.WORLD)
    local2 = cb.MoEExperts(None, [mk(g) for g in lg_], [mk(u) for u in lu_], [mk(d) for d in ld_], top_k=k)
    router_lin = cb.QuantLinear(mk(router))
    layer2 = parallel.ExpertParallelMoE(lambda t: router_lin(t), None, E, k, ep=ep, local_moe=local2)
    xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
    for _ in range(3):
        y2 = layer2(xt).cpu().numpy()
        assert np.array_equal(y2, y), (float(np.abs(y2 - y).max()), float(np.abs(y).max()), int((y2 != y).sum()), y.size)
    layer3 = parallel.ExpertParallelMoE(router_lin, None, E, k, ep=ep, local_moe=local2)       # fused router
    y3 = layer3(xt).cpu().numpy()
    assert spec.rel_err(y3, ref) <= 4e-3 and spec.rel_err(y3, y) <= 1e-3
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        yg = layer2(xt)
    for _ in range(3):
        yg.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert np.array_equal(yg.cpu().numpy(), y)
    assert cb._lib.lib().bq_status_poll() == 0
    # ---- sparse-MoE decoder, expert parallel: every rank decodes its own sequences ----
    from chadslab_b200.decoder import MoEDecoder
    cfg = dict(layers=2, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64, ffn=0, vocab=1024, fmt=1, n_experts=8, top_k=2,
               moe_ffn=256)
    w = omodel.random_weights(cfg, seed=12)
    prompts = np.random.default_rng(9).integers(0, cfg["vocab"], (world, 6))
    ref_tokens, ref_logits = omodel.OracleDecoder(cfg, w).generate(list(prompts[rank]), 3)
    ep2 = cb.PeerEP(cfg["n_experts"], cfg["hidden"], max_send_rows=6 * cfg["top_k"], group=dist.group.WORLD)
    dec = MoEDecoder.from_numpy(DecoderConfig(**cfg), w, act_dtype=torch.float32, rank=rank, world=world, max_seq=32, ep=ep2)
    pt = torch.from_numpy(prompts[rank])[None].cuda()
    lg = dec.logits(pt)[0, -1].cpu().numpy()
    assert spec.rel_err(lg, ref_logits[0]) <= 2e-3, spec.rel_err(lg, ref_logits[0])
    dec.reset()
    first = dec.next_tokens(pt)
    step, tokens = dec.make_graph_stepper(1, first, start_pos=dec.pos)
    got = [int(first[0])]
    for _ in range(2):
        step()
        got.append(int(tokens[0]))
    assert got == ref_tokens, (got, ref_tokens)
    assert cb._lib.lib().bq_status_poll() == 0
    del step
    ep2.close()
    ep.close()
    dist.barrier()
    if rank == 0:
        print("tp_worker ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
