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
    dist.barrier()
    if rank == 0:
        print("tp_worker ok")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
