"""Host logic of the tensor / expert parallel layer on 2 CPU ranks (gloo).  The math callables are the
numpy oracle, so what is tested is the sharding, the collectives and the index bookkeeping: the sharded
result must equal the unsharded oracle."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import spec

WORLD = 2


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _np(t):
    return t.detach().cpu().float().numpy()


def _oracle_linear(codes, scales, fmt):
    return lambda x: torch.from_numpy(spec.qlinear(_np(x), codes, scales, fmt))


def _cpu_backend():
    from chadslab_b200.parallel import MoEBackend

    def route(logits, k, renorm=True):
        idx, w = spec.moe_route_from_logits(_np(logits), k)
        return torch.from_numpy(idx), torch.from_numpy(w)

    def permute(idx, E):
        perm, offsets = spec.moe_permute(idx.numpy(), E)
        inv = np.empty_like(perm)
        inv[perm] = np.arange(len(perm), dtype=np.int32)
        return torch.from_numpy(perm), torch.from_numpy(inv), torch.from_numpy(offsets)

    def gather(x, perm, k):
        return x[(perm.long() // k)]

    def combine(out_p, inv, w):
        T, k = w.shape
        perm = np.empty(T * k, dtype=np.int32)
        perm[inv.numpy()] = np.arange(T * k, dtype=np.int32)
        return torch.from_numpy(spec.moe_combine(_np(out_p), perm, w.numpy()))

    return MoEBackend(route=route, permute=permute, gather=gather, combine=combine)


def _worker(rank, port, fn, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        fn(rank)
        ret[rank] = "ok"
    except Exception as e:  # pragma: no cover
        import traceback
        ret[rank] = traceback.format_exc()
    finally:
        dist.destroy_process_group()


def _run(fn):
    port = _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_worker, args=(r, port, fn, ret)) for r in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    for r in range(WORLD):
        assert ret.get(r) == "ok", ret.get(r)


def _tp_case(rank):
    from chadslab_b200 import parallel
    rng = np.random.default_rng(0)                       # identical on every rank
    K, N, V, M = 256, 192, 1000, 5
    x = rng.normal(0, 1, (M, K)).astype(np.float32)
    for fmt in (0, 1):
        Wc, Wr, Wv = (rng.normal(0, 0.02, s).astype(np.float32) for s in ((N, K), (K, N), (V, K)))
        qc, qr, qv = spec.quantize(Wc, fmt), spec.quantize(Wr, fmt), spec.quantize(Wv, fmt)
        # column-parallel then row-parallel (an MLP without the activation)
        col = parallel.ColumnParallelLinear(_oracle_linear(*spec.shard(*qc, fmt, "n", rank, WORLD), fmt))
        row = parallel.RowParallelLinear(_oracle_linear(*spec.shard(*qr, fmt, "k", rank, WORLD), fmt))
        h_local = col(torch.from_numpy(x))
        y = row(h_local)
        h_full = spec.qlinear(x, *qc, fmt)
        ref = spec.qlinear(h_full, *qr, fmt, f64=True)
        assert spec.rel_err(_np(y), ref) < 1e-5
        gathered = parallel.ColumnParallelLinear(_oracle_linear(*spec.shard(*qc, fmt, "n", rank, WORLD), fmt),
                                                 gather_output=True)(torch.from_numpy(x))
        assert np.allclose(_np(gathered), h_full, atol=1e-6)
        # vocabulary-parallel head, with an exact tie across the two shards
        Wv[700] = Wv[100]
        qv = spec.quantize(Wv, fmt)
        xq = x.copy()
        xq[0] = 50 * spec.dequantize(*qv, fmt)[100]
        head = parallel.VocabParallelHead(_oracle_linear(*spec.shard(*qv, fmt, "n", rank, WORLD), fmt), V // WORLD)
        ids = head.greedy(torch.from_numpy(xq)).numpy()
        ref_logits, ref_ids = spec.lm_head(xq, *qv, fmt)
        assert ids[0] == 100 and np.array_equal(ids, ref_ids)
        assert np.allclose(_np(head.logits(torch.from_numpy(xq))), ref_logits, atol=1e-5)


def _ep_case(rank):
    from chadslab_b200 import parallel
    rng = np.random.default_rng(1)
    E, H, F, k = 8, 64, 96, 2
    fmt = 1
    q = lambda W: spec.quantize(W.astype(np.float32), fmt)
    router = q(rng.normal(0, 0.5, (E, H)))
    gate = [q(rng.normal(0, 0.1, (F, H))) for _ in range(E)]
    up = [q(rng.normal(0, 0.1, (F, H))) for _ in range(E)]
    down = [q(rng.normal(0, 0.1, (H, F))) for _ in range(E)]
    T_all = [7, 12]                                         # ragged token counts per rank
    xs = [spec.bf16_round(rng.normal(0, 1, (t, H)).astype(np.float32)) for t in T_all]
    x = xs[rank]
    lg, lu, ld = (parallel.shard_experts(w_, rank, WORLD) for w_ in (gate, up, down))

    def experts(xl, loffsets):
        return torch.from_numpy(spec.moe_experts(_np(xl), loffsets.numpy(), lg, lu, ld, fmt))

    layer = parallel.ExpertParallelMoE(_oracle_linear(*router, fmt), experts, E, k, backend=_cpu_backend(),
                                       act_dtype=torch.float32)
    y = layer(torch.from_numpy(x))
    ref, _ = spec.moe_forward(x, router, gate, up, down, fmt, k)
    assert spec.rel_err(_np(y), ref) < 1e-6
    # an empty rank (no tokens) still takes part in the exchange
    if rank == 1:
        x = x[:0]
    y = layer(torch.from_numpy(x))
    if rank == 0:
        assert spec.rel_err(_np(y), ref) < 1e-6
    else:
        assert tuple(y.shape) == (0, H)


def _ep_layout_case(rank):
    """The device-side exchange's row bookkeeping (parallel.ep_layout restates ep_layout_kernel): rows placed by
    dest_base / returned by blk_start + blk_src must reproduce the unsharded oracle layer.  Peer memory is played
    by all-gathering every rank's rows together with their destination indices."""
    from chadslab_b200 import parallel
    rng = np.random.default_rng(4)
    E, H, F, k, fmt = 8, 64, 96, 3, 1
    El = E // WORLD
    q = lambda W: spec.quantize(W.astype(np.float32), fmt)
    router = q(rng.normal(0, 0.5, (E, H)))
    gate = [q(rng.normal(0, 0.1, (F, H))) for _ in range(E)]
    up = [q(rng.normal(0, 0.1, (F, H))) for _ in range(E)]
    down = [q(rng.normal(0, 0.1, (H, F))) for _ in range(E)]
    xs = [spec.bf16_round(rng.normal(0, 1, (t, H)).astype(np.float32)) for t in (11, 6)]
    x = xs[rank]
    lg, lu, ld = (parallel.shard_experts(w_, rank, WORLD) for w_ in (gate, up, down))
    idx, w = spec.moe_route(x, router[0], router[1], fmt, k)
    perm, offsets = spec.moe_permute(idx, E)
    inv = np.empty_like(perm)
    inv[perm] = np.arange(len(perm), dtype=np.int32)
    counts = [None] * WORLD
    dist.all_gather_object(counts, np.diff(offsets).tolist())
    dest_base, loffsets, blk_start, blk_src = parallel.ep_layout(counts, rank)
    # dispatch: sorted position p (expert e, j-th of my rows for e) -> row dest_base[e] + j on rank e // El
    ex = idx.reshape(-1)[perm]
    dst_row = dest_base[ex] + (np.arange(len(perm)) - offsets[ex])
    sent = [None] * WORLD
    dist.all_gather_object(sent, (ex // El, dst_row, x[perm // k]))
    n_recv = int(blk_start[-1])
    xrecv = np.full((n_recv, H), np.nan, np.float32)
    for owner, rows, data in sent:
        m = owner == rank
        xrecv[rows[m]] = data[m]
    assert not np.isnan(xrecv).any() and n_recv == loffsets[-1]         # every row written exactly where expected
    out = spec.moe_experts(xrecv, loffsets, lg, lu, ld, fmt)
    # way back: received row i of block b = (local expert, source s) -> position blk_src[b] + (i - blk_start[b]) on s
    blk = np.searchsorted(blk_start[1:], np.arange(n_recv), side="right")
    back = [None] * WORLD
    dist.all_gather_object(back, (blk % WORLD, blk_src[blk] + (np.arange(n_recv) - blk_start[blk]), out))
    yback = np.full((len(perm), H), np.nan, np.float32)
    for src, pos, data in back:
        m = src == rank
        yback[pos[m]] = data[m]
    assert not np.isnan(yback).any()
    y = spec.moe_combine(yback, perm, w)
    ref, _ = spec.moe_forward(x, router, gate, up, down, fmt, k)
    assert spec.rel_err(y, ref) < 1e-6


def test_tensor_parallel_two_ranks():
    _run(_tp_case)


def test_expert_parallel_two_ranks():
    _run(_ep_case)


def test_expert_parallel_device_layout_two_ranks():
    _run(_ep_layout_case)
