"""Expert-parallel exchange through peer memory, on one GPU.

With a world of one rank the whole device path runs (counts through the receive slots, rows stored into the
receive buffer, flags, wait, grouped experts on the received rows, rows stored back, combine) with the rank as its
own peer, and must reproduce the plain single-GPU layer bit for bit; the row bookkeeping every rank derives from
the exchanged counts is checked for worlds of 2, 4 and 8 by running the layout kernel on given count matrices.
The exchange between two real GPUs is covered by tests/tp_worker.py."""
import numpy as np
import pytest

from oracle import spec

pytestmark = pytest.mark.gpu


def _layer(cb, rng, E, H, F, k, fmt=1):
    q = lambda w: spec.quantize(w.astype(np.float32), fmt)
    router = q(rng.normal(0, 0.5, (E, H)))
    gate = [q(rng.normal(0, 0.05, (F, H))) for _ in range(E)]
    up = [q(rng.normal(0, 0.05, (F, H))) for _ in range(E)]
    down = [q(rng.normal(0, 0.05, (H, F))) for _ in range(E)]
    mk = lambda cs: cb.PackedWeight.from_arrays(cs[0], cs[1], fmt)
    moe = cb.MoEExperts(mk(router), [mk(g) for g in gate], [mk(u) for u in up], [mk(d) for d in down], top_k=k)
    return moe, (router, gate, up, down)


@pytest.mark.parametrize("T", [1, 37, 300])
def test_device_exchange_world_one_equals_plain_layer(cuda_lib, T):
    import torch
    import chadslab_b200 as cb
    from chadslab_b200 import parallel
    rng = np.random.default_rng(T)
    E, H, F, k = 8, 256, 256, 2
    moe, (router, gate, up, down) = _layer(cb, rng, E, H, F, k)
    ep = cb.PeerEP(E, H, max_send_rows=320 * k)
    layer = parallel.ExpertParallelMoE(moe.router, None, E, k, ep=ep, local_moe=moe)
    x = spec.bf16_round(rng.normal(0, 1, (T, H)).astype(np.float32))
    xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
    for it in range(3):                                  # several layers in a row: epochs, both parities
        y = layer(xt)
        assert torch.equal(y, moe(xt)), it
    ref, _ = spec.moe_forward(x, router, gate, up, down, 1, k)
    assert spec.rel_err(y.cpu().numpy(), ref) <= 4e-3     # layer-level bound (bf16 hidden activation between the matmuls)
    # the same layer from a replayed CUDA graph: the call counter advances on the device
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        yg = layer(xt)
    for _ in range(3):
        yg.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(yg, y)
    ep.close()
    assert cuda_lib.bq_status_poll() == 0


def test_device_exchange_refuses_what_does_not_fit(cuda_lib):
    import torch
    import chadslab_b200 as cb
    from chadslab_b200 import _lib
    ep = cb.PeerEP(8, 64, max_send_rows=16)
    x = torch.zeros((9, 64), device="cuda", dtype=torch.bfloat16)
    idx = torch.zeros((9, 2), device="cuda", dtype=torch.int32)
    perm, inv, offsets = cb.moe_permute(idx, 8)
    rc = cuda_lib.bq_ep_dispatch(ep.handle, x.data_ptr(), idx.data_ptr(), perm.data_ptr(), offsets.data_ptr(), 9, 2, None)
    assert rc == _lib.ERR_ARG and b"max_send_rows" in cuda_lib.bq_last_error()
    ep.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_layout_tables_for_given_count_matrices(cuda_lib, world):
    """ep_layout_kernel's tables against their host restatement (parallel.ep_layout), every rank of the world."""
    import torch
    from chadslab_b200 import _lib, parallel
    rng = np.random.default_rng(world)
    for E in (world, 16, 128):
        if E % world:
            continue
        El = E // world
        C = rng.integers(0, 40, (world, E)).astype(np.int32)
        C[rng.integers(0, world), :] = 0                   # a rank without tokens
        C[:, rng.integers(0, E)] = 0                       # an expert nobody chose
        d_counts = torch.from_numpy(C).cuda()
        n = E + (El + 1) + (El * world + 1) + El * world
        for rank in range(world):
            out = torch.full((n + 64,), -9, dtype=torch.int32, device="cuda")
            _lib.check(cuda_lib.bq_ep_layout_selftest(d_counts.data_ptr(), rank, world, E, out.data_ptr(), None))
            got = out.cpu().numpy()
            dest_base, loffsets, blk_start, blk_src = parallel.ep_layout(C, rank)
            o = 0
            for want in (dest_base, loffsets, blk_start, blk_src):
                assert np.array_equal(got[o:o + len(want)], want), (world, E, rank)
                o += len(want)
