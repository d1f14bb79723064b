"""MoE pieces (route, permute, gather, grouped experts, combine) and the whole layer vs the oracle."""
import numpy as np
import pytest

from oracle import spec

pytestmark = pytest.mark.gpu
TOL = 1e-3


def _bf16(a, torch):
    return torch.from_numpy(spec.bf16_round(a)).cuda().to(torch.bfloat16)


def test_route_golden_ties(cuda_lib, moegolden):
    import torch
    import chadslab_b200 as cb
    idx, w = cb.moe_route(torch.from_numpy(moegolden["route/logits"]).cuda(), 4)
    assert np.array_equal(idx.cpu().numpy(), moegolden["route/idx"])
    assert np.allclose(w.cpu().numpy(), moegolden["route/w"], rtol=2e-6, atol=1e-7)
    perm, inv, offsets = cb.moe_permute(idx, 16)
    assert np.array_equal(perm.cpu().numpy(), moegolden["route/perm"])
    assert np.array_equal(offsets.cpu().numpy(), moegolden["route/offsets"])
    assert np.array_equal(inv.cpu().numpy()[perm.cpu().numpy()], np.arange(perm.numel()))


@pytest.mark.parametrize("T,E,k", [(1, 8, 2), (256, 128, 8), (1000, 128, 8), (37, 64, 6), (20000, 128, 8), (5, 300, 4)])
def test_route_and_permute_random(cuda_lib, T, E, k):
    import torch
    import chadslab_b200 as cb
    rng = np.random.default_rng(T + E)
    logits = rng.normal(0, 1, (T, E)).astype(np.float32)
    ridx, rw = spec.moe_route_from_logits(logits, k)
    idx, w = cb.moe_route(torch.from_numpy(logits).cuda(), k)
    got = idx.cpu().numpy()
    same = (got == ridx).all(axis=1)
    assert same.mean() > 0.999                                 # fp32 exp near-ties may swap neighbours
    assert np.allclose(w.cpu().numpy()[same], rw[same], rtol=5e-6, atol=1e-7)
    # without renormalisation the weights are the plain softmax probabilities
    _, w2 = cb.moe_route(torch.from_numpy(logits).cuda(), k, renormalise=False)
    p = np.take_along_axis(spec.softmax(logits), got.astype(np.int64), axis=1)
    assert np.allclose(w2.cpu().numpy(), p, rtol=5e-6, atol=1e-8)
    # permute: stable sort by expert, exact
    perm, inv, offsets = cb.moe_permute(idx, E)
    rperm, roff = spec.moe_permute(got, E)
    assert np.array_equal(perm.cpu().numpy(), rperm) and np.array_equal(offsets.cpu().numpy(), roff)
    assert np.array_equal(inv.cpu().numpy()[rperm], np.arange(T * k))
    # gather
    x = rng.normal(0, 1, (T, 64)).astype(np.float32)
    xp = cb.moe_gather(_bf16(x, torch), perm, k)
    assert np.array_equal(xp.float().cpu().numpy(), spec.bf16_round(x)[rperm // k])


def test_combine_matches_oracle_order(cuda_lib):
    import torch
    import chadslab_b200 as cb
    rng = np.random.default_rng(11)
    T, k, H, E = 50, 4, 96, 9
    idx = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int32)
    w = rng.random((T, k)).astype(np.float32)
    perm, _ = spec.moe_permute(idx, E)
    out_p = rng.normal(0, 1, (T * k, H)).astype(np.float32)
    ref = spec.moe_combine(out_p, perm, w)
    _, inv, _ = cb.moe_permute(torch.from_numpy(idx).cuda(), E)
    y = cb.moe_combine(torch.from_numpy(out_p).cuda(), inv, torch.from_numpy(w).cuda())
    assert np.array_equal(y.cpu().numpy(), ref)                # same order, separate mul/add: bit-exact


@pytest.mark.parametrize("fmt,tag", [(0, "q8"), (1, "q4")])
def test_moe_layer_golden(cuda_lib, moegolden, fmt, tag):
    import torch
    import chadslab_b200 as cb
    E = moegolden[f"{tag}/gate_codes"].shape[0]
    mk = lambda nm: [cb.PackedWeight.from_arrays(moegolden[f"{tag}/{nm}_codes"][e], moegolden[f"{tag}/{nm}_scales"][e], fmt)
                     for e in range(E)]
    router = cb.PackedWeight.from_arrays(moegolden[f"{tag}/router_codes"], moegolden[f"{tag}/router_scales"], fmt)
    for path in (cb.PATH_SIMT, cb.PATH_AUTO):
        layer = cb.MoEExperts(router, mk("gate"), mk("up"), mk("down"), top_k=2, path=path)
        x = torch.from_numpy(moegolden["x_bf16"].astype(np.int16)).cuda().view(torch.bfloat16)
        y, (idx, w, perm, inv, offsets) = layer(x, return_aux=True)
        assert np.array_equal(idx.cpu().numpy(), moegolden[f"{tag}/idx"])
        assert np.array_equal(perm.cpu().numpy(), moegolden[f"{tag}/perm"])
        assert np.array_equal(offsets.cpu().numpy(), moegolden[f"{tag}/offsets"])
        assert spec.rel_err(y.cpu().numpy(), moegolden[f"{tag}/y"]) <= TOL


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("T", [3, 64, 300])
def test_moe_layer_random(cuda_lib, fmt, T):
    """16 experts of the benchmark's expert shape family (hidden 256, ffn 96..., top-4), some experts empty."""
    import torch
    import chadslab_b200 as cb
    rng = np.random.default_rng(100 + T + fmt)
    E, H, F, k = 16, 256, 192, 4
    x = spec.bf16_round(rng.normal(0, 1, (T, H)).astype(np.float32))
    Wr = rng.normal(0, 0.3, (E, H)).astype(np.float32)
    Wr[5] = -10.0 * np.abs(Wr[5])        # expert 5 is (almost) never chosen -> empty segment
    q = lambda W: spec.quantize(W, fmt)
    router = q(Wr)
    gate = [q(rng.normal(0, 0.05, (F, H)).astype(np.float32)) for _ in range(E)]
    up = [q(rng.normal(0, 0.05, (F, H)).astype(np.float32)) for _ in range(E)]
    down = [q(rng.normal(0, 0.05, (H, F)).astype(np.float32)) for _ in range(E)]
    ref, (ridx, rw, rperm, roff) = spec.moe_forward(x, router, gate, up, down, fmt, k)
    pw = lambda cs: cb.PackedWeight.from_arrays(cs[0], cs[1], fmt)
    for path in (cb.PATH_SIMT, cb.PATH_AUTO):
        layer = cb.MoEExperts(pw(router), [pw(g) for g in gate], [pw(u) for u in up], [pw(d) for d in down], top_k=k,
                              path=path)
        y, (idx, w, perm, inv, offsets) = layer(torch.from_numpy(x).cuda().to(torch.bfloat16), return_aux=True)
        if np.array_equal(idx.cpu().numpy(), ridx):
            assert spec.rel_err(y.cpu().numpy(), ref) <= TOL
        else:                                # a router near-tie flipped: compare with the oracle fed the kernel's routing
            gi, gw = idx.cpu().numpy(), w.cpu().numpy()
            p2, o2 = spec.moe_permute(gi, E)
            out_p = spec.moe_experts(x[p2 // k], o2, gate, up, down, fmt)
            assert spec.rel_err(y.cpu().numpy(), spec.moe_combine(out_p, p2, gw)) <= TOL
