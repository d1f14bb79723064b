"""Guards around the hot path: cache positions outside the KV cache are refused on the device without a fault,
library scratch that grows keeps graphs captured earlier valid, growth during capture is refused, a communicator
that timed out stays unusable until it is reset, and dropped expert assignments never index out of range."""
import ctypes as C

import numpy as np
import pytest

from oracle import spec

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fused", [True, False])
def test_position_outside_the_kv_cache_is_refused_not_written(cuda_lib, fused):
    """pos == S (one past the last cache row): the kernels record BQ_ERR_ARG in the status word and touch neither the
    caches nor the output; the bounds check is what makes this call safe to run."""
    import torch
    from chadslab_b200 import _lib
    from chadslab_b200.ops import _stream_ptr
    B, Hq, Hkv, D, S = 2, 4, 2, 64, 16
    g = torch.Generator(device="cuda").manual_seed(0)
    qkv = torch.randn((B, (Hq + 2 * Hkv) * D), device="cuda", generator=g)
    kc = torch.randn((B, S, Hkv, D), device="cuda", generator=g)
    vc = torch.randn((B, S, Hkv, D), device="cuda", generator=g)
    k0, v0 = kc.clone(), vc.clone()
    out = torch.full((B, Hq, D), 7.0, device="cuda")
    q = torch.full((B, Hq, D), 3.0, device="cuda")
    for bad in (S, S + 5, -1):
        pos = torch.tensor([bad], device="cuda", dtype=torch.int64)
        if fused:
            _lib.check(cuda_lib.bq_decode_attention_rope(qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(),
                                                         out.data_ptr(), B, Hq, Hkv, D, S, 10000.0, _lib.DT_F32, _stream_ptr()))
        else:
            _lib.check(cuda_lib.bq_rope_kv_append(qkv.data_ptr(), pos.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                                  B, Hq, Hkv, D, S, 10000.0, _lib.DT_F32, _stream_ptr()))
            _lib.check(cuda_lib.bq_decode_attention(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), out.data_ptr(),
                                                    B, Hq, Hkv, D, S, _lib.DT_F32, _stream_ptr()))
        assert cuda_lib.bq_status_poll() == _lib.ERR_ARG
        assert torch.equal(kc, k0) and torch.equal(vc, v0) and bool((out == 7.0).all()) and bool((q == 3.0).all())
    # the last valid position still works
    pos = torch.tensor([S - 1], device="cuda", dtype=torch.int64)
    _lib.check(cuda_lib.bq_decode_attention_rope(qkv.data_ptr(), kc.data_ptr(), vc.data_ptr(), pos.data_ptr(), out.data_ptr(),
                                                 B, Hq, Hkv, D, S, 10000.0, _lib.DT_F32, _stream_ptr()))
    assert cuda_lib.bq_status_poll() == 0
    assert not torch.equal(kc, k0) and torch.isfinite(out).all()


def test_decoder_refuses_steps_beyond_its_cache(cuda_lib):
    import torch
    from oracle import model as omodel
    from chadslab_b200.decoder import DecoderConfig, QuantDecoder
    cfg = dict(layers=1, hidden=256, n_heads=4, n_kv_heads=1, head_dim=64, ffn=512, vocab=512, fmt=0)
    dec = QuantDecoder.from_numpy(DecoderConfig(**cfg), omodel.random_weights(cfg, seed=1), act_dtype=torch.float32, max_seq=8)
    prompt = torch.arange(5, device="cuda")[None]
    first = dec.next_tokens(prompt)
    with pytest.raises(ValueError):
        dec.hidden_states(torch.zeros((1, 9), dtype=torch.int64, device="cuda"))
    step, tokens = dec.make_graph_stepper(1, first, start_pos=dec.pos)
    for _ in range(3):
        step()                               # positions 5, 6, 7
    with pytest.raises(ValueError):
        step()                               # position 8 does not exist
    with pytest.raises(ValueError):
        dec.make_graph_stepper(1, first, start_pos=7)
    assert cuda_lib.bq_status_poll() == 0


def test_scratch_growth_keeps_earlier_graphs_valid_and_is_refused_during_capture(cuda_lib):
    """A graph captured at batch 16 must replay correctly after a batch-64 call made the library's scratch grow (the
    outgrown buffers are retired, not freed); a first call of a new, larger size inside a capture returns BQ_ERR_STATE."""
    import torch
    import chadslab_b200 as cb
    from chadslab_b200 import _lib
    rng = np.random.default_rng(3)
    K, N = 9728, 384                        # a K no other test uses: the activation scratch has to grow for it
    lin = cb.QuantLinear(cb.PackedWeight.from_float(rng.normal(0, 0.02, (N, K)).astype(np.float32), 1))
    x16 = torch.randn((16, K), device="cuda").to(torch.bfloat16)
    y16 = torch.empty((16, N), dtype=torch.float32, device="cuda")
    lin(x16, out=y16)                       # warm-up outside capture sizes the scratch for 16 rows
    want16 = y16.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        lin(x16, out=y16)
    big = torch.randn((4096, K), device="cuda").to(torch.bfloat16)
    ybig = lin(big)                         # grows the scratch well past the 16-row buffers
    torch.cuda.synchronize()
    y16.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(y16, want16)
    # growth inside a capture is refused, nothing is launched, and the capture itself stays healthy
    huge = torch.randn((16384, K), device="cuda").to(torch.bfloat16)
    yh = torch.empty((16384, N), dtype=torch.float32, device="cuda")
    g2 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g2, stream=side):
        rc = cuda_lib.bq_qlinear(lin.pw.handle, huge.data_ptr(), _lib.DT_BF16, 16384, yh.data_ptr(), _lib.DT_F32,
                                 torch.cuda.current_stream().cuda_stream)
        lin(x16, out=y16)                   # a call that fits still captures
    assert rc == _lib.ERR_STATE and b"capture" in cuda_lib.bq_last_error()
    y16.zero_()
    g2.replay()
    torch.cuda.synchronize()
    assert torch.equal(y16, want16)
    del ybig
    # bq_reserve sizes the scratch up front: the same call then captures
    _lib.check(cuda_lib.bq_reserve(16384, K, N))
    g3 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g3, stream=side):
        lin(huge, out=yh)
    g3.replay()
    torch.cuda.synchronize()
    ref = huge[:4].float() @ lin.pw.dequantize().t()
    assert (yh[:4] - ref).abs().max() <= 1e-3 * ref.abs().max()
    assert cuda_lib.bq_status_poll() == 0


def test_timed_out_communicator_stays_failed_until_reset(cuda_lib):
    import torch
    from chadslab_b200 import _lib
    h = C.c_uint64(0)
    _lib.check(cuda_lib.bq_comm_create(0, 2, 1024, C.byref(h)))
    _lib.check(cuda_lib.bq_comm_connect_loopback(h.value))          # the stand-in peer never deposits
    _lib.check(cuda_lib.bq_comm_set_timeout_ms(h.value, 300))
    x = torch.ones(256, device="cuda")
    out = torch.empty_like(x)
    _lib.check(cuda_lib.bq_allreduce(h.value, x.data_ptr(), out.data_ptr(), 256, None))
    assert cuda_lib.bq_status_poll() == _lib.ERR_TIMEOUT
    # sticky: the next summing call is refused on the host ...
    assert cuda_lib.bq_allreduce(h.value, x.data_ptr(), out.data_ptr(), 256, None) == _lib.ERR_STATE
    assert b"bq_comm_reset" in cuda_lib.bq_last_error()
    # ... a reset makes it usable again (it times out again here, because nobody answers, but it runs)
    _lib.check(cuda_lib.bq_comm_reset(h.value))
    _lib.check(cuda_lib.bq_allreduce(h.value, x.data_ptr(), out.data_ptr(), 256, None))
    assert cuda_lib.bq_status_poll() == _lib.ERR_TIMEOUT
    _lib.check(cuda_lib.bq_comm_destroy(h.value))
    assert cuda_lib.bq_status_poll() == 0
    # a world of one after all that: sums work (the failure did not outlive the communicator that had it)
    _lib.check(cuda_lib.bq_comm_create(0, 1, 1024, C.byref(h)))
    _lib.check(cuda_lib.bq_allreduce(h.value, x.data_ptr(), out.data_ptr(), 256, None))
    torch.cuda.synchronize()
    assert torch.equal(out, x)
    _lib.check(cuda_lib.bq_comm_destroy(h.value))


def test_sharded_greedy_head_world_of_one(cuda_lib):
    """bq_lm_head_sharded with one rank = bq_lm_head's arg-max (tie -> lower id), ids offset by vocab_offset."""
    import torch
    import chadslab_b200 as cb
    rng = np.random.default_rng(9)
    V, K = 40000, 256
    W = rng.normal(0, 0.02, (V, K)).astype(np.float32)
    W[777] = W[123]
    head = cb.LMHead(cb.PackedWeight.from_float(W, 1))
    x = spec.bf16_round(rng.normal(0, 1, (5, K)).astype(np.float32))
    x[4] = spec.bf16_round(50 * spec.dequantize(head.pw.codes, head.pw.scales, 1)[123])
    xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
    want = head.greedy(xt).cpu().numpy()
    comm = cb.PeerComm(max_elems=1024)
    for off in (0, 1000):
        got = comm.greedy_head(head, xt, off).cpu().numpy()
        assert np.array_equal(got, want + off) and got[4] == 123 + off
    comm.close()
    assert cuda_lib.bq_status_poll() == 0


def test_dropped_assignments_are_never_dereferenced(cuda_lib):
    """Expert ids outside [0, E): inv = -1, the tail of perm = -1, gathered rows are zero, combine skips them."""
    import torch
    import chadslab_b200 as cb
    T, k, E, H = 50, 4, 8, 64
    g = torch.Generator(device="cuda").manual_seed(1)
    idx = torch.randint(0, E, (T, k), dtype=torch.int32, device="cuda", generator=g)
    idx[3, 1], idx[10, 0], idx[49, 3] = E, -2, 1 << 20
    perm, inv, offsets = cb.moe_permute(idx, E)
    valid = T * k - 3
    assert int(offsets[-1]) == valid and bool((perm[valid:] == -1).all()) and int((inv == -1).sum()) == 3
    x = torch.randn((T, H), device="cuda", generator=g).to(torch.bfloat16)
    xp = cb.moe_gather(x, perm, k)
    assert bool((xp[valid:] == 0).all())
    assert torch.equal(xp[:valid], x[(perm[:valid] // k).long()])
    w = torch.rand((T, k), device="cuda", generator=g)
    y = cb.moe_combine(xp.float(), inv, w).cpu().numpy()
    keep = (inv.reshape(T, k) >= 0).cpu().numpy()
    ref = (x.float().cpu().numpy()[:, None, :] * (w.cpu().numpy() * keep)[:, :, None]).sum(1)
    assert np.allclose(y, ref, rtol=1e-5, atol=1e-5)


def test_container_file_round_trip_on_the_device(cuda_lib, tmp_path):
    """A packed-weight container written to disk, read back tensor by tensor and uploaded: the products equal those
    of the weights it was made from, bit for bit, and match the oracle."""
    import torch
    import chadslab_b200 as cb
    from chadslab_b200 import container
    rng = np.random.default_rng(5)
    ws = {"a.q8": cb.PackedWeight.from_float(rng.normal(0, 0.02, (300, 512)).astype(np.float32), 0),
          "b.q4": cb.PackedWeight.from_float(rng.normal(0, 0.02, (1024, 2048)).astype(np.float32), 1)}
    extra = {"norm": rng.normal(0, 1, 512).astype(np.float32)}
    path = str(tmp_path / "w.safetensors")
    container.save_packed(path, ws, extra)
    names = []
    loaded = {}
    for name, pw in container.iter_packed(path):             # streaming: one weight resident on the host at a time
        names.append(name)
        loaded[name] = pw
        assert pw.codes is None                               # the host copy was dropped after the upload
    assert sorted(names) == sorted(ws)
    _, tensors = container.load_packed(path, upload=False)
    assert np.array_equal(tensors["norm"], extra["norm"])
    for name, pw in ws.items():
        x = torch.randn((3, pw.K), device="cuda").to(torch.bfloat16)
        y0, y1 = cb.QuantLinear(pw)(x), cb.QuantLinear(loaded[name])(x)
        assert torch.equal(y0, y1)
        ref = spec.qlinear(x.float().cpu().numpy(), pw.codes, pw.scales, pw.fmt, f64=True)
        assert spec.rel_err(y1.cpu().numpy(), ref) <= 1e-3
        c2, s2 = loaded[name].export()
        assert np.array_equal(c2, pw.codes) and np.array_equal(s2, pw.scales)
