"""The decode step's glue kernels against float64 restatements of the same formulas (the decoder oracle's
RMSNorm / RoPE / attention / gated activation, oracle/model.py): residual add + RMSNorm, RoPE + KV append,
single-query attention (one CTA per head, grouped heads on CUDA cores and - bf16 caches - on mma.sync, positions split
over several CTAs with an in-kernel merge),
gated activation.  Tolerances: fp32 data 2e-5, bf16 data one bf16 step (2^-8 relative)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _tol(dt):
    import torch
    return 2e-5 if dt == torch.float32 else 2.0 ** -7


def _rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


@pytest.mark.parametrize("adt", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(1, 4, 2, 64, 1024, 700), (2, 8, 1, 256, 2048, 2047), (1, 2, 2, 256, 4096, 0),
                                   (3, 4, 4, 128, 512, 5), (1, 16, 16, 256, 2112, 2048), (2, 4, 1, 64, 64, 40),
                                   (2, 32, 4, 128, 600, 531), (1, 16, 1, 128, 300, 299), (1, 32, 1, 64, 200, 77),
                                   (2, 12, 4, 128, 2048, 1999), (1, 8, 1, 256, 8192, 8000), (1, 6, 2, 64, 64, 15),
                                   (1, 32, 2, 256, 700, 16),
                                   # at least a full wave of (batch row, head) pairs: the 8-positions-per-trip variant (bf16),
                                   # unsplit with a ragged last trip, and split over two CTAs per head
                                   (32, 16, 16, 64, 300, 259), (40, 12, 12, 128, 1100, 1090)])
def test_decode_attention_matches_softmax_attention(cuda_lib, adt, shape):
    import torch
    from chadslab_b200 import _lib
    from chadslab_b200.ops import _dt_of_torch, _stream_ptr
    B, Hq, Hkv, D, S, pos = shape
    dt = getattr(torch, adt)
    g = torch.Generator(device="cuda").manual_seed(B * 131 + pos)
    q = torch.randn((B, Hq, D), device="cuda", generator=g).to(dt)
    k = torch.randn((B, S, Hkv, D), device="cuda", generator=g).to(dt)
    v = torch.randn((B, S, Hkv, D), device="cuda", generator=g).to(dt)
    pos_t = torch.tensor([pos], device="cuda", dtype=torch.int64)
    out = torch.empty_like(q)
    for _ in range(2):          # twice: the arrival counters of the split variant must be back at zero
        out.zero_()
        _lib.check(cuda_lib.bq_decode_attention(q.data_ptr(), k.data_ptr(), v.data_ptr(), pos_t.data_ptr(), out.data_ptr(),
                                                B, Hq, Hkv, D, S, _dt_of_torch(q), _stream_ptr()))
        qd, kd, vd = q.double(), k[:, :pos + 1].double(), v[:, :pos + 1].double()
        rep = Hq // Hkv
        kd, vd = kd.repeat_interleave(rep, dim=2), vd.repeat_interleave(rep, dim=2)      # [B, n, Hq, D]
        sc = torch.einsum("bhd,bnhd->bhn", qd, kd) / np.sqrt(D)
        ref = torch.einsum("bhn,bnhd->bhd", torch.softmax(sc, dim=-1), vd)
        assert _rel(out.double().cpu().numpy(), ref.cpu().numpy()) <= _tol(dt)
    assert cuda_lib.bq_status_poll() == 0


@pytest.mark.parametrize("adt", ["float32", "bfloat16"])
def test_add_rmsnorm(cuda_lib, adt):
    import torch
    from chadslab_b200 import _lib
    from chadslab_b200.ops import _dt_of_torch, _stream_ptr
    dt = getattr(torch, adt)
    for rows, H in ((1, 2048), (3, 3072), (2, 5000), (4, 96)):
        g = torch.Generator(device="cuda").manual_seed(H)
        x = torch.randn((rows, H), device="cuda", generator=g).to(dt)
        d = torch.randn((rows, H), device="cuda", generator=g)
        w = torch.rand(H, device="cuda", generator=g) + 0.5
        x0, out = x.clone(), torch.empty_like(x)
        _lib.check(cuda_lib.bq_add_rmsnorm(x.data_ptr(), d.data_ptr(), w.data_ptr(), out.data_ptr(), rows, H, 1e-6,
                                           _dt_of_torch(x), _stream_ptr()))
        want_x = (x0.float() + d).to(dt)
        assert torch.equal(x, want_x)                                            # one fp32 add, rounded to the stream's type
        xr = want_x.double()
        ref = xr * torch.rsqrt((xr * xr).mean(-1, keepdim=True) + 1e-6) * w.double()
        assert _rel(out.double().cpu().numpy(), ref.cpu().numpy()) <= _tol(dt)
        # no delta: x untouched
        x1, out1 = x0.clone(), torch.empty_like(x0)
        _lib.check(cuda_lib.bq_add_rmsnorm(x1.data_ptr(), None, w.data_ptr(), out1.data_ptr(), rows, H, 1e-6,
                                           _dt_of_torch(x1), _stream_ptr()))
        assert torch.equal(x1, x0)


@pytest.mark.parametrize("adt", ["float32", "bfloat16"])
def test_rope_kv_append(cuda_lib, adt):
    import torch
    from chadslab_b200 import _lib
    from chadslab_b200.ops import _dt_of_torch, _stream_ptr
    dt = getattr(torch, adt)
    B, Hq, Hkv, D, S, pos, base = 2, 4, 2, 64, 16, 9, 10000.0
    g = torch.Generator(device="cuda").manual_seed(1)
    qkv = torch.randn((B, (Hq + 2 * Hkv) * D), device="cuda", generator=g)
    kc = torch.zeros((B, S, Hkv, D), device="cuda", dtype=dt)
    vc = torch.zeros_like(kc)
    qo = torch.empty((B, Hq, D), device="cuda", dtype=dt)
    pos_t = torch.tensor([pos], device="cuda", dtype=torch.int64)
    _lib.check(cuda_lib.bq_rope_kv_append(qkv.data_ptr(), pos_t.data_ptr(), qo.data_ptr(), kc.data_ptr(), vc.data_ptr(), B, Hq,
                                          Hkv, D, S, base, _dt_of_torch(kc), _stream_ptr()))

    def rope(x):                       # x [B, heads, D] float64; rotate-half convention of the decoder oracle
        inv = 1.0 / (base ** (np.arange(0, D, 2) / D))
        ang = pos * inv
        c, s = np.cos(ang), np.sin(ang)
        x1, x2 = x[..., : D // 2], x[..., D // 2:]
        return np.concatenate([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    a = qkv.double().cpu().numpy()
    qr = a[:, : Hq * D].reshape(B, Hq, D)
    kr = a[:, Hq * D:(Hq + Hkv) * D].reshape(B, Hkv, D)
    vr = a[:, (Hq + Hkv) * D:].reshape(B, Hkv, D)
    assert _rel(qo.double().cpu().numpy(), rope(qr)) <= _tol(dt)
    assert _rel(kc[:, pos].double().cpu().numpy(), rope(kr)) <= _tol(dt)
    assert torch.equal(vc[:, pos], torch.from_numpy(vr).cuda().float().to(dt))   # V is copied (rounded to the cache type)
    kc[:, pos] = 0
    vc[:, pos] = 0
    assert not kc.any() and not vc.any()                                          # nothing else was written


@pytest.mark.parametrize("adt", ["float32", "bfloat16"])
@pytest.mark.parametrize("act", [0, 1])
def test_gated_activation(cuda_lib, adt, act):
    import torch
    from chadslab_b200 import _lib
    from chadslab_b200.ops import _dt_of_torch, _stream_ptr
    dt = getattr(torch, adt)
    rows, F = 3, 1000
    gu = torch.randn((rows, 2 * F), device="cuda") * 3
    out = torch.empty((rows, F), device="cuda", dtype=dt)
    _lib.check(cuda_lib.bq_gated_act(gu.data_ptr(), out.data_ptr(), rows, F, act, _dt_of_torch(out), _stream_ptr()))
    gt, up = gu[:, :F].double(), gu[:, F:].double()
    if act == 0:
        a = 0.5 * gt * (1.0 + torch.tanh(0.7978845608028654 * (gt + 0.044715 * gt ** 3)))
    else:
        a = gt / (1.0 + torch.exp(-gt))
    assert _rel(out.double().cpu().numpy(), (a * up).cpu().numpy()) <= _tol(dt)


@pytest.mark.parametrize("adt", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(2, 4, 2, 64, 64, 0), (1, 8, 1, 256, 1024, 700), (2, 4, 4, 128, 512, 511),
                                   (1, 16, 16, 256, 2112, 2048), (3, 2, 1, 64, 4096, 128), (2, 32, 4, 128, 600, 531),
                                   (1, 16, 1, 128, 4096, 3000), (1, 32, 1, 64, 200, 0), (1, 32, 2, 256, 700, 16),
                                   (32, 16, 16, 64, 300, 259), (40, 12, 12, 128, 1100, 1090)])
def test_fused_rope_append_attention_equals_the_two_kernels(cuda_lib, adt, shape):
    """bq_decode_attention_rope against bq_rope_kv_append + bq_decode_attention: the appended cache rows are
    bit-identical, the attention output agrees to rounding (the current position joins the softmax last)."""
    import torch
    from chadslab_b200 import _lib
    from chadslab_b200.ops import _dt_of_torch, _stream_ptr
    B, Hq, Hkv, D, S, pos = shape
    dt = getattr(torch, adt)
    g = torch.Generator(device="cuda").manual_seed(pos + 7)
    qkv = torch.randn((B, (Hq + 2 * Hkv) * D), device="cuda", generator=g)
    k0 = torch.randn((B, S, Hkv, D), device="cuda", generator=g).to(dt)
    v0 = torch.randn((B, S, Hkv, D), device="cuda", generator=g).to(dt)
    pos_t = torch.tensor([pos], device="cuda", dtype=torch.int64)
    ka, va = k0.clone(), v0.clone()
    qa = torch.empty((B, Hq, D), device="cuda", dtype=dt)
    oa = torch.empty_like(qa)
    d, st = _dt_of_torch(ka), _stream_ptr()
    _lib.check(cuda_lib.bq_rope_kv_append(qkv.data_ptr(), pos_t.data_ptr(), qa.data_ptr(), ka.data_ptr(), va.data_ptr(), B, Hq,
                                          Hkv, D, S, 10000.0, d, st))
    _lib.check(cuda_lib.bq_decode_attention(qa.data_ptr(), ka.data_ptr(), va.data_ptr(), pos_t.data_ptr(), oa.data_ptr(), B, Hq,
                                            Hkv, D, S, d, st))
    kb, vb = k0.clone(), v0.clone()
    ob = torch.empty_like(oa)
    for _ in range(2):
        ob.zero_()
        _lib.check(cuda_lib.bq_decode_attention_rope(qkv.data_ptr(), kb.data_ptr(), vb.data_ptr(), pos_t.data_ptr(), ob.data_ptr(),
                                                     B, Hq, Hkv, D, S, 10000.0, d, st))
        assert torch.equal(ka, kb) and torch.equal(va, vb)
        assert _rel(ob.double().cpu().numpy(), oa.double().cpu().numpy()) <= _tol(dt)
    assert cuda_lib.bq_status_poll() == 0


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("adt", ["float32", "bfloat16"])
@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("M", [1, 2, 4, 16, 200, 600])
def test_gated_linear_equals_product_then_activation(cuda_lib, fmt, adt, act, M):
    """bq_qlinear_gated on an interleaved gate|up weight against the plain products of the two weights followed by
    the activation.  bf16 activations: the exact GEMV (M <= 2), the batched GEMV (up to 16 rows) and the tcgen05
    kernel (larger batches) all apply the activation in their epilogue; fp32 activations beyond the GEMV take the
    two-kernel route (product, then activation)."""
    import torch
    import chadslab_b200 as cb
    dt = getattr(torch, adt)
    F, K = 1024, 512
    rng = np.random.default_rng(3)
    gate = cb.PackedWeight.from_float(rng.normal(0, 0.05, (F, K)).astype(np.float32), fmt)
    up = cb.PackedWeight.from_float(rng.normal(0, 0.05, (F, K)).astype(np.float32), fmt)
    fused = cb.QuantLinear(cb.interleave_gate_up(gate, up))
    x = torch.randn((M, K), device="cuda").to(dt)
    got = fused.gated(x, act)
    assert got.dtype == dt and tuple(got.shape) == (M, F)
    g, u = cb.QuantLinear(gate)(x).double(), cb.QuantLinear(up)(x).double()
    if act == 0:
        a = 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    else:
        a = g / (1.0 + torch.exp(-g))
    assert _rel(got.double().cpu().numpy(), (a * u).cpu().numpy()) <= _tol(dt)
    # the plain product of the fused weight is the interleaved pair
    from chadslab_b200.ops import split_gate_up
    g2, u2 = split_gate_up(fused(x))
    if M <= 2 or M > 16 or dt == torch.float32:      # same kernel, same K split for the fused and the separate weights
        assert torch.equal(g2, cb.QuantLinear(gate)(x)) and torch.equal(u2, cb.QuantLinear(up)(x))
    else:                                             # batched GEMV: the K split depends on the row count of the weight
        assert _rel(g2.double().cpu().numpy(), g.cpu().numpy()) <= 1e-5 and _rel(u2.double().cpu().numpy(), u.cpu().numpy()) <= 1e-5


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("act", [0, 1])
def test_gated_linear_with_split_k(cuda_lib, fmt, act):
    """Few output tiles and a long K: the tcgen05 kernel splits K over the grid and the reduction kernel applies the
    gated activation."""
    import torch
    import chadslab_b200 as cb
    F, K, M = 128, 4096, 64
    rng = np.random.default_rng(8)
    gate = cb.PackedWeight.from_float(rng.normal(0, 0.05, (F, K)).astype(np.float32), fmt)
    up = cb.PackedWeight.from_float(rng.normal(0, 0.05, (F, K)).astype(np.float32), fmt)
    fused = cb.QuantLinear(cb.interleave_gate_up(gate, up))
    x = torch.randn((M, K), device="cuda").to(torch.bfloat16)
    n0 = cuda_lib.bq_launch_count()
    got = fused.gated(x, act)
    assert cuda_lib.bq_launch_count() - n0 == 3 and cuda_lib.bq_last_path() == cb.PATH_TENSOR     # pre-pass, split GEMM, gated reduction
    g, u = cb.QuantLinear(gate)(x).double(), cb.QuantLinear(up)(x).double()
    a = 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))) if act == 0 else g / (1.0 + torch.exp(-g))
    assert _rel(got.double().cpu().numpy(), (a * u).cpu().numpy()) <= _tol(torch.bfloat16)
