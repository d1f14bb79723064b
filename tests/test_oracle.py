"""The numpy oracle against its golden fixtures and its own defining properties (CPU only)."""
import numpy as np
import pytest
from hypothesis import given, settings, strategies as st

from oracle import spec

CASES = ["rand_48x96", "rand_1x32", "rand_33x256", "zero_groups_8x64", "extremes_4x64", "range_16x128",
         "half_ties_2x32"]
FMTS = [(spec.FMT_Q8, "q8"), (spec.FMT_Q4, "q4")]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("fmt,tag", FMTS)
def test_golden_quantize_dequant(qgolden, case, fmt, tag):
    W = qgolden[f"{case}/W"]
    codes, scales = spec.quantize(W, fmt)
    assert np.array_equal(codes, qgolden[f"{case}/{tag}/codes"])
    assert np.array_equal(scales.view(np.uint16), qgolden[f"{case}/{tag}/scales"].view(np.uint16))
    assert np.array_equal(spec.codes_of(codes, fmt), qgolden[f"{case}/{tag}/unpacked"])
    d = spec.dequantize(codes, scales, fmt)
    assert np.array_equal(d.view(np.uint32), qgolden[f"{case}/{tag}/dequant"].view(np.uint32))


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("fmt,tag", FMTS)
def test_golden_qlinear(qgolden, case, fmt, tag):
    codes, scales = qgolden[f"{case}/{tag}/codes"], qgolden[f"{case}/{tag}/scales"]
    xb = spec.from_bf16_bits(qgolden[f"{case}/x_bf16"])
    y = spec.qlinear(xb, codes, scales, fmt)
    assert spec.rel_err(y, qgolden[f"{case}/{tag}/y_bf16"]) <= 1e-5   # fp32 BLAS vs float64 golden
    y = spec.qlinear(qgolden[f"{case}/x_f32"], codes, scales, fmt)
    assert spec.rel_err(y, qgolden[f"{case}/{tag}/y_f32"]) <= 1e-5


def test_known_answers():
    # hand-computed: scale = fp16(absmax/qmax), code = rint(w/scale)
    W = np.zeros((1, 32), np.float32)
    W[0, 0], W[0, 1], W[0, 2] = 1.27, -0.64, 0.005
    c, s = spec.quantize_q8_g32(W)
    assert s[0, 0] == np.float16(0.01) and list(c[0, :3]) == [127, -64, 0 if abs(0.005 / float(np.float16(0.01))) < 0.5 else 1]
    W[0, :3] = [0.7, -0.35, 0.1]
    p, s = spec.quantize_q4_g32(W)
    assert s[0, 0] == np.float16(0.1)
    u = spec.unpack_q4(p)
    assert list(u[0, :3]) == [7, -4 if -0.35 / float(np.float16(0.1)) < -3.5 else -3, 1]
    # nibble order: element 0 in the low nibble, stored as code+8
    assert p[0, 0] == ((u[0, 0] + 8) | ((u[0, 1] + 8) << 4))
    d = spec.dequantize(p, s, spec.FMT_Q4)
    assert d[0, 0] == np.float32(7) * np.float32(np.float16(0.1))


def test_zero_group_and_extremes(qgolden):
    for fmt, tag, qmax in ((spec.FMT_Q8, "q8", 127), (spec.FMT_Q4, "q4", 7)):
        u = qgolden[f"zero_groups_8x64/{tag}/unpacked"]
        s = qgolden[f"zero_groups_8x64/{tag}/scales"]
        assert s[2, 0] == 0 and not u[2, :32].any() and s[3, 1] == 0 and not u[3, 32:].any()
        u = qgolden[f"extremes_4x64/{tag}/unpacked"]
        assert (u[0] == qmax).all() and (u[1] == -qmax).all()
        assert (u[2, 0::2] == qmax).all() and (u[2, 1::2] == -qmax).all()


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 9), st.integers(1, 6), st.integers(0, 2 ** 31 - 1), st.sampled_from([0, 1]),
       st.floats(1e-4, 50.0))
def test_quantizer_properties(N, G, seed, fmt, sigma):
    rng = np.random.default_rng(seed)
    W = rng.normal(0, sigma, (N, G * 32)).astype(np.float32)
    codes, scales = spec.quantize(W, fmt)
    qmax = 127 if fmt == spec.FMT_Q8 else 7
    u = spec.codes_of(codes, fmt)
    assert u.min() >= -qmax and u.max() <= qmax
    if fmt == spec.FMT_Q4:
        assert np.array_equal(spec.unpack_q4(spec.pack_q4(u)), u)          # pack -> unpack = identity
        assert (codes & 0xF).min() >= 1 and (codes >> 4).min() >= 1         # nibble 0 never produced
    d = spec.dequantize(codes, scales, fmt)
    s = np.repeat(scales.astype(np.float32), 32, axis=1)
    # |w - dequant| <= scale/2 inside the clip range (plus the fp16 rounding of the scale at the edge)
    err = np.abs(W - d)
    c2, s2 = spec.quantize(d, fmt)
    if scales.astype(np.float32).min() >= 2.0 ** -14:    # normal fp16 scales only (subnormal ones clip)
        assert (err <= s * (0.5 + qmax * 2.0 ** -11) + 1e-30).all()
        # re-quantizing the dequantized weight reproduces the codes (idempotence)
        assert np.array_equal(spec.codes_of(c2, fmt), u)
        assert np.array_equal(s2.view(np.uint16), scales.view(np.uint16))


def test_bf16_round_matches_ml_dtypes():
    import ml_dtypes
    rng = np.random.default_rng(3)
    a = np.concatenate([rng.normal(0, 1, 4096), rng.normal(0, 1e-3, 4096), [0.0, -0.0, 1.0, 65504.0, 3.0e38]])
    a = a.astype(np.float32)
    ref = a.astype(ml_dtypes.bfloat16).astype(np.float32)
    assert np.array_equal(spec.bf16_round(a).view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(spec.from_bf16_bits(spec.to_bf16_bits(a)), ref)


def test_shard_equals_unsharded():
    rng = np.random.default_rng(4)
    W = rng.normal(0, 0.02, (64, 256)).astype(np.float32)
    x = rng.normal(0, 1, (5, 256)).astype(np.float32)
    for fmt in (spec.FMT_Q8, spec.FMT_Q4):
        codes, scales = spec.quantize(W, fmt)
        full = spec.qlinear(x, codes, scales, fmt, f64=True)
        for world in (2, 4, 8):
            cols = [spec.qlinear(x, *spec.shard(codes, scales, fmt, "n", r, world), fmt, f64=True) for r in range(world)]
            assert np.array_equal(np.concatenate(cols, axis=1), full)
            k = 256 // world
            rows = sum(spec.qlinear(x[:, r * k:(r + 1) * k], *spec.shard(codes, scales, fmt, "k", r, world), fmt, f64=True)
                       for r in range(world))
            assert spec.rel_err(rows, full) < 1e-12
    with pytest.raises(ValueError):
        spec.shard(codes, scales, fmt, "k", 0, 16)     # 256/16 = 16 is not a multiple of 32


def test_route_ties_and_golden(moegolden):
    logits = moegolden["route/logits"]
    idx, w = spec.moe_route_from_logits(logits, 4)
    assert np.array_equal(idx, moegolden["route/idx"])
    assert list(idx[1]) == [0, 1, 2, 3]                 # all equal -> lowest ids
    assert list(idx[2][:2]) == [3, 9]                   # two-way tie -> lower id first
    assert np.allclose(w.sum(-1), 1.0, atol=1e-6)
    perm, offsets = spec.moe_permute(idx, 16)
    assert np.array_equal(perm, moegolden["route/perm"]) and np.array_equal(offsets, moegolden["route/offsets"])
    flat = idx.reshape(-1)
    assert (np.diff(flat[perm]) >= 0).all()             # sorted by expert
    for e in range(16):
        seg = perm[offsets[e]:offsets[e + 1]]
        assert (np.diff(seg) > 0).all()                 # stable within an expert


@pytest.mark.parametrize("fmt,tag", FMTS)
def test_moe_equals_dense_masked(moegolden, fmt, tag):
    E = moegolden[f"{tag}/gate_codes"].shape[0]
    x = spec.from_bf16_bits(moegolden["x_bf16"])
    router = (moegolden[f"{tag}/router_codes"], moegolden[f"{tag}/router_scales"])
    pick = lambda nm: [(moegolden[f"{tag}/{nm}_codes"][e], moegolden[f"{tag}/{nm}_scales"][e]) for e in range(E)]
    y, (idx, w, perm, offsets) = spec.moe_forward(x, router, pick("gate"), pick("up"), pick("down"), fmt, 2)
    assert np.array_equal(idx, moegolden[f"{tag}/idx"])
    assert spec.rel_err(y, moegolden[f"{tag}/y"]) < 1e-6
    dense = spec.moe_dense_reference(x, router, pick("gate"), pick("up"), pick("down"), fmt, 2)
    assert spec.rel_err(y, dense) < 1e-5
