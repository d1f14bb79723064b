"""Host-side packer and PackedWeight/shard bookkeeping against the oracle (CPU only)."""
import numpy as np
import pytest

from chadslab_b200 import packing
from chadslab_b200.ops import PackedWeight, shard
from oracle import spec

CASES = ["rand_48x96", "rand_1x32", "rand_33x256", "zero_groups_8x64", "extremes_4x64", "range_16x128",
         "half_ties_2x32"]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("fmt,tag", [(0, "q8"), (1, "q4")])
def test_packer_matches_golden(qgolden, case, fmt, tag):
    codes, scales = packing.quantize(qgolden[f"{case}/W"], fmt)
    assert codes.dtype == packing.codes_dtype(fmt)
    assert np.array_equal(codes, qgolden[f"{case}/{tag}/codes"])
    assert np.array_equal(scales.view(np.uint16), qgolden[f"{case}/{tag}/scales"].view(np.uint16))


def test_packer_matches_oracle_random():
    rng = np.random.default_rng(7)
    for _ in range(10):
        N, G = int(rng.integers(1, 40)), int(rng.integers(1, 9))
        W = rng.normal(0, float(rng.uniform(1e-3, 3)), (N, 32 * G)).astype(np.float32)
        for fmt in (0, 1):
            a, b = packing.quantize(W, fmt), spec.quantize(W, fmt)
            assert np.array_equal(a[0], b[0]) and np.array_equal(a[1].view(np.uint16), b[1].view(np.uint16))
    u = rng.integers(-8, 8, (5, 64)).astype(np.int8)
    assert np.array_equal(packing.unpack_nibbles(packing.pack_nibbles(u)), u)
    assert np.array_equal(packing.pack_nibbles(u), spec.pack_q4(u))


def test_packer_rejects_bad_shapes():
    with pytest.raises(ValueError):
        packing.quantize(np.zeros((4, 48), np.float32), 0)      # K not a multiple of 32
    with pytest.raises(ValueError):
        packing.quantize(np.zeros((4,), np.float32), 0)
    with pytest.raises(ValueError):
        packing.quantize(np.zeros((4, 32), np.float32), 5)


def test_packed_weight_and_shard_bookkeeping():
    rng = np.random.default_rng(8)
    W = rng.normal(0, 0.02, (64, 256)).astype(np.float32)
    for fmt in (0, 1):
        pw = PackedWeight.from_float(W, fmt, upload=False)
        assert (pw.N, pw.K) == (64, 256)
        assert pw.nbytes == int(64 * 256 * (1.0625 if fmt == 0 else 0.5625))
        for world in (2, 4, 8):
            for r in range(world):
                a = shard(pw, "n", r, world, upload=False)
                c, s = spec.shard(pw.codes, pw.scales, fmt, "n", r, world)
                assert np.array_equal(a.codes, c) and np.array_equal(a.scales, s) and a.N == 64 // world
                b = shard(pw, "k", r, world, upload=False)
                c, s = spec.shard(pw.codes, pw.scales, fmt, "k", r, world)
                assert np.array_equal(b.codes, c) and np.array_equal(b.scales, s) and b.K == 256 // world
        with pytest.raises(ValueError):
            shard(pw, "k", 0, 16, upload=False)
        with pytest.raises(ValueError):
            shard(pw, "n", 0, 3, upload=False)
    with pytest.raises(ValueError):
        PackedWeight(np.zeros((2, 32), np.int8), np.zeros((2, 2), np.float16), 0, upload=False)
    with pytest.raises(TypeError):
        PackedWeight(np.zeros((2, 32), np.uint8), np.zeros((2, 1), np.float16), 0, upload=False)


def test_container_round_trip(tmp_path):
    from chadslab_b200 import container
    rng = np.random.default_rng(9)
    ws = {"l0.q": PackedWeight.from_float(rng.normal(0, 0.02, (24, 64)).astype(np.float32), 0, upload=False),
          "l0.down": PackedWeight.from_float(rng.normal(0, 0.02, (8, 96)).astype(np.float32), 1, upload=False)}
    extra = {"embed": rng.normal(0, 1, (10, 8)).astype(np.float32)}
    path = str(tmp_path / "w.safetensors")
    container.save_packed(path, ws, extra)
    got, tensors = container.load_packed(path, upload=False)
    assert set(got) == set(ws) and set(tensors) == {"embed"}
    for k in ws:
        assert got[k].fmt == ws[k].fmt and (got[k].N, got[k].K) == (ws[k].N, ws[k].K)
        assert np.array_equal(got[k].codes, ws[k].codes)
        assert np.array_equal(got[k].scales.view(np.uint16), ws[k].scales.view(np.uint16))
    assert np.array_equal(tensors["embed"], extra["embed"])
    with pytest.raises(ValueError):
        container.save_packed(path, ws, {"x.codes": extra["embed"]})


def test_interleave_gate_up_is_a_row_permutation():
    from chadslab_b200.ops import PackedWeight, interleave_gate_up, split_gate_up
    from oracle import spec
    rng = np.random.default_rng(4)
    for fmt in (0, 1):
        Wg, Wu = (rng.normal(0, 0.02, (24, 64)).astype(np.float32) for _ in range(2))
        g = PackedWeight(*spec.quantize(Wg, fmt), fmt, upload=False)
        u = PackedWeight(*spec.quantize(Wu, fmt), fmt, upload=False)
        f = interleave_gate_up(g, u, upload=False)
        assert f.N == 48 and f.K == 64
        d = spec.dequantize(f.codes, f.scales, fmt)                      # [48, 64]
        gg, uu = split_gate_up(d.T)                                      # split along the last axis
        assert np.array_equal(gg.T, spec.dequantize(g.codes, g.scales, fmt))
        assert np.array_equal(uu.T, spec.dequantize(u.codes, u.scales, fmt))
