"""Generates the golden fixtures in this directory from the numpy oracle (oracle/spec.py).

The reference checkout holds no code, test or vector for the quantized-matmul path, so these
fixtures pin the path to the self-authored oracle (seeded, small, both formats, edge cases).
Run from the repository root:   python tests/golden/make_golden.py
"""
from __future__ import annotations

import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import spec  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))


def weight_cases():
    rng = np.random.default_rng(0)
    cases = {}
    cases["rand_48x96"] = rng.normal(0, 0.02, (48, 96)).astype(np.float32)
    cases["rand_1x32"] = rng.normal(0, 0.02, (1, 32)).astype(np.float32)       # N=1, K=32
    cases["rand_33x256"] = rng.normal(0, 0.02, (33, 256)).astype(np.float32)   # ragged N
    w = rng.normal(0, 0.02, (8, 64)).astype(np.float32)
    w[2, :32] = 0.0                      # an all-zero group
    w[3, 32:] = 0.0
    cases["zero_groups_8x64"] = w
    w = np.zeros((4, 64), dtype=np.float32)
    w[0, :] = 0.5                        # every element = +absmax -> all codes +qmax
    w[1, :] = -0.5                       # every element = -absmax -> all codes -qmax
    w[2, 0::2], w[2, 1::2] = 0.25, -0.25  # alternating +-absmax
    w[3, :] = np.linspace(-1, 1, 64, dtype=np.float32)
    cases["extremes_4x64"] = w
    w = rng.normal(0, 0.02, (16, 128)).astype(np.float32)
    w[0, 0] = 3.0e4                      # large magnitude (scale near the top of fp16 range / 127)
    w[1, :32] = 1.0e-7                   # scale underflows towards fp16 subnormals
    w[2, 5] = 0.5                        # one outlier in a group: rint ties and tiny codes
    cases["range_16x128"] = w
    # exact half-way values: w / scale = k + 0.5 exercises round-half-to-even
    w = np.zeros((2, 32), dtype=np.float32)
    w[0] = (np.arange(32, dtype=np.float32) - 16 + 0.5) * np.float32(2.0 ** -6)
    w[0, 0] = -127 * np.float32(2.0 ** -6)
    w[1] = (np.arange(32, dtype=np.float32) % 14 - 7 + 0.5) * np.float32(2.0 ** -4)
    w[1, 0] = -7 * np.float32(2.0 ** -4)
    cases["half_ties_2x32"] = w
    return cases


def main() -> None:
    rng = np.random.default_rng(1)
    out = {}
    for name, W in weight_cases().items():
        N, K = W.shape
        out[f"{name}/W"] = W
        xb = spec.bf16_round(rng.normal(0, 1, (3, K)).astype(np.float32))    # bf16-representable
        xf = rng.normal(0, 1, (2, K)).astype(np.float32)
        out[f"{name}/x_bf16"] = spec.to_bf16_bits(xb)
        out[f"{name}/x_f32"] = xf
        for fmt, tag in ((spec.FMT_Q8, "q8"), (spec.FMT_Q4, "q4")):
            codes, scales = spec.quantize(W, fmt)
            out[f"{name}/{tag}/codes"] = codes
            out[f"{name}/{tag}/scales"] = scales
            out[f"{name}/{tag}/unpacked"] = spec.codes_of(codes, fmt)
            out[f"{name}/{tag}/dequant"] = spec.dequantize(codes, scales, fmt)
            out[f"{name}/{tag}/y_bf16"] = spec.qlinear(xb, codes, scales, fmt, f64=True).astype(np.float32)
            out[f"{name}/{tag}/y_f32"] = spec.qlinear(xf, codes, scales, fmt, f64=True).astype(np.float32)
    np.savez_compressed(os.path.join(OUT, "qlinear_golden.npz"), **out)

    # ---- MoE: 6 experts, hidden 64, ffn 96, top-2, 10 tokens, both formats; plus routing ties
    moe = {}
    rng = np.random.default_rng(2)
    E, H, F, T, k = 6, 64, 96, 10, 2
    x = spec.bf16_round(rng.normal(0, 1, (T, H)).astype(np.float32))
    moe["x_bf16"] = spec.to_bf16_bits(x)
    Wr = rng.normal(0, 0.5, (E, H)).astype(np.float32)
    Wg = rng.normal(0, 0.1, (E, F, H)).astype(np.float32)
    Wu = rng.normal(0, 0.1, (E, F, H)).astype(np.float32)
    Wd = rng.normal(0, 0.1, (E, H, F)).astype(np.float32)
    for fmt, tag in ((spec.FMT_Q8, "q8"), (spec.FMT_Q4, "q4")):
        router = spec.quantize(Wr, fmt)
        gate = [spec.quantize(Wg[e], fmt) for e in range(E)]
        up = [spec.quantize(Wu[e], fmt) for e in range(E)]
        down = [spec.quantize(Wd[e], fmt) for e in range(E)]
        y, (idx, w, perm, offsets) = spec.moe_forward(x, router, gate, up, down, fmt, k)
        moe[f"{tag}/router_codes"], moe[f"{tag}/router_scales"] = router
        for nm, lst in (("gate", gate), ("up", up), ("down", down)):
            moe[f"{tag}/{nm}_codes"] = np.stack([c for c, _ in lst])
            moe[f"{tag}/{nm}_scales"] = np.stack([s for _, s in lst])
        moe[f"{tag}/idx"], moe[f"{tag}/w"], moe[f"{tag}/perm"], moe[f"{tag}/offsets"] = idx, w, perm, offsets
        moe[f"{tag}/y"] = y
    # routing-only vectors, including exact ties (lower expert id must win)
    logits = rng.normal(0, 1, (7, 16)).astype(np.float32)
    logits[1, :] = 0.25                       # all equal
    logits[2, [3, 9]] = 5.0                   # two-way tie at the top
    logits[3, 8:] = logits[3, :8]             # every value duplicated
    idx, w = spec.moe_route_from_logits(logits, 4)
    moe["route/logits"], moe["route/idx"], moe["route/w"] = logits, idx, w
    perm, offsets = spec.moe_permute(idx, 16)
    moe["route/perm"], moe["route/offsets"] = perm, offsets
    np.savez_compressed(os.path.join(OUT, "moe_golden.npz"), **moe)
    print("wrote", sorted(f for f in os.listdir(OUT) if f.endswith(".npz")))


if __name__ == "__main__":
    main()
