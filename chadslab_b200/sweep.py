"""Standalone quantized-matmul sweep: one weight shape, several batch sizes, chosen kernel path.

    python -m chadslab_b200.sweep --n 256000 --k 2048 --fmt int8,q4 --m 1,8,64,512,4096 [--path auto|mma|tensor|simt]
                                  [--reps 20] [--copies 1] [--check]

Prints one JSON line per (format, M): microseconds per launch (CUDA events), algorithmic GB/s, TFLOP/s, the
kernel family that ran, and with --check the max-normalised error against a float32 torch evaluation of the
dequantized weights (the library's own bit-exact dequantize, so this checks the matmul, not the format).
`--copies C` rotates over C distinct weight copies (use it for shapes smaller than L2).
"""
from __future__ import annotations

import argparse
import json

from . import _lib
from .ops import PackedWeight
from .synth import algorithmic_bytes, make_device_weight

PATHS = {"auto": 0, "simt": 1, "tensor": 2, "mma": 3}
FMTS = {"int8": 0, "q4": 1}


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--n", type=int, required=True)
    ap.add_argument("--k", type=int, required=True)
    ap.add_argument("--fmt", default="int8,q4")
    ap.add_argument("--m", default="1")
    ap.add_argument("--path", default="auto", choices=sorted(PATHS))
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--copies", type=int, default=1)
    ap.add_argument("--xdtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--check", action="store_true")
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)

    import torch
    torch.cuda.set_device(0)
    lib = _lib.init(0)
    gen = torch.Generator(device="cuda").manual_seed(a.seed)
    stream = torch.cuda.current_stream().cuda_stream
    xdt = torch.bfloat16 if a.xdtype == "bf16" else torch.float32
    for fname in a.fmt.split(","):
        fmt = FMTS[fname]
        codes, scales = make_device_weight(torch, a.n, a.k, fmt, gen)
        pws = [PackedWeight.from_device(codes.roll(c, 0).contiguous() if c else codes,
                                        scales.roll(c, 0).contiguous() if c else scales, fmt) for c in range(a.copies)]
        del codes, scales
        for M in [int(v) for v in a.m.split(",")]:
            x = torch.randn((M, a.k), device="cuda", generator=gen).to(xdt)
            y = torch.empty((M, a.n), dtype=torch.float32, device="cuda")
            call = lambda i: _lib.check(lib.bq_qlinear_ex(pws[i % len(pws)].handle, x.data_ptr(), 1 if xdt == torch.bfloat16 else 0,
                                                          M, y.data_ptr(), 0, PATHS[a.path], stream))
            for i in range(3):
                call(i)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for i in range(a.reps):
                call(i)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / a.reps
            rec = {"N": a.n, "K": a.k, "fmt": fname, "M": M, "x": a.xdtype, "path": {0: "none", 1: "simt", 2: "tensor", 3: "mma"}[lib.bq_last_path()],
                   "us": round(us, 2), "GBps": round(algorithmic_bytes(a.n, a.k, fmt, M, 2 if xdt == torch.bfloat16 else 4) / us / 1e3, 1),
                   "TFLOPs": round(2.0 * M * a.n * a.k / us / 1e6, 2)}
            if a.check:
                call(0)
                rows = min(a.n, 8192)
                Wd = pws[0].dequantize()[:rows]
                ref = x.float() @ Wd.t()
                rec["rel_err"] = float(((y[:, :rows] - ref).abs().max() / ref.abs().max()).item())
            print(json.dumps(rec), flush=True)
        for p in pws:
            p.close()
    _lib.check(lib.bq_status_poll())


if __name__ == "__main__":
    main()
