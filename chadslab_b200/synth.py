"""Seeded synthetic packed weights generated on the device (benchmark / sweep data only)."""
from __future__ import annotations


def make_device_weight(torch, N: int, K: int, fmt: int, gen):
    """W ~ N(0, 0.02) quantized on the GPU with the format's rule -> (codes, scales) CUDA tensors in the
    interface layout.  Uses torch ops: this is data generation, not part of the matmul path."""
    qmax = 127.0 if fmt == 0 else 7.0
    codes = torch.empty((N, K if fmt == 0 else K // 2), dtype=torch.int8 if fmt == 0 else torch.uint8, device="cuda")
    scales = torch.empty((N, K // 32), dtype=torch.float16, device="cuda")
    rows = max(1, min(N, (64 << 20) // (K * 4)))
    for r0 in range(0, N, rows):
        r1 = min(N, r0 + rows)
        W = torch.randn((r1 - r0, K // 32, 32), device="cuda", generator=gen) * 0.02
        s = (W.abs().amax(-1) / qmax).to(torch.float16)
        s32 = s.float().clamp_min(1e-30)
        q = torch.clamp(torch.round(W / s32[..., None]), -qmax, qmax).reshape(r1 - r0, K)
        if fmt == 0:
            codes[r0:r1] = q.to(torch.int8)
        else:
            n = (q + 8).to(torch.uint8)
            codes[r0:r1] = n[:, 0::2] | (n[:, 1::2] << 4)
        scales[r0:r1] = s
    return codes, scales


def algorithmic_bytes(N: int, K: int, fmt: int, M: int, x_bytes: int = 2, y_bytes: int = 4) -> float:
    """codes + fp16 scales + activations + outputs (1.0625 / 0.5625 bytes per weight)."""
    return N * K * (1.0 if fmt == 0 else 0.5) + (N * K // 32) * 2 + M * K * x_bytes + M * N * y_bytes
