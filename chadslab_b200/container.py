"""On-disk container for packed weights: one `safetensors` file holding, per weight, `<name>.codes` (int8 [N,K]
or uint8 [N,K/2]) and `<name>.scales` (fp16 [N,K/32]) in the interface layout, plus plain tensors (embeddings,
norms) and JSON metadata (format id per weight, group size).  Loading re-tiles on upload (bq_weight_create).
`iter_packed` streams: it reads one weight at a time in row blocks of bounded size straight into device memory,
so a checkpoint larger than host memory can be served."""
from __future__ import annotations

import json
from typing import Dict, Tuple

import numpy as np

from .ops import PackedWeight
from .packing import GROUP

FORMAT_TAG = "b200q-packed-v1"


def save_packed(path: str, weights: Dict[str, PackedWeight], tensors: Dict[str, np.ndarray] = None) -> None:
    from safetensors.numpy import save_file
    blob, fmts = {}, {}
    for name, pw in weights.items():
        if pw.codes is None:
            codes, scales = pw.export()
        else:
            codes, scales = pw.codes, pw.scales
        blob[f"{name}.codes"] = np.ascontiguousarray(codes)
        blob[f"{name}.scales"] = np.ascontiguousarray(scales)
        fmts[name] = int(pw.fmt)
    for name, t in (tensors or {}).items():
        if name.endswith(".codes") or name.endswith(".scales"):
            raise ValueError(f"tensor name {name!r} collides with the packed-weight naming")
        blob[name] = np.ascontiguousarray(t)
    save_file(blob, path, metadata={"format": FORMAT_TAG, "group": str(GROUP), "weights": json.dumps(fmts)})


def load_packed(path: str, upload: bool = True, device=None) -> Tuple[Dict[str, PackedWeight], Dict[str, np.ndarray]]:
    from safetensors import safe_open
    weights, tensors = {}, {}
    with safe_open(path, framework="numpy") as f:
        meta = f.metadata() or {}
        if meta.get("format") != FORMAT_TAG:
            raise ValueError(f"{path}: not a {FORMAT_TAG} container")
        if int(meta.get("group", "0")) != GROUP:
            raise ValueError(f"{path}: group size {meta.get('group')} != {GROUP}")
        fmts = json.loads(meta["weights"])
        keys = set(f.keys())
        for name, fmt in fmts.items():
            if f"{name}.codes" not in keys or f"{name}.scales" not in keys:
                raise ValueError(f"{path}: weight {name!r} is incomplete")
            weights[name] = PackedWeight(f.get_tensor(f"{name}.codes"), f.get_tensor(f"{name}.scales"), int(fmt),
                                         upload=upload, device=device)
        for k in keys:
            base = k.rsplit(".", 1)[0]
            if not ((k.endswith(".codes") or k.endswith(".scales")) and base in fmts):
                tensors[k] = f.get_tensor(k)
    return weights, tensors


def iter_packed(path: str, chunk_bytes: int = 64 << 20):
    """Yields (name, PackedWeight) for every packed weight of the container, one at a time.  Codes and scales are
    read in blocks of rows of at most `chunk_bytes` and copied into device tensors; the weight is then created from
    the device copy (which re-tiles it) and no host copy is kept (`pw.codes is None`)."""
    import torch
    from safetensors import safe_open
    with safe_open(path, framework="numpy") as f:
        meta = f.metadata() or {}
        if meta.get("format") != FORMAT_TAG:
            raise ValueError(f"{path}: not a {FORMAT_TAG} container")
        if int(meta.get("group", "0")) != GROUP:
            raise ValueError(f"{path}: group size {meta.get('group')} != {GROUP}")
        fmts = json.loads(meta["weights"])
        keys = set(f.keys())
        for name, fmt in fmts.items():
            if f"{name}.codes" not in keys or f"{name}.scales" not in keys:
                raise ValueError(f"{path}: weight {name!r} is incomplete")
            cs, ss = f.get_slice(f"{name}.codes"), f.get_slice(f"{name}.scales")
            N, kb = cs.get_shape()
            d_codes = torch.empty((N, kb), dtype=torch.int8 if int(fmt) == 0 else torch.uint8, device="cuda")
            d_scales = torch.empty(tuple(ss.get_shape()), dtype=torch.float16, device="cuda")
            rows = max(1, int(chunk_bytes) // max(1, kb))
            for r0 in range(0, N, rows):
                r1 = min(N, r0 + rows)
                d_codes[r0:r1].copy_(torch.from_numpy(np.ascontiguousarray(cs[r0:r1])))
                d_scales[r0:r1].copy_(torch.from_numpy(np.ascontiguousarray(ss[r0:r1])))
            yield name, PackedWeight.from_device(d_codes, d_scales, int(fmt))
