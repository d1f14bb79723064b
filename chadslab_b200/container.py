"""On-disk container for packed weights: one `safetensors` file holding, per weight, `<name>.codes` (int8 [N,K]
or uint8 [N,K/2]) and `<name>.scales` (fp16 [N,K/32]) in the interface layout, plus plain tensors (embeddings,
norms) and JSON metadata (format id per weight, group size).  Loading re-tiles on upload (bq_weight_create)."""
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
