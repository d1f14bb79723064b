"""The C-ABI library loads and exports every symbol that include/b200q.h declares (no GPU needed),
and argument / state errors are reported through return codes, never by crashing."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200q.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bq_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(built_lib):
    from chadslab_b200 import _lib
    syms = declared_symbols()
    assert len(syms) >= 20
    for s in syms:
        assert hasattr(built_lib, s), f"{s} declared in b200q.h but not exported by libb200q.so"
    assert sorted(_lib.PROTOTYPES) == syms, "ctypes prototypes and header disagree"


def test_version_and_error_string(built_lib):
    assert built_lib.bq_version() >= 100
    assert isinstance(built_lib.bq_last_error(), bytes)


def test_no_cpu_fallback_without_init(built_lib):
    """Before bq_init (or with no GPU) compute calls fail with a code; nothing computes on the CPU."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("state test is for the GPU-less container")
    assert built_lib.bq_init(0) == -3                       # BQ_ERR_CUDA: no driver / device
    assert b"cuda" in built_lib.bq_last_error().lower()
    h = C.c_uint64(0)
    codes = np.zeros((2, 32), np.int8)
    scales = np.zeros((2, 1), np.float16)
    rc = built_lib.bq_weight_create(codes.ctypes.data, scales.ctypes.data, 2, 32, 0, C.byref(h))
    assert rc == -4 and h.value == 0                        # BQ_ERR_STATE
    assert built_lib.bq_qlinear(12345, None, 0, 1, None, 0, None) == -4
    assert built_lib.bq_moe_route(None, 1, 8, 2, 1, None, None, None) == -4


def test_python_surface_fails_loudly_without_gpu(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("state test is for the GPU-less container")
    import chadslab_b200 as cb
    W = np.random.default_rng(0).normal(0, 0.02, (4, 32)).astype(np.float32)
    with pytest.raises(cb.BqError):
        cb.PackedWeight.from_float(W, cb.FMT_Q8)            # upload needs a GPU: raises, no fallback
    pw = cb.PackedWeight.from_float(W, cb.FMT_Q8, upload=False)
    with pytest.raises(cb.BqError):
        cb.QuantLinear(pw)(np.zeros((1, 32), np.float32))
