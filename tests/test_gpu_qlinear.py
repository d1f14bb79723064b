"""Parity of the CUDA path (through the C ABI) with the numpy oracle: unpack / dequant bit-exact,
matmul outputs within 1e-3 (max error / max magnitude; tolerance stated by the specification)."""
import ctypes as C

import numpy as np
import pytest

from oracle import spec

pytestmark = pytest.mark.gpu

TOL = 1e-3          # matmul outputs: max|y - y_ref| / max|y_ref|
TOL_SIMT = 2e-5     # the exact-fp32 CUDA-core path is far inside it
CASES = ["rand_48x96", "rand_1x32", "rand_33x256", "zero_groups_8x64", "extremes_4x64", "range_16x128",
         "half_ties_2x32"]
FMTS = [(0, "q8"), (1, "q4")]


def _bf16_tensor(bits, torch):
    return torch.from_numpy(bits.astype(np.int16)).cuda().view(torch.bfloat16)


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("fmt,tag", FMTS)
def test_golden_unpack_dequant_bit_exact(cuda_lib, qgolden, case, fmt, tag):
    import torch
    import chadslab_b200 as cb
    pw = cb.PackedWeight.from_arrays(qgolden[f"{case}/{tag}/codes"], qgolden[f"{case}/{tag}/scales"], fmt)
    assert np.array_equal(pw.unpack().cpu().numpy(), qgolden[f"{case}/{tag}/unpacked"])
    d = pw.dequantize(torch.float32).cpu().numpy()
    assert np.array_equal(d.view(np.uint32), qgolden[f"{case}/{tag}/dequant"].view(np.uint32))
    db = pw.dequantize(torch.bfloat16).float().cpu().numpy()
    assert np.array_equal(db.view(np.uint32), spec.bf16_round(qgolden[f"{case}/{tag}/dequant"]).view(np.uint32))
    codes, scales = pw.export()                       # device layout is a pure permutation of the host one
    assert np.array_equal(codes, qgolden[f"{case}/{tag}/codes"])
    assert np.array_equal(scales.view(np.uint16), qgolden[f"{case}/{tag}/scales"].view(np.uint16))


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("fmt,tag", FMTS)
def test_golden_qlinear(cuda_lib, qgolden, case, fmt, tag):
    import torch
    import chadslab_b200 as cb
    pw = cb.PackedWeight.from_arrays(qgolden[f"{case}/{tag}/codes"], qgolden[f"{case}/{tag}/scales"], fmt)
    lin = cb.QuantLinear(pw)
    y = lin(_bf16_tensor(qgolden[f"{case}/x_bf16"], torch)).cpu().numpy()
    assert spec.rel_err(y, qgolden[f"{case}/{tag}/y_bf16"]) <= TOL
    y = lin(torch.from_numpy(qgolden[f"{case}/x_f32"]).cuda()).cpu().numpy()
    assert spec.rel_err(y, qgolden[f"{case}/{tag}/y_f32"]) <= TOL_SIMT
    y = cb.QuantLinear(pw, path=cb.PATH_SIMT)(_bf16_tensor(qgolden[f"{case}/x_bf16"], torch)).cpu().numpy()
    assert spec.rel_err(y, qgolden[f"{case}/{tag}/y_bf16"]) <= TOL_SIMT


SHAPES = [(64, 64), (96, 2048), (1000, 512), (257, 4096), (2048, 2048), (130, 768), (768, 2048), (384, 16384)]


@pytest.mark.parametrize("N,K", SHAPES)
@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("xdt", ["bf16", "f32"])
def test_qlinear_parity_sweep(cuda_lib, N, K, fmt, xdt):
    """Seeded weights N(0,0.02), activations N(0,1); every M regime the dispatcher distinguishes."""
    import torch
    import chadslab_b200 as cb
    rng = np.random.default_rng(1000 + N + K + fmt)
    W = rng.normal(0, 0.02, (N, K)).astype(np.float32)
    codes, scales = spec.quantize(W, fmt)
    pw = cb.PackedWeight.from_arrays(codes, scales, fmt)
    lin = cb.QuantLinear(pw)
    for M in (1, 2, 3, 5, 8, 9, 16, 17, 64, 130):
        x = rng.normal(0, 1, (M, K)).astype(np.float32)
        if xdt == "bf16":
            x = spec.bf16_round(x)
            xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
        else:
            xt = torch.from_numpy(x).cuda()
        ref = spec.qlinear(x, codes, scales, fmt, f64=True)
        y = lin(xt).cpu().numpy()
        err = spec.rel_err(y, ref)
        assert err <= TOL, f"M={M} rel_err={err:.3e}"
        assert spec.rel_err_elementwise(y, ref) <= 2.0, "an element is grossly wrong"
        ys = cb.QuantLinear(pw, path=cb.PATH_SIMT)(xt).cpu().numpy()
        assert spec.rel_err(ys, ref) <= TOL_SIMT, f"SIMT M={M}"


@pytest.mark.parametrize("fmt", [0, 1])
def test_bf16_output_and_strided_batches(cuda_lib, fmt):
    import torch
    import chadslab_b200 as cb
    rng = np.random.default_rng(5)
    W = rng.normal(0, 0.02, (320, 512)).astype(np.float32)
    codes, scales = spec.quantize(W, fmt)
    pw = cb.PackedWeight.from_arrays(codes, scales, fmt)
    x = spec.bf16_round(rng.normal(0, 1, (2, 3, 512)).astype(np.float32))
    ref = spec.qlinear(x.reshape(6, 512), codes, scales, fmt, f64=True).reshape(2, 3, 320)
    y = cb.QuantLinear(pw, out_dtype=torch.bfloat16)(torch.from_numpy(x).cuda().to(torch.bfloat16))
    assert y.dtype == torch.bfloat16 and tuple(y.shape) == (2, 3, 320)
    assert spec.rel_err(y.float().cpu().numpy(), ref) <= 6e-3          # bf16 output rounding (2^-8)


@pytest.mark.parametrize("fmt", [0, 1])
def test_host_buffer_entry_point(cuda_lib, fmt):
    """bq_qlinear_host: host in, host out (the end-to-end call the benchmark times)."""
    import ml_dtypes
    import chadslab_b200 as cb
    rng = np.random.default_rng(6)
    W = rng.normal(0, 0.02, (513, 1024)).astype(np.float32)
    codes, scales = spec.quantize(W, fmt)
    pw = cb.PackedWeight.from_arrays(codes, scales, fmt)
    lin = cb.QuantLinear(pw)
    for M in (1, 7):
        x = rng.normal(0, 1, (M, 1024)).astype(np.float32)
        y = lin(x)
        assert isinstance(y, np.ndarray) and spec.rel_err(y, spec.qlinear(x, codes, scales, fmt, f64=True)) <= TOL_SIMT
        xb = x.astype(ml_dtypes.bfloat16)
        y = lin(xb)
        assert spec.rel_err(y, spec.qlinear(xb.astype(np.float32), codes, scales, fmt, f64=True)) <= TOL


@pytest.mark.parametrize("fmt", [0, 1])
def test_lm_head_greedy(cuda_lib, fmt):
    import torch
    import chadslab_b200 as cb
    rng = np.random.default_rng(9)
    V, K = 40000, 256          # > 32768: exercises the two-stage argmax; rows 123 and 777 fall in different slices
    W = rng.normal(0, 0.02, (V, K)).astype(np.float32)
    W[777] = W[123]                                           # exact tie between two vocabulary rows
    codes, scales = spec.quantize(W, fmt)
    head = cb.LMHead(cb.PackedWeight.from_arrays(codes, scales, fmt))
    x = spec.bf16_round(rng.normal(0, 1, (4, K)).astype(np.float32))
    x[3] = spec.bf16_round(50 * spec.dequantize(codes, scales, fmt)[123])   # row 3 points at the tied rows
    ref_logits, ref_ids = spec.lm_head(x, codes, scales, fmt, f64=True)
    xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
    ids, logits = head.greedy(xt, return_logits=True)
    assert spec.rel_err(logits.cpu().numpy(), ref_logits) <= TOL
    got = ids.cpu().numpy()
    assert got[3] == 123 and ref_ids[3] == 123               # tie -> lower id
    # greedy ids must be the argmax of the kernel's own logits, and agree with the oracle unless near-tied
    assert np.array_equal(got, np.argmax(logits.cpu().numpy(), axis=-1))
    for m in range(3):
        if got[m] != ref_ids[m]:
            assert abs(ref_logits[m, got[m]] - ref_logits[m, ref_ids[m]]) <= TOL * np.abs(ref_logits[m]).max()
    assert np.array_equal(head.greedy(xt).cpu().numpy(), got)  # argmax-only entry (no logits buffer)


def test_size_independent_properties_full_size(cuda_lib):
    """Full-size lm_head shape (256000 x 2048): linearity and row-subset consistency, no CPU matmul."""
    import torch
    import chadslab_b200 as cb
    g = torch.Generator(device="cuda").manual_seed(0)
    N, K = 256000, 2048
    for fmt in (0, 1):
        kb = K if fmt == 0 else K // 2
        codes = torch.randint(0, 256, (N, kb), dtype=torch.uint8, device="cuda", generator=g)
        if fmt == 1:
            codes = codes | 0x11                                 # keep nibbles >= 1 (code >= -7)
        else:
            codes = torch.where(codes == 128, torch.zeros_like(codes), codes)  # avoid code -128
        scales = (torch.rand((N, K // 32), device="cuda", generator=g) * 2e-3 + 1e-4).to(torch.float16)
        pw = cb.PackedWeight.from_device(codes.view(torch.int8) if fmt == 0 else codes, scales, fmt)
        lin = cb.QuantLinear(pw)
        xa = torch.randn((1, K), device="cuda", generator=g).to(torch.bfloat16)
        xb = torch.randn((1, K), device="cuda", generator=g).to(torch.bfloat16)
        ya, yb = lin(xa), lin(xb)
        # linearity in x (fp32 activations take the exact path): W(2a) = 2 W(a); W(a+b) = W(a)+W(b)
        assert torch.equal(lin(xa * 2), ya * 2)
        yab = lin(xa.float() + xb.float())
        assert (yab - (ya + yb)).abs().max() <= 1e-4 * yab.abs().max()
        # batched rows equal single rows
        y2 = lin(torch.cat([xa, xb, xa], 0))
        scale = ya.abs().max()
        assert (y2[0] - ya[0]).abs().max() <= TOL * scale and (y2[2] - ya[0]).abs().max() <= TOL * scale
        # a sampled subset of rows against the oracle
        rows = torch.randint(0, N, (64,), device="cuda", generator=g)
        c_np = codes[rows].cpu().numpy()
        s_np = scales[rows].cpu().numpy()
        ref = spec.qlinear(xa.float().cpu().numpy(), c_np.view(np.int8) if fmt == 0 else c_np, s_np, fmt, f64=True)
        assert spec.rel_err(ya[:, rows].cpu().numpy(), ref) <= TOL_SIMT
        pw.close()


def test_edge_cases_and_errors(cuda_lib):
    import torch
    import chadslab_b200 as cb
    from chadslab_b200 import _lib
    lib = cuda_lib
    # empty weight (N = 0) and empty batch (M = 0)
    pw0 = cb.PackedWeight(np.zeros((0, 64), np.int8), np.zeros((0, 2), np.float16), 0)
    y = cb.QuantLinear(pw0)(torch.zeros((3, 64), device="cuda"))
    assert tuple(y.shape) == (3, 0)
    rng = np.random.default_rng(1)
    W = rng.normal(0, 0.02, (8, 64)).astype(np.float32)
    pw = cb.PackedWeight.from_float(W, 1)
    y = cb.QuantLinear(pw)(torch.zeros((0, 64), device="cuda", dtype=torch.bfloat16))
    assert tuple(y.shape) == (0, 8)
    # K not a multiple of 32 is rejected on the host
    h = C.c_uint64(0)
    buf = np.zeros(4096, np.uint8)
    assert lib.bq_weight_create(buf.ctypes.data, buf.ctypes.data, 4, 48, 0, C.byref(h)) == _lib.ERR_ARG
    assert b"multiple of 32" in lib.bq_last_error()
    assert lib.bq_weight_create(buf.ctypes.data, buf.ctypes.data, 4, 64, 7, C.byref(h)) == _lib.ERR_ARG
    assert lib.bq_weight_create(None, buf.ctypes.data, 4, 64, 0, C.byref(h)) == _lib.ERR_ARG
    # bad / destroyed handle
    assert lib.bq_qlinear(0xdeadbeef, None, 0, 1, None, 0, None) == _lib.ERR_HANDLE
    hh = pw.handle
    pw.close()
    assert lib.bq_weight_destroy(hh) == _lib.ERR_HANDLE
    # bad dtype, null activations
    pw = cb.PackedWeight.from_float(W, 0)
    assert lib.bq_qlinear(pw.handle, None, 0, 1, None, 0, None) == _lib.ERR_ARG
    t = torch.zeros((1, 64), device="cuda")
    assert lib.bq_qlinear(pw.handle, t.data_ptr(), 9, 1, t.data_ptr(), 0, None) == _lib.ERR_ARG
    with pytest.raises(ValueError):
        cb.QuantLinear(pw)(torch.zeros((1, 32), device="cuda"))
    with pytest.raises(TypeError):
        cb.QuantLinear(pw)(torch.zeros((1, 64), device="cuda", dtype=torch.float16))
    assert lib.bq_status_poll() == 0
    assert lib.bq_launch_count() > 0


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("wdt", ["float32", "bfloat16"])
def test_device_quantizer_is_bit_identical_to_the_oracle(cuda_lib, fmt, wdt):
    """bq_quantize against oracle.spec.quantize: codes and scales bit for bit, including the edge groups (all zero,
    exact ties x.5, values at +-absmax, an absmax that underflows fp16, a scale clamped to the fp16 maximum)."""
    import torch
    import chadslab_b200 as cb
    rng = np.random.default_rng(17)
    N, K = 96, 256
    W = rng.normal(0, 0.02, (N, K)).astype(np.float32)
    W[0, :32] = 0.0                                           # all-zero group
    if fmt == 0:
        W[1, :32] = (np.arange(-16, 16, dtype=np.float32) + 0.5) * 0.5       # w / 0.5 = -15.5 .. 15.5: every element a tie
        W[1, 0] = -63.5                                                       # absmax chosen so that scale = 0.5
    else:
        W[1, :32] = (np.arange(32, dtype=np.float32) % 14 - 7 + 0.5) * 0.5   # w / 0.5 = -6.5 .. 6.5: ties
        W[1, 0] = -3.5
    W[2, :32] = 1e-9                                          # absmax / qmax underflows fp16 -> scale 0 -> codes 0
    W[3, :32] = 3.0e7                                         # scale clamps to 65504
    W[4, 32:64] = -W[4, 32:64].max()                          # every element at -absmax
    dt = getattr(torch, wdt)
    Wt = torch.from_numpy(W).cuda().to(dt)
    Wref = Wt.float().cpu().numpy()                           # what the device sees (bf16-rounded when wdt is bf16)
    pw = cb.PackedWeight.from_float_device(Wt, fmt)
    codes, scales = pw.export()
    rc, rs = spec.quantize(Wref, fmt)
    assert np.array_equal(scales.view(np.uint16), rs.view(np.uint16))
    assert np.array_equal(codes, rc)
    # and it multiplies like a host-packed weight
    x = torch.randn((1, K), device="cuda").to(torch.bfloat16)
    host = cb.PackedWeight.from_arrays(rc, rs, fmt)
    assert torch.equal(cb.QuantLinear(pw)(x), cb.QuantLinear(host)(x))


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("odt", ["float32", "bfloat16"])
def test_tensor_path_split_k_for_few_output_tiles(cuda_lib, fmt, odt):
    """Few 128-row output tiles and a long K: the tensor-core kernel splits K over the grid and a second kernel adds
    the partial tiles in order.  Same tolerance as every other matmul; repeated calls give identical bits."""
    import torch
    import chadslab_b200 as cb
    rng = np.random.default_rng(77 + fmt)
    for N, K in ((200, 8192), (512, 16384), (130, 1024)):
        codes, scales = spec.quantize(rng.normal(0, 0.02, (N, K)).astype(np.float32), fmt)
        pw = cb.PackedWeight.from_arrays(codes, scales, fmt)
        lin = cb.QuantLinear(pw, out_dtype=getattr(torch, odt), path=cb.PATH_TENSOR)
        for M in (8, 64, 300):
            x = spec.bf16_round(rng.normal(0, 1, (M, K)).astype(np.float32))
            xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
            y1 = lin(xt)
            y2 = lin(xt)
            assert torch.equal(y1, y2)
            ref = spec.qlinear(x, codes, scales, fmt, f64=True)
            tol = TOL if odt == "float32" else TOL + 2.0 ** -8
            assert spec.rel_err(y1.float().cpu().numpy(), ref) <= tol, (N, K, M)
    assert cuda_lib.bq_status_poll() == 0


@pytest.mark.parametrize("fmt", [0, 1])
def test_tile_store_epilogue_output_types_and_edges(cuda_lib, fmt):
    """The tcgen05 kernels store their output tile through shared memory and one bulk tensor store: fp32, bf16 and gated
    (bf16, half the columns) outputs, with batch rows and weight rows that end inside a tile, on the one-CTA kernel
    (no split over K here: K = 512) and on the 2-SM kernel (M >= 512).  bf16 output must be the rounding of the fp32
    output of the same call; the gated output is checked against the two separate products."""
    import torch
    import chadslab_b200 as cb
    rng = np.random.default_rng(31 + fmt)
    K, N = 512, 8200                                         # 64 whole 128-row tiles + 8 rows
    W = rng.normal(0, 0.02, (N, K)).astype(np.float32)
    codes, scales = spec.quantize(W, fmt)
    pw = cb.PackedWeight.from_arrays(codes, scales, fmt)
    lin32, lin16 = cb.QuantLinear(pw, path=cb.PATH_TENSOR), cb.QuantLinear(pw, out_dtype=torch.bfloat16, path=cb.PATH_TENSOR)
    F = 4104                                                 # gate|up: 8208 rows, the last 16-row block ends a tile early
    g_w, u_w = rng.normal(0, 0.05, (F, K)).astype(np.float32), rng.normal(0, 0.05, (F, K)).astype(np.float32)
    gate, up = cb.PackedWeight.from_float(g_w, fmt), cb.PackedWeight.from_float(u_w, fmt)
    fused = cb.QuantLinear(cb.interleave_gate_up(gate, up))
    for M in (64, 201, 601, 1030):
        x = spec.bf16_round(rng.normal(0, 1, (M, K)).astype(np.float32))
        xt = torch.from_numpy(x).cuda().to(torch.bfloat16)
        y32 = lin32(xt)
        assert cuda_lib.bq_last_path() == cb.PATH_TENSOR
        rows = rng.choice(M, size=min(M, 48), replace=False)
        ref = spec.qlinear(x[rows], codes, scales, fmt, f64=True)
        assert spec.rel_err(y32[torch.from_numpy(rows).cuda()].cpu().numpy(), ref) <= TOL, M
        y16 = lin16(xt)
        assert torch.equal(y16, y32.to(torch.bfloat16)), M
        # an output that does not start on a 16-byte boundary takes the plain-store epilogue: same bits
        buf = torch.empty((M * N + 1,), dtype=torch.float32, device="cuda")
        yo = buf[1:].view(M, N)
        assert yo.data_ptr() % 16 == 4
        lin32(xt, out=yo)
        assert torch.equal(yo, y32), M
        got = fused.gated(xt, 1).float()
        g, u = cb.QuantLinear(gate)(xt).double(), cb.QuantLinear(up)(xt).double()
        want = (g / (1.0 + torch.exp(-g)) * u).float()
        assert tuple(got.shape) == (M, F)
        assert spec.rel_err(got.cpu().numpy(), want.cpu().numpy()) <= 6e-3, M
    assert cuda_lib.bq_status_poll() == 0
