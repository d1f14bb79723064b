"""The quantized matmul at the benchmark's own shapes and prefill batch sizes, against the oracle.

(16384, 2048), (2048, 16384) and (256000, 2048) at M = 512 and 4096, both formats: the weights are generated and
quantized on the device with the oracle's rule, 128 sampled weight rows are copied to the host and the matching
output columns are compared with the float64 oracle on the same codes and scales (tolerance 1e-3, max error over
max magnitude, the bound the specification states).  The whole product is computed on the device; only the sampled
columns are checked on the CPU, which keeps the test in seconds."""
import numpy as np
import pytest

from oracle import spec

pytestmark = pytest.mark.gpu
TOL = 1e-3


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("shape", [(16384, 2048), (2048, 16384), (256000, 2048)])
def test_prefill_batches_on_config_shapes_sampled_rows(cuda_lib, fmt, shape):
    import torch
    import chadslab_b200 as cb
    from chadslab_b200.synth import make_device_weight
    N, K = shape
    g = torch.Generator(device="cuda").manual_seed(N + K + fmt)
    codes, scales = make_device_weight(torch, N, K, fmt, g)
    pw = cb.PackedWeight.from_device(codes, scales, fmt)
    lin = cb.QuantLinear(pw)
    rows = torch.randint(0, N, (128,), device="cuda", generator=g)
    c_np, s_np = codes[rows].cpu().numpy(), scales[rows].cpu().numpy()
    for M in (300, 512, 4096):           # 300: one-CTA kernels (two weight tiles per CTA for 4-bit codes), 512+: the 2-SM kernel
        x = torch.randn((M, K), device="cuda", generator=g).to(torch.bfloat16)
        y = lin(x)
        assert cuda_lib.bq_last_path() == cb.PATH_TENSOR                   # the tcgen05 kernel, not a fallback
        ref = spec.qlinear(x.float().cpu().numpy(), c_np, s_np, fmt, f64=True)
        err = spec.rel_err(y[:, rows].cpu().numpy(), ref)
        assert err <= TOL, (shape, fmt, M, err)
        del x, y
    pw.close()
    assert cuda_lib.bq_status_poll() == 0


@pytest.mark.parametrize("fmt", [0, 1])
def test_decode_batches_on_the_head_shape_sampled_rows(cuda_lib, fmt):
    """M = 8 and 64 on (256000, 2048): the decode batch sizes of the sweep between the GEMV and the prefill tiles."""
    import torch
    import chadslab_b200 as cb
    from chadslab_b200.synth import make_device_weight
    N, K = 256000, 2048
    g = torch.Generator(device="cuda").manual_seed(7 + fmt)
    codes, scales = make_device_weight(torch, N, K, fmt, g)
    lin = cb.QuantLinear(cb.PackedWeight.from_device(codes, scales, fmt))
    rows = torch.randint(0, N, (128,), device="cuda", generator=g)
    c_np, s_np = codes[rows].cpu().numpy(), scales[rows].cpu().numpy()
    for M in (2, 4, 8, 64):
        x = torch.randn((M, K), device="cuda", generator=g).to(torch.bfloat16)
        y = lin(x)
        ref = spec.qlinear(x.float().cpu().numpy(), c_np, s_np, fmt, f64=True)
        assert spec.rel_err(y[:, rows].cpu().numpy(), ref) <= TOL, (fmt, M)
    lin.pw.close()


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("N,K,M", [(3000, 1024, 1800), (1536, 3072, 2050), (12288, 3072, 700)])
def test_large_batches_ragged_shapes_all_rows(cuda_lib, fmt, N, K, M):
    """Large batches on shapes whose row and batch counts are not multiples of the tile sizes (the last weight tile, the
    last 256-row batch tile and - for int8, which runs on pairs of CTAs here - the second CTA of the last pair are
    partly or wholly outside the matrix): every output against the float64 oracle, plain and gated epilogue."""
    import torch
    import chadslab_b200 as cb
    from chadslab_b200.synth import make_device_weight
    g = torch.Generator(device="cuda").manual_seed(N + M + fmt)
    codes, scales = make_device_weight(torch, N, K, fmt, g)
    lin = cb.QuantLinear(cb.PackedWeight.from_device(codes, scales, fmt))
    x = torch.randn((M, K), device="cuda", generator=g).to(torch.bfloat16)
    y = lin(x)
    assert cuda_lib.bq_last_path() == cb.PATH_TENSOR
    ref = spec.qlinear(x.float().cpu().numpy(), codes.cpu().numpy(), scales.cpu().numpy(), fmt, f64=True)
    assert spec.rel_err(y.cpu().numpy(), ref) <= TOL
    if N % 16 == 0:
        h = lin.gated(x, 1)                                                # silu(gate) * up on interleaved 8 + 8 row blocks
        gate = ref.reshape(M, N // 16, 2, 8)[:, :, 0, :].reshape(M, N // 2)
        up = ref.reshape(M, N // 16, 2, 8)[:, :, 1, :].reshape(M, N // 2)
        want = gate / (1.0 + np.exp(-gate)) * up
        assert spec.rel_err(h.float().cpu().numpy(), want) <= 2.0 ** -7
    lin.pw.close()
    assert cuda_lib.bq_status_poll() == 0
