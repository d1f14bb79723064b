"""Peer-memory communicator on one GPU: with a world of one rank the deposit -> signal -> wait -> sum chain must
reproduce the plain kernels bit for bit (also from a replayed CUDA graph, where the epoch advances on the device),
and with stand-in peers that never answer the bounded wait must end with BQ_ERR_TIMEOUT and a usable context.
The 2-GPU exchange itself is covered by tests/tp_worker.py."""
import ctypes as C

import numpy as np
import pytest


pytestmark = pytest.mark.gpu


def _weight(N, K, fmt, seed):
    import chadslab_b200 as cb
    rng = np.random.default_rng(seed)
    return cb.PackedWeight.from_float(rng.normal(0, 0.02, (N, K)).astype(np.float32), fmt)


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("adt", ["bfloat16", "float32"])
@pytest.mark.parametrize("shape", [(256, 512, 1), (3072, 2048, 2), (200, 8192, 1)])
def test_push_gemv_then_sum_equals_plain_gemv(cuda_lib, fmt, adt, shape):
    import torch
    import chadslab_b200 as cb
    N, K, M = shape
    lin = cb.QuantLinear(_weight(N, K, fmt, 1))
    comm = cb.PeerComm(max_elems=4 * 4096)
    g = torch.Generator(device="cuda").manual_seed(3)
    for it in range(5):                                # several calls: both parities of the receive slots
        x = torch.randn((M, K), device="cuda", generator=g).to(getattr(torch, adt))
        want = lin(x)
        assert comm.push_linear(lin, x) is None        # decode-sized: deposited by the GEMV itself
        got = comm.all_reduce(None, count=M * N).reshape(M, N)
        assert torch.equal(got, want), it
    comm.close()
    assert cuda_lib.bq_status_poll() == 0


def test_push_refuses_large_batches_and_falls_back(cuda_lib):
    import torch
    import chadslab_b200 as cb
    lin = cb.QuantLinear(_weight(512, 1024, 0, 2))
    comm = cb.PeerComm(max_elems=64 * 512)
    x = torch.randn((64, 1024), device="cuda").to(torch.bfloat16)
    y = comm.push_linear(lin, x)                       # not a GEMV shape: the partial product comes back
    assert y is not None and torch.equal(y, lin(x))
    assert torch.equal(comm.all_reduce(y), y)          # world of one: the sum is the input
    comm.close()


@pytest.mark.parametrize("adt", ["bfloat16", "float32"])
def test_fused_sum_add_rmsnorm_equals_add_rmsnorm(cuda_lib, adt):
    import torch
    import chadslab_b200 as cb
    from chadslab_b200 import _lib
    from chadslab_b200.ops import _dt_of_torch, _stream_ptr
    dt = getattr(torch, adt)
    rows, H = 3, 3072
    comm = cb.PeerComm(max_elems=rows * H)
    g = torch.Generator(device="cuda").manual_seed(5)
    x0 = torch.randn((rows, H), device="cuda", generator=g).to(dt)
    delta = torch.randn((rows, H), device="cuda", generator=g)
    gamma = torch.rand(H, device="cuda", generator=g) + 0.5
    xa, na = x0.clone(), torch.empty_like(x0)
    _lib.check(cuda_lib.bq_add_rmsnorm(xa.data_ptr(), delta.data_ptr(), gamma.data_ptr(), na.data_ptr(), rows, H, 1e-6,
                                       _dt_of_torch(xa), _stream_ptr()))
    xb, nb = x0.clone(), torch.empty_like(x0)
    comm.add_rmsnorm(delta, xb, gamma, nb, 1e-6)
    assert torch.equal(xa, xb) and torch.equal(na, nb)
    # after a depositing GEMV (M = rows would exceed the GEMV's 4 vectors for fp32, so one row)
    lin = cb.QuantLinear(_weight(H, 1024, 1, 7))
    xin = torch.randn((1, 1024), device="cuda", generator=g).to(dt)
    want_delta = lin(xin)
    xa, na = x0[:1].clone(), torch.empty_like(x0[:1])
    _lib.check(cuda_lib.bq_add_rmsnorm(xa.data_ptr(), want_delta.data_ptr(), gamma.data_ptr(), na.data_ptr(), 1, H, 1e-6,
                                       _dt_of_torch(xa), _stream_ptr()))
    xb, nb = x0[:1].clone(), torch.empty_like(x0[:1])
    assert comm.push_linear(lin, xin) is None
    comm.add_rmsnorm(None, xb, gamma, nb, 1e-6)
    assert torch.equal(xa, xb) and torch.equal(na, nb)
    comm.close()


def test_graph_replay_advances_the_epoch_on_the_device(cuda_lib):
    import torch
    import chadslab_b200 as cb
    N, K = 1024, 2048
    lin = cb.QuantLinear(_weight(N, K, 0, 9))
    comm = cb.PeerComm(max_elems=N)
    x = torch.randn((1, K), device="cuda").to(torch.bfloat16)
    out = torch.empty(N, dtype=torch.float32, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        comm.push_linear(lin, x)
        comm.all_reduce(None, count=N, out=out)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        comm.push_linear(lin, x)
        comm.all_reduce(None, count=N, out=out)
        comm.push_linear(lin, x)                       # two sums per replay: the parity flips inside the graph too
        comm.all_reduce(None, count=N, out=out)
    for _ in range(3):
        x.copy_(torch.randn((1, K), device="cuda").to(torch.bfloat16))
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, lin(x).reshape(-1))
    comm.close()
    assert cuda_lib.bq_status_poll() == 0


def test_argument_errors(cuda_lib):
    import torch
    from chadslab_b200 import _lib
    h = C.c_uint64(0)
    assert cuda_lib.bq_comm_create(0, 9, 1024, C.byref(h)) == _lib.ERR_ARG
    assert cuda_lib.bq_comm_create(2, 2, 1024, C.byref(h)) == _lib.ERR_ARG
    assert cuda_lib.bq_comm_create(0, 2, 1024, C.byref(h)) == 0
    out = torch.empty(16, device="cuda")
    assert cuda_lib.bq_allreduce(h.value, out.data_ptr(), out.data_ptr(), 16, None) == _lib.ERR_STATE   # not connected
    assert cuda_lib.bq_comm_destroy(h.value) == 0
    assert cuda_lib.bq_comm_destroy(h.value) == _lib.ERR_HANDLE
    assert cuda_lib.bq_comm_create(0, 1, 1024, C.byref(h)) == 0
    assert cuda_lib.bq_allreduce(h.value, out.data_ptr(), out.data_ptr(), 4096, None) == _lib.ERR_ARG   # > max_elems
    assert cuda_lib.bq_comm_destroy(h.value) == 0


def test_unanswered_wait_times_out_and_the_context_survives(cuda_lib):
    """A rank whose peers never raise their flag: the kernel gives up at its time limit (set to 0.5 s here), records the time-out in
    the status word and returns; later calls on the same context work."""
    import torch
    import chadslab_b200 as cb
    from chadslab_b200 import _lib
    h = C.c_uint64(0)
    _lib.check(cuda_lib.bq_comm_create(0, 2, 1024, C.byref(h)))
    _lib.check(cuda_lib.bq_comm_connect_loopback(h.value))
    _lib.check(cuda_lib.bq_comm_set_timeout_ms(h.value, 500))
    x = torch.ones(256, device="cuda")
    out = torch.empty_like(x)
    _lib.check(cuda_lib.bq_allreduce(h.value, x.data_ptr(), out.data_ptr(), 256, None))
    assert cuda_lib.bq_status_poll() == _lib.ERR_TIMEOUT
    assert cuda_lib.bq_status_poll() == 0              # reading the status clears it
    _lib.check(cuda_lib.bq_comm_destroy(h.value))
    lin = cb.QuantLinear(_weight(64, 128, 0, 4))
    y = lin(torch.ones((1, 128), device="cuda"))
    assert np.isfinite(y.cpu().numpy()).all()
