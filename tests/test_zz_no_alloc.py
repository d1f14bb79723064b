"""bq_moe_permute_noalloc: the token sort for callers that may not allocate device memory.

A serving process that has handed all free HBM to its KV-cache pool, or a plugin running under an allocator
it does not own, cannot give bq_moe_permute the scratch buffer it asks for.  The variant keeps the per-chunk
histograms in a fixed array inside the library instead.  This file checks, through the C ABI, that it returns
exactly what bq_moe_permute returns (integer outputs: perm, inv, offsets must be identical), on two calls in a
row whose sizes differ (the second call sees the first call's leftovers in the array), and that sizes beyond
the built-in array are refused without launching anything.  It is collected last on purpose.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _permute_both(lib, torch, idx, E):
    T, k = idx.shape
    A = T * k
    dev = idx.device
    out = []
    stream = torch.cuda.current_stream().cuda_stream
    for variant in ("scratch", "noalloc"):
        perm = torch.full((A,), -7, dtype=torch.int32, device=dev)
        inv = torch.full((A,), -7, dtype=torch.int32, device=dev)
        offsets = torch.full((E + 1,), -7, dtype=torch.int32, device=dev)
        if variant == "scratch":
            nbytes = max(int(lib.bq_moe_permute_scratch_bytes(T, k, E)), 16)
            scratch = torch.empty((nbytes,), dtype=torch.uint8, device=dev)
            rc = lib.bq_moe_permute(idx.data_ptr(), T, k, E, perm.data_ptr(), inv.data_ptr(), offsets.data_ptr(),
                                    scratch.data_ptr(), stream)
        else:
            rc = lib.bq_moe_permute_noalloc(idx.data_ptr(), T, k, E, perm.data_ptr(), inv.data_ptr(),
                                            offsets.data_ptr(), stream)
        assert rc == 0, lib.bq_last_error()
        torch.cuda.synchronize()
        out.append((perm.cpu().numpy(), inv.cpu().numpy(), offsets.cpu().numpy()))
    return out


def test_noalloc_permute_matches_scratch_variant_twice(cuda_lib):
    import torch
    lib = cuda_lib
    assert lib.bq_moe_permute_noalloc_max_bytes() == 512 * 1024
    g = torch.Generator(device="cuda").manual_seed(123)
    # first call: many chunks (fills a large part of the array); second call: small, different expert count
    for (T, k, E) in ((40000, 8, 128), (300, 4, 16)):
        idx = torch.randint(0, E, (T, k), dtype=torch.int32, device="cuda", generator=g)
        (p0, i0, o0), (p1, i1, o1) = _permute_both(lib, torch, idx, E)
        assert np.array_equal(p0, p1) and np.array_equal(i0, i1) and np.array_equal(o0, o1)
        flat = idx.cpu().numpy().reshape(-1)
        assert (np.diff(flat[p1]) >= 0).all() and o1[-1] == T * k          # sorted by expert, all placed
        assert np.array_equal(i1[p1], np.arange(T * k))


def test_noalloc_permute_allocates_nothing_and_handles_edge_inputs(cuda_lib):
    """After its first call on the device the entry point leaves the amount of free device memory unchanged (it may
    not allocate: that is its reason to exist), an empty batch gives all-zero offsets, and expert ids outside
    [0, E) are dropped exactly as bq_moe_permute drops them."""
    import torch
    lib = cuda_lib
    E, k = 16, 2
    g = torch.Generator(device="cuda").manual_seed(5)
    idx = torch.randint(0, E, (500, k), dtype=torch.int32, device="cuda", generator=g)
    idx[7, 0], idx[100, 1] = E + 3, -1
    (p0, i0, o0), (p1, i1, o1) = _permute_both(lib, torch, idx, E)          # includes this device's first call
    assert np.array_equal(p0, p1) and np.array_equal(i0, i1) and np.array_equal(o0, o1)
    assert o1[-1] == 500 * k - 2 and (i1 == -1).sum() == 2 and (p1[o1[-1]:] == -1).all()
    perm = torch.empty((500 * k,), dtype=torch.int32, device="cuda")
    inv = torch.empty_like(perm)
    offsets = torch.empty((E + 1,), dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    for _ in range(3):
        assert lib.bq_moe_permute_noalloc(idx.data_ptr(), 500, k, E, perm.data_ptr(), inv.data_ptr(), offsets.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert np.array_equal(perm.cpu().numpy(), p1)
    offsets.fill_(-7)
    assert lib.bq_moe_permute_noalloc(idx.data_ptr(), 0, k, E, perm.data_ptr(), inv.data_ptr(), offsets.data_ptr(),
                                      torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert bool((offsets == 0).all())


def test_noalloc_permute_rejects_sizes_beyond_the_array(cuda_lib):
    import torch
    from chadslab_b200 import _lib
    lib = cuda_lib
    T, k, E = 200000, 8, 1024            # 1024 chunks x 1024 experts x 4 B = 4 MiB > 512 KiB
    assert lib.bq_moe_permute_scratch_bytes(T, k, E) > lib.bq_moe_permute_noalloc_max_bytes()
    before = lib.bq_launch_count()
    dummy = torch.zeros((8,), dtype=torch.int32, device="cuda")
    rc = lib.bq_moe_permute_noalloc(dummy.data_ptr(), T, k, E, dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), None)
    assert rc == _lib.ERR_ARG
    assert b"built-in array" in lib.bq_last_error()
    assert lib.bq_launch_count() == before                       # nothing was launched
