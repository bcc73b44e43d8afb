"""The allocation-free RMSNorm entry point against the ordinary one.

Kept in a file that sorts last so that a run stopping at the first failure has already run every
other test. The entry point is for hosts that may not allocate while running (a server that gave
all of HBM away at start-up, a latency-critical loop, a plugin host that owns the allocator); its
scratch is an array built into the library, shared by every call on a device.
"""
import ctypes as C

import numpy as np
import pytest

import synth

pkg = synth.pkg
pytestmark = pytest.mark.gpu


def _host_reference(x, w, eps):
    y = np.zeros_like(x)
    rc = pkg.lib().g5b_rmsnorm_host(y.ctypes.data, x.ctypes.data, w.ctypes.data if w is not None else None,
                                    x.shape[1], x.shape[0], eps, 0)
    assert rc == 0
    return y


def _free_bytes(torch):
    """Free device memory as the driver counts it (cudaMemGetInfo): unlike torch's own counters it
    also moves when a library calls cudaMalloc or cudaFree behind torch's back."""
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_rmsnorm_noalloc_matches_allocating_entry_point(gpu_lib):
    import torch
    L = pkg.lib()
    torch.cuda.set_device(0)
    rng = np.random.default_rng(99)
    # a first call outside the measurement: it loads the module and resolves the scratch address
    wx = torch.ones((2, 64), device="cuda")
    assert L.g5b_rmsnorm_noalloc(wx.data_ptr(), wx.data_ptr(), None, 64, 2, C.c_float(1e-5), None) == 0
    side = torch.cuda.Stream()
    # calls in a row on the shared scratch, different shapes and contents: none must see anything of
    # the one before; one of them on a stream of its own, one in place (y == x)
    for rows, n, with_w, how in ((4096, 512, True, "default"), (7, 4096, False, "default"),
                                 (300, 1000, True, "stream"), (64, 256, True, "inplace")):
        x = rng.standard_normal((rows, n)).astype(np.float32) * (1.0 + rows % 5)
        w = rng.standard_normal(n).astype(np.float32) if with_w else None
        want = _host_reference(x, w, 1e-5)
        xd = torch.from_numpy(x).cuda()
        wd = torch.from_numpy(w).cuda() if with_w else None
        yd = xd if how == "inplace" else torch.empty_like(xd)
        stream = side.cuda_stream if how == "stream" else None
        before_torch = torch.cuda.memory_allocated()
        before = _free_bytes(torch)
        rc = L.g5b_rmsnorm_noalloc(yd.data_ptr(), xd.data_ptr(), wd.data_ptr() if with_w else None, n, rows,
                                   C.c_float(1e-5), stream)
        assert rc == 0, L.g5b_last_error()
        # the property the entry point exists for: neither the driver's nor torch's count moved
        assert _free_bytes(torch) == before
        assert torch.cuda.memory_allocated() == before_torch
        got = yd.cpu().numpy()
        # same kernels, same order of operations: the tolerance of the RMSNorm parity test, which
        # these results meet with room to spare (they are bit-equal)
        assert np.max(np.abs(got - want)) <= 1e-6 * np.max(np.abs(want))
        assert np.array_equal(got, want)


def test_rmsnorm_noalloc_refuses_more_rows_than_its_scratch(gpu_lib):
    import torch
    L = pkg.lib()
    torch.cuda.set_device(0)
    xd = torch.zeros((4097, 8), device="cuda")
    yd = torch.empty_like(xd)
    rc = L.g5b_rmsnorm_noalloc(yd.data_ptr(), xd.data_ptr(), None, 8, 4097, C.c_float(1e-5), None)
    assert rc == -1
    assert b"4096" in L.g5b_last_error()
