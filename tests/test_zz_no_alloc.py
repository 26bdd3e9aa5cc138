"""The allocation-free flat search against the regular device search.

Who needs it: hosts that must not allocate GPU memory while a search runs - a
database worker held to a fixed memory budget, a caller that records searches into
a CUDA graph, a thread that cannot tolerate the device-wide stalls of cudaMalloc /
cudaFree.  The regular entry points grow a scratch pool; this one keeps all
scratch in one fixed device array, which every call shares.  So the test runs two
different calls back to back (the second must not see anything the first left
behind) and checks each against ann_cuda_index_search_device, through the C ABI.
This file sorts last on purpose: a run that stops at the first failure has then
already run every other test."""
import ctypes as C

import numpy as np
import pytest

from parity import assert_topk_matches

pytestmark = pytest.mark.gpu


def _free_bytes(torch):
    free, _ = torch.cuda.mem_get_info()
    return free


def test_static_scratch_search_matches_regular_search_twice_in_a_row(pkg, oracle):
    import torch
    rng = np.random.default_rng(77)
    d, nv = 96, 30000
    xb = rng.uniform(-1, 1, (nv, d)).astype(np.float32)
    idx = pkg.CudaIndexFlat(d, pkg.METRIC_L2)
    idx.add(xb)
    lib = pkg.lib()
    stream = torch.cuda.current_stream()
    calls = [(rng.uniform(-1, 1, (128, d)).astype(np.float32), 16),  # the limits themselves
             (rng.uniform(-1, 1, (5, d)).astype(np.float32), 3)]     # smaller call right after: stale scratch must not leak in
    outs = []
    for xq, k in calls:
        x = torch.from_numpy(xq).cuda()
        D = torch.empty((len(xq), k), dtype=torch.float32, device="cuda")
        I = torch.empty((len(xq), k), dtype=torch.int64, device="cuda")
        outs.append((x, k, D, I))
    # regular entry point first (it may allocate), so the comparison data exists up front
    want = []
    for x, k, _, _ in outs:
        Dw, Iw = idx.search_device(x, k)
        torch.cuda.synchronize()
        want.append((Dw.cpu().numpy(), Iw.cpu().numpy()))
    # first call performs the one-time address look-up
    x, k, D, I = outs[0]
    rc = lib.ann_cuda_flat_search_small_static(idx._h, x.shape[0], C.c_void_p(x.data_ptr()), k, C.c_void_p(D.data_ptr()),
                                               C.c_void_p(I.data_ptr()), 0, C.c_void_p(stream.cuda_stream))
    assert rc == 0, pkg.last_error()
    torch.cuda.synchronize()
    free_before = _free_bytes(torch)
    for (x, k, D, I), (Dw, Iw) in zip(outs, want):
        rc = lib.ann_cuda_flat_search_small_static(idx._h, x.shape[0], C.c_void_p(x.data_ptr()), k,
                                                   C.c_void_p(D.data_ptr()), C.c_void_p(I.data_ptr()), 0,
                                                   C.c_void_p(stream.cuda_stream))
        assert rc == 0, pkg.last_error()
        torch.cuda.synchronize()
        assert (I.cpu().numpy() == Iw).all()
        np.testing.assert_allclose(D.cpu().numpy(), Dw, rtol=1e-4, atol=0)  # the tolerance of the parity tests
        # ... and against the CPU oracle, like every other search path
        Dref, Iref = oracle.flat_search(xb, x.cpu().numpy(), k, oracle.METRIC_L2)
        assert_topk_matches(oracle, xb, x.cpu().numpy(), oracle.METRIC_L2, D.cpu().numpy(), I.cpu().numpy(), Dref, Iref,
                            "allocation-free search")
    assert lib.ann_cuda_flat_search_small_static_status(0, C.c_void_p(stream.cuda_stream)) == 0, pkg.last_error()
    assert _free_bytes(torch) == free_before, "the allocation-free entry point changed the amount of free device memory"
    idx.close()


def test_static_scratch_search_inner_product_and_label_offset(pkg):
    import torch
    rng = np.random.default_rng(78)
    xb = rng.standard_normal((5000, 256)).astype(np.float32)
    idx = pkg.CudaIndexFlat(256, pkg.METRIC_INNER_PRODUCT)
    idx.add(xb)
    x = torch.from_numpy(rng.standard_normal((17, 256)).astype(np.float32)).cuda()
    Dw, Iw = idx.search_device(x, 7, label_offset=1000)
    D, I = idx.search_small_static(x, 7, label_offset=1000)
    torch.cuda.synchronize()
    assert (I == Iw).all() and (I >= 1000).all()
    np.testing.assert_allclose(D.cpu().numpy(), Dw.cpu().numpy(), rtol=1e-4, atol=0)
    idx.close()


def test_static_scratch_search_rejects_what_does_not_fit(pkg):
    import torch
    idx = pkg.CudaIndexFlat(64, pkg.METRIC_L2)
    idx.add(np.zeros((300, 64), np.float32))
    x = torch.zeros((129, 64), device="cuda")
    with pytest.raises(pkg.AnnCudaError, match="128"):
        idx.search_small_static(x, 4)            # too many queries
    with pytest.raises(pkg.AnnCudaError, match="16"):
        idx.search_small_static(x[:4].contiguous(), 17)        # k too large
    big = pkg.CudaIndexFlat(1100, pkg.METRIC_L2)
    big.add(np.zeros((10, 1100), np.float32))
    with pytest.raises(pkg.AnnCudaError, match="1024"):
        big.search_small_static(torch.zeros((1, 1100), device="cuda"), 1)  # dimension too large
    ivf = pkg.CudaIndexIVFFlat(64, 4, pkg.METRIC_L2)
    with pytest.raises(pkg.AnnCudaError):
        lib = pkg.lib()
        pkg.check(lib.ann_cuda_flat_search_small_static(ivf._h, 1, C.c_void_p(x.data_ptr()), 1, C.c_void_p(x.data_ptr()),
                                                        C.c_void_p(x.data_ptr()), 0, None), "static search on IVF")
    idx.close(); big.close(); ivf.close()
