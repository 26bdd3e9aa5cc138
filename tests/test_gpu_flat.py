"""Flat (exact) search on the GPU against the CPU oracle, through the C ABI.

Shapes and data follow the reference's own tests: uniform(-1, 1) rows, seed 42,
(nv, nq, d, k) from faiss-metal/tests/test_metal_flat.mm:489-508, the edge cases
of :451-474, the reconstruct / round-trip checks of :173-222; plus ragged sizes
and a scaled-down copy of the headline configuration."""
import json
import os
import threading

import numpy as np
import pytest

from parity import assert_topk_matches

pytestmark = pytest.mark.gpu

REF_SHAPES = [(1000, 10, 32, 5), (1000, 10, 128, 10), (500, 5, 768, 5), (500, 5, 1536, 5),
              (5000, 5, 128, 33), (5000, 5, 128, 64), (5000, 5, 128, 128), (100, 1, 32, 1)]
EXTRA_SHAPES = [(1, 1, 3, 1), (257, 3, 5, 16), (256, 129, 33, 17), (3000, 130, 100, 100), (70000, 4, 64, 10),
                (20000, 300, 96, 40), (4099, 7, 384, 600)]


def _data(seed, nv, nq, d, lo=-1.0, hi=1.0):
    rng = np.random.default_rng(seed)
    return (rng.uniform(lo, hi, (nv, d)).astype(np.float32), rng.uniform(lo, hi, (nq, d)).astype(np.float32))


def _metric(pkg, name):
    return pkg.METRIC_L2 if name == "L2" else pkg.METRIC_INNER_PRODUCT


@pytest.fixture(params=["tcgen05", "tcgen05-screened", "simt"])
def kernel(request, pkg):
    assert pkg.lib().ann_cuda_set_flat_kernel(request.param.encode()) == 0
    yield request.param
    pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")


@pytest.mark.parametrize("shape", REF_SHAPES + EXTRA_SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("metric_name", ["L2", "IP"])
def test_flat_matches_oracle(pkg, oracle, kernel, shape, metric_name):
    nv, nq, d, k = shape
    xb, xq = _data(42, nv, nq, d)
    m = _metric(pkg, metric_name)
    idx = pkg.CudaIndexFlat(d, m)
    idx.add(xb)
    assert idx.ntotal == nv and idx.d == d and idx.metric_type == m and idx.is_trained
    D, I = idx.search(xq, k)
    Dref, Iref = oracle.flat_search(xb, xq, k, m)
    assert_topk_matches(oracle, xb, xq, m, D, I, Dref, Iref, f"{kernel} {metric_name} {shape}")
    idx.close()


@pytest.mark.parametrize("metric_name", ["L2", "IP"])
def test_screened_search_with_norms_over_four_decades(pkg, oracle, metric_name):
    """One-MMA screening bounds its error with the LARGEST row norm of the store: rows whose
    norms span 1e-2 .. 1e2 and queries of all sizes must still give the oracle's answer."""
    rng = np.random.default_rng(5)
    nv, nq, d, k = 30000, 64, 96, 50
    xb = rng.standard_normal((nv, d)).astype(np.float32)
    xb *= (10.0 ** rng.uniform(-2, 2, (nv, 1))).astype(np.float32)
    xq = rng.standard_normal((nq, d)).astype(np.float32) * (10.0 ** rng.uniform(-2, 2, (nq, 1))).astype(np.float32)
    m = _metric(pkg, metric_name)
    assert pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05-screened") == 0
    try:
        idx = pkg.CudaIndexFlat(d, m)
        idx.add(xb[:10000])
        idx.add(xb[10000:])
        D, I = idx.search(xq, k)
        Dref, Iref = oracle.flat_search(xb, xq, k, m)
        assert_topk_matches(oracle, xb, xq, m, D, I, Dref, Iref, f"screened {metric_name}")
        idx.close()
    finally:
        pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")


def test_screening_falls_back_when_its_spare_candidates_run_out(pkg, oracle):
    """600 rows whose distances to the query are 1e-4 apart (resolved by the split product, far
    inside the error band of the one-MMA keys, whose size is set by the largest norm in the
    store): more than the screened search keeps in reserve.  The host entry point must notice
    and answer with the split product."""
    rng = np.random.default_rng(17)
    d, k = 64, 40
    q = rng.standard_normal(d)
    q /= np.linalg.norm(q)
    u = rng.standard_normal((600, d))
    u /= np.linalg.norm(u, axis=1, keepdims=True)
    far = rng.standard_normal((20000, d)).astype(np.float32)        # norms ~8: they set the band
    xq = q[None, :].astype(np.float32)
    assert pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05-screened") == 0
    try:
        for metric_name in ("L2", "IP"):
            if metric_name == "L2":     # squared distances 0.5, 0.5001, 0.5002, ...
                near = q[None, :] + np.sqrt(0.5 + 1e-4 * np.arange(600))[:, None] * u
            else:                       # dot products 50, 49.9998, 49.9996, ... (the other rows: |q.x| < 5)
                r = u - (u @ q)[:, None] * q[None, :]
                near = (50.0 - 2e-4 * np.arange(600))[:, None] * q[None, :] + 0.1 * r
            xb = np.concatenate([far, near.astype(np.float32)])
            xb = xb[np.random.default_rng(3).permutation(len(xb))]
            m = _metric(pkg, metric_name)
            idx = pkg.CudaIndexFlat(d, m)
            idx.add(xb)
            before = pkg.lib().ann_cuda_screen_fallbacks()
            D, I = idx.search(xq, k)
            assert pkg.lib().ann_cuda_screen_fallbacks() == before + 1, "the overflow went unnoticed"
            Dref, Iref = oracle.flat_search(xb, xq, k, m)
            assert_topk_matches(oracle, xb, xq, m, D, I, Dref, Iref, f"screen overflow {metric_name}")
            Da, Ia = idx.search_async(xq, k).wait()      # the token's wait repeats the search the same way
            assert pkg.lib().ann_cuda_screen_fallbacks() == before + 2
            np.testing.assert_array_equal(Ia, I)
            np.testing.assert_array_equal(Da, D)
            idx.close()
    finally:
        pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")


def test_known_answers_from_reference_sql(pkg, kernel):
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")) as f:
        golden = json.load(f)
    for case in golden["flat"]:
        db = np.array(case["db"], np.float32)
        idx = pkg.CudaIndexFlat(db.shape[1], _metric(pkg, case["metric"]))
        idx.add(db)
        D, I = idx.search(np.array([case["query"]], np.float32), case["k"])
        np.testing.assert_allclose(D[0], np.array(case["distances"], np.float32), rtol=1e-6, atol=1e-7,
                                   err_msg=case["source"])
        n = len(case["labels_first"])
        assert I[0, :n].tolist() == case["labels_first"], case["source"]
        idx.close()


def test_edge_cases(pkg, kernel):
    idx = pkg.CudaIndexFlat(32, pkg.METRIC_L2)
    q = np.ones((3, 32), np.float32)
    D, I = idx.search(q, 4)  # empty index -> (+inf, -1) (MetalIndexFlat.mm:303-309)
    assert (I == -1).all() and np.isposinf(D).all()
    D, I = idx.search(np.zeros((0, 32), np.float32), 4)  # n == 0
    assert D.shape == (0, 4)
    with pytest.raises(pkg.AnnCudaError):
        idx.search(q, 0)  # k must be > 0 (:297)
    xb = np.random.default_rng(0).uniform(-1, 1, (5, 32)).astype(np.float32)
    idx.add(xb)
    D, I = idx.search(q, 8)  # k > ntotal -> padded (:363-367)
    assert (I[:, 5:] == -1).all() and np.isposinf(D[:, 5:]).all() and (I[:, :5] >= 0).all()
    ip = pkg.CudaIndexFlat(32, pkg.METRIC_INNER_PRODUCT)
    ip.add(xb)
    D, I = ip.search(q, 8)
    assert (I[:, 5:] == -1).all() and np.isneginf(D[:, 5:]).all()
    idx.reset()
    assert idx.ntotal == 0
    D, I = idx.search(q, 2)
    assert (I == -1).all()
    idx.close(); ip.close()


def test_incremental_add_reconstruct_and_duplicates(pkg, oracle, kernel):
    xb, xq = _data(7, 3000, 20, 48)
    idx = pkg.CudaIndexFlat(48, pkg.METRIC_L2)
    for s in range(0, 3000, 700):  # grows past the initial capacity several times
        idx.add(xb[s:s + 700])
    assert idx.ntotal == 3000
    for key in (0, 1, 1023, 1024, 2999):
        assert idx.reconstruct(key).tobytes() == xb[key].tobytes()  # bit-exact (test_metal_flat.mm:216-222)
    assert idx.get_rows(0, 3000).tobytes() == xb.tobytes()
    with pytest.raises(pkg.AnnCudaError):
        idx.reconstruct(3000)
    # queries that ARE database rows: distance exactly 0, found first
    D, I = idx.search(xb[:20], 3)
    assert (I[:, 0] == np.arange(20)).all() and (D[:, 0] == 0).all()
    Dref, Iref = oracle.flat_search(xb, xb[:20], 3, oracle.METRIC_L2)
    assert_topk_matches(oracle, xb, xb[:20], oracle.METRIC_L2, D, I, Dref, Iref, "self queries")
    idx.close()


def test_kernels_agree(pkg):
    """Tensor-core path and exact-fp32 path give the same ids on the same data."""
    xb, xq = _data(11, 30000, 200, 256, 0.0, 1.0)
    idx = pkg.CudaIndexFlat(256, pkg.METRIC_L2)
    idx.add(xb)
    pkg.lib().ann_cuda_set_flat_kernel(b"simt")
    Ds, Is = idx.search(xq, 10)
    pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")
    Dt, It = idx.search(xq, 10)
    assert (Is == It).mean() > 0.999
    np.testing.assert_allclose(Dt, Ds, rtol=1e-5)
    idx.close()


def test_headline_config_scaled_down(pkg, oracle):
    """Flat L2, uniform[0,1) rows, d=384, k=10 (the reference's CPU-runnable case) at 1/5 of its rows."""
    xb, xq = _data(42, 20000, 250, 384, 0.0, 1.0)
    idx = pkg.CudaIndexFlat(384, pkg.METRIC_L2)
    idx.add(xb)
    D, I = idx.search(xq, 10)
    Dref, Iref = oracle.flat_search(xb, xq, 10, oracle.METRIC_L2)
    assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, "C1 scaled")
    idx.close()


def test_unit_norm_inner_product_k100(pkg, oracle):
    """Flat IP, unit-norm Gaussian rows, d=768, k=100 (the sharded configuration) scaled down."""
    rng = np.random.default_rng(43)
    xb = rng.standard_normal((30000, 768)).astype(np.float32)
    xb /= np.linalg.norm(xb, axis=1, keepdims=True)
    xq = rng.standard_normal((130, 768)).astype(np.float32)
    xq /= np.linalg.norm(xq, axis=1, keepdims=True)
    idx = pkg.CudaIndexFlat(768, pkg.METRIC_INNER_PRODUCT)
    idx.add(xb)
    D, I = idx.search(xq, 100)
    Dref, Iref = oracle.flat_search(xb, xq, 100, oracle.METRIC_IP)
    assert_topk_matches(oracle, xb, xq, oracle.METRIC_IP, D, I, Dref, Iref, "C4 scaled")
    idx.close()


@pytest.mark.parametrize("flat_kernel", ["tcgen05", "tcgen05-screened"])
@pytest.mark.parametrize("shape", [(160_000, 4096, 32, 24), (620_000, 300, 16, 100), (310_000, 200, 24, 17), (310_000, 200, 24, 10)],
                         ids=lambda s: "x".join(map(str, s)))
def test_large_store_static_schedule(pkg, oracle, flat_kernel, shape):
    """Stores of several hundred row tiles and more, k <= 128: every CTA owns a fixed share of each
    chunk of the store and alternates between the lists of two query tiles (32 query tiles: shares
    of 8 units out of 37 per tile; 3 and 2 query tiles: one CTA in 49 / 74 straddles two tiles).
    Ragged last chunk, ragged last query tile."""
    nv, nq, d, k = shape
    xb, xq = _data(7, nv, nq, d)
    assert pkg.lib().ann_cuda_set_flat_kernel(flat_kernel.encode()) == 0
    try:
        for metric_name in ("L2", "IP"):
            m = _metric(pkg, metric_name)
            idx = pkg.CudaIndexFlat(d, m)
            idx.add(xb)
            D, I = idx.search(xq, k)
            idx.close()
            Dref, Iref = oracle.flat_search(xb, xq, k, m)
            assert_topk_matches(oracle, xb, xq, m, D, I, Dref, Iref, f"{flat_kernel} {metric_name} {shape}")
    finally:
        pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")


def test_static_schedule_with_searches_in_flight(pkg, oracle):
    """Three screened searches of a large store enqueued at once on their own streams: their CTAs
    compete for the SMs, so the CTAs of one launch are not all running together and its pacing has
    to give way.  Same answers as the synchronous search."""
    xb, xq = _data(19, 200_000, 1024, 32)
    assert pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05-screened") == 0
    try:
        idx = pkg.CudaIndexFlat(32, pkg.METRIC_L2)
        idx.add(xb)
        D, I = idx.search(xq, 30)
        tokens = [idx.search_async(xq, 30) for _ in range(3)]
        for t in tokens:
            Da, Ia = t.wait()
            np.testing.assert_array_equal(Ia, I)
            np.testing.assert_array_equal(Da, D)
        Dref, Iref = oracle.flat_search(xb, xq, 30, pkg.METRIC_L2)
        assert_topk_matches(oracle, xb, xq, pkg.METRIC_L2, D, I, Dref, Iref, "static schedule, searches in flight")
        idx.close()
    finally:
        pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")


def test_search_async_tokens(pkg, oracle, kernel):
    """searchAsync (faiss-metal/src/MetalIndexFlat.mm:371-443): several tokens in flight on one
    index, waited on out of order, give what search() gives; n == 0 and an empty index answer at
    once; a token may be dropped without a wait."""
    xb, xq = _data(11, 6000, 40, 96)
    for metric_name in ("L2", "IP"):
        m = _metric(pkg, metric_name)
        idx = pkg.CudaIndexFlat(96, m)
        empty = idx.search_async(xq[:2], 3)            # ntotal == 0: sentinels (MetalIndexFlat.mm:385-395)
        De, Ie = empty.wait()
        assert (Ie == -1).all() and np.isinf(De).all()
        idx.add(xb)
        Dsync, Isync = idx.search(xq, 20)
        tokens = [idx.search_async(xq[i:i + 8], 20) for i in range(0, 40, 8)]
        dropped = idx.search_async(xq, 20)
        dropped.close()
        for j in (3, 0, 4, 1, 2):
            D, I = tokens[j].wait()
            assert tokens[j].is_ready()
            np.testing.assert_array_equal(I, Isync[8 * j:8 * j + 8])
            np.testing.assert_array_equal(D, Dsync[8 * j:8 * j + 8])
            assert tokens[j].wait()[1] is I            # a second wait is a no-op
        none = idx.search_async(xq[:0], 20)
        assert none.is_ready() and none.wait()[0].shape == (0, 20)
        Dref, Iref = oracle.flat_search(xb, xq, 20, m)
        assert_topk_matches(oracle, xb, xq, m, Dsync, Isync, Dref, Iref, f"async {metric_name}")
        with pytest.raises(RuntimeError):
            idx.search_async(xq, 0)
        idx.close()


def test_concurrent_search(pkg, oracle):
    """search() runs from several host threads on one index (src/faiss_index.cpp:729-737)."""
    xb, xq = _data(3, 5000, 64, 128)
    idx = pkg.CudaIndexFlat(128, pkg.METRIC_L2)
    idx.add(xb)
    Dref, Iref = oracle.flat_search(xb, xq, 5, oracle.METRIC_L2)
    bad = []

    def work(t):
        for i in range(t, 64, 8):
            D, I = idx.search(xq[i:i + 1], 5)  # one query per call, as the extension does
            if I[0].tolist() != Iref[i].tolist():
                bad.append(i)

    ths = [threading.Thread(target=work, args=(t,)) for t in range(8)]
    [t.start() for t in ths]
    [t.join() for t in ths]
    assert not bad
    idx.close()


def test_device_buffers_and_merge(pkg, oracle):
    """search_device on two row shards + merge kernel == unsharded search."""
    import torch
    xb, xq = _data(5, 9001, 70, 160)
    m = pkg.METRIC_L2
    full = pkg.CudaIndexFlat(160, m)
    full.add(xb)
    Dfull, Ifull = full.search(xq, 20)
    parts_d, parts_i = [], []
    xq_dev = torch.from_numpy(xq).cuda()
    shards = []
    for lo, hi in [(0, 4000), (4000, 9001)]:
        s = pkg.CudaIndexFlat(160, m)
        s.add_device(torch.from_numpy(xb[lo:hi]).cuda())
        d, i = s.search_device(xq_dev, 20, label_offset=lo)
        parts_d.append(d); parts_i.append(i); shards.append(s)
    D, I = pkg.merge_topk_device(torch.stack(parts_d).contiguous(), torch.stack(parts_i).contiguous(), m)
    torch.cuda.synchronize()
    assert (I.cpu().numpy() == Ifull).all()
    np.testing.assert_array_equal(D.cpu().numpy(), Dfull)
    Dref, Iref = oracle.flat_search(xb, xq, 20, oracle.METRIC_L2)
    assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D.cpu().numpy(), I.cpu().numpy(), Dref, Iref, "sharded")
    for s in shards:
        s.close()
    full.close()
