"""The three tiers of the flat search (one-MMA screening -> three-MMA split product -> exact fp32
scan) and what moves a query block from one to the next, through every entry point of the C ABI.

The acceptance rule is the one of the other parity tests: distances within 1e-4 relative of the
CPU oracle, identical id sets except for tolerance ties at the k-th place
(faiss-metal/tests/test_metal_flat.mm:25-60 is the reference's own, looser, form of it)."""
import ctypes as C

import numpy as np
import pytest

from parity import assert_topk_matches

pytestmark = pytest.mark.gpu


def _metric(pkg, name):
    return pkg.METRIC_L2 if name == "L2" else pkg.METRIC_INNER_PRODUCT


def _near_tie_store(rng, d, n_far, n_near, metric_name, step):
    """`n_near` rows whose distance to the query q grows by `step` from one to the next, among
    `n_far` Gaussian rows that are all much farther away."""
    q = rng.standard_normal(d)
    q /= np.linalg.norm(q)
    u = rng.standard_normal((n_near, d))
    u /= np.linalg.norm(u, axis=1, keepdims=True)
    far = rng.standard_normal((n_far, d)).astype(np.float32)
    if metric_name == "L2":
        near = q[None, :] + np.sqrt(0.5 + step * np.arange(n_near))[:, None] * u
    else:
        r = u - (u @ q)[:, None] * q[None, :]
        near = (50.0 - 2 * step * np.arange(n_near))[:, None] * q[None, :] + 0.1 * r
    xb = np.concatenate([far, near.astype(np.float32)])
    xb = xb[np.random.default_rng(3).permutation(len(xb))]
    return xb, q[None, :].astype(np.float32)


def test_tight_clusters_far_from_the_origin(pkg, oracle):
    """The flat twin of the IVF test of the same name: neighbour distances ~1e-4 of the operands'
    squared norms, so that split-product keys alone cannot rank the neighbours.  The band check
    has to notice and the exact tier has to answer."""
    rng = np.random.default_rng(11)
    nc, d = 32, 96
    centers = (rng.standard_normal((nc, d)) * 3 + 2).astype(np.float32)
    xb = (centers[rng.integers(0, nc, 8000)] + 0.05 * rng.standard_normal((8000, d))).astype(np.float32)
    xq = (centers[rng.integers(0, nc, 150)] + 0.05 * rng.standard_normal((150, d))).astype(np.float32)
    xq[:20] = xb[rng.integers(0, len(xb), 20)]
    xq[20:40] = xb[rng.integers(0, len(xb), 20)] + np.float32(1e-3)
    for kernel in ("tcgen05", "tcgen05-screened", "tcgen05-split"):
        assert pkg.lib().ann_cuda_set_flat_kernel(kernel.encode()) == 0
        try:
            for metric_name in ("L2", "IP"):
                m = _metric(pkg, metric_name)
                idx = pkg.CudaIndexFlat(d, m)
                idx.add(xb)
                for k in (5, 20, 300):
                    D, I = idx.search(xq, k)
                    Dref, Iref = oracle.flat_search(xb, xq, k, m)
                    assert_topk_matches(oracle, xb, xq, m, D, I, Dref, Iref, f"tight clusters {kernel} {metric_name} k={k}")
                if metric_name == "L2":
                    assert (D[:20, 0] == 0.0).all()
                idx.close()
        finally:
            pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")


def test_near_ties_far_denser_than_the_split_product_resolves(pkg, oracle):
    """400 rows whose distances to the query differ by 1e-7 of |q||x|max each: more than the 256
    candidates a banded list holds sit inside the split product's error band, so its band check
    must flag it (k = 8: first the 16-list, then the banded lists; k = 40: the banded lists) and the
    exact scan settles the order.  The counter shows that the fallbacks really ran."""
    rng = np.random.default_rng(23)
    for metric_name in ("L2", "IP"):
        xb, xq = _near_tie_store(rng, 64, 20000, 400, metric_name, 1e-6)
        m = _metric(pkg, metric_name)
        idx = pkg.CudaIndexFlat(64, m)
        idx.add(xb)
        before = pkg.lib().ann_cuda_screen_fallbacks()
        for k in (8, 40):
            D, I = idx.search(xq, k)
            Dref, Iref = oracle.flat_search(xb, xq, k, m)
            assert_topk_matches(oracle, xb, xq, m, D, I, Dref, Iref, f"dense ties {metric_name} k={k}")
        assert pkg.lib().ann_cuda_screen_fallbacks() == before + 3, "the split product's band overflow went unnoticed"
        idx.close()


@pytest.mark.parametrize("entry", ["host", "device"])
def test_the_exact_scan_repairs_the_flagged_queries_only(pkg, oracle, entry):
    """One query in 300 sits on 400 near ties that no tensor-core tier can order; the other 299 are
    ordinary.  The exact scan that settles it runs for the flagged query alone - the others keep the
    answers of the tier before, which must still be the oracle's - whether the host repeats the
    search tier by tier or the tiers were enqueued behind one another on the device."""
    import torch
    rng = np.random.default_rng(29)
    xb, q0 = _near_tie_store(rng, 64, 20000, 400, "L2", 1e-6)
    xq = (rng.standard_normal((300, 64))).astype(np.float32)
    xq[137] = q0
    idx = pkg.CudaIndexFlat(64, pkg.METRIC_L2)
    idx.add(xb)
    before = pkg.lib().ann_cuda_screen_fallbacks()
    for k in (8, 40):
        if entry == "host":
            D, I = idx.search(xq, k)
        else:
            Dd, Id = idx.search_device(torch.from_numpy(xq).cuda(), k)
            idx.search_status()
            D, I = Dd.cpu().numpy(), Id.cpu().numpy()
        Dref, Iref = oracle.flat_search(xb, xq, k, oracle.METRIC_L2)
        assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, f"one hard query among 300, k={k}, {entry}")
    assert pkg.lib().ann_cuda_screen_fallbacks() >= before + 2, "the exact scan never ran"
    idx.close()


@pytest.mark.parametrize("storage_kind", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("metric_name", ["L2", "IP"])
def test_many_flagged_queries_share_one_pass_over_the_store(pkg, oracle, metric_name, storage_kind):
    """23 of 300 queries sit on the near ties (copies of the hard query, some moved by 1e-6): the exact
    tier compacts them, scans the store once with the k-th distance of the tier before as the bound
    (16 queries per row tile and CTA, the last group ragged) and sorts what passed; k below and above one list."""
    import torch
    rng = np.random.default_rng(41)
    d = 64
    xb, q0 = _near_tie_store(rng, d, 20000, 400, metric_name, 1e-6)
    xq = rng.standard_normal((300, d)).astype(np.float32)
    hard = rng.choice(300, 23, replace=False)
    for j, h in enumerate(hard):
        xq[h] = q0[0] + (1e-6 * rng.standard_normal(d) if j % 3 == 0 else 0.0)
    storage = {"f32": pkg.STORAGE_F32, "f16": pkg.STORAGE_F16, "bf16": pkg.STORAGE_BF16}[storage_kind]
    xr = xb if storage_kind == "f32" else oracle.round_storage(xb, storage_kind)
    m, om = _metric(pkg, metric_name), (oracle.METRIC_L2 if metric_name == "L2" else oracle.METRIC_IP)
    idx = pkg.CudaIndexFlat(d, m, 0, storage)
    idx.add(xb)
    before = pkg.lib().ann_cuda_screen_fallbacks()
    for k in (8, 40, 300):
        D, I = idx.search(xq, k)
        Dref, Iref = oracle.flat_search(xr, xq, k, om)
        assert_topk_matches(oracle, xr, xq, om, D, I, Dref, Iref, f"23 hard queries, {metric_name}, {storage_kind}, k={k}")
        Dd, Id = idx.search_device(torch.from_numpy(xq).cuda(), k)
        idx.search_status()
        np.testing.assert_array_equal(Id.cpu().numpy(), I)
        np.testing.assert_array_equal(Dd.cpu().numpy(), D)
    assert pkg.lib().ann_cuda_screen_fallbacks() > before, "no tier flagged anything"
    idx.close()


@pytest.mark.parametrize("d", [768, 2000, 4000])
def test_the_threshold_scan_at_larger_dimensions(pkg, oracle, d):
    """Shared memory holds a group of 16 queries up to 3,200 floats each, of 8 beyond; at 768 floats the
    group fills exactly the 48 KB a launch gets without asking for more."""
    rng = np.random.default_rng(43)
    xb, q0 = _near_tie_store(rng, d, 3000, 300, "L2", 1e-6)
    xq = rng.standard_normal((9, d)).astype(np.float32)
    xq[1] = xq[4] = xq[5] = xq[8] = q0[0]
    idx = pkg.CudaIndexFlat(d, pkg.METRIC_L2)
    idx.add(xb)
    D, I = idx.search(xq, 20)
    Dref, Iref = oracle.flat_search(xb, xq, 20, oracle.METRIC_L2)
    assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, f"near ties at d={d}")
    idx.close()


@pytest.mark.parametrize("metric_name", ["L2", "IP"])
def test_duplicates_by_the_thousand_overflow_the_threshold_scan(pkg, oracle, metric_name):
    """5,000 copies of one row next to the query: every one of them is at the k-th distance, more than a
    candidate buffer holds, so the query is handed on to the scan that keeps k rows per item.  Any k of
    the copies are a right answer (ties at the k-th place)."""
    rng = np.random.default_rng(47)
    d = 48
    far = rng.standard_normal((12000, d)).astype(np.float32)
    q = rng.standard_normal(d).astype(np.float32)
    q /= np.linalg.norm(q)
    # (inner product: Gaussian rows reach ~4 along the unit query, the copies 6)
    row = (6.0 * q if metric_name == "IP" else q + 0.05 * rng.standard_normal(d)).astype(np.float32)
    xb = np.concatenate([far, np.repeat(row[None, :], 5000, 0)])
    xb = xb[np.random.default_rng(5).permutation(len(xb))]
    xq = np.stack([q, rng.standard_normal(d).astype(np.float32), q]).astype(np.float32)
    m, om = _metric(pkg, metric_name), (oracle.METRIC_L2 if metric_name == "L2" else oracle.METRIC_IP)
    idx = pkg.CudaIndexFlat(d, m)
    idx.add(xb)
    for k in (10, 100):
        D, I = idx.search(xq, k)
        Dref, Iref = oracle.flat_search(xb, xq, k, om)
        assert_topk_matches(oracle, xb, xq, om, D, I, Dref, Iref, f"5,000 duplicates, {metric_name}, k={k}")
    idx.close()


def test_more_flagged_queries_than_candidate_buffers(pkg, oracle):
    """4,200 queries of one block sit on the near ties; the candidate buffers of a block (16 M entries, 4,096
    per query at k = 8) serve the first 4,096 flagged queries, the item scan the other 104."""
    rng = np.random.default_rng(53)
    d = 64
    xb, q0 = _near_tie_store(rng, d, 20000, 400, "L2", 1e-6)
    xq = np.repeat(q0, 4200, 0)
    xq[::7] += (1e-6 * rng.standard_normal((len(xq[::7]), d))).astype(np.float32)
    idx = pkg.CudaIndexFlat(d, pkg.METRIC_L2)
    idx.add(xb)
    before = pkg.lib().ann_cuda_screen_fallbacks()
    D, I = idx.search(xq, 8)
    assert pkg.lib().ann_cuda_screen_fallbacks() == before + 2, "the exact tier did not run"
    Dref, Iref = oracle.flat_search(xb, xq, 8, oracle.METRIC_L2)
    assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, "4,200 flagged queries in one block")
    idx.close()


@pytest.mark.parametrize("entry", ["device", "async"])
def test_fallback_passes_run_on_the_device_for_the_entries_that_do_not_wait(pkg, oracle, entry):
    """search_device and search_async return before anything has run: the higher tiers are enqueued
    behind the first, gated by its band check.  More than two query blocks (16384 queries each),
    with the near ties that overflow the screened tier visible to the queries of block 0 only -
    a clean later block must not hide what an earlier one needed."""
    import torch
    rng = np.random.default_rng(31)
    d, k = 32, 20
    xb, q0 = _near_tie_store(rng, d, 6000, 600, "L2", 1e-4)
    nq = 2 * 16384 + 100
    xq = (rng.standard_normal((nq, d)) * 4).astype(np.float32)      # far from the tie cluster: clean blocks
    xq[:3] = q0
    assert pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05-screened") == 0
    try:
        idx = pkg.CudaIndexFlat(d, pkg.METRIC_L2)
        idx.add(xb)
        before = pkg.lib().ann_cuda_screen_fallbacks()
        if entry == "device":
            Dd, Id = idx.search_device(torch.from_numpy(xq).cuda(), k)
            idx.search_status()                                       # waits; raises on a device-side failure
            D, I = Dd.cpu().numpy(), Id.cpu().numpy()
        else:
            D, I = idx.search_async(xq, k).wait()
        assert pkg.lib().ann_cuda_screen_fallbacks() >= before + 1, "no fallback pass ran"
        sample = np.concatenate([np.arange(0, 40), np.arange(16384 - 5, 16384 + 5), np.arange(nq - 20, nq)])
        Dref, Iref = oracle.flat_search(xb, xq[sample], k, oracle.METRIC_L2)
        assert_topk_matches(oracle, xb, xq[sample], oracle.METRIC_L2, D[sample], I[sample], Dref, Iref, f"gated tiers ({entry})")
        # the synchronous entry point repeats on the host instead and must give the same answer
        Ds, Is = idx.search(xq[sample], k)
        np.testing.assert_array_equal(Is, I[sample])
        np.testing.assert_array_equal(Ds, D[sample])
        idx.close()
    finally:
        pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")


@pytest.mark.parametrize("k", [130, 200, 256, 1024, 2048])
def test_large_k(pkg, oracle, k):
    """k beyond the shared-memory and one-MMA modes: append-and-compact lists up to 256 entries,
    replace-max lists up to the limit of 2048 (the reference's block select takes k up to 4096 on
    its newest GPUs, faiss-metal/src/MetalSelect.mm:53-56), screened search up to k = 224."""
    rng = np.random.default_rng(k)
    nv, nq, d = 9000, 130, 40
    xb = rng.uniform(-1, 1, (nv, d)).astype(np.float32)
    xq = rng.uniform(-1, 1, (nq, d)).astype(np.float32)
    for kernel in ("tcgen05", "tcgen05-screened"):
        assert pkg.lib().ann_cuda_set_flat_kernel(kernel.encode()) == 0
        try:
            for metric_name in ("L2", "IP"):
                m = _metric(pkg, metric_name)
                idx = pkg.CudaIndexFlat(d, m)
                idx.add(xb)
                D, I = idx.search(xq, k)
                Dref, Iref = oracle.flat_search(xb, xq, k, m)
                assert_topk_matches(oracle, xb, xq, m, D, I, Dref, Iref, f"{kernel} {metric_name} k={k}")
                idx.close()
        finally:
            pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")
    idx = pkg.CudaIndexFlat(d, pkg.METRIC_L2)
    idx.add(xb)
    with pytest.raises(pkg.AnnCudaError, match="2048"):
        idx.search(xq, 2049)
    idx.close()


@pytest.mark.parametrize("shape", ["split", "screened-pairs"])
def test_a_wait_that_runs_out_fails_the_search_and_leaves_the_device_usable(pkg, oracle, shape):
    """Every wait inside the tensor-core kernel is bounded.  With the bound lowered to 20 ms and the
    loader told to stop after three blocks of the dimension, the MMA issuer waits for a stage that
    never arrives: the kernel must give up in order, the search must FAIL (not return partial
    lists), and the next search on the same index must work.  "screened-pairs" is the same on the
    kernel that runs as clusters of two CTAs (tcgen05 cta_group::2): both CTAs of every pair have
    to find their way out, the one that issues the MMAs and the one that only feeds it."""
    rng = np.random.default_rng(5)
    if shape == "split":
        n, d, nq, k, kernel = 20000, 128, 40, 10, b"tcgen05"
    else:
        n, d, nq, k, kernel = 200_000, 32, 256, 30, b"tcgen05-screened"
    xb = rng.uniform(-1, 1, (n, d)).astype(np.float32)
    xq = rng.uniform(-1, 1, (nq, d)).astype(np.float32)
    lib = pkg.lib()
    assert lib.ann_cuda_set_flat_kernel(kernel) == 0
    try:
        idx = pkg.CudaIndexFlat(d, pkg.METRIC_L2)
        idx.add(xb)
        D0, I0 = idx.search(xq, k)
        lib.ann_cuda_set_wait_limit_ms(20)
        lib.ann_cuda_test_withhold_loads(3)
        try:
            with pytest.raises(pkg.AnnCudaError, match="gave up on a wait"):
                idx.search(xq, k)
            tok = idx.search_async(xq, k)
            with pytest.raises(pkg.AnnCudaError, match="gave up on a wait"):
                tok.wait()
            import torch
            idx.search_device(torch.from_numpy(xq).cuda(), k)
            with pytest.raises(pkg.AnnCudaError, match="gave up on a wait"):
                idx.search_status()
            idx.search_status()          # collected: the stream's record is clean again
        finally:
            lib.ann_cuda_test_withhold_loads(-1)
            lib.ann_cuda_set_wait_limit_ms(0)
        D1, I1 = idx.search(xq, k)
        np.testing.assert_array_equal(I1, I0)
        np.testing.assert_array_equal(D1, D0)
        Dref, Iref = oracle.flat_search(xb, xq, k, oracle.METRIC_L2)
        assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D1, I1, Dref, Iref, "after a failed search")
        idx.close()
    finally:
        lib.ann_cuda_set_flat_kernel(b"tcgen05")


@pytest.mark.parametrize("nq", [11 * 128 - 5, 13 * 128, 9 * 128 + 1])
def test_an_odd_number_of_query_tiles(pkg, oracle, nq):
    """The kernel that runs as clusters of two CTAs gives each CTA of a pair one query tile.  Eleven or thirteen
    tiles are planned as twelve or fourteen, the last one holding no query; nine tiles (and a ragged tenth) stay
    as they are.  Every query must come back with the oracle's answer either way."""
    rng = np.random.default_rng(41)
    xb = rng.uniform(-1, 1, (200_000, 32)).astype(np.float32)
    xq = rng.uniform(-1, 1, (nq, 32)).astype(np.float32)
    assert pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05-screened") == 0
    try:
        idx = pkg.CudaIndexFlat(32, pkg.METRIC_INNER_PRODUCT)
        idx.add(xb)
        D, I = idx.search(xq, 30)
        Dref, Iref = oracle.flat_search(xb, xq, 30, oracle.METRIC_IP)
        assert_topk_matches(oracle, xb, xq, oracle.METRIC_IP, D, I, Dref, Iref, f"{nq} queries")
        idx.close()
    finally:
        pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")


@pytest.mark.parametrize("flat_kernel", ["tcgen05-screened", "tcgen05-split"])
def test_every_repetition_gives_the_oracle_answer(pkg, oracle, flat_kernel):
    """Thresholds travel between CTAs through memory, so WHICH rows reach the candidate lists depends on
    timing; the answer must not.  Twelve searches in a row and four in flight at once, 1,024 queries
    whose error bands differ from row to row, every single result against the oracle (a compaction
    that applied one row's band to another row's buffer passed a one-shot test here)."""
    rng = np.random.default_rng(19)
    xb = rng.uniform(-1, 1, (200_000, 32)).astype(np.float32)
    xq = (rng.uniform(-1, 1, (1024, 32)) * rng.uniform(0.2, 3.0, (1024, 1))).astype(np.float32)
    Dref, Iref = oracle.flat_search(xb, xq, 30, oracle.METRIC_L2)
    assert pkg.lib().ann_cuda_set_flat_kernel(flat_kernel.encode()) == 0
    try:
        idx = pkg.CudaIndexFlat(32, pkg.METRIC_L2)
        idx.add(xb)
        for rep in range(12):
            D, I = idx.search(xq, 30)
            assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, f"{flat_kernel}, repetition {rep}")
        for i, t in enumerate([idx.search_async(xq, 30) for _ in range(4)]):
            D, I = t.wait()
            assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, f"{flat_kernel}, in flight {i}")
        idx.close()
    finally:
        pkg.lib().ann_cuda_set_flat_kernel(b"tcgen05")
