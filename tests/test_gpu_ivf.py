"""IVFFlat search on the GPU against the CPU oracle, with the SAME centroids and nprobe.

Shapes from faiss-metal/tests/test_metal_ivfflat.mm:31-36 (L2: nv=2000, d=64,
nlist=16, nprobe=4, nq=10, k=5) and :105-112 (IP: nv=1000, d=128, nlist=8,
nprobe=2, nq=5, k=10, seed 123), the empty-index cases of :328-351, the
round trip of :215-224, plus a scaled-down copy of the clustered configuration."""
import json
import os

import numpy as np
import pytest

from parity import RTOL, assert_topk_matches

pytestmark = pytest.mark.gpu


def _build(pkg, oracle, xb, nlist, metric, seed=1, via="add_list"):
    cent = oracle.kmeans(xb, nlist, niter=6, seed=seed)
    assign = oracle.ivf_assign(xb, cent, metric)
    off, rows = oracle.lists_from_assign(assign, nlist)
    idx = pkg.CudaIndexIVFFlat(xb.shape[1], nlist, metric)
    assert not idx.is_trained
    idx.set_centroids(cent)
    assert idx.is_trained
    if via == "add_list":  # the CpuToGpu conversion path
        for l in range(nlist):
            r = rows[off[l]:off[l + 1]]
            if len(r):
                idx.add_list(l, r, xb[r])
    else:  # faiss::Index::add: assignment on the GPU
        idx.add(xb)
    return idx, cent, off, rows


def _check(pkg, oracle, idx, xb, cent, off, rows, xq, k, nprobe, metric, what):
    idx.setNprobe(nprobe)
    D, I = idx.search(xq, k)
    Dref, Iref, probes = oracle.ivf_search(xb, cent, off, rows, xq, k, nprobe, metric, return_probes=True)
    # Where a query's nprobe-th and (nprobe+1)-th centroid distances are a tolerance
    # tie the probe set itself may legitimately differ; such queries are compared
    # against the oracle run over the union of both candidate probe sets.
    cd = np.stack([oracle.all_distances(cent, q, metric) for q in xq])
    order = np.argsort(cd if metric == oracle.METRIC_L2 else -cd, axis=1, kind="stable")
    cands = []
    for q in range(len(xq)):
        p = probes[q][probes[q] >= 0]
        cands.append(set(np.concatenate([rows[off[c]:off[c + 1]] for c in p]).tolist()) if len(p) else set())
    ambiguous = []
    if nprobe < cent.shape[0]:
        a = np.take_along_axis(cd, order[:, nprobe - 1:nprobe], 1)[:, 0]
        b = np.take_along_axis(cd, order[:, nprobe:nprobe + 1], 1)[:, 0]
        ambiguous = np.nonzero(np.abs(a - b) <= 4 * RTOL * np.maximum(np.abs(a), 1e-30))[0].tolist()
    keep = [q for q in range(len(xq)) if q not in ambiguous]
    assert_topk_matches(oracle, xb, xq[keep], metric, D[keep], I[keep], Dref[keep], Iref[keep], what,
                        candidates=[cands[q] for q in keep])
    # a query whose nprobe-th / (nprobe+1)-th centroids tie may take either of them
    for q in ambiguous:
        alt = order[q, :nprobe + 1].copy()
        alt = np.delete(alt, nprobe - 1)[None, :].astype(np.int64)
        Da, Ia = oracle.ivf_search_given_probes(xb, off, rows, xq[q:q + 1], k, alt, metric)
        try:
            assert_topk_matches(oracle, xb, xq[q:q + 1], metric, D[q:q + 1], I[q:q + 1], Dref[q:q + 1], Iref[q:q + 1],
                                what + " (tie, first probe set)", candidates=None)
        except AssertionError:
            assert_topk_matches(oracle, xb, xq[q:q + 1], metric, D[q:q + 1], I[q:q + 1], Da, Ia,
                                what + " (tie, second probe set)", candidates=None)
    # recall@k against the oracle with the same centroids and nprobe must be 1.0
    hits = sum(len(set(I[q][I[q] >= 0].tolist()) & set(Iref[q][Iref[q] >= 0].tolist())) for q in keep)
    total = sum(int((Iref[q] >= 0).sum()) for q in keep)
    assert total == 0 or hits / total >= 1.0 - 1e-3, f"{what}: recall {hits / total}"
    return D, I


@pytest.mark.parametrize("via", ["add_list", "add"])
def test_l2_reference_shape(pkg, oracle, via):
    rng = np.random.default_rng(42)
    xb = rng.uniform(-1, 1, (2000, 64)).astype(np.float32)
    xq = rng.uniform(-1, 1, (10, 64)).astype(np.float32)
    idx, cent, off, rows = _build(pkg, oracle, xb, 16, pkg.METRIC_L2, via=via)
    assert idx.ntotal == 2000 and idx.getNlist() == 16
    for nprobe in (1, 4, 16):
        _check(pkg, oracle, idx, xb, cent, off, rows, xq, 5, nprobe, pkg.METRIC_L2, f"L2 {via} nprobe={nprobe}")
    idx.close()


def test_ip_reference_shape(pkg, oracle):
    rng = np.random.default_rng(123)
    xb = rng.uniform(-1, 1, (1000, 128)).astype(np.float32)
    xq = rng.uniform(-1, 1, (5, 128)).astype(np.float32)
    idx, cent, off, rows = _build(pkg, oracle, xb, 8, pkg.METRIC_INNER_PRODUCT)
    _check(pkg, oracle, idx, xb, cent, off, rows, xq, 10, 2, pkg.METRIC_INNER_PRODUCT, "IP")
    idx.close()


def test_search_async_on_an_ivf_index(pkg, oracle):
    """The token interface of the flat index also serves IVFFlat: same answers as search()."""
    rng = np.random.default_rng(7)
    xb = rng.uniform(-1, 1, (3000, 48)).astype(np.float32)
    xq = rng.uniform(-1, 1, (24, 48)).astype(np.float32)
    idx, cent, off, rows = _build(pkg, oracle, xb, 12, pkg.METRIC_L2)
    idx.setNprobe(3)
    D, I = idx.search(xq, 9)
    tokens = [idx.search_async(xq[i:i + 6], 9) for i in range(0, 24, 6)]
    for j in (2, 3, 0, 1):
        Da, Ia = tokens[j].wait()
        np.testing.assert_array_equal(Ia, I[6 * j:6 * j + 6])
        np.testing.assert_array_equal(Da, D[6 * j:6 * j + 6])
    idx.close()


def test_known_answer_from_reference_sql(pkg, oracle):
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")) as f:
        case = json.load(f)["ivfflat"][0]
    db = np.array(case["db"], np.float32)
    idx, cent, off, rows = _build(pkg, oracle, db, case["nlist"], pkg.METRIC_L2, seed=7)
    idx.setNprobe(case["nprobe"])
    D, I = idx.search(np.array([case["query"]], np.float32), case["k"])
    assert I[0].tolist() == case["labels"] and D[0, 0] == 0.0
    idx.close()


def test_full_probe_equals_flat_and_ragged_lists(pkg, oracle):
    rng = np.random.default_rng(8)
    xb = rng.standard_normal((5000, 100)).astype(np.float32)  # d not a multiple of 32
    xq = rng.standard_normal((37, 100)).astype(np.float32)
    idx, cent, off, rows = _build(pkg, oracle, xb, 50, pkg.METRIC_L2)
    D, I = _check(pkg, oracle, idx, xb, cent, off, rows, xq, 70, 50, pkg.METRIC_L2, "full probe")
    Df, If = oracle.flat_search(xb, xq, 70, oracle.METRIC_L2)
    assert (I == If).mean() > 0.999
    idx.close()


def test_edge_cases_and_round_trip(pkg, oracle):
    rng = np.random.default_rng(2)
    xb = rng.uniform(-1, 1, (300, 32)).astype(np.float32)
    idx = pkg.CudaIndexIVFFlat(32, 4, pkg.METRIC_L2)
    with pytest.raises(pkg.AnnCudaError):
        idx.search(xb[:2], 3)  # not trained (MetalIndexIVFFlat.mm:125)
    with pytest.raises(pkg.AnnCudaError):
        idx.add(xb)
    cent = oracle.kmeans(xb, 4, niter=4, seed=3)
    idx.set_centroids(cent)
    D, I = idx.search(xb[:2], 3)  # trained but empty -> sentinels (:328-351)
    assert (I == -1).all() and np.isposinf(D).all()
    idx.add(xb[:200])
    idx.add(xb[200:])  # second add interleaves lists: regrouped lazily
    assert idx.ntotal == 300
    assign = oracle.ivf_assign(xb, cent, oracle.METRIC_L2)
    off, rows = oracle.lists_from_assign(assign, 4)
    got_cent = idx.get_centroids()
    assert got_cent.tobytes() == cent.tobytes()
    for l in range(4):  # GPU assignment == oracle assignment; rows come back bit for bit, in add order
        ids, vecs = idx.get_list(l)
        assert ids.tolist() == rows[off[l]:off[l + 1]].tolist()
        assert vecs.tobytes() == xb[ids].tobytes()
    assert idx.reconstruct(123).tobytes() == xb[123].tobytes()
    idx.setNprobe(100)
    assert idx.getNprobe() == 4  # clamped to nlist (:275-279)
    D, I = idx.search(xb[:5], 500)  # k > ntotal
    assert (I[:, 300:] == -1).all() and (I[:, :300] >= 0).all()
    idx.reset()
    assert idx.ntotal == 0 and (idx.search(xb[:1], 2)[1] == -1).all()
    idx.close()


def test_gpu_train_gives_usable_centroids(pkg, oracle):
    rng = np.random.default_rng(4)
    centers = rng.standard_normal((8, 48)).astype(np.float32) * 4
    lab = rng.integers(0, 8, 4000)
    xb = (centers[lab] + 0.1 * rng.standard_normal((4000, 48))).astype(np.float32)
    idx = pkg.CudaIndexIVFFlat(48, 8, pkg.METRIC_L2)
    idx.train(xb)
    assert idx.is_trained
    idx.add(xb)
    cent = idx.get_centroids()
    # Lloyd iterations only ever lower the quantisation error: the trained centroids
    # must beat the initial ones (rows spread evenly over the training set)
    init = xb[(np.arange(8) * len(xb)) // 8]

    def qerr(c):
        return ((xb[:, None, :].astype(np.float64) - c[None].astype(np.float64)) ** 2).sum(-1).min(1).mean()

    assert qerr(cent) < 0.7 * qerr(init)
    assign = oracle.ivf_assign(xb, cent, oracle.METRIC_L2)
    off, rows = oracle.lists_from_assign(assign, 8)
    xq = xb[:50] + 0.01
    _check(pkg, oracle, idx, xb, cent, off, rows, xq.astype(np.float32), 10, 2, pkg.METRIC_L2, "after GPU train")
    idx.close()


def test_tight_clusters_far_from_the_origin(pkg, oracle):
    """Distances ~1e-4 of the operands' squared norms, several centroids inside one cluster,
    some queries equal to stored rows: neither the choice of probe lists nor the list scan's
    norm expansion may lose them to cancellation."""
    rng = np.random.default_rng(11)
    nc, d = 32, 96
    centers = (rng.standard_normal((nc, d)) * 3 + 2).astype(np.float32)   # |c|^2 ~ 1.2e3, in-cluster d^2 ~ 0.5
    xb = (centers[rng.integers(0, nc, 8000)] + 0.05 * rng.standard_normal((8000, d))).astype(np.float32)
    xq = (centers[rng.integers(0, nc, 300)] + 0.05 * rng.standard_normal((300, d))).astype(np.float32)
    xq[:40] = xb[rng.integers(0, len(xb), 40)]          # exact duplicates of stored rows
    xq[40:80] = xb[rng.integers(0, len(xb), 40)] + np.float32(1e-3)
    idx, cent, off, rows = _build(pkg, oracle, xb, nc, pkg.METRIC_L2, seed=5)
    D, I = _check(pkg, oracle, idx, xb, cent, off, rows, xq, 20, 4, pkg.METRIC_L2, "tight clusters")
    assert (D[:40, 0] == 0.0).all()
    idx.close()


def test_clustered_config_scaled_down(pkg, oracle):
    """Gaussian clusters (centres N(0,1), offsets N(0, 0.1^2)), d=768, k=100, nprobe=16, scaled 1/50."""
    rng = np.random.default_rng(45)
    nc, d = 64, 768
    centers = rng.standard_normal((nc, d)).astype(np.float32)
    xb = (centers[rng.integers(0, nc, 20000)] + 0.1 * rng.standard_normal((20000, d))).astype(np.float32)
    xq = (centers[rng.integers(0, nc, 64)] + 0.1 * rng.standard_normal((64, d))).astype(np.float32)
    sample = xb[::10]  # every 10th row, the train_sample rule of src/faiss_index.cpp:304-315
    cent = oracle.kmeans(sample, nc, niter=8, seed=45)
    assign = oracle.ivf_assign(xb, cent, oracle.METRIC_L2)
    off, rows = oracle.lists_from_assign(assign, nc)
    idx = pkg.CudaIndexIVFFlat(d, nc, pkg.METRIC_L2)
    idx.set_centroids(cent)
    for l in range(nc):
        r = rows[off[l]:off[l + 1]]
        if len(r):
            idx.add_list(l, r, xb[r])
    _check(pkg, oracle, idx, xb, cent, off, rows, xq, 100, 16, pkg.METRIC_L2, "C3 scaled")
    idx.close()


def test_list_sharding_matches_unsharded(pkg, oracle):
    import torch
    rng = np.random.default_rng(6)
    xb = rng.standard_normal((6000, 64)).astype(np.float32)
    xq = rng.standard_normal((40, 64)).astype(np.float32)
    cent = oracle.kmeans(xb, 32, niter=5, seed=6)
    assign = oracle.ivf_assign(xb, cent, oracle.METRIC_L2)
    off, rows = oracle.lists_from_assign(assign, 32)
    xq_dev = torch.from_numpy(xq).cuda()
    parts_d, parts_i, shards = [], [], []
    for rank in range(3):
        s = pkg.CudaIndexIVFFlat(64, 32, pkg.METRIC_L2)
        s.set_shard(rank, 3)
        s.set_centroids(cent)
        for l in range(32):
            r = rows[off[l]:off[l + 1]]
            if len(r):
                s.add_list(l, r, xb[r])
        assert s.ntotal == 6000  # labels stay global
        s.setNprobe(8)
        d, i = s.search_device(xq_dev, 10)
        parts_d.append(d); parts_i.append(i); shards.append(s)
    D, I = pkg.merge_topk_device(torch.stack(parts_d).contiguous(), torch.stack(parts_i).contiguous(), pkg.METRIC_L2)
    torch.cuda.synchronize()
    Dref, Iref = oracle.ivf_search(xb, cent, off, rows, xq, 10, 8, oracle.METRIC_L2)
    assert (I.cpu().numpy() == Iref).mean() > 0.995
    np.testing.assert_allclose(D.cpu().numpy(), Dref, rtol=1e-4)
    # The same without a replicated coarse quantiser (what the sharded searcher does over several ranks):
    # every shard ranks the centroids for ITS slice of the queries, the slices are put together (the
    # all-gather), and every shard scans its lists for all queries with the probes given.
    per = (len(xq) + 2) // 3
    probes = torch.full((3 * per, 8), -1, dtype=torch.int32, device="cuda")
    for rank, sh in enumerate(shards):
        lo, hi = min(len(xq), rank * per), min(len(xq), (rank + 1) * per)
        sh.coarse_device(xq_dev[lo:hi], out=probes[lo:hi])
    np.testing.assert_array_equal(probes[:len(xq)].cpu().numpy(), shards[0].coarse(xq, 8))
    parts2 = [sh.search_preassigned_device(xq_dev, probes[:len(xq)], 10) for sh in shards]
    for sh in shards:
        sh.search_status()
    D2, I2 = pkg.merge_topk_device(torch.stack([p[0] for p in parts2]).contiguous(),
                                   torch.stack([p[1] for p in parts2]).contiguous(), pkg.METRIC_L2)
    np.testing.assert_array_equal(I2.cpu().numpy(), I.cpu().numpy())
    np.testing.assert_array_equal(D2.cpu().numpy(), D.cpu().numpy())
    # the coarse quantiser as the FIRST call on an index and stream leaves a clean status behind
    fresh = pkg.CudaIndexIVFFlat(64, 32, pkg.METRIC_L2)
    fresh.set_centroids(cent)
    fresh.setNprobe(8)
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        p0 = fresh.coarse_device(xq_dev, stream=st)
        fresh.search_status(stream=st)
    np.testing.assert_array_equal(p0.cpu().numpy(), shards[0].coarse(xq, 8))
    fresh.close()
    # a probe list of "no list" entries finds nothing
    none = torch.full((len(xq), 8), -1, dtype=torch.int32, device="cuda")
    D3, I3 = shards[0].search_preassigned_device(xq_dev, none, 10)
    torch.cuda.synchronize()
    assert (I3.cpu().numpy() == -1).all() and np.isinf(D3.cpu().numpy()).all()
    for s in shards:
        s.close()


@pytest.mark.parametrize("k,nprobe", [(100, 256), (10, 256), (300, 64), (2048, 4)])
def test_any_nprobe_and_k(pkg, oracle, k, nprobe):
    """The reference scans whatever nprobe <= nlist asks for (faiss-metal/src/MetalIndexIVFFlat.mm:122-256,
    275-279).  nprobe = nlist = 256 with k = 100 is 27,648 candidates per query; the per-query merge
    streams them, so no product of nprobe and k is too large.  All three selection modes of the scan."""
    rng = np.random.default_rng(k + nprobe)
    xb = rng.standard_normal((20000, 32)).astype(np.float32)
    xq = rng.standard_normal((40, 32)).astype(np.float32)
    idx, cent, off, rows = _build(pkg, oracle, xb, 256, pkg.METRIC_L2, seed=3)
    _check(pkg, oracle, idx, xb, cent, off, rows, xq, k, nprobe, pkg.METRIC_L2, f"k={k} nprobe={nprobe}")
    if nprobe == 256:   # every list probed: the flat answer
        D, I = idx.search(xq, k)
        Dref, Iref = oracle.flat_search(xb, xq, k, oracle.METRIC_L2)
        assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, "nprobe = nlist equals flat")
    with pytest.raises(pkg.AnnCudaError, match="2048"):
        idx.search(xq, 2049)     # an error, as for Flat, not a silently shortened result
    idx.close()
