"""The search loop that feeds the by-id batch-distance entry points: lock-step batched graph
search over a ".diskann" image resident in GPU memory (diskann_cuda_searcher_*), against the
oracle's restatement of DiskProvider::search_batch (rust_lib/src/disk_provider.rs:470-652) and
against brute force."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _knn_graph_image(oracle, rng, n, d, degree, metric, with_sq8=False):
    x = rng.standard_normal((n, d)).astype(np.float32)
    # exact k-nearest-neighbour graph plus a few random long edges, padded with the "unused" mark
    g = (x @ x.T).astype(np.float64)
    if metric == 0:
        sq = (x.astype(np.float64) ** 2).sum(1)
        g = -(sq[:, None] + sq[None, :] - 2 * g)
    np.fill_diagonal(g, -np.inf)
    nn = np.argsort(-g, axis=1)[:, :degree - 6].astype(np.uint32)
    adj = np.full((n, degree), 0xFFFFFFFF, np.uint32)
    adj[:, :degree - 6] = nn
    adj[:, degree - 6:degree - 2] = rng.integers(0, n, (n, 4)).astype(np.uint32)
    entry = np.array([0, n // 2], np.uint32)
    sq8 = None
    if with_sq8:
        mins, scale = oracle.sq8_train(x)
        sq8 = (mins, scale, oracle.sq8_encode(x, mins, scale))
    return x, oracle.write_diskann_image(x, adj, entry, metric=metric, sq8=sq8)


@pytest.mark.parametrize("metric", [0, 1])
@pytest.mark.parametrize("use_sq8", [False, True])
def test_lock_step_search_matches_the_oracle_loop(pkg, oracle, metric, use_sq8):
    rng = np.random.default_rng(12 + metric)
    n, d, degree, nq, k, l = 3000, 64, 32, 24, 10, 48
    x, image = _knn_graph_image(oracle, rng, n, d, degree, metric, with_sq8=use_sq8)
    queries = (x[rng.integers(0, n, nq)] + 0.3 * rng.standard_normal((nq, d))).astype(np.float32)
    s = pkg.diskann_bridge.DiskSearcher(image, use_sq8=use_sq8)
    assert s.info.num_vectors == n and s.info.max_degree == degree
    s.set_trace(True)
    got = s.search_batch(queries, k, l)
    st = s.stats()
    want = oracle.disk_search_batch(image, queries, k, l, use_sq8=use_sq8)
    hits = total = 0
    for (gi, gd), (wi, wd) in zip(got, want):
        assert len(gi) == k and (np.diff(gd) >= 0).all()
        common = set(gi.tolist()) & set(wi.tolist())
        hits += len(common); total += k
        # the distance of every id both report agrees to the tolerance of the batch-distance tests
        wmap = dict(zip(wi.tolist(), wd.tolist()))
        for i, dist in zip(gi.tolist(), gd.tolist()):
            if i in wmap:
                assert abs(dist - wmap[i]) <= 1e-4 * max(abs(wmap[i]), 1e-2 * d ** 0.5)
    # the traversal is decided by float comparisons: a distance that differs in its last bits may swap
    # two candidates, so the sets may differ in rare ties - not more
    assert hits >= 0.98 * total, f"only {hits} of {total} results agree with the oracle loop"
    # one distance call per iteration (plus the entry points), all queries in it: the batches a real search makes
    batches = s.trace()
    assert len(batches) == st["distance_calls"] and sum(len(b[0]) for b in batches) == st["pairs_scored"]
    assert st["distance_calls"] <= st["iterations"] + 1
    assert max(len(np.unique(b[1])) for b in batches) > nq // 2        # many queries share one launch
    if not use_sq8:
        # against brute force: the graph is good enough to find most true neighbours
        dd = ((queries[:, None, :].astype(np.float64) - x[None].astype(np.float64)) ** 2).sum(-1) if metric == 0 \
            else -(queries.astype(np.float64) @ x.T.astype(np.float64))
        truth = np.argsort(dd, axis=1)[:, :k]
        recall = np.mean([len(set(g[0].tolist()) & set(t.tolist())) / k for g, t in zip(got, truth)])
        assert recall > 0.8, recall
    s.close()


def test_edge_cases(pkg, oracle):
    rng = np.random.default_rng(3)
    x, image = _knn_graph_image(oracle, rng, 200, 16, 16, 0)
    s = pkg.diskann_bridge.DiskSearcher(image)
    assert s.search_batch(np.zeros((0, 16), np.float32), 5, 10) == []
    one = s.search_batch(x[:1], 5, 10)                      # a single query takes the same loop
    assert one[0][0][0] == 0 and one[0][1][0] == 0.0
    big = s.search_batch(x[:2], 500, 10)                    # k > num_vectors: clamped (disk_provider.rs:485)
    assert len(big[0][0]) <= 200
    with pytest.raises(pkg.AnnCudaError):
        pkg.diskann_bridge.DiskSearcher(image, use_sq8=True)   # no SQ8 trailer in this image
    with pytest.raises(pkg.AnnCudaError):
        pkg.diskann_bridge.DiskSearcher(image[:100])
    s.close()
