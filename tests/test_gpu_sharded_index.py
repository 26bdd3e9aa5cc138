"""One index over several shards in one process (ann_cuda_sharded_*): the search of every shard,
the copy of the per-shard lists into the merging GPU and the merge give exactly what a single
index gives.  Shards may share a device, so the whole path runs on a one-GPU box; with two or more
GPUs the same tests also run with one shard per GPU."""
import numpy as np
import pytest

from parity import assert_topk_matches

pytestmark = pytest.mark.gpu


def _device_lists():
    import torch
    lists = [(0, 0, 0)]
    if torch.cuda.device_count() >= 2:
        lists.append(tuple(range(min(torch.cuda.device_count(), 4))))
    return lists


@pytest.mark.parametrize("metric_name", ["L2", "IP"])
def test_flat_rows_sharded(pkg, oracle, metric_name):
    rng = np.random.default_rng(5)
    xb = rng.uniform(-1, 1, (9001, 160)).astype(np.float32)
    xq = rng.uniform(-1, 1, (70, 160)).astype(np.float32)
    m = pkg.METRIC_L2 if metric_name == "L2" else pkg.METRIC_INNER_PRODUCT
    single = pkg.CudaIndexFlat(160, m)
    single.add(xb)
    D0, I0 = single.search(xq, 20)
    Dref, Iref = oracle.flat_search(xb, xq, 20, m)
    for devices in _device_lists():
        idx = pkg.CudaShardedIndex(160, m, devices)
        assert idx.shard_count == len(devices)
        D, I = idx.search(xq[:3], 4)                      # empty: sentinels
        assert (I == -1).all() and np.isinf(D).all()
        idx.add(xb[:8000])                                 # first add: equal contiguous ranges
        sizes = [idx.shard(g).ntotal for g in range(len(devices))]
        assert sum(sizes) == 8000 and max(sizes) - min(sizes) <= 1
        idx.add(xb[8000:])                                 # later rows go behind the last shard's
        assert idx.ntotal == 9001 and idx.shard(len(devices) - 1).ntotal == sizes[-1] + 1001
        D, I = idx.search(xq, 20)
        np.testing.assert_array_equal(I, I0)
        np.testing.assert_array_equal(D, D0)
        assert_topk_matches(oracle, xb, xq, m, D, I, Dref, Iref, f"flat sharded over {devices}")
        for key in (0, sizes[0] - 1, sizes[0], 8999, 9000):
            assert idx.reconstruct(key).tobytes() == xb[key].tobytes()
        assert idx.get_rows(sizes[0] - 2, 5).tobytes() == xb[sizes[0] - 2:sizes[0] + 3].tobytes()
        with pytest.raises(pkg.AnnCudaError):
            idx.reconstruct(9001)
        idx.reset()
        assert idx.ntotal == 0
        idx.add(xb[:7])                                    # fewer rows than shards x k: k > ntotal is padded
        D, I = idx.search(xq[:2], 12)
        assert (I[:, 7:] == -1).all() and (np.sort(I[0, :7]) == np.arange(7)).all() and np.isinf(D[:, 7:]).all()
        idx.close()
    single.close()


def test_ivf_lists_sharded(pkg, oracle):
    rng = np.random.default_rng(6)
    xb = rng.standard_normal((6000, 64)).astype(np.float32)
    xq = rng.standard_normal((40, 64)).astype(np.float32)
    cent = oracle.kmeans(xb, 32, niter=5, seed=6)
    assign = oracle.ivf_assign(xb, cent, oracle.METRIC_L2)
    off, rows = oracle.lists_from_assign(assign, 32)
    Dref, Iref = oracle.ivf_search(xb, cent, off, rows, xq, 10, 8, oracle.METRIC_L2)
    for devices in _device_lists():
        for via in ("add_list", "add"):
            idx = pkg.CudaShardedIndex(64, pkg.METRIC_L2, devices, nlist=32)
            idx.set_centroids(cent)
            if via == "add_list":                           # the CpuToGpu conversion path
                for l in range(32):
                    r = rows[off[l]:off[l + 1]]
                    if len(r):
                        idx.add_list(l, r, xb[r])
            else:                                           # faiss::Index::add: every shard keeps its lists' rows
                idx.add(xb)
            assert idx.ntotal == 6000
            idx.setNprobe(8)
            D, I = idx.search(xq, 10)
            assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, f"ivf sharded over {devices} via {via}")
            assert idx.reconstruct(4321).tobytes() == xb[4321].tobytes()
            idx.close()


def test_sharded_training_gives_every_shard_the_same_centroids(pkg):
    rng = np.random.default_rng(9)
    centers = rng.standard_normal((8, 32)) * 4
    xb = (centers[rng.integers(0, 8, 4000)] + 0.3 * rng.standard_normal((4000, 32))).astype(np.float32)
    idx = pkg.CudaShardedIndex(32, pkg.METRIC_L2, (0, 0), nlist=8)
    idx.train(xb)
    lib = pkg.lib()
    import ctypes as C
    cents = []
    for g in range(2):
        out = np.empty((8, 32), np.float32)
        assert lib.ann_cuda_ivfflat_get_centroids(idx.shard(g)._h, C.c_void_p(out.ctypes.data)) == 0
        cents.append(out)
    np.testing.assert_array_equal(cents[0], cents[1])
    idx.add(xb)
    idx.setNprobe(8)
    D, I = idx.search(xb[:30], 1)
    assert (I[:, 0] == np.arange(30)).all() and (D[:, 0] == 0).all()
    idx.close()
