"""The benchmark configurations at (or near) their full sizes against the CPU oracle.

These are the shapes the benchmark times: Flat L2 100,000 x 384 with 1,000 queries and k = 10 in
full; a flat inner-product store of 2.1 million unit-norm rows of 768 floats with k = 100, large
enough that the library chooses one-MMA screening and the static schedule BY ITSELF (the
sharded 20M-row configuration puts 2.5 million rows on each of 8 GPUs); the same for L2 with the
store's mean far from the origin; a million rows with planted groups of duplicates, which only the exact
tier can answer; one full aggregated batch of the DiskANN batch distance
(256 x 128 rows of 1536 floats) and of the SQ8 distance (1,024 x 128 rows of 384 codes).
The oracle runs on a sample of the queries where the full set would take minutes."""
import numpy as np
import pytest

from parity import RTOL, assert_distances_close, assert_topk_matches

pytestmark = pytest.mark.gpu


def test_flat_l2_100k_full_size(pkg, oracle):
    rng = np.random.default_rng(42)
    xb = rng.uniform(0, 1, (100_000, 384)).astype(np.float32)
    xq = rng.uniform(0, 1, (1000, 384)).astype(np.float32)
    idx = pkg.CudaIndexFlat(384, pkg.METRIC_L2)
    idx.add(xb)
    D, I = idx.search(xq, 10)
    Dref, Iref = oracle.flat_search(xb, xq, 10, oracle.METRIC_L2)
    assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, "Flat L2 100k x 384, full size")
    idx.close()


def _big_store(torch, n, d, kind, seed):
    chunks = []
    for c in range(0, n, 300_000):
        rows = min(300_000, n - c)
        g = torch.Generator(device="cuda").manual_seed(seed + c)
        x = torch.randn((rows, d), generator=g, device="cuda", dtype=torch.float32)
        if kind == "unit":
            x /= x.norm(dim=1, keepdim=True)
        else:                       # a store whose mean is far from the origin
            x = x * 0.25 + 3.0
        chunks.append(x)
    return chunks


@pytest.mark.parametrize("kind,metric_name", [("unit", "IP"), ("shifted", "L2")])
def test_screening_chosen_by_the_library_at_two_million_rows(pkg, oracle, kind, metric_name):
    import torch
    n, d, nq, k = 2_100_000, 768, 300, 100
    m = pkg.METRIC_INNER_PRODUCT if metric_name == "IP" else pkg.METRIC_L2
    assert pkg.lib().ann_cuda_flat_kernel_name() == b"tcgen05"
    idx = pkg.CudaIndexFlat(d, m)
    idx.reserve(n)
    chunks = _big_store(torch, n, d, kind, 1000)
    for x in chunks:
        idx.add_device(x.contiguous())
    xb = np.concatenate([x.cpu().numpy() for x in chunks])
    del chunks
    torch.cuda.empty_cache()
    g = torch.Generator().manual_seed(43)
    q = torch.randn((nq, d), generator=g)
    xq = (q / q.norm(dim=1, keepdim=True) if kind == "unit" else q * 0.25 + 3.0).numpy().astype(np.float32)
    xq[0] = xb[12345]            # a stored row: best hit is itself
    before = pkg.lib().ann_cuda_screen_fallbacks()
    D, I = idx.search(xq, k)
    # ... the same through the device entry point on torch's stream (what the sharded search calls)
    Dd, Id = idx.search_device(torch.from_numpy(xq).cuda(), k)
    idx.search_status()
    np.testing.assert_array_equal(Id.cpu().numpy(), I)
    np.testing.assert_array_equal(Dd.cpu().numpy(), D)
    assert I[0, 0] == 12345
    # sortedness and label range over ALL queries, the oracle on a sample of them
    sgn = -1.0 if metric_name == "IP" else 1.0
    assert (np.diff(sgn * D, axis=1) >= 0).all() and (I >= 0).all() and (I < n).all()
    sample = np.concatenate([np.arange(0, 12), np.arange(122, 134), np.arange(nq - 8, nq)])
    om = oracle.METRIC_IP if metric_name == "IP" else oracle.METRIC_L2
    Dref, Iref = oracle.flat_search(xb, xq[sample], k, om)
    assert_topk_matches(oracle, xb, xq[sample], om, D[sample], I[sample], Dref, Iref,
                        f"screened by the library's own choice, {metric_name}, 2.1M x 768")
    # Unit-norm rows: the screened search answers by itself.  The shifted store is the hard case of
    # the tensor-core tiers: their proven error bands scale with |q - mean| |x|max, and |x|max is twelve
    # times the spread of the rows here, so at d = 768 even the split product's band (0.75 on squared
    # distances of ~78) holds ~240 rows above the 100th - about what a banded list can keep.  Queries
    # that exceed it send the block on, up to the exact scan: at most two passes more per entry point.
    fell_back = pkg.lib().ann_cuda_screen_fallbacks() - before
    assert fell_back <= (0 if kind == "unit" else 4), f"{fell_back} fallback passes"
    # 300 queries are three tiles of 128, an odd number, which the kernel that runs as clusters of two
    # CTAs (one query tile each on a shared row tile, tcgen05 cta_group::2) does not take.  The first
    # 200 are two tiles, the second one ragged: the same answers must come back from that kernel
    # (2.1M rows end in a ragged row tile whose second half lies wholly past the store).
    D2, I2 = idx.search(xq[:200], k)
    np.testing.assert_array_equal(I2, I[:200])
    np.testing.assert_array_equal(D2, D[:200])
    idx.close()


@pytest.mark.parametrize("metric_name", ["L2", "IP"])
def test_duplicate_groups_at_one_million_rows(pkg, oracle, metric_name):
    """200 groups of 400 identical rows planted in a million: a query equal to a group's row has 400 neighbours
    at one distance, more than a candidate list of the tensor-core tiers holds, so every tier's band check flags
    it and the exact tier answers - for the 200 flagged queries among 600 only, with one threshold scan of the
    store per 16 of them.  Size-independent properties over all queries (a flagged query gets ten members of its
    own group, at distance exactly 0 for L2), the oracle on a sample."""
    import torch
    n, d, nq, k, groups, copies = 1_000_000, 256, 600, 10, 200, 400
    m = pkg.METRIC_INNER_PRODUCT if metric_name == "IP" else pkg.METRIC_L2
    g = torch.Generator(device="cuda").manual_seed(77)
    x = torch.randn((n, d), generator=g, device="cuda", dtype=torch.float32)
    member = torch.randperm(n, generator=g, device="cuda")[: groups * copies].view(groups, copies)
    x[member.flatten()] = x[member[:, 0]].repeat_interleave(copies, 0)
    idx = pkg.CudaIndexFlat(d, m)
    idx.add_device(x)
    q = torch.randn((nq, d), generator=g, device="cuda", dtype=torch.float32)
    hard = torch.randperm(nq, generator=g, device="cuda")[:groups]
    # (inner product: three times the row, so that nothing but the copies comes near |row|^2 * 3)
    q[hard] = x[member[:, 0]] * (3.0 if metric_name == "IP" else 1.0)
    before = pkg.lib().ann_cuda_screen_fallbacks()
    Dd, Id = idx.search_device(q, k)
    idx.search_status()
    assert pkg.lib().ann_cuda_screen_fallbacks() > before, "no band check flagged the duplicates"
    in_group = (Id[hard].unsqueeze(2) == member.unsqueeze(1)).any(2)
    assert bool(in_group.all()), f"{int((~in_group).sum())} neighbours of flagged queries are outside their group"
    if metric_name == "L2":
        assert bool((Dd[hard] == 0).all())
    xq = q.cpu().numpy()
    D, I = idx.search(xq, k)                      # the host entry repeats tier by tier from the host
    np.testing.assert_array_equal(Id.cpu().numpy(), I)
    np.testing.assert_array_equal(Dd.cpu().numpy(), D)
    xb = x.cpu().numpy()
    del x
    hs = hard.cpu().numpy()
    sample = np.concatenate([hs[:12], np.setdiff1d(np.arange(nq), hs)[:12]])
    om = oracle.METRIC_IP if metric_name == "IP" else oracle.METRIC_L2
    Dref, Iref = oracle.flat_search(xb, xq[sample], k, om)
    assert_topk_matches(oracle, xb, xq[sample], om, D[sample], I[sample], Dref, Iref,
                        f"duplicate groups, {metric_name}, 1M x 256")
    idx.close()


def test_batch_distance_one_full_aggregated_batch(pkg, oracle):
    """256 queries x 128 random rows of a 1536-float table, L2 and IP, ids in / distances out."""
    rng = np.random.default_rng(44)
    num, dim, nq, per = 200_000, 1536, 256, 128      # the table is cut to 1.2 GB; the batch is full size
    table = rng.standard_normal((num, dim)).astype(np.float32)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    ids = rng.integers(0, num, nq * per).astype(np.uint32)
    qmap = np.repeat(np.arange(nq, dtype=np.uint32), per)
    t = pkg.diskann_bridge.DeviceTable.from_host(table)
    for metric in (0, 1):
        got = t.batch_distances_by_id(q, ids, qmap, metric)
        want = oracle.batch_distances_by_id(table, q, ids, qmap, metric, exact=True)
        if metric == 0:
            assert_distances_close(got, want, "full aggregated batch, L2")
        else:   # a dot product near zero is judged against the size of its terms
            scale = (np.abs(q[qmap]).astype(np.float64) * np.abs(table[ids])).sum(1)
            assert (np.abs(got - want) <= RTOL * np.maximum(np.abs(want), 1e-2 * scale)).all()
    t.close()


def test_sq8_one_full_batch(pkg, oracle):
    """1,024 queries x 128 random rows of 384 codes (asymmetric L2 and IP against the uint8 codes)."""
    rng = np.random.default_rng(45)
    num, dim, nq, per = 1_000_000, 384, 1024, 128
    x = rng.standard_normal((num, dim)).astype(np.float32)
    mins, scale = oracle.sq8_train(x)
    codes = oracle.sq8_encode(x, mins, scale)
    del x
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    ids = rng.integers(0, num, nq * per).astype(np.uint32)
    qmap = np.repeat(np.arange(nq, dtype=np.uint32), per)
    t = pkg.diskann_bridge.DeviceTable.sq8_from_host(codes, mins, scale)
    for metric in (0, 1):
        got = t.batch_distances_by_id(q, ids, qmap, metric)
        want = oracle.sq8_batch_distances_by_id(codes, mins, scale, q, ids, qmap, metric, exact=True)
        if metric == 0:
            assert_distances_close(got, want, "full SQ8 batch, L2")
        else:
            xh = oracle.sq8_decode(codes[ids], mins, scale)
            sc = (np.abs(q[qmap]).astype(np.float64) * np.abs(xh)).sum(1)
            assert (np.abs(got - want) <= RTOL * np.maximum(np.abs(want), 1e-2 * sc)).all()
    t.close()
