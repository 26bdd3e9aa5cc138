"""DiskANN batch-distance bridge on the GPU against the CPU oracle, through the C ABI.

Shapes follow the reference's callers and benches: single query x n gathered rows
(bench/metal_distance_bench.mm, README.md:140-145), lock-step multi-query batches
(bench/metal_distance_bench_v2.mm:205-212), plus ragged dimensions."""
import threading

import numpy as np
import pytest

from parity import assert_distances_close

pytestmark = pytest.mark.gpu


def _data(seed, n, dim, nq=1):
    rng = np.random.default_rng(seed)
    return (rng.standard_normal((nq, dim)).astype(np.float32),
            rng.standard_normal((n, dim)).astype(np.float32))


@pytest.mark.parametrize("n,dim", [(64, 128), (64, 768), (128, 1536), (256, 1536), (512, 1536), (1024, 768),
                                   (1, 3), (7, 5), (33, 130), (100, 1537), (5000, 96)])
@pytest.mark.parametrize("metric", [0, 1])
def test_single_query_host_abi(pkg, oracle, n, dim, metric):
    q, c = _data(42, n, dim)
    out = np.full(n, np.nan, np.float32)
    rc = pkg.diskann_bridge.batch_distances_raw(q[0], c, n, dim, metric, out)
    assert rc == 0, pkg.last_error()
    want = oracle.batch_distances(q[0], c, metric, exact=True)
    # relative to the scale of the terms (an inner product can cancel to ~0)
    scale = np.abs(q[0]).astype(np.float64) @ np.abs(c.T).astype(np.float64) if metric else None
    if metric == 0:
        assert_distances_close(out, want, f"L2 n={n} dim={dim}")
    else:
        assert (np.abs(out - want) <= 1e-4 * np.maximum(np.abs(want), 1e-2 * scale)).all()


def test_known_answers_from_reference_sql(pkg, oracle):
    import json, os
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")) as f:
        golden = json.load(f)
    for case in golden["batch_distance"]:
        qs = np.array(case["queries"], np.float32)
        c = np.array(case["candidates"], np.float32)
        qm = np.array(case["query_map"], np.uint32)
        out = np.empty(len(c), np.float32)
        rc = pkg.diskann_bridge.multi_batch_distances_raw(qs, c, qm, len(c), len(qs), c.shape[1], case["metric"], out)
        assert rc == 0
        np.testing.assert_allclose(out, np.array(case["distances"], np.float32), rtol=1e-6, atol=1e-7)


@pytest.mark.parametrize("nq,per,dim", [(10, 40, 768), (100, 40, 1536), (200, 40, 768), (3, 5, 17), (256, 128, 384)])
@pytest.mark.parametrize("metric", [0, 1])
def test_multi_query_host_abi(pkg, oracle, nq, per, dim, metric):
    q, c = _data(7, nq * per, dim, nq)
    qm = np.repeat(np.arange(nq, dtype=np.uint32), per)
    rng = np.random.default_rng(3)
    rng.shuffle(qm)  # the map need not be grouped
    out = np.empty(nq * per, np.float32)
    rc = pkg.diskann_bridge.multi_batch_distances_raw(q, c, qm, nq * per, nq, dim, metric, out)
    assert rc == 0, pkg.last_error()
    want = oracle.multi_batch_distances(q, c, qm, metric, exact=True)
    if metric == 0:
        assert_distances_close(out, want)
    else:
        scale = (np.abs(q[qm]).astype(np.float64) * np.abs(c)).sum(1)
        assert (np.abs(out - want) <= 1e-4 * np.maximum(np.abs(want), 1e-2 * scale)).all()


def test_gated_wrappers_follow_metal_ffi(pkg):
    br = pkg.diskann_bridge
    assert br.is_metal_available() is True
    q, c = _data(1, 8, 16)
    out = np.empty(8, np.float32)
    # below MIN_GPU_WORK the single-query wrapper declines (metal_ffi.rs:78-80)
    assert br.metal_batch_distances(q[0], c.ravel(), 8, 16, 0, out) is False
    q, c = _data(1, 128, 1536)
    out = np.empty(128, np.float32)
    assert br.metal_batch_distances(q[0], c.ravel(), 128, 1536, 0, out) is True
    assert np.isfinite(out).all()
    # the multi wrapper does not gate on size (metal_ffi.rs:104-106)
    qm = np.zeros(8, np.uint32)
    out = np.empty(8, np.float32)
    assert br.metal_multi_batch_distances(q, c[:8].ravel(), qm, 8, 1, 1536, 1, out) is True


def test_error_returns(pkg):
    br = pkg.diskann_bridge
    q, c = _data(1, 8, 16, nq=2)
    out = np.empty(8, np.float32)
    qm = np.array([0, 1, 2, 0, 0, 0, 0, 0], np.uint32)  # 2 >= nq
    assert br.multi_batch_distances_raw(q, c, qm, 8, 2, 16, 0, out) == -1
    assert "out of range" in pkg.last_error()


@pytest.mark.parametrize("dim", [1536, 100, 384])
@pytest.mark.parametrize("metric", [0, 1])
def test_by_id_fp32_table(pkg, oracle, dim, metric):
    rng = np.random.default_rng(44)
    table = rng.standard_normal((20000, dim)).astype(np.float32)
    t = pkg.diskann_bridge.DeviceTable.from_host(table)
    for nq, per in [(1, 64), (1, 1024), (256, 128), (5, 3)]:
        q = rng.standard_normal((nq, dim)).astype(np.float32)
        ids = rng.integers(0, len(table), nq * per).astype(np.uint32)
        qm = np.repeat(np.arange(nq, dtype=np.uint32), per)
        out = t.batch_distances_by_id(q, ids, qm if nq > 1 else None, metric)
        want = oracle.batch_distances_by_id(table, q, ids, qm, metric, exact=True)
        if metric == 0:
            assert_distances_close(out, want, f"by-id nq={nq}")
        else:
            scale = (np.abs(q[qm]).astype(np.float64) * np.abs(table[ids])).sum(1)
            assert (np.abs(out - want) <= 1e-4 * np.maximum(np.abs(want), 1e-2 * scale)).all()
    bad = np.array([len(table)], np.uint32)
    with pytest.raises(pkg.AnnCudaError):
        t.batch_distances_by_id(q[:1], bad, None, metric)
    t.close()


@pytest.mark.parametrize("dim", [384, 64, 100, 528])
@pytest.mark.parametrize("metric", [0, 1])
def test_by_id_sq8_table(pkg, oracle, dim, metric):
    rng = np.random.default_rng(45)
    x = rng.standard_normal((30000, dim)).astype(np.float32)
    mins, scale = oracle.sq8_train(x)
    codes = oracle.sq8_encode(x, mins, scale)
    t = pkg.diskann_bridge.DeviceTable.sq8_from_host(codes, mins, scale)
    for nq, per in [(1, 100), (64, 128), (7, 9)]:
        q = rng.standard_normal((nq, dim)).astype(np.float32)
        ids = rng.integers(0, len(x), nq * per).astype(np.uint32)
        qm = np.repeat(np.arange(nq, dtype=np.uint32), per)
        out = t.batch_distances_by_id(q, ids, qm if nq > 1 else None, metric)
        want = oracle.sq8_batch_distances_by_id(codes, mins, scale, q, ids, qm, metric, exact=True)
        if metric == 0:
            assert_distances_close(out, want, f"sq8 nq={nq} dim={dim}")
        else:
            xh = oracle.sq8_decode(codes[ids], mins, scale)
            sc = (np.abs(q[qm]).astype(np.float64) * np.abs(xh)).sum(1)
            assert (np.abs(out - want) <= 1e-4 * np.maximum(np.abs(want), 1e-2 * sc)).all()
    t.close()


@pytest.mark.parametrize("dim", [384, 256, 80])
def test_sq8_rows_that_almost_coincide_with_the_query(pkg, oracle, dim):
    """L2 distances far below the norms of their operands (the query is a decoded row plus a
    little noise): a kernel that expands (q - x)^2 into norms and a cross term must not lose
    them to cancellation."""
    rng = np.random.default_rng(77)
    x = rng.standard_normal((20000, dim)).astype(np.float32)
    mins, scale = oracle.sq8_train(x)
    codes = oracle.sq8_encode(x, mins, scale)
    t = pkg.diskann_bridge.DeviceTable.sq8_from_host(codes, mins, scale)
    nq, per = 64, 128
    anchor = rng.integers(0, len(x), nq).astype(np.uint32)
    noise = np.repeat(np.array([0.0, 1e-4, 1e-3, 1e-2], np.float32), nq // 4)[:, None]
    q = (oracle.sq8_decode(codes[anchor], mins, scale) +
         noise * rng.standard_normal((nq, dim))).astype(np.float32)
    ids = rng.integers(0, len(x), nq * per).astype(np.uint32)
    ids[::per] = anchor          # first candidate of every query: the row it was made from
    ids[1::per] = anchor         # and once more
    qm = np.repeat(np.arange(nq, dtype=np.uint32), per)
    out = t.batch_distances_by_id(q, ids, qm, 0)
    want = oracle.sq8_batch_distances_by_id(codes, mins, scale, q, ids, qm, 0, exact=True)
    near = want < 1e-2 * want.max()
    assert near.sum() >= nq
    err = np.abs(out - want)
    # the decoded value is formed as code * (scale / 255) + min, an ulp or two off the oracle's
    # (code / 255) * scale + min: an absolute term of that size on top of the relative bound
    assert (err <= 1e-4 * np.abs(want) + 1e-10 * dim).all(), (err / np.maximum(want, 1e-10 * dim)).max()
    t.close()


@pytest.mark.parametrize("kind", ["f32", "sq8", "sq8_odd_dim"])
@pytest.mark.parametrize("metric", [0, 1])
def test_multi_batch_launch_equals_single_launches(pkg, oracle, kind, metric):
    """Several batches of different sizes in one launch: every batch gets the result of its own
    single-batch call (same kernels; only the summation order of a row may differ)."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(3)
    dim = {"f32": 200, "sq8": 256, "sq8_odd_dim": 72}[kind]
    num = 60000
    if kind == "f32":
        table = torch.randn((num, dim), generator=g, device="cuda")
        t = pkg.diskann_bridge.DeviceTable.from_device(table)
    else:
        codes = torch.randint(0, 256, (num, dim), generator=g, device="cuda", dtype=torch.uint8)
        mins = np.linspace(-2, -1, dim).astype(np.float32)
        scale = np.linspace(2, 4, dim).astype(np.float32)
        t = pkg.diskann_bridge.DeviceTable.sq8_from_device(codes, mins, scale)
    shapes = [(64, 128), (1, 77), (33, 100), (64, 128), (5, 3)]   # (queries, rows per query)
    batches, singles = [], []
    for nq, per in shapes:
        q = torch.randn((nq, dim), generator=g, device="cuda")
        ids = torch.randint(0, num, (nq * per,), generator=g, device="cuda", dtype=torch.int32)
        qm = None if nq == 1 else torch.arange(nq, device="cuda", dtype=torch.int32).repeat_interleave(per)
        out = torch.full((nq * per,), float("nan"), device="cuda")
        batches.append((q, ids, qm, out))
        singles.append(t.batch_distances_by_id_device(q, ids, qm, metric).clone())
    t.batch_distances_by_id_device_multi(batches, metric)
    torch.cuda.synchronize()
    for (q, ids, qm, out), want in zip(batches, singles):
        # not bit for bit: a small single batch puts four warps on a row, which sums in another order
        assert torch.allclose(out, want, rtol=3e-6, atol=1e-4 if metric else 0) and torch.isfinite(out).all()
    with pytest.raises(pkg.AnnCudaError):
        t.batch_distances_by_id_device_multi([(batches[0][0], batches[0][1], None, batches[0][3])], metric)
    t.close()


def test_sq8_nearest_neighbour_known_answer(pkg, oracle):
    import json, os
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")) as f:
        case = json.load(f)["sq8"][0]
    db = np.array(case["db"], np.float32)
    qs = np.array(case["queries"], np.float32)
    mins, scale = oracle.sq8_train(db)
    t = pkg.diskann_bridge.DeviceTable.sq8_from_host(oracle.sq8_encode(db, mins, scale), mins, scale)
    ids = np.tile(np.arange(len(db), dtype=np.uint32), len(qs))
    qm = np.repeat(np.arange(len(qs), dtype=np.uint32), len(db))
    d = t.batch_distances_by_id(qs, ids, qm, 0).reshape(len(qs), -1)
    assert d.argmin(1).tolist() == case["nearest"]
    t.close()


def test_device_pointer_entry_point(pkg, oracle):
    import torch
    g = torch.Generator(device="cuda").manual_seed(9)
    table = torch.randn((50000, 256), generator=g, device="cuda")
    q = torch.randn((32, 256), generator=g, device="cuda")
    ids = torch.randint(0, 50000, (32 * 128,), generator=g, device="cuda", dtype=torch.int32)
    qm = torch.arange(32, device="cuda", dtype=torch.int32).repeat_interleave(128)
    t = pkg.diskann_bridge.DeviceTable.from_device(table)
    out = t.batch_distances_by_id_device(q, ids, qm, 0)
    torch.cuda.synchronize()
    want = oracle.batch_distances_by_id(table.cpu().numpy(), q.cpu().numpy(), ids.cpu().numpy().astype(np.uint32),
                                        qm.cpu().numpy().astype(np.uint32), 0, exact=True)
    assert_distances_close(out.cpu().numpy(), want)
    t.close()


def test_concurrent_callers(pkg, oracle):
    """The bridge is called from many threads at once (tokio workers + DuckDB threads)."""
    q, c = _data(5, 300, 257, nq=8)
    qm = (np.arange(300) % 8).astype(np.uint32)
    want = oracle.multi_batch_distances(q, c, qm, 0, exact=True)
    errors = []

    def work():
        for _ in range(20):
            out = np.empty(300, np.float32)
            rc = pkg.diskann_bridge.multi_batch_distances_raw(q, c, qm, 300, 8, 257, 0, out)
            if rc != 0 or not np.allclose(out, want, rtol=1e-4):
                errors.append(rc)

    threads = [threading.Thread(target=work) for _ in range(8)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errors
