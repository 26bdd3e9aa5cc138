"""The CPU oracle against the reference's own known answers (tests/golden) and
against itself (float-order path vs double path, fast paths vs exact paths)."""
import json
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_known_answers.json")


@pytest.fixture(scope="module")
def golden():
    with open(GOLDEN) as f:
        return json.load(f)


def _metric(o, name):
    return o.METRIC_L2 if name == "L2" else o.METRIC_IP


def test_flat_known_answers(oracle, golden):
    for case in golden["flat"]:
        db = np.array(case["db"], np.float32)
        q = np.array([case["query"]], np.float32)
        D, I = oracle.flat_search(db, q, case["k"], _metric(oracle, case["metric"]))
        # The SQL results are printed fp32 values.  FAISS's own summation order is not
        # in the reference tree, and its 0.020000001 is 2 fp32 ulps from the
        # double-accumulated 0.020000005: compare at 1e-6 relative, far inside the
        # 1e-4 contract.
        np.testing.assert_allclose(D[0], np.array(case["distances"], np.float32), rtol=1e-6, atol=0,
                                   err_msg=case["source"])
        n = len(case["labels_first"])
        assert I[0, :n].tolist() == case["labels_first"], case["source"]


def test_ivfflat_known_answers(oracle, golden):
    for case in golden["ivfflat"]:
        db = np.array(case["db"], np.float32)
        q = np.array([case["query"]], np.float32)
        m = _metric(oracle, case["metric"])
        cent = oracle.kmeans(db, case["nlist"], niter=10, seed=7)
        off, rows = oracle.lists_from_assign(oracle.ivf_assign(db, cent, m), case["nlist"])
        D, I = oracle.ivf_search(db, cent, off, rows, q, case["k"], case["nprobe"], m)
        assert I[0].tolist() == case["labels"], case["source"]
        assert D[0, 0] == np.float32(case["first_distance"])
        Df, If = oracle.ivf_search(db, cent, off, rows, q, case["k"], case["nprobe"], m, fast=True)
        assert If[0].tolist() == case["labels"]


def test_batch_known_answers(oracle, golden):
    for case in golden["batch_distance"]:
        qs = np.array(case["queries"], np.float32)
        c = np.array(case["candidates"], np.float32)
        qm = np.array(case["query_map"], np.uint32)
        want = np.array(case["distances"], np.float32)
        for exact in (False, True):
            got = oracle.multi_batch_distances(qs, c, qm, case["metric"], exact=exact)
            np.testing.assert_allclose(got, want, rtol=1e-6, atol=0, err_msg=case["source"])
        if len(qs) == 1:
            got = oracle.batch_distances(qs[0], c, case["metric"])
            np.testing.assert_allclose(got, want, rtol=1e-6, atol=0)


def test_sq8_known_answers(oracle, golden):
    for case in golden["sq8"]:
        db = np.array(case["db"], np.float32)
        qs = np.array(case["queries"], np.float32)
        mins, scale = oracle.sq8_train(db)
        codes = oracle.sq8_encode(db, mins, scale)
        ids = np.tile(np.arange(len(db), dtype=np.uint32), len(qs))
        qm = np.repeat(np.arange(len(qs), dtype=np.uint32), len(db))
        d = oracle.sq8_batch_distances_by_id(codes, mins, scale, qs, ids, qm, oracle.BATCH_L2).reshape(len(qs), -1)
        assert d.argmin(1).tolist() == case["nearest"], case["source"]
        # every value here is a multiple of 1/4 of the range: the codes decode exactly
        np.testing.assert_allclose(oracle.sq8_decode(codes, mins, scale), db, atol=2e-3)


def test_batch_rejects_bad_arguments(oracle):
    q = np.zeros(4, np.float32)
    with pytest.raises(ValueError):
        oracle.batch_distances(q, np.zeros((0, 4), np.float32), 0)  # n <= 0 -> -1 (bridge.mm:157-159)
    with pytest.raises(ValueError):
        oracle.multi_batch_distances(np.zeros((2, 4), np.float32), np.zeros((3, 4), np.float32),
                                     np.array([0, 1, 2], np.uint32), 0)  # query_map out of range


def test_float_order_matches_numpy_reference_loop(oracle):
    rng = np.random.default_rng(5)
    q = rng.standard_normal(97).astype(np.float32)
    c = rng.standard_normal((13, 97)).astype(np.float32)
    got = oracle.batch_distances(q, c, 0)
    # the same sequential float loop, in numpy scalars
    want = []
    for row in c:
        s = np.float32(0)
        for a, b in zip(q, row):
            df = np.float32(a - b)
            s = np.float32(s + np.float32(df * df))
        want.append(s)
    assert got.tolist() == np.array(want, np.float32).tolist()
    got64 = oracle.batch_distances(q, c, 0, exact=True)
    np.testing.assert_allclose(got, got64, rtol=1e-5)
    ip = oracle.batch_distances(q, c, 1, exact=True)
    np.testing.assert_allclose(ip, -(c.astype(np.float64) @ q.astype(np.float64)), rtol=1e-6)


def test_sq8_roundtrip_formula(oracle):
    rng = np.random.default_rng(11)
    x = rng.standard_normal((500, 24)).astype(np.float32)
    x[:, 3] = 0.25  # constant dimension: range 0 -> scale 1.0 (provider.rs:190-193)
    mins, scale = oracle.sq8_train(x)
    assert scale[3] == 1.0 and mins[3] == np.float32(0.25)
    np.testing.assert_array_equal(mins, x.min(0))
    codes = oracle.sq8_encode(x, mins, scale)
    want = np.clip(np.floor(((x - mins) / scale) * np.float32(255.0) + np.float32(0.5)), 0, 255).astype(np.uint8)
    assert (codes != want).mean() < 1e-3  # floor(v+.5) differs from round() only at representable ties
    xh = oracle.sq8_decode(codes, mins, scale)
    assert np.abs(xh - x).max() <= (scale.max() / 255.0) * 0.5 + 1e-6
    ids = np.arange(500, dtype=np.uint32)
    q = rng.standard_normal((1, 24)).astype(np.float32)
    d = oracle.sq8_batch_distances_by_id(codes, mins, scale, q, ids, None, 0, exact=True)
    np.testing.assert_allclose(d, ((xh.astype(np.float64) - q.astype(np.float64)) ** 2).sum(1), rtol=1e-6)


@pytest.mark.parametrize("metric_name", ["L2", "IP"])
def test_flat_matches_numpy_bruteforce(oracle, metric_name):
    rng = np.random.default_rng(42)
    xb = rng.uniform(-1, 1, (1000, 32)).astype(np.float32)  # shapes of faiss-metal/tests/test_metal_flat.mm:489-508
    xq = rng.uniform(-1, 1, (10, 32)).astype(np.float32)
    m = _metric(oracle, metric_name)
    D, I = oracle.flat_search(xb, xq, 5, m)
    b64, q64 = xb.astype(np.float64), xq.astype(np.float64)
    full = ((q64[:, None, :] - b64[None]) ** 2).sum(-1) if metric_name == "L2" else -(q64 @ b64.T)
    want = np.argsort(full, axis=1, kind="stable")[:, :5]
    np.testing.assert_array_equal(I, want)
    np.testing.assert_allclose(np.abs(D), np.abs(np.take_along_axis(full, want, 1)), rtol=1e-6)
    Db, Ib = oracle.flat_search_blas(xb, xq, 5, m)
    np.testing.assert_array_equal(Ib, want)
    np.testing.assert_allclose(Db, D, rtol=1e-4, atol=1e-5)
    one = oracle.all_distances(xb, xq[0], m)
    np.testing.assert_allclose(np.sort(one if metric_name == "L2" else -one)[:5], np.abs(D[0]) if metric_name == "L2"
                               else -D[0], rtol=1e-6)


def test_flat_edge_cases(oracle):
    xb = np.eye(3, dtype=np.float32)
    q = np.array([[1, 0, 0]], np.float32)
    D, I = oracle.flat_search(xb, q, 5, oracle.METRIC_L2)  # k > ntotal -> (+inf, -1) padding (MetalIndexFlat.mm:363-367)
    assert I[0].tolist()[3:] == [-1, -1] and np.isinf(D[0, 3:]).all() and (D[0, 3:] > 0).all()
    D, I = oracle.flat_search(xb, q, 5, oracle.METRIC_IP)
    assert I[0].tolist()[3:] == [-1, -1] and (D[0, 3:] == -np.inf).all()
    D, I = oracle.flat_search(np.zeros((0, 3), np.float32), q, 2, oracle.METRIC_L2)  # empty index (:303-309)
    assert I.tolist() == [[-1, -1]] and np.isinf(D).all()


def test_ivf_full_probe_equals_flat(oracle):
    rng = np.random.default_rng(123)
    xb = rng.uniform(-1, 1, (2000, 64)).astype(np.float32)  # faiss-metal/tests/test_metal_ivfflat.mm:31-36
    xq = rng.uniform(-1, 1, (10, 64)).astype(np.float32)
    cent = oracle.kmeans(xb, 16, niter=5, seed=1)
    assign = oracle.ivf_assign(xb, cent, oracle.METRIC_L2)
    off, rows = oracle.lists_from_assign(assign, 16)
    assert off[-1] == 2000 and sorted(rows.tolist()) == list(range(2000))
    Df, If = oracle.flat_search(xb, xq, 5, oracle.METRIC_L2)
    D, I = oracle.ivf_search(xb, cent, off, rows, xq, 5, 16, oracle.METRIC_L2)
    np.testing.assert_array_equal(I, If)
    np.testing.assert_array_equal(D, Df)
    D4, I4, probes = oracle.ivf_search(xb, cent, off, rows, xq, 5, 4, oracle.METRIC_L2, return_probes=True)
    Dg, Ig = oracle.ivf_search_given_probes(xb, off, rows, xq, 5, probes, oracle.METRIC_L2)
    np.testing.assert_array_equal(I4, Ig)
    np.testing.assert_array_equal(D4, Dg)
    Dq, Iq = oracle.ivf_search(xb, cent, off, rows, xq, 5, 4, oracle.METRIC_L2, fast=True)
    assert (Iq == I4).mean() > 0.98
