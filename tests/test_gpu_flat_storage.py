"""Reduced-precision row storage of the flat index (fp16 / bf16), through the C ABI.

The reference's form of the feature: faiss-metal/include/faiss-metal/MetalIndexFlat.h:38-60 (StorageType,
queries stay fp32), rows rounded when they are added (faiss-metal/src/MetalIndexFlat.mm:211-236), its own
test (faiss-metal/tests/test_metal_flat.mm:225-270): uniform(-1, 1) rows, 1000 x 64, 10 queries, k = 5,
the fp16 index against the UNROUNDED CPU index with tolerance 5e-2 and a top-1 match, reconstruct within
2e-3 of the row that was added.

Here the contract is tighter: the index answers for the rows it keeps - the rounded ones - to the same
1e-4 as the fp32 index, so the oracle searches `oracle.round_storage(xb)`.  The reference's looser check
against the unrounded rows is repeated as well."""
import numpy as np
import pytest

from parity import assert_topk_matches

pytestmark = pytest.mark.gpu

KINDS = [("f16", 1), ("bf16", 2)]


def _metric(pkg, name):
    return pkg.METRIC_L2 if name == "L2" else pkg.METRIC_INNER_PRODUCT


@pytest.mark.parametrize("kind,storage", KINDS)
@pytest.mark.parametrize("metric_name", ["L2", "IP"])
@pytest.mark.parametrize("shape", [(1000, 10, 64, 5), (5000, 7, 128, 33), (70000, 130, 96, 10), (300000, 256, 64, 100),
                                   (400000, 256, 64, 50), (200, 3, 32, 4), (4099, 5, 384, 300)],
                         ids=lambda s: "x".join(map(str, s)))
def test_search_answers_for_the_rounded_rows(pkg, oracle, kind, storage, metric_name, shape):
    nv, nq, d, k = shape
    rng = np.random.default_rng(42)
    xb = rng.uniform(-1, 1, (nv, d)).astype(np.float32)
    xq = rng.uniform(-1, 1, (nq, d)).astype(np.float32)
    xr = oracle.round_storage(xb, kind)
    om = oracle.METRIC_L2 if metric_name == "L2" else oracle.METRIC_IP
    idx = pkg.CudaIndexFlat(d, _metric(pkg, metric_name), 0, storage)
    assert idx.storage == storage
    idx.add(xb[: nv // 2])
    idx.add(xb[nv // 2:])          # growth copies the 16-bit plane
    assert idx.ntotal == nv
    D, I = idx.search(xq, k)
    Dref, Iref = oracle.flat_search(xr, xq, k, om)
    assert_topk_matches(oracle, xr, xq, om, D, I, Dref, Iref, f"{kind} storage, {metric_name}, {shape}")
    # the entry points that do not wait give the same answer
    import torch
    Dd, Id = idx.search_device(torch.from_numpy(xq).cuda(), k)
    idx.search_status()
    np.testing.assert_array_equal(Id.cpu().numpy(), I)
    np.testing.assert_array_equal(Dd.cpu().numpy(), D)
    # reconstruct / get_rows: the rounded rows, bit for bit (test_metal_flat.mm:262-268 allows 2e-3 for fp16)
    for key in (0, nv // 2, nv - 1):
        np.testing.assert_array_equal(idx.reconstruct(key), xr[key])
    np.testing.assert_array_equal(idx.get_rows(3, min(50, nv - 3)), xr[3:3 + min(50, nv - 3)])
    if kind == "f16":
        assert np.abs(idx.reconstruct(0) - xb[0]).max() < 2e-3
    idx.close()


@pytest.mark.parametrize("kind,storage", KINDS)
def test_the_reference_check_against_the_unrounded_rows(pkg, oracle, kind, storage):
    """test_metal_flat.mm:225-261: 1000 x 64, 10 queries, k = 5; distances within 5e-2 of the fp32 CPU
    index, the nearest neighbour the same."""
    rng = np.random.default_rng(42)
    xb = rng.uniform(-1, 1, (1000, 64)).astype(np.float32)
    xq = rng.uniform(-1, 1, (10, 64)).astype(np.float32)
    idx = pkg.CudaIndexFlat(64, pkg.METRIC_L2, 0, storage)
    idx.add(xb)
    D, I = idx.search(xq, 5)
    Dref, Iref = oracle.flat_search(xb, xq, 5, oracle.METRIC_L2)
    np.testing.assert_array_equal(I[:, 0], Iref[:, 0])
    np.testing.assert_allclose(D, Dref, rtol=5e-2)
    idx.close()


@pytest.mark.parametrize("kind,storage", KINDS)
def test_a_query_the_16_bit_type_cannot_hold_goes_to_the_exact_scan(pkg, oracle, kind, storage):
    """fp16 ends at 65504: a query element beyond it cannot be fed to the 16-bit tensor-core product.  The
    block is then answered by the exact scan, which reads the query in fp32 (bf16 has the range of fp32 and
    stays on the tensor cores).  The rows themselves stay within range."""
    rng = np.random.default_rng(9)
    xb = rng.uniform(-1, 1, (20000, 64)).astype(np.float32)
    xq = rng.uniform(-1, 1, (6, 64)).astype(np.float32)
    xq[2] *= 3.0e5
    xr = oracle.round_storage(xb, kind)
    idx = pkg.CudaIndexFlat(64, pkg.METRIC_INNER_PRODUCT, 0, storage)
    idx.add(xb)
    before = pkg.lib().ann_cuda_screen_fallbacks()
    D, I = idx.search(xq, 10)
    Dref, Iref = oracle.flat_search(xr, xq, 10, oracle.METRIC_IP)
    assert_topk_matches(oracle, xr, xq, oracle.METRIC_IP, D, I, Dref, Iref, f"{kind}: query beyond the fp16 range")
    if kind == "f16":
        assert pkg.lib().ann_cuda_screen_fallbacks() > before
    import torch
    Dd, Id = idx.search_device(torch.from_numpy(xq).cuda(), 10)
    idx.search_status()
    np.testing.assert_array_equal(Id.cpu().numpy(), I)
    idx.close()


@pytest.mark.parametrize("kind,storage", KINDS)
def test_near_ties_closer_than_one_16_bit_part_resolves(pkg, oracle, kind, storage):
    """Rows whose keys differ by far less than the rounding of a single 16-bit query part: the first tier's
    band overflows, the two-part product (or the exact scan) settles it, and the answer is still the
    oracle's."""
    rng = np.random.default_rng(3)
    d, n_far, n_near = 64, 30000, 600
    q = rng.standard_normal(d)
    q /= np.linalg.norm(q)
    u = rng.standard_normal((n_near, d))
    u /= np.linalg.norm(u, axis=1, keepdims=True)
    near = q[None, :] + np.sqrt(0.5 + 2e-5 * np.arange(n_near))[:, None] * u
    xb = np.concatenate([rng.standard_normal((n_far, d)), near]).astype(np.float32)
    xb = xb[np.random.default_rng(4).permutation(len(xb))]
    xq = q[None, :].astype(np.float32)
    xr = oracle.round_storage(xb, kind)
    idx = pkg.CudaIndexFlat(d, pkg.METRIC_L2, 0, storage)
    idx.add(xb)
    D, I = idx.search(xq, 20)
    Dref, Iref = oracle.flat_search(xr, xq, 20, oracle.METRIC_L2)
    assert_topk_matches(oracle, xr, xq, oracle.METRIC_L2, D, I, Dref, Iref, f"{kind}: dense near ties")
    idx.close()


def test_storage_is_a_flat_index_option_only(pkg):
    lib = pkg.lib()
    import ctypes as C
    h = C.c_void_p()
    assert lib.ann_cuda_flat_create_storage(0, 16, pkg.METRIC_L2, 7, C.byref(h)) != 0
    idx = pkg.CudaIndexFlat(16, pkg.METRIC_L2)
    assert idx.storage == pkg.STORAGE_F32
    idx.close()
