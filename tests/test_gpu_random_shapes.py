"""Seeded random shapes: every tensor-core path of the library against its own exact-fp32 scan kernels.

The scan kernels (`ann_cuda_set_flat_kernel("simt")`: one warp per (query, row chunk / inverted list), direct-form
fp32, no tensor cores, no bands) are checked against the CPU oracle shape by shape in the other test files; here
they stand in for it on shapes too many and too large to search on the CPU: dimensions that are not multiples of
anything, one query and ragged query tiles, k on both sides of every switch between selection modes (16 / 17,
160, 224 / 225, 256), stores far from the origin or of large magnitude, 16-bit row storage, IVFFlat with
nprobe = 1 .. nlist.  Same acceptance rule as `parity.py`: distances within 1e-4 (of the query's largest
distance: the two paths sum in different orders), identical id sets except for tolerance ties at the k-th place."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _same_answers(D, I, De, Ie):
    for q in range(D.shape[0]):
        v = Ie[q] >= 0
        scale = float(np.abs(De[q][v]).max()) if v.any() else 1.0
        if int((I[q] >= 0).sum()) != int(v.sum()):
            return f"query {q}: {int((I[q] >= 0).sum())} results, the exact scan has {int(v.sum())}"
        if not np.allclose(np.sort(D[q][v]), np.sort(De[q][v]), rtol=2e-4, atol=1e-5 * scale):
            return f"query {q}: distances differ"
        diff = set(I[q].tolist()) ^ set(Ie[q].tolist())
        if diff:
            kth = float(De[q][v][-1])
            dist = {int(i): float(d) for i, d in zip(I[q], D[q])}
            dist.update({int(i): float(d) for i, d in zip(Ie[q], De[q])})
            for i in diff:
                if abs(dist[i] - kth) > 2e-4 * abs(kth) + 1e-5 * scale:
                    return f"query {q}: id {i} (distance {dist[i]}) is not a tie with the k-th ({kth})"
    return None


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_tensor_core_paths_against_the_exact_scan(pkg, seed):
    lib = pkg.lib()
    rng = np.random.default_rng(seed)
    problems = []
    for case in range(14):
        kind = str(rng.choice(["flat", "flat", "flat16", "ivf"]))
        d = int(rng.choice([3, 17, 32, 64, 100, 128, 384, 768, 1000]))
        metric = int(rng.choice([0, 1]))
        nq = int(rng.choice([1, 5, 127, 128, 129, 300, 700]))
        k = int(rng.choice([1, 5, 10, 16, 17, 50, 100, 160, 200, 224, 225, 300, 600]))
        scale = float(rng.choice([1.0, 1.0, 20.0]))
        shift = float(rng.choice([0.0, 0.0, 5.0]))
        if kind == "ivf":
            n, nlist = int(rng.choice([3000, 20000, 60000])), int(rng.choice([8, 64, 200]))
            nprobe, k = int(rng.choice([1, 4, 8, nlist])), min(k, 300)
        else:
            n = int(rng.choice([200, 3000, 40000, 150000, 400000]))
            if d >= 768:
                n = min(n, 150000)
        xb = (rng.standard_normal((n, d)) * scale + shift).astype(np.float32)
        xq = (rng.standard_normal((nq, d)) * scale + shift).astype(np.float32)
        m = pkg.METRIC_L2 if metric == 1 else pkg.METRIC_INNER_PRODUCT
        what = f"{kind} n={n} d={d} nq={nq} k={k} metric={metric} scale={scale} shift={shift}"
        screened = bool(rng.integers(0, 2))
        try:
            if kind == "ivf":
                what += f" nlist={nlist} nprobe={nprobe}"
                idx = pkg.CudaIndexIVFFlat(d, nlist, m)
                idx.train(xb)
                idx.add(xb)
                idx.setNprobe(nprobe)
            elif kind == "flat16":
                storage = int(rng.choice([pkg.STORAGE_F16, pkg.STORAGE_BF16]))
                what += f" storage={storage}"
                idx = pkg.CudaIndexFlat(d, m, 0, storage)
                idx.add(xb)
            else:
                idx = pkg.CudaIndexFlat(d, m)
                idx.add(xb)
                if screened:
                    what += " screening forced"
                    assert lib.ann_cuda_set_flat_kernel(b"tcgen05-screened") == 0
            D, I = idx.search(xq, k)
            assert lib.ann_cuda_set_flat_kernel(b"simt") == 0
            De, Ie = idx.search(xq, k)
            idx.close()
        finally:
            lib.ann_cuda_set_flat_kernel(b"tcgen05")
        bad = _same_answers(D, I, De, Ie)
        if bad:
            problems.append(f"{what}: {bad}")
    assert not problems, "\n".join(problems)
