"""The C++ plugin surface (duckdb::GetGpuBackend / CpuToGpu / faiss::Index::search /
GpuToCpu) exercised by the compiled driver, checked against the CPU oracle."""
import json
import os
import subprocess

import numpy as np
import pytest

from conftest import ROOT
from parity import assert_topk_matches

pytestmark = pytest.mark.gpu
DRIVER = os.path.join(ROOT, "duckdb-ann_b200", "backend_driver")


def _run(tmp_path, mode, d, k, metric, xb, xq, nlist=0, nprobe=0, cent=None, assign=None, devices=None, extra=(),
         storage=None):
    inp, out = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        f.write(np.array([d, len(xb), len(xq), k, metric, nlist, nprobe], np.int64).tobytes())
        f.write(xb.tobytes()); f.write(xq.tobytes())
        if cent is not None:
            f.write(cent.tobytes()); f.write(assign.astype(np.int64).tobytes())
    env = dict(os.environ)
    env.pop("ANN_CUDA_DEVICES", None)
    env.pop("ANN_CUDA_STORAGE", None)
    if storage:
        env["ANN_CUDA_STORAGE"] = storage
    if devices:
        env["ANN_CUDA_DEVICES"] = devices
    res = subprocess.run([DRIVER, mode, str(inp), str(out), *extra], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stderr
    info = json.loads(res.stdout.strip().splitlines()[-1])
    raw = open(out, "rb").read()
    nq = len(xq)
    o = 0
    D = np.frombuffer(raw, np.float32, nq * k, o).reshape(nq, k); o += nq * k * 4
    I = np.frombuffer(raw, np.int64, nq * k, o).reshape(nq, k); o += nq * k * 8
    D1 = np.frombuffer(raw, np.float32, nq * k, o).reshape(nq, k); o += nq * k * 4
    I1 = np.frombuffer(raw, np.int64, nq * k, o).reshape(nq, k)
    return info, D, I, D1, I1


def test_info():
    out = json.loads(subprocess.check_output([DRIVER, "info"], text=True))
    assert out["available"] is True and out["backend"] == "cuda" and "B200" in out["device"]  # faiss_gpu_info()


@pytest.mark.parametrize("metric", [1, 0])
def test_flat_through_gpu_backend(tmp_path, oracle, metric):
    rng = np.random.default_rng(42)
    xb = rng.uniform(-1, 1, (3000, 96)).astype(np.float32)
    xq = rng.uniform(-1, 1, (12, 96)).astype(np.float32)
    info, D, I, D1, I1 = _run(tmp_path, "flat", 96, 7, metric, xb, xq)
    assert info == {"backend": "cuda", "roundtrip_ok": 1, "rejects_unknown": 1, "async_ok": 1, "shards": 1}
    Dref, Iref = oracle.flat_search(xb, xq, 7, metric)
    assert_topk_matches(oracle, xb, xq, metric, D, I, Dref, Iref, "batch")
    assert_topk_matches(oracle, xb, xq, metric, D1, I1, Dref, Iref, "one query per call")


@pytest.mark.parametrize("kind", ["f16", "bf16"])
@pytest.mark.parametrize("metric", [1, 0])
def test_reduced_precision_storage_through_the_cpp_class(tmp_path, oracle, kind, metric):
    """faiss_cuda::CudaIndexFlat(device, d, metric, StorageType) (the extended constructor of
    faiss-metal/include/faiss-metal/MetalIndexFlat.h:60): the index answers for the rounded rows."""
    rng = np.random.default_rng(42)
    xb = rng.uniform(-1, 1, (3000, 96)).astype(np.float32)
    xq = rng.uniform(-1, 1, (12, 96)).astype(np.float32)
    info, D, I, D1, I1 = _run(tmp_path, "storage", 96, 7, metric, xb, xq, extra=(kind,))
    assert info["backend"] == "cuda" and info["flags_ok"] == 1 and info["roundtrip_ok"] == 1
    assert 0 < info["worst_rounding"] < (2e-3 if kind == "f16" else 8e-3)   # test_metal_flat.mm:262-268
    xr = oracle.round_storage(xb, kind)
    Dref, Iref = oracle.flat_search(xr, xq, 7, metric)
    assert_topk_matches(oracle, xr, xq, metric, D, I, Dref, Iref, f"{kind} batch")
    assert_topk_matches(oracle, xr, xq, metric, D1, I1, Dref, Iref, f"{kind} one query per call")


@pytest.mark.parametrize("kind", ["f16", "bf16"])
def test_reduced_precision_storage_chosen_by_the_environment(tmp_path, oracle, kind):
    """ANN_CUDA_STORAGE=f16|bf16: GetGpuBackend().CpuToGpu keeps a flat index's rows in 16 bits without a change
    to the caller; the searches answer for the rounded rows, and GpuToCpu hands those out (so the round trip is
    no longer bit for bit - the extension keeps its own fp32 CPU index, src/faiss_index.cpp:108-149)."""
    rng = np.random.default_rng(42)
    xb = rng.uniform(-1, 1, (3000, 96)).astype(np.float32)
    xq = rng.uniform(-1, 1, (12, 96)).astype(np.float32)
    info, D, I, D1, I1 = _run(tmp_path, "flat", 96, 7, 1, xb, xq, storage=kind)
    assert info["backend"] == "cuda" and info["roundtrip_ok"] == 0 and info["async_ok"] == 1
    xr = oracle.round_storage(xb, kind)
    Dref, Iref = oracle.flat_search(xr, xq, 7, 1)
    assert_topk_matches(oracle, xr, xq, 1, D, I, Dref, Iref, f"{kind} by environment, batch")
    assert_topk_matches(oracle, xr, xq, 1, D1, I1, Dref, Iref, f"{kind} by environment, one query per call")


def test_ivf_through_gpu_backend(tmp_path, oracle):
    rng = np.random.default_rng(43)
    xb = rng.uniform(-1, 1, (2500, 64)).astype(np.float32)
    xq = rng.uniform(-1, 1, (9, 64)).astype(np.float32)
    cent = oracle.kmeans(xb, 12, niter=5, seed=2)
    assign = oracle.ivf_assign(xb, cent, oracle.METRIC_L2)
    off, rows = oracle.lists_from_assign(assign, 12)
    info, D, I, D1, I1 = _run(tmp_path, "ivf", 64, 6, 1, xb, xq, 12, 12, cent, assign)
    assert info["roundtrip_ok"] == 1
    Dref, Iref = oracle.ivf_search(xb, cent, off, rows, xq, 6, 12, oracle.METRIC_L2)
    assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, "ivf batch")
    assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D1, I1, Dref, Iref, "ivf one query per call")


def _device_lists():
    """Device lists for the sharded runs: three shards on device 0 always (the same code path as
    one shard per GPU), and one shard on each of the first two GPUs where the box has them."""
    import torch
    lists = ["0,0,0"]
    if torch.cuda.device_count() >= 2:
        lists.append("0,1")
    return lists


@pytest.mark.parametrize("metric", [1, 0])
def test_flat_sharded_behind_the_plugin(tmp_path, oracle, metric):
    """ANN_CUDA_DEVICES with more than one entry: CpuToGpu hands out ONE index object spread over the
    devices, and the process that owns it searches all of them through faiss::Index::search
    (src/faiss_index.cpp:108-149, 729-737).  Same answers as on one device, bit for bit."""
    rng = np.random.default_rng(42)
    xb = rng.uniform(-1, 1, (3001, 96)).astype(np.float32)
    xq = rng.uniform(-1, 1, (12, 96)).astype(np.float32)
    _, D0, I0, _, _ = _run(tmp_path, "flat", 96, 7, metric, xb, xq)
    Dref, Iref = oracle.flat_search(xb, xq, 7, metric)
    for devices in _device_lists():
        info, D, I, D1, I1 = _run(tmp_path, "flat", 96, 7, metric, xb, xq, devices=devices)
        assert info["shards"] == len(devices.split(",")) and info["roundtrip_ok"] == 1, (devices, info)
        np.testing.assert_array_equal(I, I0)
        np.testing.assert_array_equal(D, D0)
        assert_topk_matches(oracle, xb, xq, metric, D, I, Dref, Iref, f"sharded over {devices}")
        assert_topk_matches(oracle, xb, xq, metric, D1, I1, Dref, Iref, f"sharded over {devices}, one query per call")


def test_ivf_sharded_behind_the_plugin(tmp_path, oracle):
    rng = np.random.default_rng(43)
    xb = rng.uniform(-1, 1, (2500, 64)).astype(np.float32)
    xq = rng.uniform(-1, 1, (9, 64)).astype(np.float32)
    cent = oracle.kmeans(xb, 12, niter=5, seed=2)
    assign = oracle.ivf_assign(xb, cent, oracle.METRIC_L2)
    off, rows = oracle.lists_from_assign(assign, 12)
    Dref, Iref = oracle.ivf_search(xb, cent, off, rows, xq, 6, 5, oracle.METRIC_L2)
    for devices in _device_lists():
        info, D, I, D1, I1 = _run(tmp_path, "ivf", 64, 6, 1, xb, xq, 12, 5, cent, assign, devices=devices)
        assert info["shards"] == len(devices.split(",")) and info["roundtrip_ok"] == 1, (devices, info)
        assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D, I, Dref, Iref, f"ivf sharded over {devices}")
        assert_topk_matches(oracle, xb, xq, oracle.METRIC_L2, D1, I1, Dref, Iref, f"ivf sharded over {devices}, one per call")


@pytest.mark.parametrize("devices", [None, "0,0"])
def test_faiss_index_glue(tmp_path, oracle, devices):
    """The FaissIndex glue (EnsureGpuIndex / InvalidateGpuIndex / Search, src/faiss_index.cpp:108-153,
    708-762) over the CUDA backend: an append drops the GPU copy and the NEXT search uploads it
    again; deleted labels are skipped and k results still come back; SearchBatch answers all
    queries with one search(n, ...) call and agrees with one Search per query."""
    rng = np.random.default_rng(8)
    d, n, n0, nq, k = 128, 4000, 3000, 11, 6
    xb = rng.uniform(-1, 1, (n, d)).astype(np.float32)
    xq = rng.uniform(-1, 1, (nq, d)).astype(np.float32)
    xq[0] = xb[3600] + np.float32(1e-3)        # its best hit arrives with the append
    Dfull, Ifull = oracle.flat_search(xb, xq, k + 4, oracle.METRIC_L2)
    tomb = np.array([Ifull[1, 0], Ifull[2, 1], Ifull[2, 2], 3500], np.int64)   # best hits of some queries
    inp, out = tmp_path / "in.bin", tmp_path / "out.bin"
    with open(inp, "wb") as f:
        f.write(np.array([d, n, nq, k, 1, n0, len(tomb)], np.int64).tobytes())
        f.write(xb.tobytes()); f.write(xq.tobytes()); f.write(tomb.tobytes())
    env = dict(os.environ)
    env.pop("ANN_CUDA_DEVICES", None)
    env.pop("ANN_CUDA_STORAGE", None)
    if devices:
        env["ANN_CUDA_DEVICES"] = devices
    res = subprocess.run([DRIVER, "glue", str(inp), str(out), "auto"], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0, res.stderr
    info = json.loads(res.stdout.strip().splitlines()[-1])
    assert info == {"on_gpu_after_build": 1, "on_gpu_after_append": 0, "on_gpu_at_end": 1, "gpu_uploads": 2,
                    "wrong_dimension_is_empty": 1}
    raw = np.frombuffer(open(out, "rb").read(), np.uint8)
    blocks, o = [], 0
    for _ in range(4):
        D = raw[o:o + nq * k * 4].view(np.float32).reshape(nq, k); o += nq * k * 4
        I = raw[o:o + nq * k * 8].view(np.int64).reshape(nq, k); o += nq * k * 8
        blocks.append((D, I))
    # before the append: the first n0 rows
    Dref, Iref = oracle.flat_search(xb[:n0], xq, k, oracle.METRIC_L2)
    for D, I in blocks[:2]:
        assert_topk_matches(oracle, xb[:n0], xq, oracle.METRIC_L2, D, I, Dref, Iref, "glue, before the append")
    np.testing.assert_array_equal(blocks[0][1], blocks[1][1])
    # after: all rows, minus the deleted labels
    Dw = np.empty((nq, k), np.float32); Iw = np.empty((nq, k), np.int64)
    for q in range(nq):
        keep = [j for j in range(k + 4) if Ifull[q, j] not in set(tomb.tolist())][:k]
        Dw[q], Iw[q] = Dfull[q, keep], Ifull[q, keep]
    for D, I in blocks[2:]:
        assert not np.isin(I, tomb).any()
        np.testing.assert_array_equal(I, Iw)
        np.testing.assert_allclose(D, Dw, rtol=1e-4)
    np.testing.assert_array_equal(blocks[2][0], blocks[3][0])
    assert blocks[2][1][0, 0] == 3600 and 3600 not in blocks[0][1][0]
