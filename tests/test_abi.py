"""CPU checks of the drop-in boundary: the shared library builds, loads, and
exports exactly the symbols include/*.h declare (no compute without a GPU)."""
import os
import re
import subprocess

import pytest

from conftest import ROOT, load_package


def _declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"\b((?:ann_cuda|diskann_metal|diskann_cuda)_[a-z0-9_]+)\s*\(", text)
    return sorted(set(names))


def test_library_exports_every_declared_symbol():
    pkg = load_package()
    lib = pkg.lib()
    declared = _declared("ann_cuda.h") + _declared("cuda_diskann_bridge.h")
    assert len(declared) > 40
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
    assert sorted(pkg.SIGNATURES) == sorted(declared), "ctypes signature table and headers disagree"


def test_reference_symbol_names_are_kept():
    # the three names rust_lib/src/metal_ffi.rs:10-30 binds
    names = _declared("cuda_diskann_bridge.h")
    for n in ("diskann_metal_available", "diskann_metal_batch_distances", "diskann_metal_multi_batch_distances"):
        assert n in names


def test_cpp_symbols_exported():
    lib = os.path.join(ROOT, "duckdb-ann_b200", "libann_cuda.so")
    out = subprocess.check_output(["nm", "-D", "--defined-only", "-C", lib], text=True)
    assert "duckdb::GetGpuBackend()" in out
    assert "faiss_cuda::index_cpu_to_cuda(" in out
    assert "faiss_cuda::CudaIndexIVFFlat::search(" in out


def test_fails_loudly_without_a_device():
    pkg = load_package()
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    assert pkg.get_gpu_backend().IsAvailable() is False
    assert pkg.get_gpu_backend().BackendName() == "cuda"
    with pytest.raises(pkg.AnnCudaError):
        pkg.CudaIndexFlat(8)
    # the bridge reports unavailable and returns -1, as the reference's stub does
    # (src/metal_diskann_stub.cpp:9-24): callers then use their own CPU loop
    assert pkg.diskann_bridge.is_metal_available() is False
    import numpy as np
    out = np.zeros(4, np.float32)
    assert pkg.diskann_bridge.batch_distances_raw(np.zeros(8, np.float32), np.zeros(32, np.float32), 4, 8, 0, out) == -1


def test_backend_driver_reports_backend():
    drv = os.path.join(ROOT, "duckdb-ann_b200", "backend_driver")
    out = subprocess.check_output([drv, "info"], text=True)
    assert '"backend": "cuda"' in out


def test_bridge_argument_validation_needs_no_device():
    pkg = load_package()
    import numpy as np
    out = np.zeros(4, np.float32)
    br = pkg.diskann_bridge
    # null pointers / non-positive sizes -> -1 (src/metal_diskann_bridge.mm:157-159, 258-260)
    assert br.batch_distances_raw(None, np.zeros(32, np.float32), 4, 8, 0, out) == -1
    assert br.batch_distances_raw(np.zeros(8, np.float32), np.zeros(32, np.float32), 0, 8, 0, out) == -1
    assert br.batch_distances_raw(np.zeros(8, np.float32), np.zeros(32, np.float32), 4, -1, 0, out) == -1
    assert br.multi_batch_distances_raw(np.zeros(8, np.float32), np.zeros(32, np.float32), None, 4, 1, 8, 0, out) == -1
    # metal_ffi.rs:75-77: nothing to compute -> true without calling
    assert br.metal_batch_distances(np.zeros(8, np.float32), np.zeros(0, np.float32), 0, 8, 0, out) is True
