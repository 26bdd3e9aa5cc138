"""B200-native GPU search path of duckdb-ann: Python host side over the C ABI.

The product is `libann_cuda.so` (hand-written CUDA for sm_100a, C ABI declared in
`include/ann_cuda.h` and `include/cuda_diskann_bridge.h`).  This package is the
thin host layer the tests and the benchmark use:

  * `faiss_like`  -- `CudaIndexFlat`, `CudaIndexIVFFlat`, `get_gpu_backend()`:
                     the reference's `faiss::Index`-shaped classes and GpuBackend
                     plugin (src/include/gpu_backend.hpp:12-33), same method names;
  * `diskann_bridge` -- the batch-distance calls of rust_lib/src/metal_ffi.rs:67-141
                     plus the device-resident table entry points;
  * `sharded`     -- row / inverted-list sharding over torch.distributed.

There is no CPU implementation behind any of it: if the shared library is
missing or no sm_100 device is present, calls raise.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("ANN_CUDA_LIB") or os.path.join(HERE, "libann_cuda.so")

_lib = None


class AnnCudaError(RuntimeError):
    pass


def lib() -> C.CDLL:
    """Loads the CUDA library; raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise AnnCudaError(f"{LIB_PATH} is missing: build it with `python duckdb-ann_b200/build.py` "
                               "(there is no CPU fallback)")
        _lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
        _declare(_lib)
    return _lib


# Every exported symbol with its signature; tests check the list against include/*.h.
_P = C.c_void_p
_I64 = C.c_int64
SIGNATURES = {
    # include/ann_cuda.h
    "ann_cuda_last_error": (C.c_char_p, []),
    "ann_cuda_available": (C.c_int, []),
    "ann_cuda_device_count": (C.c_int, []),
    "ann_cuda_device_info": (C.c_int, [C.c_char_p, C.c_size_t]),
    "ann_cuda_flat_create": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(_P)]),
    "ann_cuda_flat_create_storage": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(_P)]),
    "ann_cuda_index_storage": (C.c_int, [_P]),
    "ann_cuda_ivfflat_create": (C.c_int, [C.c_int, C.c_int, _I64, C.c_int, C.POINTER(_P)]),
    "ann_cuda_ivfflat_set_centroids": (C.c_int, [_P, _P]),
    "ann_cuda_ivfflat_train": (C.c_int, [_P, _I64, _P]),
    "ann_cuda_ivfflat_add_list": (C.c_int, [_P, _I64, _I64, _P, _P]),
    "ann_cuda_ivfflat_list_size": (_I64, [_P, _I64]),
    "ann_cuda_ivfflat_get_list": (C.c_int, [_P, _I64, _P, _P]),
    "ann_cuda_ivfflat_get_centroids": (C.c_int, [_P, _P]),
    "ann_cuda_ivfflat_coarse": (C.c_int, [_P, _I64, _P, _I64, _P]),
    "ann_cuda_ivfflat_coarse_device": (C.c_int, [_P, C.c_int64, _P, _P, _P]),
    "ann_cuda_ivfflat_search_preassigned_device": (C.c_int, [_P, C.c_int64, _P, _P, C.c_int64, _P, _P, C.c_int64, _P]),
    "ann_cuda_ivfflat_set_nprobe": (C.c_int, [_P, _I64]),
    "ann_cuda_ivfflat_get_nprobe": (_I64, [_P]),
    "ann_cuda_ivfflat_nlist": (_I64, [_P]),
    "ann_cuda_ivfflat_set_shard": (C.c_int, [_P, C.c_int, C.c_int]),
    "ann_cuda_index_add": (C.c_int, [_P, _I64, _P]),
    "ann_cuda_index_add_device": (C.c_int, [_P, _I64, _P]),
    "ann_cuda_index_reserve": (C.c_int, [_P, _I64]),
    "ann_cuda_index_search": (C.c_int, [_P, _I64, _P, _I64, _P, _P]),
    "ann_cuda_index_search_device": (C.c_int, [_P, _I64, _P, _I64, _P, _P, _I64, _P]),
    "ann_cuda_index_search_async": (C.c_int, [_P, _I64, _P, _I64, _P, _P, _P]),
    "ann_cuda_search_token_ready": (C.c_int, [_P]),
    "ann_cuda_search_token_wait": (C.c_int, [_P]),
    "ann_cuda_search_token_free": (None, [_P]),
    "ann_cuda_flat_search_small_static": (C.c_int, [_P, _I64, _P, _I64, _P, _P, _I64, _P]),
    "ann_cuda_flat_search_small_static_status": (C.c_int, [C.c_int, _P]),
    "ann_cuda_index_search_status": (C.c_int, [_P, _P]),
    "ann_cuda_set_wait_limit_ms": (None, [C.c_int]),
    "ann_cuda_test_withhold_loads": (None, [C.c_int]),
    "ann_cuda_index_reset": (C.c_int, [_P]),
    "ann_cuda_index_reconstruct": (C.c_int, [_P, _I64, _P]),
    "ann_cuda_flat_get_rows": (C.c_int, [_P, _I64, _I64, _P]),
    "ann_cuda_index_ntotal": (_I64, [_P]),
    "ann_cuda_index_d": (C.c_int, [_P]),
    "ann_cuda_index_metric": (C.c_int, [_P]),
    "ann_cuda_index_is_trained": (C.c_int, [_P]),
    "ann_cuda_index_is_ivf": (C.c_int, [_P]),
    "ann_cuda_index_device": (C.c_int, [_P]),
    "ann_cuda_index_free": (None, [_P]),
    "ann_cuda_sharded_create": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, _I64, C.POINTER(_P)]),
    "ann_cuda_sharded_free": (None, [_P]),
    "ann_cuda_sharded_shard_count": (C.c_int, [_P]),
    "ann_cuda_sharded_shard": (_P, [_P, C.c_int]),
    "ann_cuda_sharded_ntotal": (_I64, [_P]),
    "ann_cuda_sharded_add": (C.c_int, [_P, _I64, _P]),
    "ann_cuda_sharded_train": (C.c_int, [_P, _I64, _P]),
    "ann_cuda_sharded_set_centroids": (C.c_int, [_P, _P]),
    "ann_cuda_sharded_add_list": (C.c_int, [_P, _I64, _I64, _P, _P]),
    "ann_cuda_sharded_set_nprobe": (C.c_int, [_P, _I64]),
    "ann_cuda_sharded_search": (C.c_int, [_P, _I64, _P, _I64, _P, _P]),
    "ann_cuda_sharded_reset": (C.c_int, [_P]),
    "ann_cuda_sharded_reconstruct": (C.c_int, [_P, _I64, _P]),
    "ann_cuda_sharded_get_rows": (C.c_int, [_P, _I64, _I64, _P]),
    "ann_cuda_merge_topk_device": (C.c_int, [C.c_int, _P, _P, C.c_int, _I64, _I64, C.c_int, _P, _P, _P]),
    "ann_cuda_flat_kernel_name": (C.c_char_p, []),
    "ann_cuda_set_flat_kernel": (C.c_int, [C.c_char_p]),
    "ann_cuda_set_kernel_timing": (None, [C.c_int]),
    "ann_cuda_index_last_flat_kernel_ms": (C.c_float, [_P]),
    "ann_cuda_launch_count": (C.c_uint64, []),
    "ann_cuda_screen_fallbacks": (C.c_uint64, []),
    # include/cuda_diskann_bridge.h
    "diskann_metal_available": (C.c_int, []),
    "diskann_metal_batch_distances": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "diskann_metal_multi_batch_distances": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "diskann_cuda_last_error": (C.c_char_p, []),
    "diskann_cuda_register_table": (C.c_int, [C.c_int, _P, C.c_size_t, C.c_int, C.POINTER(_P)]),
    "diskann_cuda_register_table_device": (C.c_int, [C.c_int, _P, C.c_size_t, C.c_int, C.POINTER(_P)]),
    "diskann_cuda_register_sq8": (C.c_int, [C.c_int, _P, _P, _P, C.c_size_t, C.c_int, C.POINTER(_P)]),
    "diskann_cuda_register_sq8_device": (C.c_int, [C.c_int, _P, _P, _P, C.c_size_t, C.c_int, C.POINTER(_P)]),
    "diskann_cuda_unregister": (C.c_int, [_P]),
    "diskann_cuda_parse_index": (C.c_int, [_P, C.c_size_t, _P]),
    "diskann_cuda_load_index": (C.c_int, [C.c_int, _P, C.c_size_t, _P, _P, _P]),
    "diskann_cuda_load_index_file": (C.c_int, [C.c_int, C.c_char_p, _P, _P, _P]),
    "diskann_cuda_batch_distances_by_id": (C.c_int, [_P, _P, C.c_int, _P, _P, C.c_int, C.c_int, _P]),
    "diskann_cuda_batch_distances_by_id_device": (C.c_int, [_P, _P, C.c_int, _P, _P, C.c_int, C.c_int, _P, _P]),
    "diskann_cuda_batch_distances_by_id_device_multi": (C.c_int, [_P, _P, C.c_int, C.c_int, _P]),
    "diskann_cuda_searcher_last_error": (C.c_char_p, []),
    "diskann_cuda_searcher_open": (C.c_int, [C.c_int, _P, C.c_size_t, C.c_int, C.POINTER(_P)]),
    "diskann_cuda_searcher_close": (None, [_P]),
    "diskann_cuda_searcher_info": (C.c_int, [_P, _P]),
    "diskann_cuda_searcher_search_batch": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P]),
    "diskann_cuda_searcher_stats": (C.c_int, [_P, _P, _P, _P]),
    "diskann_cuda_searcher_set_trace": (None, [_P, C.c_int]),
    "diskann_cuda_searcher_trace": (_I64, [_P, _P, _P, _P, _I64, _I64]),
}


def _declare(l: C.CDLL) -> None:
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(l, name)  # AttributeError here = the library does not export a declared symbol
        fn.restype = res
        fn.argtypes = args


def last_error() -> str:
    l = lib()
    a = (l.ann_cuda_last_error() or b"").decode()
    b = (l.diskann_cuda_last_error() or b"").decode()
    c = (l.diskann_cuda_searcher_last_error() or b"").decode()
    return a or c or b


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise AnnCudaError(f"{what}: {last_error()}")


from .faiss_like import (METRIC_INNER_PRODUCT, METRIC_L2, STORAGE_BF16, STORAGE_F16, STORAGE_F32,  # noqa: E402
                         CudaGpuBackend, CudaIndexFlat, CudaIndexIVFFlat, CudaShardedIndex, SearchToken,
                         get_gpu_backend, merge_topk_device)
from . import diskann_bridge  # noqa: E402
from . import sharded  # noqa: E402

__all__ = ["lib", "last_error", "AnnCudaError", "CudaIndexFlat", "CudaIndexIVFFlat", "CudaShardedIndex", "CudaGpuBackend",
           "get_gpu_backend", "merge_topk_device", "METRIC_L2", "METRIC_INNER_PRODUCT", "STORAGE_F32",
           "STORAGE_F16", "STORAGE_BF16", "diskann_bridge", "sharded"]
