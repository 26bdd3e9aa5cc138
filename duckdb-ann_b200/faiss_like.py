"""Python mirror of the reference's C++ plugin surface for FAISS indexes.

Same names and argument meaning as the classes a maintainer sees in C++
(`faiss::Index` members used at src/faiss_index.cpp:108-153, 708-762; index
classes of faiss-metal/include/faiss-metal/MetalIndexFlat.h:47-101 and
MetalIndexIVFFlat.h:25-76; backend of src/gpu_backend_metal.mm:15-84), so the
parity tests read like the reference's own tests.  Every method is one call into
the C ABI; numpy arrays are host buffers, torch CUDA tensors are device buffers.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

METRIC_INNER_PRODUCT = 0  # faiss::METRIC_INNER_PRODUCT
METRIC_L2 = 1             # faiss::METRIC_L2


def _pkg():
    import sys
    return sys.modules[__name__.rsplit(".", 1)[0]]


def _np_f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return C.c_void_p(a.ctypes.data) if a is not None else None


class SearchToken:
    """MetalSearchToken (MetalIndexFlat.h:15-36): owns one in-flight search."""

    def __init__(self, handle, D, I, index):
        self._t, self._D, self._I, self._index = handle, D, I, index  # the index outlives its tokens

    def is_ready(self) -> bool:
        """Non-blocking: True once the device work has finished."""
        return not self._t or _pkg().lib().ann_cuda_search_token_ready(self._t) == 1

    def wait(self):
        """Blocks until the search has finished; returns (D, I)."""
        if self._t:
            p = _pkg()
            rc = p.lib().ann_cuda_search_token_wait(self._t)
            self.close()
            p.check(rc, "search_async wait")
        return self._D, self._I

    def close(self) -> None:
        if self._t:
            _pkg().lib().ann_cuda_search_token_free(self._t)
            self._t = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _CudaIndex:
    """Common faiss::Index surface: d, ntotal, metric_type, is_trained, add,
    search, reset, reconstruct."""

    def __init__(self):
        self._h = C.c_void_p()

    # -- fields of faiss::Index
    @property
    def d(self) -> int:
        return _pkg().lib().ann_cuda_index_d(self._h)

    @property
    def ntotal(self) -> int:
        return _pkg().lib().ann_cuda_index_ntotal(self._h)

    @property
    def metric_type(self) -> int:
        return _pkg().lib().ann_cuda_index_metric(self._h)

    @property
    def is_trained(self) -> bool:
        return bool(_pkg().lib().ann_cuda_index_is_trained(self._h))

    @property
    def device(self) -> int:
        return _pkg().lib().ann_cuda_index_device(self._h)

    def add(self, x) -> None:
        """faiss::Index::add(n, x); x is (n, d) float32 on the host."""
        x = _np_f32(x)
        if x.ndim != 2 or x.shape[1] != self.d:
            raise ValueError(f"add: expected (n, {self.d}) rows")
        p = _pkg()
        p.check(p.lib().ann_cuda_index_add(self._h, x.shape[0], _ptr(x)), "add")

    def add_device(self, x) -> None:
        """add() with the rows already on this index's GPU (a torch CUDA tensor)."""
        assert x.is_cuda and x.is_contiguous() and x.dim() == 2 and x.shape[1] == self.d
        p = _pkg()
        p.check(p.lib().ann_cuda_index_add_device(self._h, x.shape[0], C.c_void_p(x.data_ptr())), "add_device")

    def reserve(self, n_total: int) -> None:
        p = _pkg()
        p.check(p.lib().ann_cuda_index_reserve(self._h, n_total), "reserve")

    def search(self, x, k: int):
        """faiss::Index::search(n, x, k, D, I) with host buffers -> (D, I)."""
        x = _np_f32(x)
        if x.ndim != 2 or x.shape[1] != self.d:
            raise ValueError(f"search: expected (n, {self.d}) queries")
        n = x.shape[0]
        D = np.empty((n, max(k, 0)), np.float32)
        I = np.empty((n, max(k, 0)), np.int64)
        p = _pkg()
        p.check(p.lib().ann_cuda_index_search(self._h, n, _ptr(x), k, _ptr(D), _ptr(I)), "search")
        return D, I

    def search_async(self, x, k: int) -> "SearchToken":
        """MetalIndexFlat::searchAsync (MetalIndexFlat.h:71-76): enqueue the search and return
        a token; token.wait() -> (D, I).  Several tokens may be in flight on one index."""
        x = _np_f32(x)
        if x.ndim != 2 or x.shape[1] != self.d:
            raise ValueError(f"search_async: expected (n, {self.d}) queries")
        n = x.shape[0]
        D = np.empty((n, max(k, 0)), np.float32)
        I = np.empty((n, max(k, 0)), np.int64)
        tok = C.c_void_p()
        p = _pkg()
        p.check(p.lib().ann_cuda_index_search_async(self._h, n, _ptr(x), k, _ptr(D), _ptr(I), C.byref(tok)),
                "search_async")
        return SearchToken(tok, D, I, self)

    def search_device(self, x, k: int, D=None, I=None, label_offset: int = 0, stream=None):
        """search() on device buffers (torch CUDA tensors), enqueued on `stream`
        (a torch.cuda.Stream; default: torch's current stream), not synchronised."""
        import torch
        assert x.is_cuda and x.is_contiguous() and x.dtype == torch.float32 and x.shape[1] == self.d
        n = x.shape[0]
        if D is None:
            D = torch.empty((n, k), dtype=torch.float32, device=x.device)
        if I is None:
            I = torch.empty((n, k), dtype=torch.int64, device=x.device)
        s = stream if stream is not None else torch.cuda.current_stream(x.device)
        p = _pkg()
        p.check(p.lib().ann_cuda_index_search_device(self._h, n, C.c_void_p(x.data_ptr()), k,
                                                     C.c_void_p(D.data_ptr()), C.c_void_p(I.data_ptr()),
                                                     label_offset, C.c_void_p(s.cuda_stream)), "search_device")
        return D, I

    def search_status(self, stream=None) -> None:
        """Waits for `stream` (default: torch's current stream) and raises if a search_device call
        made on it since the last check failed on the device."""
        import torch
        s = stream if stream is not None else torch.cuda.current_stream(self.device)
        p = _pkg()
        p.check(p.lib().ann_cuda_index_search_status(self._h, C.c_void_p(s.cuda_stream)), "search_status")

    def reset(self) -> None:
        p = _pkg()
        p.check(p.lib().ann_cuda_index_reset(self._h), "reset")

    def reconstruct(self, key: int):
        out = np.empty(self.d, np.float32)
        p = _pkg()
        p.check(p.lib().ann_cuda_index_reconstruct(self._h, key, _ptr(out)), "reconstruct")
        return out

    def close(self) -> None:
        if self._h:
            _pkg().lib().ann_cuda_index_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# StorageType of faiss-metal/include/faiss-metal/MetalIndexFlat.h:38-43
STORAGE_F32, STORAGE_F16, STORAGE_BF16 = 0, 1, 2


class CudaIndexFlat(_CudaIndex):
    """MetalIndexFlat(resources, d, metric[, storage]) -> CudaIndexFlat(d, metric, device, storage).

    storage = STORAGE_F16 / STORAGE_BF16 keeps the rows rounded to that type (2 bytes per element) and
    searches the rounded rows; queries stay fp32 (MetalIndexFlat.h:53-60)."""

    def __init__(self, d: int, metric: int = METRIC_L2, device: int = 0, storage: int = STORAGE_F32):
        super().__init__()
        p = _pkg()
        if storage == STORAGE_F32:
            p.check(p.lib().ann_cuda_flat_create(device, d, metric, C.byref(self._h)), "CudaIndexFlat")
        else:
            p.check(p.lib().ann_cuda_flat_create_storage(device, d, metric, storage, C.byref(self._h)), "CudaIndexFlat")

    @property
    def storage(self) -> int:
        """MetalIndexFlat::getStorageType (MetalIndexFlat.h:90)."""
        return _pkg().lib().ann_cuda_index_storage(self._h)

    def search_small_static(self, x, k: int, D=None, I=None, label_offset: int = 0, stream=None):
        """search_device() for callers that may not allocate device memory (a worker under a
        fixed memory budget): at most 128 queries, k <= 16,
        d <= 1024, all scratch in a fixed device array.  Calls must not overlap on the GPU.
        D and I must be passed in if torch itself must not allocate either."""
        import torch
        assert x.is_cuda and x.is_contiguous() and x.dtype == torch.float32 and x.shape[1] == self.d
        n = x.shape[0]
        if D is None:
            D = torch.empty((n, k), dtype=torch.float32, device=x.device)
        if I is None:
            I = torch.empty((n, k), dtype=torch.int64, device=x.device)
        s = stream if stream is not None else torch.cuda.current_stream(x.device)
        p = _pkg()
        p.check(p.lib().ann_cuda_flat_search_small_static(self._h, n, C.c_void_p(x.data_ptr()), k,
                                                          C.c_void_p(D.data_ptr()), C.c_void_p(I.data_ptr()),
                                                          label_offset, C.c_void_p(s.cuda_stream)),
                "search_small_static")
        return D, I

    def get_rows(self, first: int, n: int):
        out = np.empty((n, self.d), np.float32)
        p = _pkg()
        p.check(p.lib().ann_cuda_flat_get_rows(self._h, first, n, _ptr(out)), "get_rows")
        return out


class CudaIndexIVFFlat(_CudaIndex):
    """MetalIndexIVFFlat(resources, d, nlist, metric) -> CudaIndexIVFFlat(d, nlist, metric, device)."""

    def __init__(self, d: int, nlist: int, metric: int = METRIC_L2, device: int = 0):
        super().__init__()
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_create(device, d, nlist, metric, C.byref(self._h)), "CudaIndexIVFFlat")

    def train(self, x) -> None:
        x = _np_f32(x)
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_train(self._h, x.shape[0], _ptr(x)), "train")

    def set_centroids(self, centroids) -> None:
        c = _np_f32(centroids)
        if c.shape != (self.getNlist(), self.d):
            raise ValueError("set_centroids: expected (nlist, d)")
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_set_centroids(self._h, _ptr(c)), "set_centroids")

    def get_centroids(self):
        out = np.empty((self.getNlist(), self.d), np.float32)
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_get_centroids(self._h, _ptr(out)), "get_centroids")
        return out

    def add_list(self, list_no: int, ids, rows) -> None:
        ids = np.ascontiguousarray(ids, np.int64)
        rows = _np_f32(rows).reshape(len(ids), self.d)
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_add_list(self._h, list_no, len(ids), _ptr(ids), _ptr(rows)), "add_list")

    def list_size(self, list_no: int) -> int:
        return _pkg().lib().ann_cuda_ivfflat_list_size(self._h, list_no)

    def get_list(self, list_no: int):
        n = self.list_size(list_no)
        ids = np.empty(n, np.int64)
        rows = np.empty((n, self.d), np.float32)
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_get_list(self._h, list_no, _ptr(ids), _ptr(rows)), "get_list")
        return ids, rows

    def coarse(self, x, nprobe: int):
        """Coarse quantiser only: (n, nprobe) list numbers, nearest centroid first."""
        x = _np_f32(x)
        out = np.empty((x.shape[0], nprobe), np.int64)
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_coarse(self._h, x.shape[0], _ptr(x), nprobe, _ptr(out)), "coarse")
        return out

    def coarse_device(self, x, out=None, stream=None):
        """Coarse quantiser on device buffers: (n, nprobe) int32 list numbers, nearest centroid first
        (nprobe = the index's), enqueued on `stream`, not synchronised."""
        import torch
        assert x.is_cuda and x.is_contiguous() and x.dtype == torch.float32 and x.shape[1] == self.d
        n, nprobe = x.shape[0], min(self.getNprobe(), self.getNlist())
        if out is None:
            out = torch.empty((n, nprobe), dtype=torch.int32, device=x.device)
        assert out.is_contiguous() and out.dtype == torch.int32 and tuple(out.shape) == (n, nprobe)
        s = stream if stream is not None else torch.cuda.current_stream(x.device)
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_coarse_device(self._h, n, C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()),
                                                       C.c_void_p(s.cuda_stream)), "coarse_device")
        return out

    def search_preassigned_device(self, x, assign, k: int, D=None, I=None, label_offset: int = 0, stream=None):
        """search_device() with the probe lists given (faiss::IndexIVF::search_preassigned): assign is an
        (n, nprobe) int32 CUDA tensor of list numbers, -1 = none.  Lists this shard does not store are skipped."""
        import torch
        assert x.is_cuda and x.is_contiguous() and x.dtype == torch.float32 and x.shape[1] == self.d
        n = x.shape[0]
        assert assign.is_cuda and assign.is_contiguous() and assign.dtype == torch.int32
        assert tuple(assign.shape) == (n, min(self.getNprobe(), self.getNlist()))
        if D is None:
            D = torch.empty((n, k), dtype=torch.float32, device=x.device)
        if I is None:
            I = torch.empty((n, k), dtype=torch.int64, device=x.device)
        s = stream if stream is not None else torch.cuda.current_stream(x.device)
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_search_preassigned_device(self._h, n, C.c_void_p(x.data_ptr()),
                                                                   C.c_void_p(assign.data_ptr()), k, C.c_void_p(D.data_ptr()),
                                                                   C.c_void_p(I.data_ptr()), label_offset,
                                                                   C.c_void_p(s.cuda_stream)), "search_preassigned_device")
        return D, I

    def getNlist(self) -> int:
        return _pkg().lib().ann_cuda_ivfflat_nlist(self._h)

    def getNprobe(self) -> int:
        return _pkg().lib().ann_cuda_ivfflat_get_nprobe(self._h)

    def setNprobe(self, nprobe: int) -> None:
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_set_nprobe(self._h, nprobe), "setNprobe")

    def set_shard(self, rank: int, count: int) -> None:
        p = _pkg()
        p.check(p.lib().ann_cuda_ivfflat_set_shard(self._h, rank, count), "set_shard")


class _ShardView(_CudaIndex):
    """A borrowed shard of a CudaShardedIndex (never freed from here)."""

    def __init__(self, handle):
        super().__init__()
        self._h = handle

    def close(self) -> None:
        self._h = C.c_void_p()


class CudaShardedIndex:
    """One Flat (nlist = 0) or IVFFlat index over several GPUs in this process: what
    CudaGpuBackend::CpuToGpu hands out when ANN_CUDA_DEVICES names more than one device.
    `devices` may repeat a device (several shards on one GPU)."""

    def __init__(self, d: int, metric: int = METRIC_L2, devices=(0,), nlist: int = 0):
        self._h = C.c_void_p()
        self.d, self.metric_type, self.nlist = d, metric, nlist
        dev = (C.c_int * len(devices))(*devices)
        p = _pkg()
        p.check(p.lib().ann_cuda_sharded_create(dev, len(devices), d, metric, nlist, C.byref(self._h)), "CudaShardedIndex")

    @property
    def ntotal(self) -> int:
        return _pkg().lib().ann_cuda_sharded_ntotal(self._h)

    @property
    def shard_count(self) -> int:
        return _pkg().lib().ann_cuda_sharded_shard_count(self._h)

    def shard(self, i: int) -> _ShardView:
        h = _pkg().lib().ann_cuda_sharded_shard(self._h, i)
        if not h:
            raise IndexError(i)
        return _ShardView(C.c_void_p(h))

    def add(self, x) -> None:
        x = _np_f32(x)
        p = _pkg()
        p.check(p.lib().ann_cuda_sharded_add(self._h, x.shape[0], _ptr(x)), "sharded add")

    def train(self, x) -> None:
        x = _np_f32(x)
        p = _pkg()
        p.check(p.lib().ann_cuda_sharded_train(self._h, x.shape[0], _ptr(x)), "sharded train")

    def set_centroids(self, centroids) -> None:
        c = _np_f32(centroids)
        p = _pkg()
        p.check(p.lib().ann_cuda_sharded_set_centroids(self._h, _ptr(c)), "sharded set_centroids")

    def add_list(self, list_no: int, ids, rows) -> None:
        ids = np.ascontiguousarray(ids, np.int64)
        rows = _np_f32(rows).reshape(len(ids), self.d)
        p = _pkg()
        p.check(p.lib().ann_cuda_sharded_add_list(self._h, list_no, len(ids), _ptr(ids), _ptr(rows)), "sharded add_list")

    def setNprobe(self, nprobe: int) -> None:
        p = _pkg()
        p.check(p.lib().ann_cuda_sharded_set_nprobe(self._h, nprobe), "sharded setNprobe")

    def search(self, x, k: int):
        x = _np_f32(x)
        n = x.shape[0]
        D = np.empty((n, max(k, 0)), np.float32)
        I = np.empty((n, max(k, 0)), np.int64)
        p = _pkg()
        p.check(p.lib().ann_cuda_sharded_search(self._h, n, _ptr(x), k, _ptr(D), _ptr(I)), "sharded search")
        return D, I

    def reset(self) -> None:
        p = _pkg()
        p.check(p.lib().ann_cuda_sharded_reset(self._h), "sharded reset")

    def reconstruct(self, key: int):
        out = np.empty(self.d, np.float32)
        p = _pkg()
        p.check(p.lib().ann_cuda_sharded_reconstruct(self._h, key, _ptr(out)), "sharded reconstruct")
        return out

    def get_rows(self, first: int, n: int):
        out = np.empty((n, self.d), np.float32)
        p = _pkg()
        p.check(p.lib().ann_cuda_sharded_get_rows(self._h, first, n, _ptr(out)), "sharded get_rows")
        return out

    def close(self) -> None:
        if self._h:
            _pkg().lib().ann_cuda_sharded_free(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CudaGpuBackend:
    """duckdb::GpuBackend for CUDA: IsAvailable / DeviceInfo / BackendName
    (src/include/gpu_backend.hpp:12-33, src/faiss_fn_gpu.cpp:33-46)."""

    def IsAvailable(self) -> bool:
        return bool(_pkg().lib().ann_cuda_available())

    def DeviceInfo(self) -> str:
        buf = C.create_string_buffer(256)
        p = _pkg()
        p.check(p.lib().ann_cuda_device_info(buf, 256), "DeviceInfo")
        return buf.value.decode()

    def BackendName(self) -> str:
        return "cuda"


_backend = None


def get_gpu_backend() -> CudaGpuBackend:
    global _backend
    if _backend is None:
        _backend = CudaGpuBackend()
    return _backend


def merge_topk_device(parts_d, parts_i, metric: int, out_d=None, out_i=None, stream=None):
    """Final k-select over per-shard results: (nparts, nq, k) CUDA tensors -> (nq, k)."""
    import torch
    assert parts_d.is_cuda and parts_d.is_contiguous() and parts_i.is_contiguous()
    nparts, nq, k = parts_d.shape
    if out_d is None:
        out_d = torch.empty((nq, k), dtype=torch.float32, device=parts_d.device)
    if out_i is None:
        out_i = torch.empty((nq, k), dtype=torch.int64, device=parts_d.device)
    s = stream if stream is not None else torch.cuda.current_stream(parts_d.device)
    p = _pkg()
    p.check(p.lib().ann_cuda_merge_topk_device(parts_d.device.index or 0, C.c_void_p(parts_d.data_ptr()),
                                               C.c_void_p(parts_i.data_ptr()), nparts, nq, k, metric,
                                               C.c_void_p(out_d.data_ptr()), C.c_void_p(out_i.data_ptr()),
                                               C.c_void_p(s.cuda_stream)), "merge_topk_device")
    return out_d, out_i
