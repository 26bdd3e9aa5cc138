"""Host-side wrappers of the DiskANN batch-distance ABI.

`metal_batch_distances` / `metal_multi_batch_distances` mirror the safe wrappers
of rust_lib/src/metal_ffi.rs:67-141 (same names, same gating and return
convention: True = `out` is valid, False = caller must use its CPU loop), with
the thresholds re-derived for a discrete GPU.  `DeviceTable` wraps the
device-resident table entry points.  `cuda_ffi.rs` beside the CUDA sources is
the Rust form of this file.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

# Minimum n*dim for one call to be worth a launch plus two PCIe copies.  The
# reference uses 131072 (iterative search) and 49152 (one-shot) for Metal's
# ~100-450 us dispatch (rust_lib/src/metal_ffi.rs:36-46); a CUDA launch with
# pageable copies costs ~20-30 us, so the break-even moves down.
MIN_GPU_WORK = 65536
MIN_GPU_WORK_ONESHOT = 32768

_status = -1  # cached availability: -1 unchecked, 0 no, 1 yes (metal_ffi.rs:33,49-57)


def _pkg():
    import sys
    return sys.modules[__name__.rsplit(".", 1)[0]]


def _p(a):
    return C.c_void_p(a.ctypes.data) if a is not None else None


def is_metal_available() -> bool:
    """Name kept from metal_ffi.rs:49; reports the CUDA bridge."""
    global _status
    if _status < 0:
        _status = int(_pkg().lib().diskann_metal_available())
    return _status == 1


def metal_batch_distances(query, candidates, n: int, dim: int, metric: int, out) -> bool:
    """metal_ffi.rs:67-96.  query (dim,), candidates (n*dim,), out (>= n)."""
    if n == 0 or dim == 0:
        return True
    if n * dim < MIN_GPU_WORK or not is_metal_available():
        return False
    return batch_distances_raw(query, candidates, n, dim, metric, out) == 0


def metal_multi_batch_distances(queries, candidates, query_map, total_n: int, nq: int, dim: int, metric: int,
                                out) -> bool:
    """metal_ffi.rs:107-141.  Does not check MIN_GPU_WORK: the caller does."""
    if total_n == 0 or nq == 0 or dim == 0:
        return True
    if not is_metal_available():
        return False
    return multi_batch_distances_raw(queries, candidates, query_map, total_n, nq, dim, metric, out) == 0


def batch_distances_raw(query, candidates, n, dim, metric, out) -> int:
    """diskann_metal_batch_distances, ungated; returns the C return code."""
    q = np.ascontiguousarray(query, np.float32) if query is not None else None
    c = np.ascontiguousarray(candidates, np.float32) if candidates is not None else None
    return int(_pkg().lib().diskann_metal_batch_distances(_p(q), _p(c), n, dim, metric, _p(out)))


def multi_batch_distances_raw(queries, candidates, query_map, total_n, nq, dim, metric, out) -> int:
    q = np.ascontiguousarray(queries, np.float32) if queries is not None else None
    c = np.ascontiguousarray(candidates, np.float32) if candidates is not None else None
    m = np.ascontiguousarray(query_map, np.uint32) if query_map is not None else None
    return int(_pkg().lib().diskann_metal_multi_batch_distances(_p(q), _p(c), _p(m), total_n, nq, dim, metric,
                                                               _p(out)))


class IndexInfo(C.Structure):
    """struct diskann_cuda_index_info of include/cuda_diskann_bridge.h"""
    _fields_ = [("num_vectors", C.c_uint32), ("dimension", C.c_uint32), ("max_degree", C.c_uint32),
                ("num_entry_points", C.c_uint32), ("build_complexity", C.c_uint32), ("metric", C.c_uint32),
                ("entry_points_offset", C.c_uint64), ("vectors_offset", C.c_uint64), ("adjacency_offset", C.c_uint64),
                ("standard_size", C.c_uint64), ("has_sq8", C.c_int), ("sq8_min_offset", C.c_uint64),
                ("sq8_scale_offset", C.c_uint64), ("sq8_codes_offset", C.c_uint64), ("sq8_codes_size", C.c_uint64)]


def parse_index(image: bytes) -> IndexInfo:
    """Header and segment offsets of a serialized DiskANN index (no GPU needed)."""
    info = IndexInfo()
    p = _pkg()
    p.check(p.lib().diskann_cuda_parse_index(image, len(image), C.byref(info)), "parse_index")
    return info


def load_index(image_or_path, device: int = 0):
    """Registers the vector segment (and the SQ8 codes, if the image carries them) of a
    serialized DiskANN index.  Returns (info, fp32 DeviceTable, SQ8 DeviceTable or None)."""
    info = IndexInfo()
    hv, hq = C.c_void_p(), C.c_void_p()
    p = _pkg()
    if isinstance(image_or_path, (bytes, bytearray, memoryview)):
        image = bytes(image_or_path)
        rc = p.lib().diskann_cuda_load_index(device, image, len(image), C.byref(info), C.byref(hv), C.byref(hq))
    else:
        rc = p.lib().diskann_cuda_load_index_file(device, str(image_or_path).encode(), C.byref(info), C.byref(hv),
                                                  C.byref(hq))
    p.check(rc, "load_index")
    vec = DeviceTable(hv, info.num_vectors, info.dimension, False)
    sq8 = DeviceTable(hq, info.num_vectors, info.dimension, True) if hq.value else None
    return info, vec, sq8


class _BatchDesc(C.Structure):
    """struct diskann_cuda_batch of include/cuda_diskann_bridge.h"""
    _fields_ = [("queries", C.c_void_p), ("ids", C.c_void_p), ("query_map", C.c_void_p),
                ("out_distances", C.c_void_p), ("nq", C.c_int), ("total_n", C.c_int)]


class DeviceTable:
    """A vector table resident in GPU memory (fp32 rows, or SQ8 codes + min/scale),
    scored by row id: diskann_cuda_register_* / diskann_cuda_batch_distances_by_id."""

    def __init__(self, handle, num: int, dim: int, sq8: bool, keepalive=None):
        self._h = handle
        self.num, self.dim, self.sq8 = num, dim, sq8
        self._keepalive = keepalive

    @staticmethod
    def from_host(rows, device: int = 0) -> "DeviceTable":
        rows = np.ascontiguousarray(rows, np.float32)
        h = C.c_void_p()
        p = _pkg()
        p.check(p.lib().diskann_cuda_register_table(device, _p(rows), rows.shape[0], rows.shape[1], C.byref(h)),
                "register_table")
        return DeviceTable(h, rows.shape[0], rows.shape[1], False)

    @staticmethod
    def from_device(rows) -> "DeviceTable":
        """rows: contiguous float32 torch CUDA tensor (num, dim); kept alive by the table."""
        h = C.c_void_p()
        p = _pkg()
        p.check(p.lib().diskann_cuda_register_table_device(rows.device.index or 0, C.c_void_p(rows.data_ptr()),
                                                           rows.shape[0], rows.shape[1], C.byref(h)),
                "register_table_device")
        return DeviceTable(h, rows.shape[0], rows.shape[1], False, keepalive=rows)

    @staticmethod
    def sq8_from_host(codes, mins, scale, device: int = 0) -> "DeviceTable":
        codes = np.ascontiguousarray(codes, np.uint8)
        mins = np.ascontiguousarray(mins, np.float32)
        scale = np.ascontiguousarray(scale, np.float32)
        h = C.c_void_p()
        p = _pkg()
        p.check(p.lib().diskann_cuda_register_sq8(device, _p(codes), _p(mins), _p(scale), codes.shape[0],
                                                  codes.shape[1], C.byref(h)), "register_sq8")
        return DeviceTable(h, codes.shape[0], codes.shape[1], True)

    @staticmethod
    def sq8_from_device(codes, mins, scale) -> "DeviceTable":
        """codes: contiguous uint8 torch CUDA tensor; mins/scale: host float32 arrays."""
        mins = np.ascontiguousarray(mins, np.float32)
        scale = np.ascontiguousarray(scale, np.float32)
        h = C.c_void_p()
        p = _pkg()
        p.check(p.lib().diskann_cuda_register_sq8_device(codes.device.index or 0, C.c_void_p(codes.data_ptr()),
                                                         _p(mins), _p(scale), codes.shape[0], codes.shape[1],
                                                         C.byref(h)), "register_sq8_device")
        return DeviceTable(h, codes.shape[0], codes.shape[1], True, keepalive=codes)

    def batch_distances_by_id(self, queries, ids, query_map, metric: int):
        """Host buffers in, host distances out (synchronous)."""
        q = np.ascontiguousarray(queries, np.float32).reshape(-1, self.dim)
        ids = np.ascontiguousarray(ids, np.uint32)
        qm = None if query_map is None else np.ascontiguousarray(query_map, np.uint32)
        out = np.empty(ids.shape[0], np.float32)
        p = _pkg()
        p.check(p.lib().diskann_cuda_batch_distances_by_id(self._h, _p(q), q.shape[0], _p(ids), _p(qm),
                                                           ids.shape[0], metric, _p(out)), "batch_distances_by_id")
        return out

    def batch_distances_by_id_device(self, queries, ids, query_map, metric: int, out=None, stream=None):
        """torch CUDA tensors in and out; enqueued on `stream`, not synchronised.
        ids / query_map are int32 tensors holding the uint32 values."""
        import torch
        nq = queries.shape[0]
        total_n = ids.shape[0]
        if out is None:
            out = torch.empty(total_n, dtype=torch.float32, device=queries.device)
        s = stream if stream is not None else torch.cuda.current_stream(queries.device)
        p = _pkg()
        p.check(p.lib().diskann_cuda_batch_distances_by_id_device(
            self._h, C.c_void_p(queries.data_ptr()), nq, C.c_void_p(ids.data_ptr()),
            C.c_void_p(query_map.data_ptr()) if query_map is not None else None, total_n, metric,
            C.c_void_p(out.data_ptr()), C.c_void_p(s.cuda_stream)), "batch_distances_by_id_device")
        return out

    @staticmethod
    def pack_batches(batches):
        """The descriptor array of a multi-batch launch (struct diskann_cuda_batch[]), built once
        and reusable: `batches` is a list of (queries, ids, query_map, out) torch CUDA tensors,
        query_map None for a single query.  The tensors must outlive the launches."""
        arr = (_BatchDesc * len(batches))()
        for d, (q, ids, qm, out) in zip(arr, batches):
            d.queries = q.data_ptr()
            d.ids = ids.data_ptr()
            d.query_map = qm.data_ptr() if qm is not None else None
            d.out_distances = out.data_ptr()
            d.nq = q.shape[0]
            d.total_n = ids.shape[0]
        return arr

    def batch_distances_by_id_device_multi(self, batches, metric: int, stream=None, device=None):
        """Several batches in one launch.  `batches` is a list of (queries, ids, query_map, out)
        torch CUDA tensors or the result of pack_batches(); enqueued on `stream`."""
        import torch
        arr = batches if isinstance(batches, C.Array) else self.pack_batches(batches)
        if stream is None:
            if device is None and not isinstance(batches, C.Array):
                device = batches[0][0].device
            stream = torch.cuda.current_stream(device)
        p = _pkg()
        p.check(p.lib().diskann_cuda_batch_distances_by_id_device_multi(self._h, arr, len(arr), metric,
                                                                         C.c_void_p(stream.cuda_stream)),
                "batch_distances_by_id_device_multi")

    def close(self) -> None:
        if self._h:
            _pkg().lib().diskann_cuda_unregister(self._h)
            self._h = C.c_void_p()
            self._keepalive = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class DiskSearcher:
    """Lock-step batched graph search over a ".diskann" image whose vectors live in GPU memory:
    DiskProvider::search_batch (rust_lib/src/disk_provider.rs:470-652) with the neighbour rows named
    by id (diskann_cuda_searcher_*)."""

    def __init__(self, image: bytes, device: int = 0, use_sq8: bool = False):
        self._h = C.c_void_p()
        self._image = bytes(image)
        p = _pkg()
        p.check(p.lib().diskann_cuda_searcher_open(device, self._image, len(self._image), int(use_sq8), C.byref(self._h)),
                "DiskSearcher")
        self.info = IndexInfo()
        p.check(p.lib().diskann_cuda_searcher_info(self._h, C.byref(self.info)), "DiskSearcher info")

    def search_batch(self, queries, k: int, l_search: int):
        """-> list of (ids uint64, distances float32) per query, best first."""
        q = np.ascontiguousarray(queries, np.float32)
        nq = q.shape[0]
        ids = np.zeros((nq, max(k, 1)), np.uint64)
        dist = np.zeros((nq, max(k, 1)), np.float32)
        counts = np.zeros(nq, np.int32)
        p = _pkg()
        p.check(p.lib().diskann_cuda_searcher_search_batch(self._h, _p(q), nq, k, l_search, _p(ids), _p(dist), _p(counts)),
                "search_batch")
        return [(ids[i, :counts[i]].copy(), dist[i, :counts[i]].copy()) for i in range(nq)]

    def stats(self) -> dict:
        it, pairs, calls = C.c_uint64(), C.c_uint64(), C.c_uint64()
        p = _pkg()
        p.check(p.lib().diskann_cuda_searcher_stats(self._h, C.byref(it), C.byref(pairs), C.byref(calls)), "stats")
        return {"iterations": it.value, "pairs_scored": pairs.value, "distance_calls": calls.value}

    def set_trace(self, on: bool) -> None:
        _pkg().lib().diskann_cuda_searcher_set_trace(self._h, int(on))

    def trace(self):
        """The id batches of the last traced search: list of (ids uint32, query_map uint32)."""
        lib = _pkg().lib()
        nb = lib.diskann_cuda_searcher_trace(self._h, None, None, None, 0, 0)
        if nb <= 0:
            return []
        st = self.stats()
        ids = np.empty(st["pairs_scored"], np.uint32)
        qm = np.empty(st["pairs_scored"], np.uint32)
        off = np.empty(nb + 1, np.uint64)
        got = lib.diskann_cuda_searcher_trace(self._h, _p(ids), _p(qm), _p(off), len(ids), nb)
        _pkg().check(0 if got == nb else -1, "trace")
        return [(ids[int(off[i]):int(off[i + 1])], qm[int(off[i]):int(off[i + 1])]) for i in range(nb)]

    def close(self) -> None:
        if self._h:
            _pkg().lib().diskann_cuda_searcher_close(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
