"""ctypes front end of the CPU oracle (oracle.c).  TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the CPU-baseline / reference arm of the
benchmark import this module.  The CUDA library never does: it has no CPU path.

The reference's FAISS / diskann-vector results for the large seeded
configurations are not stored anywhere in the reference, so for those the
oracle is "parity unpinned"; it is pinned on the reference's own known answers
(tests/golden/reference_known_answers.json).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

METRIC_IP = 0  # faiss::METRIC_INNER_PRODUCT
METRIC_L2 = 1  # faiss::METRIC_L2
BATCH_L2 = 0   # batch-distance ABI: 0 = L2, anything else = IP
BATCH_IP = 1


def build(force: bool = False) -> str:
    """Compile oracle.c with the Makefile beside it (gcc, OpenMP)."""
    src = os.path.join(_HERE, "oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s", "liboracle.so"])
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_num_threads.restype = C.c_int
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(C.c_int(int(n)))


# --------------------------------------------------------------------------- batch distance
def batch_distances(query, candidates, metric: int, exact: bool = False):
    """One query against n gathered rows (src/ann_search.cpp:702-720)."""
    query, candidates = _f32(query), _f32(candidates)
    n, dim = candidates.shape
    out = np.empty(n, np.float32)
    rc = lib().oracle_batch_distances(_p(query, C.c_float), _p(candidates, C.c_float), C.c_int64(n), C.c_int64(dim),
                                      C.c_int(metric), C.c_int(int(exact)), _p(out, C.c_float))
    if rc != 0:
        raise ValueError("oracle_batch_distances: invalid arguments")
    return out


def multi_batch_distances(queries, candidates, query_map, metric: int, exact: bool = False):
    """query_map[i] picks the query of row i (src/metal_diskann_bridge.mm:255-323)."""
    queries, candidates = _f32(queries), _f32(candidates)
    query_map = np.ascontiguousarray(query_map, dtype=np.uint32)
    total_n, dim = candidates.shape
    out = np.empty(total_n, np.float32)
    rc = lib().oracle_multi_batch_distances(_p(queries, C.c_float), _p(candidates, C.c_float),
                                            _p(query_map, C.c_uint32), C.c_int64(total_n),
                                            C.c_int64(queries.shape[0]), C.c_int64(dim), C.c_int(metric),
                                            C.c_int(int(exact)), _p(out, C.c_float))
    if rc != 0:
        raise ValueError("oracle_multi_batch_distances: invalid arguments")
    return out


def batch_distances_by_id(table, queries, ids, query_map, metric: int, exact: bool = False):
    table, queries = _f32(table), _f32(queries)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    qm = None if query_map is None else np.ascontiguousarray(query_map, dtype=np.uint32)
    out = np.empty(ids.shape[0], np.float32)
    rc = lib().oracle_batch_distances_by_id(_p(table, C.c_float), C.c_int64(table.shape[0]),
                                            C.c_int64(table.shape[1]), _p(queries, C.c_float),
                                            C.c_int64(queries.shape[0]), _p(ids, C.c_uint32), _p(qm, C.c_uint32),
                                            C.c_int64(ids.shape[0]), C.c_int(metric), C.c_int(int(exact)),
                                            _p(out, C.c_float))
    if rc != 0:
        raise ValueError("oracle_batch_distances_by_id: invalid arguments")
    return out


# --------------------------------------------------------------------------- SQ8
def sq8_train(x):
    """Per-dimension min and scale (rust_lib/src/provider.rs:170-194)."""
    x = _f32(x)
    n, dim = x.shape
    mins, scale = np.empty(dim, np.float32), np.empty(dim, np.float32)
    rc = lib().oracle_sq8_train(_p(x, C.c_float), C.c_int64(n), C.c_int64(dim), _p(mins, C.c_float),
                                _p(scale, C.c_float))
    if rc != 0:
        raise ValueError("oracle_sq8_train: invalid arguments")
    return mins, scale


def sq8_encode(x, mins, scale):
    """u8 codes (rust_lib/src/provider.rs:196-203)."""
    x = _f32(x)
    n, dim = x.shape
    codes = np.empty((n, dim), np.uint8)
    rc = lib().oracle_sq8_encode(_p(x, C.c_float), C.c_int64(n), C.c_int64(dim), _p(_f32(mins), C.c_float),
                                 _p(_f32(scale), C.c_float), _p(codes, C.c_uint8))
    if rc != 0:
        raise ValueError("oracle_sq8_encode: invalid arguments")
    return codes


def sq8_decode(codes, mins, scale):
    """(code/255)*scale+min (rust_lib/src/provider.rs:138-147)."""
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    n, dim = codes.shape
    x = np.empty((n, dim), np.float32)
    rc = lib().oracle_sq8_decode(_p(codes, C.c_uint8), C.c_int64(n), C.c_int64(dim), _p(_f32(mins), C.c_float),
                                 _p(_f32(scale), C.c_float), _p(x, C.c_float))
    if rc != 0:
        raise ValueError("oracle_sq8_decode: invalid arguments")
    return x


def sq8_batch_distances_by_id(codes, mins, scale, queries, ids, query_map, metric: int, exact: bool = False):
    codes = np.ascontiguousarray(codes, dtype=np.uint8)
    queries = _f32(queries)
    ids = np.ascontiguousarray(ids, dtype=np.uint32)
    qm = None if query_map is None else np.ascontiguousarray(query_map, dtype=np.uint32)
    out = np.empty(ids.shape[0], np.float32)
    rc = lib().oracle_sq8_batch_distances_by_id(_p(codes, C.c_uint8), C.c_int64(codes.shape[0]),
                                                C.c_int64(codes.shape[1]), _p(_f32(mins), C.c_float),
                                                _p(_f32(scale), C.c_float), _p(queries, C.c_float),
                                                C.c_int64(queries.shape[0]), _p(ids, C.c_uint32),
                                                _p(qm, C.c_uint32), C.c_int64(ids.shape[0]), C.c_int(metric),
                                                C.c_int(int(exact)), _p(out, C.c_float))
    if rc != 0:
        raise ValueError("oracle_sq8_batch_distances_by_id: invalid arguments")
    return out


# --------------------------------------------------------------------------- flat
def round_storage(x, kind: str):
    """Rows as a reduced-precision flat index keeps them: rounded to nearest even to fp16 ("f16": the
    (__fp16) cast of faiss-metal/src/MetalIndexFlat.mm:228-236) or bf16 ("bf16": bits + 0x7FFF + lsb, then
    the upper half, :211-226), widened back to float32 (reconstruct, :461-478)."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    if kind == "f16":
        with np.errstate(over="ignore"):
            return x.astype(np.float16).astype(np.float32)
    if kind == "bf16":
        bits = x.view(np.uint32).astype(np.uint64)
        lsb = (bits >> 16) & 1
        return (((bits + 0x7FFF + lsb) >> 16) << 16).astype(np.uint32).view(np.float32).reshape(x.shape)
    raise ValueError(kind)


def flat_search(xb, xq, k: int, metric: int):
    """Exact top-k, distances accumulated in double (faiss-metal/src/MetalIndexFlat.mm:294-369)."""
    xb, xq = _f32(xb), _f32(xq)
    n = xb.shape[0]
    d = xb.shape[1] if xb.ndim == 2 else xq.shape[1]
    nq = xq.shape[0]
    D = np.empty((nq, k), np.float32)
    I = np.empty((nq, k), np.int64)
    rc = lib().oracle_flat_search(_p(xb, C.c_float), C.c_int64(n), C.c_int64(d), _p(xq, C.c_float), C.c_int64(nq),
                                  C.c_int64(k), C.c_int(metric), _p(D, C.c_float), _p(I, C.c_int64))
    if rc != 0:
        raise ValueError("oracle_flat_search: invalid arguments")
    return D, I


def all_distances(xb, q, metric: int):
    """Double-precision distance of one query to every row (squared L2 or raw dot)."""
    xb, q = _f32(xb), _f32(q)
    out = np.empty(xb.shape[0], np.float64)
    rc = lib().oracle_all_distances(_p(xb, C.c_float), C.c_int64(xb.shape[0]), C.c_int64(xb.shape[1]),
                                    _p(q, C.c_float), C.c_int(metric), _p(out, C.c_double))
    if rc != 0:
        raise ValueError("oracle_all_distances: invalid arguments")
    return out


def flat_search_blas(xb, xq, k: int, metric: int, block: int = 16384):
    """Blocked sgemm + heap form of a CPU flat search (the shape of FAISS's CPU
    path for batched queries): numpy's BLAS does Q.X^T per row block, the C heap
    merges.  This is the timed CPU baseline, not a parity reference."""
    xb, xq = _f32(xb), _f32(xq)
    nq = xq.shape[0]
    runD = np.full((nq, k), np.inf, np.float32)
    runI = np.full((nq, k), -1, np.int64)
    qn = (xq * xq).sum(1, dtype=np.float32) if metric == METRIC_L2 else None
    for s in range(0, xb.shape[0], block):
        blk = xb[s:s + block]
        keys = xq @ blk.T
        if metric == METRIC_L2:
            keys *= -2.0
            keys += (blk * blk).sum(1, dtype=np.float32)[None, :]
        else:
            np.negative(keys, out=keys)
        keys = np.ascontiguousarray(keys)
        lib().oracle_select_block(_p(keys, C.c_float), C.c_int64(nq), C.c_int64(blk.shape[0]), C.c_int64(s),
                                  C.c_int64(k), _p(runD, C.c_float), _p(runI, C.c_int64))
    if metric == METRIC_L2:
        D = np.where(runI >= 0, np.maximum(runD + qn[:, None], 0.0), np.inf).astype(np.float32)
    else:
        D = np.where(runI >= 0, -runD, -np.inf).astype(np.float32)
    return D, runI


# --------------------------------------------------------------------------- IVFFlat
def kmeans(x, nlist: int, niter: int = 10, seed: int = 1234):
    x = _f32(x)
    n, d = x.shape
    cent = np.empty((nlist, d), np.float32)
    rc = lib().oracle_kmeans(_p(x, C.c_float), C.c_int64(n), C.c_int64(d), C.c_int64(nlist), C.c_int(niter),
                             C.c_uint64(seed), _p(cent, C.c_float))
    if rc != 0:
        raise ValueError("oracle_kmeans: invalid arguments")
    return cent


def ivf_assign(x, centroids, metric: int):
    """Nearest centroid under the index metric (faiss-metal/src/MetalIndexIVFFlat.mm:102-120)."""
    x, centroids = _f32(x), _f32(centroids)
    out = np.empty(x.shape[0], np.int64)
    rc = lib().oracle_ivf_assign(_p(x, C.c_float), C.c_int64(x.shape[0]), C.c_int64(x.shape[1]),
                                 _p(centroids, C.c_float), C.c_int64(centroids.shape[0]), C.c_int(metric),
                                 _p(out, C.c_int64))
    if rc != 0:
        raise ValueError("oracle_ivf_assign: invalid arguments")
    return out


def lists_from_assign(assign, nlist: int):
    """CSR inverted lists; within a list rows keep add order."""
    assign = np.asarray(assign, np.int64)
    order = np.argsort(assign, kind="stable").astype(np.int64)
    counts = np.bincount(assign, minlength=nlist).astype(np.int64)
    off = np.zeros(nlist + 1, np.int64)
    np.cumsum(counts, out=off[1:])
    return off, order


def ivf_search(xb, centroids, list_off, list_rows, xq, k: int, nprobe: int, metric: int, fast: bool = False,
               return_probes: bool = False):
    """Probe the nprobe nearest centroids, exact top-k of their union
    (faiss-metal/src/MetalIndexIVFFlat.mm:122-256)."""
    xb, centroids, xq = _f32(xb), _f32(centroids), _f32(xq)
    list_off = np.ascontiguousarray(list_off, np.int64)
    list_rows = np.ascontiguousarray(list_rows, np.int64)
    nq, d = xq.shape
    nlist = centroids.shape[0]
    D = np.empty((nq, k), np.float32)
    I = np.empty((nq, k), np.int64)
    if fast:
        rc = lib().oracle_ivf_search_fast(_p(xb, C.c_float), C.c_int64(d), _p(centroids, C.c_float),
                                          C.c_int64(nlist), _p(list_off, C.c_int64), _p(list_rows, C.c_int64),
                                          _p(xq, C.c_float), C.c_int64(nq), C.c_int64(k), C.c_int64(nprobe),
                                          C.c_int(metric), _p(D, C.c_float), _p(I, C.c_int64))
        probes = None
    else:
        probes = np.empty((nq, min(nprobe, nlist)), np.int64) if return_probes else None
        rc = lib().oracle_ivf_search(_p(xb, C.c_float), C.c_int64(xb.shape[0]), C.c_int64(d),
                                     _p(centroids, C.c_float), C.c_int64(nlist), _p(list_off, C.c_int64),
                                     _p(list_rows, C.c_int64), _p(xq, C.c_float), C.c_int64(nq), C.c_int64(k),
                                     C.c_int64(nprobe), C.c_int(metric), _p(D, C.c_float), _p(I, C.c_int64),
                                     _p(probes, C.c_int64))
    if rc != 0:
        raise ValueError("oracle_ivf_search: invalid arguments")
    return (D, I, probes) if return_probes else (D, I)


def ivf_search_given_probes(xb, list_off, list_rows, xq, k: int, probes, metric: int):
    xb, xq = _f32(xb), _f32(xq)
    list_off = np.ascontiguousarray(list_off, np.int64)
    list_rows = np.ascontiguousarray(list_rows, np.int64)
    probes = np.ascontiguousarray(probes, np.int64)
    nq, d = xq.shape
    D = np.empty((nq, k), np.float32)
    I = np.empty((nq, k), np.int64)
    rc = lib().oracle_ivf_search_given_probes(_p(xb, C.c_float), C.c_int64(d), _p(list_off, C.c_int64),
                                              _p(list_rows, C.c_int64), _p(xq, C.c_float), C.c_int64(nq),
                                              C.c_int64(k), C.c_int64(probes.shape[1]), _p(probes, C.c_int64),
                                              C.c_int(metric), _p(D, C.c_float), _p(I, C.c_int64))
    if rc != 0:
        raise ValueError("oracle_ivf_search_given_probes: invalid arguments")
    return D, I


# ---- serialized DiskANN index (".diskann" v2 image, rust_lib/src/file_format.rs:3-18, with the
# ---- optional SQ8 trailer of rust_lib/src/index_manager.rs:513-533) ---------------------------
def write_diskann_image(vectors, adjacency, entry_points, metric: int = 0, build_complexity: int = 64, sq8=None) -> bytes:
    """vectors (n, d) float32; adjacency (n, max_degree) uint32 with 0xFFFFFFFF in unused slots;
    entry_points: ids; sq8 = (mins, scale, codes) appends the trailer.  All little-endian."""
    import struct
    v = np.ascontiguousarray(vectors, "<f4")
    a = np.ascontiguousarray(adjacency, "<u4")
    e = np.ascontiguousarray(entry_points, "<u4")
    out = bytearray()
    out += b"DANN" + struct.pack("<IIIII", 2, v.shape[0], v.shape[1], a.shape[1], len(e))
    out += struct.pack("<B3xI", metric, build_complexity)
    assert len(out) == 32
    out += e.tobytes() + v.tobytes() + a.tobytes()
    if sq8 is not None:
        mins, scale, codes = sq8
        codes = np.ascontiguousarray(codes, np.uint8)
        out += b"SQ8\0" + struct.pack("<IQ", v.shape[1], codes.size)
        out += np.ascontiguousarray(mins, "<f4").tobytes() + np.ascontiguousarray(scale, "<f4").tobytes()
        out += codes.tobytes()
    return bytes(out)


def parse_diskann_image(image: bytes) -> dict:
    """Restates FileHeader::read and InMemoryIndex::from_bytes (rust_lib/src/index_manager.rs:560-668):
    returns the header fields, the segments as arrays and, if present, the SQ8 section."""
    import struct
    if len(image) < 32 or image[:4] != b"DANN":
        raise ValueError("not a .diskann image")
    version, n, d, deg, ne = struct.unpack_from("<IIIII", image, 4)
    metric = image[24]
    (bc,) = struct.unpack_from("<I", image, 28)
    if version != 2:
        raise ValueError("unsupported version")
    off = 32
    entry = np.frombuffer(image, "<u4", ne, off)
    off += ne * 4
    if off + n * d * 4 + n * deg * 4 > len(image):
        raise ValueError("truncated")
    vec = np.frombuffer(image, "<f4", n * d, off).reshape(n, d)
    off += n * d * 4
    adj = np.frombuffer(image, "<u4", n * deg, off).reshape(n, deg)
    off += n * deg * 4
    res = {"num_vectors": n, "dimension": d, "max_degree": deg, "metric": metric, "build_complexity": bc,
           "entry_points": entry, "vectors": vec, "adjacency": adj, "standard_size": off, "sq8": None}
    if len(image) > off + 4 and image[off:off + 4] == b"SQ8\0":
        sq_dim, qlen = struct.unpack_from("<IQ", image, off + 4)
        p = off + 16
        if p + sq_dim * 8 + qlen > len(image):
            raise ValueError("SQ8 section truncated")
        mins = np.frombuffer(image, "<f4", sq_dim, p)
        scale = np.frombuffer(image, "<f4", sq_dim, p + sq_dim * 4)
        codes = np.frombuffer(image, np.uint8, qlen, p + sq_dim * 8).reshape(n, sq_dim)
        res["sq8"] = (mins, scale, codes)
    return res


def disk_search_batch(image: bytes, queries, k: int, l_search: int, use_sq8: bool = False):
    """Restates DiskProvider::search_batch (rust_lib/src/disk_provider.rs:470-652) with its
    insert_result (:655-678): lock-step best-first search, one popped candidate per active query and
    iteration, the unvisited neighbours of all of them scored together.  Distances in double
    (`exact`), squared L2 or negated dot as rust_lib/src/distance.rs:15-25 returns them.  Pure
    Python loops: small cases only.  Returns a list of (ids, distances) per query."""
    import bisect
    import heapq
    im = parse_diskann_image(image)
    n, deg, metric = im["num_vectors"], im["max_degree"], (BATCH_L2 if im["metric"] == 0 else BATCH_IP)
    queries = _f32(queries)
    nq = queries.shape[0]
    if nq == 0 or n == 0 or k <= 0:
        return [(np.zeros(0, np.uint64), np.zeros(0, np.float32)) for _ in range(nq)]
    k = min(k, n)
    l = max(l_search, k)
    if use_sq8:
        mins, scale, codes = im["sq8"]

    def score(ids, qmap):
        ids, qmap = np.asarray(ids, np.uint32), np.asarray(qmap, np.uint32)
        if use_sq8:
            return sq8_batch_distances_by_id(codes, mins, scale, queries, ids, qmap, metric, exact=True)
        return batch_distances_by_id(im["vectors"], queries, ids, qmap, metric, exact=True)

    visited = [set() for _ in range(nq)]
    cands = [[] for _ in range(nq)]
    result = [[] for _ in range(nq)]      # sorted (dist, id), at most l
    active = [True] * nq
    ids, qmap = [], []
    for q in range(nq):
        for ep in im["entry_points"].tolist():
            if ep < n and ep not in visited[q]:
                visited[q].add(ep)
                ids.append(ep); qmap.append(q)
    for d, i, q in zip(score(ids, qmap).tolist() if ids else [], ids, qmap):
        d = float(np.float32(d))
        heapq.heappush(cands[q], (d, i))
        result[q].append((d, i))
    for q in range(nq):
        result[q].sort(key=lambda t: t[0])
    while True:
        ids, qmap = [], []
        any_active = False
        for q in range(nq):
            if not active[q]:
                continue
            if not cands[q]:
                active[q] = False
                continue
            c_dist, c_id = heapq.heappop(cands[q])
            if len(result[q]) >= l and c_dist > result[q][l - 1][0]:
                active[q] = False
                continue
            any_active = True
            for v in im["adjacency"][c_id].tolist():
                if v >= n or v in visited[q]:
                    continue
                visited[q].add(v)
                ids.append(v); qmap.append(q)
        if not any_active:
            break
        if not ids:
            continue
        for d, i, q in zip(score(ids, qmap).tolist(), ids, qmap):
            d = float(np.float32(d))
            r = result[q]
            if len(r) < l or d < r[-1][0]:
                pos = bisect.bisect_left([t[0] for t in r], d)
                r.insert(pos, (d, i))
                del r[l:]
                heapq.heappush(cands[q], (d, i))
    return [(np.array([t[1] for t in result[q][:k]], np.uint64), np.array([t[0] for t in result[q][:k]], np.float32))
            for q in range(nq)]
