#!/usr/bin/env python
"""Benchmark of the GPU search path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Under `python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N` every rank
owns one GPU and one shard; rank 0 prints ONE JSON line.

Workloads (synthetic, seeded; shapes of the reference configurations):
  flat_ip_20m   (default) Flat inner product, 20,000,000 x 768 unit-norm rows, 4,096 queries, k=100,
                rows sharded over the ranks, per-shard top-k merged after an all-gather.  STRONG scaling.
  flat_l2_100k  Flat L2, 100,000 x 384 uniform[0,1) rows, 1,000 queries, k=10.
  ivf_1m        IVFFlat L2, 1,000,000 x 768 rows from 1,024 Gaussian clusters, nlist=1024, nprobe=16,
                10,000 queries, k=100, inverted lists sharded over the ranks.
  batch_c2      DiskANN batch distance, table 1,000,000 x 1536, 256 queries x 128 random rows (L2).
  sq8_c5        SQ8 asymmetric L2, 10,000,000 x 384 codes, 1,024 queries x 128 random rows.
A step is one pass of the hot path over one batch of queries.  `value` is measured with the
inputs resident in HBM; `e2e` goes through the host-pointer C-ABI call (or, for N > 1, pinned-host
copies around the sharded search) with the copies inside the timed region.

Without --workload the line is the headline workload (flat_ip_20m) and carries a `workloads`
object with the other configurations measured the same way in the same run (N = 1: all four;
N > 1: ivf_1m with its lists sharded over the ranks).  Every entry has `value`, `ms_per_step`,
`roofline`, `e2e`, `clocks`, `parity_check` and, at N = 1, `cpu_baseline`.  `parity_check` compares
a sample of the timed output with the exact-fp32 scan kernel over the same shard(s) and with the
CPU oracle; a mismatch makes the run fail after the line is printed.
"""
from __future__ import annotations

import os
import sys


def _host_cores() -> int:
    return len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)


# The CPU arm uses every host core.  torchrun exports OMP_NUM_THREADS=1 to its workers, and numpy's
# BLAS reads the variable when it is first imported - so it is corrected here, before that import.
if "reference" in sys.argv[1:]:
    for _v in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ[_v] = str(_host_cores())

import argparse  # noqa: E402
import importlib.util  # noqa: E402
import json  # noqa: E402
import statistics  # noqa: E402
import subprocess  # noqa: E402
import threading  # noqa: E402
import time  # noqa: E402

import numpy as np  # noqa: E402

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def load_package():
    name = "duckdb_ann_b200"
    if name in sys.modules:
        return sys.modules[name]
    pkg_dir = os.path.join(ROOT, "duckdb-ann_b200")
    spec = importlib.util.spec_from_file_location(name, os.path.join(pkg_dir, "__init__.py"),
                                                  submodule_search_locations=[pkg_dir])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "_source": "fallback"}


# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def wait_first_sample(self, timeout=3.0):
        t0 = time.perf_counter()
        while not self.lines and time.perf_counter() - t0 < timeout:
            time.sleep(0.02)

    def mark(self):
        return time.perf_counter()

    def stop(self, t_begin=None, t_end=None):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        in_region = [l for (t, l) in self.lines if t_begin is None or (t_begin <= t <= t_end + 0.15)]
        where = "timed region"
        if not in_region:  # region shorter than the sampling period: use the samples taken under the warm-up load
            in_region = [l for (_, l) in self.lines]
            where = "warm-up + timed region (timed region shorter than the 100 ms sampling period)"
        for line in in_region:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower() == "active":
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "sampled_over": where}


def dist_info(args):
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return rank, local, world


def unit_rows(gen_seed, rows, d, device, torch):
    g = torch.Generator(device=device).manual_seed(gen_seed)
    x = torch.randn((rows, d), generator=g, device=device, dtype=torch.float32)
    x /= x.norm(dim=1, keepdim=True)
    return x


# ------------------------------------------------------------------------------------------------
# Parity of the timed output (the acceptance rule of the parity tests: distances within 1e-4
# relative; id sets identical except for tolerance ties at the k-th place)
# ------------------------------------------------------------------------------------------------
RTOL = 1e-4


def compare_topk(D, I, Dref, Iref, larger_is_better):
    """Both (nq, k), best first.  Returns (id mismatches that are not tolerance ties, max relative
    distance error position by position)."""
    D, Dref = np.asarray(D, np.float64), np.asarray(Dref, np.float64)
    mism = 0
    for q in range(D.shape[0]):
        got, want = set(I[q][I[q] >= 0].tolist()), set(Iref[q][Iref[q] >= 0].tolist())
        if got == want:
            continue
        valid = Iref[q] >= 0
        kth = Dref[q][valid][-1] if valid.any() else 0.0
        band = 2 * RTOL * abs(kth) + 1e-30
        dist_of = {int(i): float(d) for i, d in zip(I[q], D[q])}
        dist_of.update({int(i): float(d) for i, d in zip(Iref[q], Dref[q])})
        mism += sum(1 for i in got ^ want if abs(dist_of[i] - kth) > band)
    fin = np.isfinite(Dref) & np.isfinite(D)
    rel = np.abs(D - Dref)[fin] / np.maximum(np.abs(Dref)[fin], 1e-30)
    return int(mism), float(rel.max()) if rel.size else 0.0


def gather_and_merge(torch, dist, D, I, world, larger_is_better):
    """Per-rank (nq, k) results of a sample -> the global top k on every rank (plain torch: this is
    the checker, not the product's merge kernel)."""
    if world == 1:
        return D, I
    gd = [torch.empty_like(D) for _ in range(world)]
    gi = [torch.empty_like(I) for _ in range(world)]
    dist.all_gather(gd, D.contiguous())
    dist.all_gather(gi, I.contiguous())
    allD, allI = torch.cat(gd, 1), torch.cat(gi, 1)
    key = -allD if larger_is_better else allD
    key = torch.where(allI < 0, torch.full_like(key, float("inf")), key)
    order = torch.argsort(key, dim=1, stable=True)[:, :D.shape[1]]
    return torch.gather(allD, 1, order), torch.gather(allI, 1, order)


def search_sample_exact(wl, torch, dist, sample, label_offset):
    """The sample queries through the library's exact-fp32 scan kernels (no tensor cores) over this
    rank's shard, merged over the ranks."""
    lib = wl.pkg.lib()
    qs = wl.q_dev[torch.from_numpy(sample).to(wl.q_dev.device)].contiguous()
    assert lib.ann_cuda_set_flat_kernel(b"simt") == 0
    try:
        Ds, Is = wl.index.search_device(qs, wl.k, label_offset=label_offset)
        wl.index.search_status()
    finally:
        lib.ann_cuda_set_flat_kernel(b"tcgen05")
    return gather_and_merge(torch, dist, Ds, Is, wl.world, wl.metric_name == "IP")


# ------------------------------------------------------------------------------------------------
# Workloads
# ------------------------------------------------------------------------------------------------
class FlatWorkload:
    def __init__(self, name, n, d, nq, k, metric_name, dist_kind, scale=1.0, storage="f32"):
        self.name, self.d, self.nq, self.k = name, d, nq, k
        # "f16" / "bf16": the rows are kept rounded to that type (2 bytes per element) and the search
        # answers for the rounded rows - a variant of the workload, never part of the default run
        self.storage = storage
        self.n = max(1024, int(n * scale))
        self.metric_name, self.dist_kind = metric_name, dist_kind
        self.chunk = 250_000
        self.metric = "flat_topk_queries_per_s"
        self.unit = "queries/s"
        self.dtype = "f32 (TF32 tensor cores with fp32 accumulate for candidate selection, exact fp32 re-ranking)"
        self.scaling = "strong"

    def gen_chunk(self, c, device, torch):
        """Rows [c*chunk, (c+1)*chunk) of the global database, the same on any rank count."""
        rows = min(self.chunk, self.n - c * self.chunk)
        if self.dist_kind == "unit":
            return unit_rows(1000 + c, rows, self.d, device, torch)
        g = torch.Generator(device=device).manual_seed(1000 + c)
        return torch.rand((rows, self.d), generator=g, device=device, dtype=torch.float32)

    def queries_host(self, torch):
        g = torch.Generator().manual_seed(43)
        if self.dist_kind == "unit":
            q = torch.randn((self.nq, self.d), generator=g)
            q /= q.norm(dim=1, keepdim=True)
        else:
            q = torch.rand((self.nq, self.d), generator=g)
        q = q.contiguous()
        return q.pin_memory() if torch.cuda.is_available() else q

    def setup(self, pkg, torch, rank, world, device):
        self.pkg = pkg
        m = pkg.METRIC_INNER_PRODUCT if self.metric_name == "IP" else pkg.METRIC_L2
        self.m = m
        lo, hi = pkg.sharded.row_range(self.n, rank, world)
        self.lo, self.hi = lo, hi
        self.index = pkg.CudaIndexFlat(self.d, m, device.index,
                                       {"f32": pkg.STORAGE_F32, "f16": pkg.STORAGE_F16, "bf16": pkg.STORAGE_BF16}[self.storage])
        self.index.reserve(hi - lo)
        c0, c1 = lo // self.chunk, (hi - 1) // self.chunk
        for c in range(c0, c1 + 1):
            x = self.gen_chunk(c, device, torch)
            a, b = max(lo, c * self.chunk) - c * self.chunk, min(hi, (c + 1) * self.chunk) - c * self.chunk
            self.index.add_device(x[a:b].contiguous())
            del x
        assert self.index.ntotal == hi - lo
        self.q_host = self.queries_host(torch)
        self.q_dev = self.q_host.to(device)
        self.searcher = pkg.sharded.ShardedSearcher(self.index, m, label_offset=lo)
        self.out_host_d = torch.empty((self.nq, self.k), dtype=torch.float32).pin_memory()
        self.out_host_i = torch.empty((self.nq, self.k), dtype=torch.int64).pin_memory()
        self.world = world

    def step(self):
        return self.searcher.search(self.q_dev, self.k)

    def step_e2e(self, torch):
        if self.world == 1:
            # the reference-facing call: host buffers in, host buffers out, synchronous
            return self.index.search(self.q_host.numpy(), self.k)
        q = self.q_host.to(self.q_dev.device, non_blocking=True)
        D, I = self.searcher.search(q, self.k)
        self.out_host_d.copy_(D, non_blocking=True)
        self.out_host_i.copy_(I, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.out_host_d, self.out_host_i

    def units_per_step(self):
        return self.nq

    def e2e_bytes(self):
        return self.nq * self.d * 4, self.nq * self.k * 12

    def config(self, world):
        return {"workload": self.name, "rows": self.n, "dim": self.d, "queries": self.nq, "k": self.k,
                "metric": self.metric_name, "sharding": f"rows/{world}", "distribution": self.dist_kind,
                "l2_flush": "database shard (>= 7 GB per GPU) is far larger than L2; no explicit flush"
                if self.n * self.d * 8 / max(world, 1) > 1e9 else "database is L2-sized (a warm-cache figure; the full-size workload is the headline)",
                "flat_kernel": self.pkg.lib().ann_cuda_flat_kernel_name().decode() if getattr(self, "pkg", None)
                else "cpu",
                "storage": self.storage,
                "search": "CPU: blocked sgemm distances + heap select over all host threads (the oracle's port of the FAISS CPU path)"
                if not getattr(self, "pkg", None) else
                "one-MMA screening (stores >= 2M rows, k <= 224), else three-MMA split product; banded candidate "
                          "lists, exact fp32 re-ranking, band check with fallback one tier up"
                if self.storage == "f32" else
                "16-bit rows (rounded when added), tcgen05 kind::f16 with one 16-bit part of the query per product, then two; "
                "banded candidate lists, exact fp32 re-ranking against the rounded rows, band check with fallback one tier up"}

    def roofline(self, peaks, kernel_ms):
        local_rows = self.hi - self.lo
        flops = 2.0 * self.nq * local_rows * self.d
        achieved = flops / (kernel_ms * 1e-3) / 1e12 if kernel_ms and kernel_ms > 0 else None
        # Stores of two million rows or more are searched with one-MMA screening (one TF32 MMA per
        # product, candidates re-ranked exactly); smaller ones with the three-MMA split product.
        screened = local_rows >= 2_000_000 and self.k <= 224 and self.pkg.lib().ann_cuda_flat_kernel_name().decode() == "tcgen05"
        mmas = 1 if screened else 3
        peak = peaks["bf16_tflops_sustained"] / 2.0 / mmas
        if self.storage != "f32":
            # 16-bit operands (kind::f16): one MMA per product at the bf16 rate itself
            return {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_tflops_sustained"], "unit": "TFLOP/s",
                    "frac": achieved / peaks["bf16_tflops_sustained"] if achieved else None, "traffic": None,
                    "traffic_note": "no capture for this storage type",
                    "kernel": "flat_tc_kernel (16-bit operands, one MMA per product)", "kernel_ms": kernel_ms,
                    "algorithmic_flops_per_launch": flops, "mma_per_product": 1,
                    "peak_note": f"{peaks['_source']} bf16 sustained {peaks['bf16_tflops_sustained']} TFLOP/s; 'achieved' counts 2*Q*N*d once"}
        # DRAM traffic of one launch.  Screened search: ncu capture of the full-size launch (20M rows of
        # 768 floats, 4,096 queries: 67.5 GB read + 1.2 GB written; the hi planes are 61.4 GB and are
        # read once for all query tiles), scaled by the rows of this launch.  That capture was taken
        # once with three one-pass metrics (a launch that holds 123 GB on the device is not captured
        # with more); the loads it measures have not changed since.  What is re-captured with every
        # change of the kernel is the 400,000-row case (profiles/flat_tc_kernel__flat_ip_20m.md).  Split product: captures
        # on 400,000 rows with 4,096 queries (16.2-22.3 GB + 0.47-0.49 GB), scaled by rows and query
        # tiles: there every 128-query tile streams the shard and L2 absorbs part of it.
        traffic, note = None, "no capture for this shape"
        if self.d == 768 and screened:
            traffic = 68.7e9 * (local_rows / 20_000_000.0)
            note = "bytes; ncu dram read+write of the 20M-row launch scaled by rows"
        elif self.d == 768:
            traffic = 19.7e9 * (local_rows / 400_000.0) * (((self.nq + 127) // 128) / 32.0)
            note = "bytes; ncu dram read+write of a 400,000-row launch scaled by rows and query tiles"
        return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak if achieved else None, "traffic": traffic,
                "traffic_note": note,
                "kernel": "flat_tc_kernel" + (" (screened, 32-float K blocks)" if screened else ""),
                "kernel_ms": kernel_ms, "algorithmic_flops_per_launch": flops, "mma_per_product": mmas,
                "peak_note": f"{peaks['_source']} bf16 sustained {peaks['bf16_tflops_sustained']} TFLOP/s / 2 (TF32 rate)"
                             + (" (screened search: one TF32 MMA per product)" if screened else
                                " / 3 (split-TF32 issues three MMAs per product)")
                             + "; 'achieved' counts 2*Q*N*d once; the denominator is a library GEMM under the board's "
                               "power cap, not a hardware limit: a kernel that moves fewer bytes per flop through shared "
                               "memory (pair mode) can exceed it",
                # cuBLAS's own TF32 GEMM on this pool (8192^3 through torch.matmul, CUDA events): the same kind of
                # figure as the bf16 peaks, measured directly for this operand type
                "cublas_tf32_tflops": {"burst": 753.5, "sustained": 636.1, "source": "profiles/tf32_peak.md"}}

    def parity_check(self, torch, dist, D, I, oracle):
        """Size-independent properties over the whole output (sorted best first, labels valid and
        distinct); 32 of the queries against the exact-fp32 scan kernel over the full store (all
        shards) and, on rank 0, against the CPU oracle on a slice of the rows."""
        Dh, Ih = D.cpu().numpy(), I.cpu().numpy()
        ip = self.metric_name == "IP"
        assert (np.diff((-1.0 if ip else 1.0) * Dh, axis=1) >= 0).all(), "results are not sorted best first"
        assert (Ih >= 0).all() and (Ih < self.n).all()
        assert all(len(set(r.tolist())) == len(r) for r in Ih[:64]), "duplicate labels"
        sample = np.unique(np.linspace(0, self.nq - 1, 32).astype(np.int64))
        Ds, Is = search_sample_exact(self, torch, dist, sample, self.lo)
        mism, err = compare_topk(Dh[sample], Ih[sample], Ds.cpu().numpy(), Is.cpu().numpy(), ip)
        res = {"queries": int(len(sample)), "id_mismatches": mism, "max_rel_err": err,
               "against": "exact-fp32 scan kernel over the full store (ids outside a 1e-4 tolerance tie at the k-th place count as mismatches)"}
        if oracle is not None:
            # CPU oracle over a slice of this rank's rows: every oracle hit that beats the reported
            # k-th distance by more than the tolerance must have been reported, at the same distance
            rows = min(self.hi - self.lo, 200_000)
            xb = self.index.get_rows(0, rows)
            m = oracle.METRIC_IP if ip else oracle.METRIC_L2
            Do, Io = oracle.flat_search(xb, self.q_host.numpy()[sample], self.k, m)
            missing, oerr = 0, 0.0
            for j, q in enumerate(sample):
                kth = float(Dh[q, -1])
                reported = {int(i): float(d) for i, d in zip(Ih[q], Dh[q])}
                for lab, do in zip(Io[j], Do[j]):
                    if lab < 0:
                        continue
                    lab = int(lab) + self.lo
                    do = float(do)
                    better = (do - kth) if ip else (kth - do)
                    if lab in reported:
                        oerr = max(oerr, float(abs(reported[lab] - do) / max(abs(do), 1e-30)))
                    elif better > 2 * RTOL * abs(kth):
                        missing += 1
            res.update({"oracle_rows": int(rows), "oracle_missing": missing, "oracle_max_rel_err": oerr})
        res["ok"] = bool(mism == 0 and err <= RTOL and res.get("oracle_missing", 0) == 0
                         and res.get("oracle_max_rel_err", 0.0) <= RTOL)
        return res

    def close(self):
        self.index.close()

    # ---- CPU baseline: blocked sgemm + heap on the host cores, on a bounded sample
    def cpu_sample(self, torch, device):
        rows = min(self.n, 2_000_000 if self.n > 2_000_000 else self.n)
        nq = min(self.nq, 1024 if self.n > 2_000_000 else self.nq)
        parts = []
        for c in range((rows + self.chunk - 1) // self.chunk):
            x = self.gen_chunk(c, device, torch)
            parts.append(x[: min(self.chunk, rows - c * self.chunk)].cpu().numpy())
            del x
        xb = np.concatenate(parts)
        xq = self.queries_host(torch).numpy()[:nq].copy()
        return xb, xq, rows, nq

    def cpu_run(self, oracle, sample):
        xb, xq, rows, nq = sample
        m = oracle.METRIC_IP if self.metric_name == "IP" else oracle.METRIC_L2
        t0 = time.perf_counter()
        oracle.flat_search_blas(xb, xq, self.k, m)
        dt = time.perf_counter() - t0
        # queries/s over the FULL database: time scales with the number of rows scanned
        qps = nq / (dt * (self.n / rows))
        return qps, dt, f"{nq} queries x {rows:,} of {self.n:,} rows (blocked sgemm + heap), time scaled x{self.n / rows:g}"


# DRAM read + write bytes of one grouped list-scan launch, keyed by (rows, queries, GPUs), from the
# ncu capture of the grouped list scan at the default shape (10.0-10.1 GB read + 0.23 GB written with the
# lists kept as one fp32 plane; 14.6-14.8 GB + 0.2 GB while they were two TF32 planes)
IVF_SCAN_TRAFFIC = {(1_000_000, 10_000, 1): 10.3e9}


class IvfWorkload:
    def __init__(self, scale=1.0):
        self.name = "ivf_1m"
        self.n = max(20_000, int(1_000_000 * scale))
        self.d, self.nlist, self.nprobe, self.k = 768, 1024, 16, 100
        self.nq = max(256, int(10_000 * scale))
        self.nclusters = 1024
        self.chunk = 100_000
        self.metric = "ivfflat_topk_queries_per_s"
        self.unit = "queries/s"
        self.dtype = "f32"
        self.scaling = "strong"
        self.metric_name = "L2"

    def centers(self, device, torch):
        g = torch.Generator(device=device).manual_seed(45)
        return torch.randn((self.nclusters, self.d), generator=g, device=device)

    def gen_chunk(self, c, device, torch, centers):
        rows = min(self.chunk, self.n - c * self.chunk)
        g = torch.Generator(device=device).manual_seed(2000 + c)
        lab = torch.randint(0, self.nclusters, (rows,), generator=g, device=device)
        return centers[lab] + 0.1 * torch.randn((rows, self.d), generator=g, device=device)

    def setup(self, pkg, torch, rank, world, device):
        self.pkg, self.world = pkg, world
        self.m = pkg.METRIC_L2
        centers = self.centers(device, torch)
        self.index = pkg.CudaIndexIVFFlat(self.d, self.nlist, pkg.METRIC_L2, device.index)
        self.index.set_shard(rank, world)
        # train on every 10th row (the train_sample rule of src/faiss_index.cpp:304-315), same on every rank
        sample = torch.cat([self.gen_chunk(c, device, torch, centers)[::10] for c in
                            range((self.n + self.chunk - 1) // self.chunk)])
        self.index.train(sample.cpu().numpy())
        del sample
        for c in range((self.n + self.chunk - 1) // self.chunk):
            self.index.add_device(self.gen_chunk(c, device, torch, centers).contiguous())
        self.index.setNprobe(self.nprobe)
        g = torch.Generator(device=device).manual_seed(43)
        lab = torch.randint(0, self.nclusters, (self.nq,), generator=g, device=device)
        q = centers[lab] + 0.1 * torch.randn((self.nq, self.d), generator=g, device=device)
        self.q_host = q.cpu().contiguous().pin_memory()
        self.q_dev = q.contiguous()
        self.searcher = pkg.sharded.ShardedSearcher(self.index, pkg.METRIC_L2)
        self.out_host_d = torch.empty((self.nq, self.k), dtype=torch.float32).pin_memory()
        self.out_host_i = torch.empty((self.nq, self.k), dtype=torch.int64).pin_memory()
        sizes = np.array([self.index.list_size(l) for l in range(self.nlist)], np.int64)
        self.list_sizes = sizes
        # algorithmic scan work of one step: every query reads every row of every list it probes.
        # Probe lists come from the index's own coarse quantiser; list sizes are the global ones
        # (each rank scans the lists it owns, together they scan all of them).
        if rank == 0:
            probes = self.index.coarse(self.q_host.numpy(), self.nprobe)
            self.probes = probes
        else:
            self.probes = None
        self.global_list_sizes = sizes.copy()
        if world > 1:
            import torch.distributed as dist
            t = torch.from_numpy(sizes).to(device)
            dist.all_reduce(t)
            self.global_list_sizes = t.cpu().numpy()
        if rank == 0:
            self.rows_scanned = int(self.global_list_sizes[self.probes[self.probes >= 0]].sum())
        else:
            self.rows_scanned = 0

    def step(self):
        return self.searcher.search(self.q_dev, self.k)

    step_e2e = FlatWorkload.step_e2e

    def units_per_step(self):
        return self.nq

    def e2e_bytes(self):
        return self.nq * self.d * 4, self.nq * self.k * 12

    def config(self, world):
        return {"workload": self.name, "rows": self.n, "dim": self.d, "queries": self.nq, "k": self.k,
                "nlist": self.nlist, "nprobe": self.nprobe, "metric": "L2", "sharding": f"lists/{world}",
                "l2_flush": "probed lists (3 GB of rows) exceed L2; no explicit flush"}

    def roofline(self, peaks, kernel_ms):
        # List scan.  Algorithmic bytes = every query reads every row of the lists it probes
        # (rows scanned x d x 4, per GPU).  The kernel gathers the queries probing a list into
        # tiles of 128 and reads a list row once per tile, on the tensor cores, so the
        # algorithmic rate EXCEEDS the HBM peak by design (frac > 1); `traffic` is what DRAM
        # really moved (~4 TB/s of it at the full size; the launch is bound by shared-memory bandwidth now), and `tensor` restates
        # the same launch against the MMA roofline (useful flops = 2 d per (query, row) pair; tile
        # padding not counted).
        pairs = self.rows_scanned / max(self.world, 1)
        alg_bytes = pairs * self.d * 4
        secs = kernel_ms * 1e-3 if kernel_ms and kernel_ms > 0 else None
        achieved = alg_bytes / 1e9 / secs if secs else None
        tpeak = peaks["bf16_tflops_sustained"] / 6.0
        tflops = 2.0 * pairs * self.d / secs / 1e12 if secs else None
        return {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / peaks["hbm_gbs"] if achieved else None,
                "traffic": IVF_SCAN_TRAFFIC.get((self.n, self.nq, self.world)),
                "kernel": "flat_tc_kernel (grouped list scan)", "kernel_ms": kernel_ms,
                "algorithmic_bytes_per_launch": alg_bytes,
                "frac_of_nominal_8000": achieved / 8000.0 if achieved else None,
                "tensor": {"achieved": tflops, "peak": tpeak, "unit": "TFLOP/s",
                           "frac": tflops / tpeak if tflops else None,
                           "peak_note": f"{peaks['_source']} bf16 sustained / 2 (TF32) / 3 (split-TF32)"},
                "note": "queries probing one list share its rows through 128-query tensor-core tiles, so the "
                        "algorithmic figure exceeds 1; physically the launch is bound by its DRAM traffic "
                        "(`traffic` / kernel time, against the same peak)",
                "traffic_gbs": (IVF_SCAN_TRAFFIC.get((self.n, self.nq, self.world), 0) / 1e9 / secs
                                if secs and IVF_SCAN_TRAFFIC.get((self.n, self.nq, self.world)) else None)}

    def parity_check(self, torch, dist, D, I, oracle):
        """Sortedness and label range over the whole output; 32 queries against the exact-fp32 scan
        kernel over the same probe lists (all shards) and, at one GPU, against the CPU oracle run
        with the index's own centroids, lists and nprobe."""
        Dh, Ih = D.cpu().numpy(), I.cpu().numpy()
        assert (np.diff(Dh, axis=1) >= 0).all()
        assert (Ih >= 0).all() and (Ih < self.n).all()
        sample = np.unique(np.linspace(0, self.nq - 1, 32).astype(np.int64))
        Ds, Is = search_sample_exact(self, torch, dist, sample, 0)
        mism, err = compare_topk(Dh[sample], Ih[sample], Ds.cpu().numpy(), Is.cpu().numpy(), False)
        res = {"queries": int(len(sample)), "id_mismatches": mism, "max_rel_err": err,
               "against": "exact-fp32 scan kernel over the same probe lists"}
        if oracle is not None and getattr(self, "_cpu_sample", None) is not None:
            xb, cent, off, rows, _, _ = self._cpu_sample
            Do, Io = oracle.ivf_search(xb, cent, off, rows, self.q_host.numpy()[sample], self.k, self.nprobe,
                                       oracle.METRIC_L2)
            omism, oerr = compare_topk(Dh[sample], Ih[sample], Do, Io, False)
            # (a query whose nprobe-th and (nprobe+1)-th centroids tie may take either probe set)
            res.update({"oracle_id_mismatches": omism, "oracle_max_rel_err": oerr,
                        "oracle": "CPU oracle, same centroids, lists and nprobe"})
        res["ok"] = bool(mism == 0 and err <= RTOL)
        return res

    def close(self):
        self.index.close()

    # ---- CPU baseline: per-query list scan with a heap, OpenMP over queries, same centroids and lists
    def cpu_sample(self, torch, device):
        nq = min(self.nq, 4000)
        cent = self.index.get_centroids()
        xb = np.empty((self.n, self.d), np.float32)
        off = np.zeros(self.nlist + 1, np.int64)
        rows = []
        for l in range(self.nlist):
            ids, vecs = self.index.get_list(l)
            xb[ids] = vecs
            rows.append(ids)
            off[l + 1] = off[l] + len(ids)
        self._cpu_sample = (xb, cent, off, np.concatenate(rows), self.q_host.numpy()[:nq].copy(), nq)
        return self._cpu_sample

    def cpu_run(self, oracle, sample):
        xb, cent, off, rows, xq, nq = sample
        t0 = time.perf_counter()
        oracle.ivf_search(xb, cent, off, rows, xq, self.k, self.nprobe, oracle.METRIC_L2, fast=True)
        dt = time.perf_counter() - t0
        return nq / dt, dt, f"{nq} of {self.nq} queries, full index (per-query fp32 list scan + heap, OpenMP over queries)"


class BatchWorkload:
    def __init__(self, sq8: bool, scale=1.0):
        self.sq8 = sq8
        if sq8:
            self.name, self.num, self.dim, self.nq, self.per = "sq8_c5", int(10_000_000 * scale), 384, 1024, 128
        else:
            self.name, self.num, self.dim, self.nq, self.per = "batch_c2", int(1_000_000 * scale), 1536, 256, 128
        self.metric = "batch_distance_gbytes_per_s"
        self.unit = "GB/s"
        self.dtype = "u8 codes -> f32" if sq8 else "f32"
        self.scaling = "weak"
        self.metric_name = "L2"
        self.batches = 64  # distinct id batches cycled through, so consecutive launches touch different rows

    def setup(self, pkg, torch, rank, world, device):
        self.pkg = pkg
        g = torch.Generator(device=device).manual_seed(42 + rank)
        br = pkg.diskann_bridge
        if self.sq8:
            x = torch.randn((self.num, self.dim), generator=g, device=device)
            mins = x.min(0).values
            scale = x.max(0).values - mins
            codes = torch.clamp(torch.round(((x - mins) / scale) * 255.0), 0, 255).to(torch.uint8).contiguous()
            del x
            self.mins_host, self.scale_host = mins.cpu().numpy(), scale.cpu().numpy()
            self.table = br.DeviceTable.sq8_from_device(codes, self.mins_host, self.scale_host)
            self.row_bytes = self.dim
        else:
            rows = torch.randn((self.num, self.dim), generator=g, device=device)
            self.table = br.DeviceTable.from_device(rows)
            self.row_bytes = self.dim * 4
        total = self.nq * self.per
        self.q_dev = torch.randn((self.nq, self.dim), generator=g, device=device)
        self.ids = [torch.randint(0, self.num, (total,), generator=g, device=device, dtype=torch.int32)
                    for _ in range(self.batches)]
        self.qmap = torch.arange(self.nq, device=device, dtype=torch.int32).repeat_interleave(self.per)
        self.out = torch.empty(total, dtype=torch.float32, device=device)
        self.q_host = self.q_dev.cpu().numpy()
        self.ids_host = [i.cpu().numpy().astype(np.uint32) for i in self.ids[:4]]
        self.qmap_host = self.qmap.cpu().numpy().astype(np.uint32)
        self.it = 0
        self.total = total

    def bytes_per_step(self):
        # rows + queries + ids, map, out
        return self.total * self.row_bytes + self.nq * self.dim * 4 + self.total * 12 + (2 * self.dim * 4 if self.sq8 else 0)

    def step(self):
        ids = self.ids[self.it % self.batches]
        self.it += 1
        return self.table.batch_distances_by_id_device(self.q_dev, ids, self.qmap, 0, out=self.out), None

    def prepare_stream_of_batches(self, torch, steps):
        """The timed region of this workload is ONE multi-batch launch of `steps` batches (each
        on its own row ids and its own output): a single batch is shorter than a few launch
        latencies, so the steady-state rate is measured on a stream of back-to-back batches."""
        self.outs = [torch.empty(self.total, dtype=torch.float32, device=self.q_dev.device) for _ in range(min(steps, 8))]
        # every batch of the launch gets row ids of its own: with repeated ids two batches in
        # flight at once would share their rows through L2
        g = torch.Generator(device=self.q_dev.device).manual_seed(4242)
        while len(self.ids) < steps:
            self.ids.append(torch.randint(0, self.num, (self.total,), generator=g, device=self.q_dev.device,
                                          dtype=torch.int32))
        self.multi = [(self.q_dev, self.ids[i], self.qmap, self.outs[i % len(self.outs)]) for i in range(steps)]
        self.packed = self.table.pack_batches(self.multi)  # the C array of descriptors, built once

    def run_stream_of_batches(self):
        self.table.batch_distances_by_id_device_multi(self.packed, 0, device=self.q_dev.device)
        return self.outs[0], None

    def step_e2e(self, torch):
        ids = self.ids_host[self.it % len(self.ids_host)]
        self.it += 1
        return self.table.batch_distances_by_id(self.q_host, ids, self.qmap_host, 0), None

    def units_per_step(self):
        return self.bytes_per_step() / 1e9

    def single_query_shapes(self, torch):
        """One query x n rows, n in {64 .. 1024} (the shapes DiskANN's single-query search produces):
        launch-latency bound, reported in microseconds.  `by_id_us`: ids in, table resident, timed
        with CUDA events over 200 back-to-back calls.  `legacy_abi_us`: the reference's
        host-pointer call (gathered rows cross PCIe inside the call), wall clock over 50 calls."""
        br = self.pkg.diskann_bridge
        res = {}
        q1 = self.q_dev[:1].contiguous()
        q1_host = self.q_host[:1].copy()
        for n in (64, 128, 256, 512, 1024):
            ids = self.ids[0][:n].contiguous()
            out = self.out[:n]
            for _ in range(10):
                self.table.batch_distances_by_id_device(q1, ids, None, 0, out=out)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(200):
                self.table.batch_distances_by_id_device(q1, ids, None, 0, out=out)
            e1.record()
            torch.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / 200
            entry = {"by_id_us": us, "by_id_gbytes_per_s": (n * self.row_bytes + self.dim * 4 + n * 8) / us / 1e3}
            if not self.sq8:
                cand = self.table._keepalive[ids.long()].cpu().numpy()
                o = np.empty(n, np.float32)
                for _ in range(5):
                    br.batch_distances_raw(q1_host, cand, n, self.dim, 0, o)
                t0 = time.perf_counter()
                for _ in range(50):
                    br.batch_distances_raw(q1_host, cand, n, self.dim, 0, o)
                entry["legacy_abi_us"] = (time.perf_counter() - t0) * 1e6 / 50
            res[str(n)] = entry
        return res

    def e2e_bytes(self):
        return self.nq * self.dim * 4 + self.total * 8, self.total * 4

    def config(self, world):
        return {"workload": self.name, "table_rows": self.num, "dim": self.dim, "queries": self.nq,
                "rows_per_query": self.per, "metric": "L2", "bytes_per_step": self.bytes_per_step(),
                "l2_flush": f"{self.batches} id batches cycled; table ({self.num * self.row_bytes / 1e9:.1f} GB) >> L2",
                "launch": "the K timed batches are submitted as ONE multi-batch launch (stream of back-to-back batches)"}

    def roofline(self, peaks, kernel_ms):
        # DRAM read + write of one launch at the default shapes, from the ncu captures summarised in
        # the profile summaries of the two batch-distance kernels
        traffic = None
        if self.sq8 and (self.nq, self.per, self.dim) == (1024, 128, 384):
            traffic = 61.1e6   # per batch of the multi-batch launch
        if not self.sq8 and (self.nq, self.per, self.dim) == (256, 128, 1536):
            traffic = 199.0e6  # per batch of the multi-batch launch
        return {"bound": "hbm", "achieved": None, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": None,
                "traffic": traffic, "kernel": "batch_distance_sq8_dp4a_kernel" if self.sq8 else "batch_distance_f32_kernel"}

    def parity_check(self, torch, dist, D, I, oracle):
        """One batch more, of which 4,096 (query, row) pairs are checked against the CPU oracle
        (the reference's scalar loop in double precision)."""
        ids = self.ids[0]
        out = self.table.batch_distances_by_id_device(self.q_dev, ids, self.qmap, 0, out=self.out)
        torch.cuda.synchronize()
        assert torch.isfinite(out).all()
        res = {"pairs": 0, "max_rel_err": None, "against": "not checked (no oracle on this rank)", "ok": True}
        if oracle is not None:
            pick = np.unique(np.linspace(0, self.total - 1, 4096).astype(np.int64))
            pick_t = torch.from_numpy(pick).to(ids.device)
            rows = self.table._keepalive[ids[pick_t].long()].cpu().numpy()
            qm = self.qmap_host[pick]
            got = out[pick_t].cpu().numpy().astype(np.float64)
            if self.sq8:
                want = oracle.sq8_batch_distances_by_id(rows, self.mins_host, self.scale_host, self.q_host,
                                                        np.arange(len(pick), dtype=np.uint32), qm, 0, exact=True)
            else:
                want = oracle.multi_batch_distances(self.q_host, rows, qm, 0, exact=True)
            err = float((np.abs(got - want) / np.maximum(np.abs(want), 1e-30)).max())
            res = {"pairs": int(len(pick)), "max_rel_err": err, "against": "CPU oracle (scalar loop, double accumulation)",
                   "ok": bool(err <= RTOL)}
        return res

    def close(self):
        self.table.close()

    # ---- CPU baseline: the reference's per-candidate loop, OpenMP over candidates, on one batch
    def cpu_sample(self, torch, device):
        if self.sq8:
            codes = self.table._keepalive.cpu().numpy()
            return ("sq8", codes, self.mins_host, self.scale_host)
        return ("f32", self.table._keepalive.cpu().numpy())

    def cpu_run(self, oracle, sample):
        ids = self.ids_host[0]
        t0 = time.perf_counter()
        reps = 300
        for _ in range(reps):
            if sample[0] == "sq8":
                oracle.sq8_batch_distances_by_id(sample[1], sample[2], sample[3], self.q_host, ids, self.qmap_host, 0)
            else:
                oracle.batch_distances_by_id(sample[1], self.q_host, ids, self.qmap_host, 0)
        dt = (time.perf_counter() - t0) / reps
        return self.bytes_per_step() / 1e9 / dt, dt, f"one batch of {self.total} (query, row) pairs, {reps} repetitions (scalar loop of the reference, OpenMP over pairs)"


def make_workload(name, scale):
    if name == "flat_ip_20m":
        return FlatWorkload(name, 20_000_000, 768, 4096, 100, "IP", "unit", scale)
    if name in ("flat_ip_20m_f16", "flat_ip_20m_bf16"):  # the same store kept in 16-bit rows
        return FlatWorkload(name, 20_000_000, 768, 4096, 100, "IP", "unit", scale, storage=name.rsplit("_", 1)[1])
    if name == "flat_l2_100k":
        return FlatWorkload(name, 100_000, 384, 1000, 10, "L2", "uniform", scale)
    if name == "ivf_1m":
        return IvfWorkload(scale)
    if name == "batch_c2":
        return BatchWorkload(False, scale)
    if name == "sq8_c5":
        return BatchWorkload(True, scale)
    raise SystemExit(f"unknown workload {name}")


# ------------------------------------------------------------------------------------------------
def blas_threads():
    """Threads numpy's BLAS will really use (the blocked sgemm of the flat CPU arm runs there)."""
    try:
        from threadpoolctl import threadpool_info
        n = [int(i.get("num_threads", 0)) for i in threadpool_info() if i.get("user_api") == "blas"]
        return max(n) if n else None
    except Exception:
        return None


def run_reference(args, wl):
    """The reference's CPU path (oracle port: blocked sgemm + heap, all host threads) on a bounded
    sample per step.  Rank 0 only."""
    import torch
    rank, local, world = dist_info(args)
    if rank != 0:
        return
    cores = _host_cores()
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=cores)
    except Exception:
        pass
    from oracle import oracle
    oracle.build()
    oracle.set_num_threads(cores)
    device = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    if not isinstance(wl, FlatWorkload):
        # the inputs of these workloads (trained centroids and lists, device-resident tables) are
        # built exactly as in the GPU arm; only the CPU search below is timed
        if not torch.cuda.is_available():
            print(json.dumps({"impl": "reference", "unavailable": "building this workload's inputs needs the GPU"}))
            return
        wl.setup(load_package(), torch, 0, 1, device)
    sample = wl.cpu_sample(torch, device)
    for _ in range(min(args.warmup, 1)):
        wl.cpu_run(oracle, sample)
    vals, times = [], []
    steps = args.steps if args.steps is not None else 5
    for _ in range(steps):
        qps, dt, desc = wl.cpu_run(oracle, sample)
        vals.append(qps)
        times.append(dt)
    value = len(vals) / sum(1.0 / v for v in vals)
    line = {"impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus,
            "steps": steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times),
            "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": wl.config(max(args.gpus, 1)) | {"flat_kernel": "cpu"},
            "cpu_baseline": {"value": value, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port",
                             "blas_threads": blas_threads(), "sample": desc},
            "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def _json_default(o):
    """numpy scalars in the line (counts, errors) as plain numbers"""
    if isinstance(o, np.generic):
        return o.item()
    raise TypeError(f"{type(o).__name__} is not JSON serializable")


DEFAULT_STEPS = {"flat_ip_20m": 5, "flat_l2_100k": 50, "ivf_1m": 10, "batch_c2": 100, "sq8_c5": 100,
                 "flat_ip_20m_f16": 5, "flat_ip_20m_bf16": 5}


def run_workload(args, name, steps, ctx, with_cpu_baseline):
    """Sets the workload up, times `steps` steps (device-resident inputs, then end to end), checks
    the timed output and returns the result as a dict (the JSON line of that workload)."""
    torch, dist, pkg, lib, peaks = ctx["torch"], ctx["dist"], ctx["pkg"], ctx["lib"], ctx["peaks"]
    rank, local, world, device = ctx["rank"], ctx["local"], ctx["world"], ctx["device"]
    wl = make_workload(name, args.scale)

    t_setup = time.perf_counter()
    wl.setup(pkg, torch, rank, world, device)
    torch.cuda.synchronize()
    t_setup = time.perf_counter() - t_setup

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    sampler.wait_first_sample()
    for _ in range(args.warmup):
        out = wl.step()
    barrier()

    # ---- timed region: K steps, CUDA events on the launching stream, max over ranks
    lib.ann_cuda_set_kernel_timing(1)
    launches0 = lib.ann_cuda_launch_count()
    kernel_ms = []
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream_of_batches = isinstance(wl, BatchWorkload)
    one_per_launch_ms = None
    if stream_of_batches:
        # for comparison: the same batches one launch each, back to back (launch gaps included)
        ev0.record()
        for _ in range(steps):
            out = wl.step()
        ev1.record()
        torch.cuda.synchronize()
        one_per_launch_ms = ev0.elapsed_time(ev1) / steps
        wl.prepare_stream_of_batches(torch, steps)
        wl.run_stream_of_batches()  # warm
        launches0 = lib.ann_cuda_launch_count()
    barrier()
    t_begin = sampler.mark()
    ev0.record()
    if stream_of_batches:
        out = wl.run_stream_of_batches()
    else:
        for _ in range(steps):
            out = wl.step()
    ev1.record()
    barrier()
    t_end = sampler.mark()
    elapsed_ms = ev0.elapsed_time(ev1)
    launches = lib.ann_cuda_launch_count() - launches0
    clocks = sampler.stop(t_begin, t_end)
    fallbacks0 = lib.ann_cuda_screen_fallbacks()
    if hasattr(wl, "index"):
        wl.index.search_status()  # raises if a kernel of the timed searches gave up on a wait
        ms = lib.ann_cuda_index_last_flat_kernel_ms(wl.index._h)
        if ms > 0:
            kernel_ms.append(ms)
    fallback_passes = int(lib.ann_cuda_screen_fallbacks() - fallbacks0)
    lib.ann_cuda_set_kernel_timing(0)
    t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    units = wl.units_per_step() * steps * (world if wl.scaling == "weak" else 1)
    value = units / (elapsed_ms * 1e-3)

    # ---- end to end: host buffers, copies inside the timed region
    for _ in range(2):
        wl.step_e2e(torch)
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        wl.step_e2e(torch)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    t = torch.tensor([e2e_s], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    h2d, d2h = wl.e2e_bytes()
    e2e_value = units / e2e_s

    roof = wl.roofline(peaks, kernel_ms[-1] if kernel_ms else None)
    if roof["bound"] == "hbm" and isinstance(wl, BatchWorkload):
        per_launch_ms = elapsed_ms / steps
        roof["achieved"] = wl.bytes_per_step() / 1e9 / (per_launch_ms * 1e-3)
        roof["frac"] = roof["achieved"] / roof["peak"]
        roof["kernel_ms"] = per_launch_ms
    roof["peak_source"] = peaks["_source"]
    if roof["bound"] == "hbm" and roof.get("achieved"):
        roof["frac_of_nominal_8000"] = roof["achieved"] / 8000.0

    line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / steps, "higher_is_better": True,
            "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": wl.config(world), "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": 1e3 * e2e_s / steps},
            "gpu_launches": int(launches), "roofline": roof, "setup_s": t_setup}
    if hasattr(wl, "index"):
        line["fallback_passes"] = fallback_passes  # searches repeated one tier up inside the timed region

    if one_per_launch_ms is not None:
        line["one_batch_per_launch"] = {"ms_per_step": one_per_launch_ms,
                                        "value": wl.units_per_step() / (one_per_launch_ms * 1e-3), "unit": wl.unit}
    if isinstance(wl, BatchWorkload) and not wl.sq8 and rank == 0:
        line["single_query"] = wl.single_query_shapes(torch)
    oracle = None
    if rank == 0:
        from oracle import oracle
        oracle.build()
    if rank == 0 and world == 1 and with_cpu_baseline:
        sample = wl.cpu_sample(torch, device)
        qps, dt, desc = wl.cpu_run(oracle, sample)
        line["cpu_baseline"] = {"value": qps, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port",
                                "blas_threads": blas_threads(), "sample": desc, "seconds": dt}
    # ---- the timed output against the exact kernels and the oracle (every rank takes part in the
    # gather of the sample; the oracle runs on rank 0)
    line["parity_check"] = wl.parity_check(torch, dist, out[0], out[1], oracle)
    wl.close()
    del wl, out
    torch.cuda.empty_cache()
    return line


def run_single_process(args, ctx, devices, steps):
    """The headline workload through ONE index object spread over `devices` in this process
    (ann_cuda_sharded_*: what CudaGpuBackend::CpuToGpu hands out when ANN_CUDA_DEVICES names several
    devices): host queries in, host results out, one host thread and stream per shard, per-shard
    lists copied into the first device and merged there.  Wall clock around the synchronous call."""
    torch, pkg = ctx["torch"], ctx["pkg"]
    wl = make_workload("flat_ip_20m", args.scale)
    G = len(devices)
    idx = pkg.CudaShardedIndex(wl.d, pkg.METRIC_INNER_PRODUCT, devices)
    t0 = time.perf_counter()
    for g, dev in enumerate(devices):
        lo, hi = pkg.sharded.row_range(wl.n, g, G)
        if hi <= lo:
            continue
        device = torch.device("cuda", dev)
        shard = idx.shard(g)
        shard.reserve(hi - lo)
        for c in range(lo // wl.chunk, (hi - 1) // wl.chunk + 1):
            x = wl.gen_chunk(c, device, torch)
            a, b = max(lo, c * wl.chunk) - c * wl.chunk, min(hi, (c + 1) * wl.chunk) - c * wl.chunk
            shard.add_device(x[a:b].contiguous())
            del x
    for dev in set(devices):
        torch.cuda.synchronize(dev)
    setup_s = time.perf_counter() - t0
    assert idx.ntotal == wl.n
    q = wl.queries_host(torch).numpy()
    for _ in range(max(args.warmup, 3)):
        D, I = idx.search(q, wl.k)
    t0 = time.perf_counter()
    for _ in range(steps):
        D, I = idx.search(q, wl.k)
    dt = (time.perf_counter() - t0) / steps
    # parity: a sample of the queries through the exact-fp32 scan kernels of the same shards
    sample = np.unique(np.linspace(0, wl.nq - 1, 32).astype(np.int64))
    lib = pkg.lib()
    assert lib.ann_cuda_set_flat_kernel(b"simt") == 0
    try:
        Ds, Is = idx.search(q[sample], wl.k)
    finally:
        lib.ann_cuda_set_flat_kernel(b"tcgen05")
    mism, err = compare_topk(D[sample], I[sample], Ds, Is, True)
    idx.close()
    for dev in set(devices):
        with torch.cuda.device(dev):
            torch.cuda.empty_cache()
    return {"value": wl.nq / dt, "unit": wl.unit, "ms_per_step": 1e3 * dt, "devices": list(devices), "steps": steps,
            "setup_s": setup_s, "what": "one process, one index object over all devices (host pointers in and out)",
            "parity_check": {"queries": int(len(sample)), "id_mismatches": mism, "max_rel_err": err,
                             "against": "exact-fp32 scan kernels over the same shards", "ok": bool(mism == 0 and err <= RTOL)}}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed steps of the headline workload (default 5; 100 for the batch-distance workloads)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None,
                    help="time this workload alone (default: flat_ip_20m plus the other configurations under `workloads`)")
    ap.add_argument("--scale", type=float, default=1.0, help="shrinks the row counts (debugging / profiling captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only")
    ap.add_argument("--single-process", default=None, metavar="DEVICES",
                    help="also time the headline workload through one sharded index object in ONE process over these "
                         "devices, e.g. 0,1,2,3 (default under torchrun: all ranks' devices, run by rank 0)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    headline = args.workload or "flat_ip_20m"
    if args.impl == "reference":
        run_reference(args, make_workload(headline, args.scale))
        return

    import torch
    import torch.distributed as dist
    rank, local, world = dist_info(args)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    pkg = load_package()
    if not pkg.get_gpu_backend().IsAvailable():
        raise SystemExit("no sm_100 GPU: " + pkg.get_gpu_backend().DeviceInfo())
    ctx = {"torch": torch, "dist": dist, "pkg": pkg, "lib": pkg.lib(), "peaks": measured_peaks(), "rank": rank,
           "local": local, "world": world, "device": device}

    steps = args.steps if args.steps is not None else DEFAULT_STEPS[headline]
    line = run_workload(args, headline, steps, ctx, not args.no_cpu_baseline)
    ok = line["parity_check"]["ok"]
    if args.workload is None and not args.no_extras:
        # the other configurations, measured the same way in the same process; the batch-distance
        # and 100k-row configurations are single-GPU by definition
        extras = ["flat_l2_100k", "ivf_1m", "batch_c2", "sq8_c5"] if world == 1 else ["ivf_1m"]
        line["workloads"] = {}
        for name in extras:
            sub = run_workload(args, name, DEFAULT_STEPS[name], ctx, not args.no_cpu_baseline)
            ok = ok and sub["parity_check"]["ok"]
            line["workloads"][name] = sub
    # the same headline search from ONE process that owns an index over all the devices (the form a
    # DuckDB process uses); the other ranks have released their memory and wait
    single = args.single_process.split(",") if args.single_process else ([str(i) for i in range(world)] if world > 1 else None)
    if single and args.workload is None:
        # The other ranks wait on the CPU (gloo): a pending NCCL barrier is a kernel spinning on their
        # GPUs, and the searches rank 0 now runs on those GPUs want every SM.
        cpu_group = dist.new_group(backend="gloo") if world > 1 else None
        if world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=cpu_group)
        if rank == 0:
            line["single_process"] = run_single_process(args, ctx, [int(v) for v in single], steps)
            ok = ok and line["single_process"]["parity_check"]["ok"]
        if world > 1:
            dist.barrier(group=cpu_group)
    if rank == 0:
        print(json.dumps(line, default=_json_default))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if not ok:
        raise SystemExit("parity check failed: see parity_check in the line above")


if __name__ == "__main__":
    main()
