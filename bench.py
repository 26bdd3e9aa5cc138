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
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

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
# Workloads
# ------------------------------------------------------------------------------------------------
class FlatWorkload:
    def __init__(self, name, n, d, nq, k, metric_name, dist_kind, scale=1.0):
        self.name, self.d, self.nq, self.k = name, d, nq, k
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
        return q.contiguous().pin_memory()

    def setup(self, pkg, torch, rank, world, device):
        self.pkg = pkg
        m = pkg.METRIC_INNER_PRODUCT if self.metric_name == "IP" else pkg.METRIC_L2
        self.m = m
        lo, hi = pkg.sharded.row_range(self.n, rank, world)
        self.lo, self.hi = lo, hi
        self.index = pkg.CudaIndexFlat(self.d, m, device.index)
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
                "search": "one-MMA screening + exact re-ranking (stores >= 2M rows, k <= 128), else three-MMA split product"}

    def roofline(self, peaks, kernel_ms):
        local_rows = self.hi - self.lo
        flops = 2.0 * self.nq * local_rows * self.d
        achieved = flops / (kernel_ms * 1e-3) / 1e12 if kernel_ms and kernel_ms > 0 else None
        # Stores of two million rows or more are searched with one-MMA screening (one TF32 MMA per
        # product, candidates re-ranked exactly); smaller ones with the three-MMA split product.
        screened = local_rows >= 2_000_000 and self.k <= 128 and self.pkg.lib().ann_cuda_flat_kernel_name().decode() == "tcgen05"
        mmas = 1 if screened else 3
        peak = peaks["bf16_tflops_sustained"] / 2.0 / mmas
        # DRAM traffic of one launch.  Screened search: ncu capture of the full-size launch (20M rows of
        # 768 floats, 4,096 queries: 67.5 GB read + 1.2 GB written; the hi planes are 61.4 GB and are
        # read once for all query tiles), scaled by the rows of this launch.  Split product: captures
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
                             + "; 'achieved' counts 2*Q*N*d once"}

    def verify(self, torch, D, I):
        """Size-independent properties: sorted best first, labels valid and distinct, and the
        reported distance of a sample of (query, label) pairs equals the exact dot / L2."""
        D, I = D.cpu().numpy(), I.cpu().numpy()
        sgn = -1.0 if self.metric_name == "IP" else 1.0
        assert (np.diff(sgn * D, axis=1) >= 0).all(), "results are not sorted best first"
        assert (I >= 0).all() and (I < self.n).all()
        assert all(len(set(r.tolist())) == len(r) for r in I[:64]), "duplicate labels"
        q = self.q_host.numpy()
        for qi in (0, self.nq // 2, self.nq - 1):
            for j in (0, self.k - 1):
                lab = int(I[qi, j])
                if not (self.lo <= lab < self.hi):
                    continue
                row = self.index.reconstruct(lab - self.lo).astype(np.float64)
                true = float(row @ q[qi].astype(np.float64)) if self.metric_name == "IP" else float(
                    ((row - q[qi].astype(np.float64)) ** 2).sum())
                assert abs(true - float(D[qi, j])) <= 1e-4 * abs(true) + 1e-7, (qi, j, true, float(D[qi, j]))

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
# ncu capture of the grouped list scan at the default shape (14.6-14.8 GB read + 0.2 GB written)
IVF_SCAN_TRAFFIC = {(1_000_000, 10_000, 1): 14.8e9}


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
        # really moved (the physical bound: ~5.5 TB/s of it at the full size), and `tensor` restates
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

    def verify(self, torch, D, I):
        D = D.cpu().numpy()
        assert (np.diff(D, axis=1) >= 0).all()
        I = I.cpu().numpy()
        assert (I >= 0).all() and (I < self.n).all()

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
        return xb, cent, off, np.concatenate(rows), self.q_host.numpy()[:nq].copy(), nq

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

    def verify(self, torch, D, I):
        assert torch.isfinite(D).all()

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
def run_reference(args, wl):
    """The reference's CPU path (oracle port: blocked sgemm + heap, all host threads) on a bounded
    sample per step.  Rank 0 only."""
    import torch
    rank, local, world = dist_info(args)
    if rank != 0:
        return
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every host core it can get
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    os.environ["OMP_NUM_THREADS"] = str(cores)
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
    for _ in range(args.steps):
        qps, dt, desc = wl.cpu_run(oracle, sample)
        vals.append(qps)
        times.append(dt)
    value = len(vals) / sum(1.0 / v for v in vals)
    line = {"impl": "reference", "metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times),
            "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": wl.config(max(args.gpus, 1)) | {"flat_kernel": "cpu"},
            "cpu_baseline": {"value": value, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port",
                             "sample": desc},
            "e2e": {"value": value, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default 5; 100 for the batch-distance workloads)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="flat_ip_20m")
    ap.add_argument("--scale", type=float, default=1.0, help="shrinks the row counts (debugging / profiling captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    wl = make_workload(args.workload, args.scale)
    if args.steps is None:
        # a batch-distance step is ~20-40 us: the steady-state rate needs a stream of >= 100 of them
        args.steps = 100 if isinstance(wl, BatchWorkload) and args.impl == "ours" else 5
    if args.impl == "reference":
        run_reference(args, wl)
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
    peaks = measured_peaks()
    lib = pkg.lib()

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
        for _ in range(args.steps):
            out = wl.step()
        ev1.record()
        torch.cuda.synchronize()
        one_per_launch_ms = ev0.elapsed_time(ev1) / args.steps
        wl.prepare_stream_of_batches(torch, args.steps)
        wl.run_stream_of_batches()  # warm
        launches0 = lib.ann_cuda_launch_count()
    barrier()
    t_begin = sampler.mark()
    ev0.record()
    if stream_of_batches:
        out = wl.run_stream_of_batches()
    else:
        for _ in range(args.steps):
            out = wl.step()
    ev1.record()
    barrier()
    t_end = sampler.mark()
    elapsed_ms = ev0.elapsed_time(ev1)
    launches = lib.ann_cuda_launch_count() - launches0
    clocks = sampler.stop(t_begin, t_end)
    if hasattr(wl, "index"):
        ms = lib.ann_cuda_index_last_flat_kernel_ms(wl.index._h)
        if ms > 0:
            kernel_ms.append(ms)
    lib.ann_cuda_set_kernel_timing(0)
    t = torch.tensor([elapsed_ms], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    elapsed_ms = float(t.item())
    units = wl.units_per_step() * args.steps * (world if wl.scaling == "weak" else 1)
    value = units / (elapsed_ms * 1e-3)
    wl.verify(torch, out[0], out[1])

    # ---- end to end: host buffers, copies inside the timed region
    for _ in range(2):
        wl.step_e2e(torch)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
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
        per_launch_ms = elapsed_ms / args.steps
        roof["achieved"] = wl.bytes_per_step() / 1e9 / (per_launch_ms * 1e-3)
        roof["frac"] = roof["achieved"] / roof["peak"]
        roof["kernel_ms"] = per_launch_ms
    roof["peak_source"] = peaks["_source"]
    if roof["bound"] == "hbm" and roof.get("achieved"):
        roof["frac_of_nominal_8000"] = roof["achieved"] / 8000.0

    line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed_ms / args.steps, "higher_is_better": True,
            "scaling": wl.scaling, "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
            "config": wl.config(world), "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": wl.unit, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": 1e3 * e2e_s / args.steps},
            "gpu_launches": int(launches), "roofline": roof, "setup_s": t_setup}

    if one_per_launch_ms is not None:
        line["one_batch_per_launch"] = {"ms_per_step": one_per_launch_ms,
                                        "value": wl.units_per_step() / (one_per_launch_ms * 1e-3), "unit": wl.unit}
    if isinstance(wl, BatchWorkload) and not wl.sq8 and rank == 0:
        line["single_query"] = wl.single_query_shapes(torch)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import oracle
        oracle.build()
        sample = wl.cpu_sample(torch, device)
        qps, dt, desc = wl.cpu_run(oracle, sample)
        line["cpu_baseline"] = {"value": qps, "unit": wl.unit, "cores": oracle.num_threads(), "kind": "port",
                                "sample": desc, "seconds": dt}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
