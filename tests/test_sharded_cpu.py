"""Host-side logic of the multi-GPU path on CPU: shard planning, and the
local-search -> all-gather -> merge flow over torch.distributed (gloo, 2 ranks).
The local search and the merge are injected (oracle + numpy) because the real
ones are CUDA kernels."""
import os
import socket
import subprocess
import sys

import numpy as np

from conftest import ROOT, load_package


def test_row_ranges_partition_the_rows():
    sh = load_package().sharded
    for n in (0, 1, 7, 20_000_000, 1001):
        for w in (1, 2, 3, 4, 8):
            r = [sh.row_range(n, i, w) for i in range(w)]
            assert r[0][0] == 0 and r[-1][1] == n
            assert all(r[i][1] == r[i + 1][0] for i in range(w - 1))
            sizes = [b - a for a, b in r]
            assert max(sizes) - min(sizes) <= 1


def test_lists_are_dealt_round_robin():
    sh = load_package().sharded
    for w in (1, 2, 4, 8):
        seen = sorted(l for r in range(w) for l in sh.lists_of_rank(1024, r, w))
        assert seen == list(range(1024))
        assert all(sh.list_owner(l, w) == r for r in range(w) for l in sh.lists_of_rank(1024, r, w))


WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
from conftest import load_package
from oracle import oracle as o
pkg = load_package()
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=int(sys.argv[3]), world_size=2)
rank, world = dist.get_rank(), dist.get_world_size()
rng = np.random.default_rng(0)
xb = rng.uniform(-1, 1, (1001, 24)).astype(np.float32)
xq = rng.uniform(-1, 1, (9, 24)).astype(np.float32)
lo, hi = pkg.sharded.row_range(len(xb), rank, world)

def local_search(x, k):
    D, I = o.flat_search(xb[lo:hi], x.numpy(), k, o.METRIC_L2)
    I = np.where(I >= 0, I + lo, -1)
    return torch.from_numpy(D), torch.from_numpy(I)

def merge(pd, pi):
    d = pd.numpy().transpose(1, 0, 2).reshape(pd.shape[1], -1)
    i = pi.numpy().transpose(1, 0, 2).reshape(pd.shape[1], -1)
    d = np.where(i >= 0, d, np.inf)
    order = np.argsort(d, axis=1, kind="stable")[:, :pd.shape[2]]
    return torch.from_numpy(np.take_along_axis(d, order, 1)), torch.from_numpy(np.take_along_axis(i, order, 1))

s = pkg.sharded.ShardedSearcher(local_search=local_search, merge=merge)
D, I = s.search(torch.from_numpy(xq), 12)
Dref, Iref = o.flat_search(xb, xq, 12, o.METRIC_L2)
assert (I.numpy() == Iref).all() and np.allclose(D.numpy(), Dref)
D2, I2 = s.search(torch.from_numpy(xq), 12)  # gather buffers are reused
assert (I2.numpy() == Iref).all()
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_two_rank_flow_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(port), str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        assert "ok" in o


IVF_WORKER = r'''
import os, sys
import numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
from conftest import load_package
from oracle import oracle as o
pkg = load_package()
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{sys.argv[2]}", rank=int(sys.argv[3]), world_size=2)
rank, world = dist.get_rank(), dist.get_world_size()
rng = np.random.default_rng(1)
xb = rng.standard_normal((900, 16)).astype(np.float32)
xq = rng.standard_normal((11, 16)).astype(np.float32)      # 11 queries over 2 ranks: slices of 6 and 5
nlist, nprobe, k = 12, 5, 7
cent = o.kmeans(xb, nlist, niter=4, seed=3)
off, rows = o.lists_from_assign(o.ivf_assign(xb, cent, o.METRIC_L2), nlist)

class FakeShard:
    """The two calls the sharded searcher makes on an IVFFlat shard, answered by the oracle for the lists this
    rank stores (list l lives on rank l % world)."""
    calls = []
    def getNprobe(self): return nprobe
    def getNlist(self): return nlist
    def coarse_device(self, x, out=None, stream=None):
        FakeShard.calls.append(("coarse", x.shape[0]))
        d2 = ((x.numpy()[:, None, :] - cent[None, :, :]) ** 2).sum(-1)
        out.copy_(torch.from_numpy(np.argsort(d2, axis=1, kind="stable")[:, :nprobe].astype(np.int32)))
        return out
    def search_preassigned_device(self, x, assign, k, label_offset=0):
        FakeShard.calls.append(("scan", x.shape[0]))
        probes = assign.numpy().copy()
        probes[(probes % world) != rank] = -1                 # lists stored elsewhere
        D, I = o.ivf_search_given_probes(xb, off, rows, x.numpy(), k, probes, o.METRIC_L2)
        return torch.from_numpy(D), torch.from_numpy(I)

def merge(pd, pi):
    d = pd.numpy().transpose(1, 0, 2).reshape(pd.shape[1], -1)
    i = pi.numpy().transpose(1, 0, 2).reshape(pd.shape[1], -1)
    d = np.where(i >= 0, d, np.inf)
    order = np.argsort(d, axis=1, kind="stable")[:, :pd.shape[2]]
    return torch.from_numpy(np.take_along_axis(d, order, 1)), torch.from_numpy(np.take_along_axis(i, order, 1))

s = pkg.sharded.ShardedSearcher(index=FakeShard(), merge=merge)
D, I = s.search(torch.from_numpy(xq), k)
Dref, Iref = o.ivf_search(xb, cent, off, rows, xq, k, nprobe, o.METRIC_L2)
assert (I.numpy() == Iref).all() and np.allclose(D.numpy(), Dref, rtol=1e-5), (I.numpy(), Iref)
# the coarse quantiser saw this rank's slice only, the scan all queries
assert FakeShard.calls == [("coarse", 6 if rank == 0 else 5), ("scan", 11)], FakeShard.calls
dist.barrier()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_ivf_probe_lists_are_chosen_by_slices_and_gathered(tmp_path):
    """IVFFlat over two ranks: each rank runs the coarse quantiser for its slice of the queries, the probe
    lists are all-gathered, and each rank scans the lists it stores for ALL queries."""
    script = tmp_path / "worker_ivf.py"
    script.write_text(IVF_WORKER)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = [subprocess.Popen([sys.executable, str(script), ROOT, str(port), str(r)], stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for p, o in zip(procs, outs):
        assert p.returncode == 0, o
        assert "ok" in o


def test_searcher_without_index_raises():
    import pytest
    import torch
    s = load_package().sharded.ShardedSearcher()
    with pytest.raises(RuntimeError):
        s.search(torch.zeros(1, 4), 1)
