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


def test_searcher_without_index_raises():
    import pytest
    import torch
    s = load_package().sharded.ShardedSearcher()
    with pytest.raises(RuntimeError):
        s.search(torch.zeros(1, 4), 1)
