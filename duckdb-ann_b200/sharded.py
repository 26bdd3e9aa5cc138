"""Multi-GPU sharding of Flat / IVFFlat search inside one box.

One process per GPU (torch.distributed).  Flat: database rows are split into
contiguous ranges, one per rank.  IVFFlat: inverted list l lives on rank
l % world; every rank runs the coarse quantiser for its slice of the queries and
the probe lists are all-gathered (centroids are replicated).  Every rank searches its shard
for ALL queries, the per-shard (distance, label) top-k lists are exchanged with
one all-gather (k * 12 bytes per query per rank) and a final k-select kernel
merges them on every rank.  The reference has no multi-GPU path; this follows
the sharding the benchmark configurations describe.

The planner functions are pure Python and are unit-tested on CPU; the search
itself needs CUDA (the local search and the merge are CUDA kernels) unless a
test injects its own `local_search` / `merge`.
"""
from __future__ import annotations

from typing import Callable, Optional


def row_range(n_rows: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous row range [begin, end) of `rank`: ranges differ by at most one row."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("bad rank / world")
    base, rem = divmod(n_rows, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def list_owner(list_no: int, world: int) -> int:
    """Rank that stores inverted list `list_no` (round-robin deal)."""
    return list_no % world


def lists_of_rank(nlist: int, rank: int, world: int) -> list[int]:
    return list(range(rank, nlist, world))


class ShardedSearcher:
    """Searches a sharded index: local search -> all-gather -> merge.

    `local_search(x, k) -> (D, I)` returns this rank's (nq, k) results with GLOBAL
    labels, best first, missing = (+-inf, -1).  `merge(parts_d, parts_i) -> (D, I)`
    reduces the gathered (world, nq, k) lists.  With a CUDA index both default to
    the library's kernels.
    """

    def __init__(self, index=None, metric: int = 1, label_offset: int = 0, group=None,
                 local_search: Optional[Callable] = None, merge: Optional[Callable] = None):
        self.index = index
        self.metric = metric
        self.label_offset = label_offset
        self.group = group
        self._local_search = local_search
        self._merge = merge
        self._gather_d = None
        self._gather_i = None
        # IVFFlat over several ranks: each rank runs the coarse quantiser for its slice of the queries only
        self.split_coarse = True
        self._probes = None
        self._my_probes = None

    def _ivf_search_split_coarse(self, x, k: int, world: int):
        """IVFFlat over several ranks without a replicated coarse quantiser: this rank ranks the centroids
        for ITS slice of the queries, the probe lists are all-gathered (nq * nprobe * 4 bytes in total) and
        the lists stored here are scanned for all queries with the probes given."""
        import torch
        import torch.distributed as dist
        rank = dist.get_rank(self.group)
        nq = x.shape[0]
        per = (nq + world - 1) // world          # equal slices, the last ones padded with "no list"
        lo, hi = min(nq, rank * per), min(nq, (rank + 1) * per)
        nprobe = min(self.index.getNprobe(), self.index.getNlist())
        if self._probes is None or tuple(self._probes.shape) != (world * per, nprobe) or self._probes.device != x.device:
            self._probes = torch.empty((world * per, nprobe), dtype=torch.int32, device=x.device)
            self._my_probes = torch.empty((per, nprobe), dtype=torch.int32, device=x.device)
        self._my_probes.fill_(-1)
        if hi > lo:
            self.index.coarse_device(x[lo:hi], out=self._my_probes[: hi - lo])
        dist.all_gather_into_tensor(self._probes, self._my_probes, group=self.group)
        return self.index.search_preassigned_device(x, self._probes[:nq], k, label_offset=self.label_offset)

    def _world(self) -> int:
        import torch.distributed as dist
        return dist.get_world_size(self.group) if dist.is_available() and dist.is_initialized() else 1

    def search(self, x, k: int):
        import torch
        import torch.distributed as dist
        world = self._world()
        if self._local_search is not None:
            d_loc, i_loc = self._local_search(x, k)
        else:
            if self.index is None:
                raise RuntimeError("ShardedSearcher needs a CUDA index (there is no CPU search path)")
            if world > 1 and self.split_coarse and hasattr(self.index, "search_preassigned_device"):
                d_loc, i_loc = self._ivf_search_split_coarse(x, k, world)
            else:
                d_loc, i_loc = self.index.search_device(x, k, label_offset=self.label_offset)
        if world == 1:
            return d_loc, i_loc
        shape = (world,) + tuple(d_loc.shape)
        if self._gather_d is None or tuple(self._gather_d.shape) != shape or self._gather_d.device != d_loc.device:
            self._gather_d = torch.empty(shape, dtype=d_loc.dtype, device=d_loc.device)
            self._gather_i = torch.empty(shape, dtype=i_loc.dtype, device=i_loc.device)
        dist.all_gather_into_tensor(self._gather_d.view(-1, d_loc.shape[-1]), d_loc.contiguous(), group=self.group)
        dist.all_gather_into_tensor(self._gather_i.view(-1, i_loc.shape[-1]), i_loc.contiguous(), group=self.group)
        if self._merge is not None:
            return self._merge(self._gather_d, self._gather_i)
        from .faiss_like import merge_topk_device
        return merge_topk_device(self._gather_d, self._gather_i, self.metric)
