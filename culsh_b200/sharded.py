"""Row-sharded indexes over the GPUs of one box (one process per GPU, torch.distributed).

Upstream cuLSH is single-GPU; sharding follows from its semantics: a bucket is an equality
class of signatures, so splitting the rows splits every bucket's member list, and a query's
candidate set over all rows is the union of its candidate sets over the shards
(core/fit.cuh:160-208, core/query.cuh:199-237).  Every rank fits its own row range with the
SAME seed (hence the same hash functions), all ranks answer the same queries, and the one
exchange step moves the per-shard CSR results to the destination rank, where a kernel
shifts local ids by the shard's first row and concatenates the per-query lists in rank
order - shard id ranges are disjoint and increasing, so the result is sorted and
duplicate-free, i.e. identical to the single-GPU CSR.
"""
from __future__ import annotations

from typing import List, Optional, Tuple


def shard_bounds(n_rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Row range [lo, hi) of `rank`: ceil(n/world) rows per rank, the last ranks may be short."""
    per = -(-n_rows // world)
    lo = min(n_rows, rank * per)
    return lo, min(n_rows, lo + per)


def exchange_to_root(indices, offsets, dst: int = 0, group=None):
    """Move every rank's (indices int32 [total_r], offsets int64 [n_q+1]) tensors to `dst`.

    Returns (list_of_indices, list_of_offsets) in rank order on `dst`, None elsewhere.
    Works with any backend (NCCL for CUDA tensors, gloo for CPU tensors): sizes travel in an
    all_gather, payloads as point-to-point sends.
    """
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    total = torch.tensor([indices.numel()], dtype=torch.int64, device=indices.device)
    totals = [torch.zeros_like(total) for _ in range(world)]
    dist.all_gather(totals, total, group=group)
    totals = [int(t.item()) for t in totals]
    if rank != dst:
        reqs = [dist.isend(offsets, dst, group=group)]
        if indices.numel():
            reqs.append(dist.isend(indices, dst, group=group))
        for r in reqs:
            r.wait()
        return None
    idx_list, off_list, reqs = [], [], []
    for r in range(world):
        if r == dst:
            idx_list.append(indices)
            off_list.append(offsets)
            continue
        o = torch.empty_like(offsets)
        i = torch.empty(totals[r], dtype=indices.dtype, device=indices.device)
        reqs.append(dist.irecv(o, r, group=group))
        if totals[r]:
            reqs.append(dist.irecv(i, r, group=group))
        idx_list.append(i)
        off_list.append(o)
    for r in reqs:
        r.wait()
    return idx_list, off_list


def gather_candidates(cand, row_base: int, dst: int = 0, group=None, row_bases: Optional[List[int]] = None):
    """Merge the per-shard results of the same queries into one CSR with global row ids on
    rank `dst` (returns None on the other ranks).  `row_base` is this rank's first row."""
    import torch
    import torch.distributed as dist
    from . import _culsh_core
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    idx = cand.get_indices(as_torch=True)
    off = cand.get_offsets(as_torch=True).view(torch.int64)  # uint64 payload, int64 for the backend
    if row_bases is None:
        b = torch.tensor([row_base], dtype=torch.int64, device=idx.device)
        bs = [torch.zeros_like(b) for _ in range(world)]
        dist.all_gather(bs, b, group=group)
        row_bases = [int(x.item()) for x in bs]
    got = exchange_to_root(idx, off, dst, group)
    if rank != dst:
        return None
    idx_list, off_list = got
    torch.cuda.synchronize()
    merged = _culsh_core.merge_shard_candidates(
        [t.data_ptr() if t.numel() else 0 for t in idx_list], [t.data_ptr() for t in off_list],
        row_bases, cand.n_queries, device=idx.device.index)
    return merged
