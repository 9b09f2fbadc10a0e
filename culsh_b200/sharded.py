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


class _DeviceView:
    """Zero-copy window on an array owned by a Candidates object (kept alive through `owner`)."""

    def __init__(self, ptr: int, n: int, typestr: str, owner):
        self.__cuda_array_interface__ = {"shape": (int(n),), "typestr": typestr, "data": (int(ptr), False),
                                         "version": 3, "strides": None}
        self._owner = owner


def _csr_tensors(cand):
    """(indices int32, offsets int64) torch tensors that alias the result's device arrays."""
    import torch
    ip, _, op = cand.device_pointers()
    dev = f"cuda:{cand._h.device}"
    n = cand.n_total_candidates
    idx = (torch.as_tensor(_DeviceView(ip, n, "<i4", cand), device=dev) if n
           else torch.empty(0, dtype=torch.int32, device=dev))
    off = torch.as_tensor(_DeviceView(op, cand.n_queries + 1, "<i8", cand), device=dev)
    return idx, off


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
    idx, off = _csr_tensors(cand)  # uint64 offsets travel as int64
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


def exchange_by_query(cand, row_base: int, group=None, row_bases: Optional[List[int]] = None):
    """Balanced form of the exchange: rank j ends up with the merged CSR (global row ids) of the
    query slice ``shard_bounds(n_queries, world, j)``; returns ``(Candidates, (q_lo, q_hi))``.

    Every rank sends each peer only the lists of that peer's queries - a contiguous piece of its
    own CSR - in one all-to-all, so no GPU receives more than one shard's worth of ids, where
    gathering on a single root receives all of them.
    """
    import torch
    import torch.distributed as dist
    from . import _culsh_core
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    nq = cand.n_queries
    idx, off = _csr_tensors(cand)
    dev = off.device
    bounds = [shard_bounds(nq, world, j) for j in range(world)]
    cuts = torch.tensor([b[0] for b in bounds] + [nq], dtype=torch.int64, device=dev)
    cut_vals = off[cuts].tolist()                      # world + 1 numbers to the host
    send_counts = [cut_vals[j + 1] - cut_vals[j] for j in range(world)]
    if row_bases is None:
        b = torch.tensor([row_base], dtype=torch.int64, device=dev)
        bs = [torch.zeros_like(b) for _ in range(world)]
        dist.all_gather(bs, b, group=group)
        row_bases = [int(x.item()) for x in bs]
    # offsets first (small): the last entry of each received slice is that shard's id count for
    # my queries, so no separate exchange of sizes is needed
    send_off = torch.cat([off[lo:hi + 1] - off[lo] for lo, hi in bounds])
    lo_r, hi_r = bounds[rank]
    my_len = hi_r - lo_r + 1
    recv_off = torch.empty(world * my_len, dtype=torch.int64, device=dev)
    dist.all_to_all_single(recv_off, send_off, output_split_sizes=[my_len] * world,
                           input_split_sizes=[hi - lo + 1 for lo, hi in bounds], group=group)
    recv_counts = [int(x) for x in recv_off[my_len - 1::my_len].tolist()]
    recv_idx = torch.empty(max(1, sum(recv_counts)), dtype=torch.int32, device=dev)
    dist.all_to_all_single(recv_idx[:sum(recv_counts)], idx, output_split_sizes=recv_counts,
                           input_split_sizes=send_counts, group=group)
    torch.cuda.synchronize()
    idx_ptrs, off_ptrs, start = [], [], 0
    for s in range(world):
        idx_ptrs.append(recv_idx.data_ptr() + 4 * start)
        off_ptrs.append(recv_off.data_ptr() + 8 * s * my_len)
        start += recv_counts[s]
    merged = _culsh_core.merge_shard_candidates(idx_ptrs, off_ptrs, row_bases, my_len - 1,
                                                device=dev.index)
    return merged, (lo_r, hi_r)


class PeerExchange:
    """Shard exchange over peer memory, push form.  Rank j owns the j-th slice of the queries and
    keeps a receive buffer that the other processes of the box have mapped (CUDA IPC).  Per
    exchange the ranks all-gather their per-query candidate counts (small), every rank works out
    where each of its lists belongs inside the owner's merged id array, and one kernel per rank
    stores its lists, shifted to global row ids, straight into the owners' buffers over NVLink
    (plain coalesced stores to peer memory; the reads are local).  A barrier later the owners'
    buffers hold the merged CSR of their slices - there is no staging copy and no collective on
    the data path.

    A receive buffer has two halves used alternately, and the returned result's ids live in the
    half just filled: a result stays valid until the second exchange after the one that made it
    (and no longer than this object).  When a result outgrows the halves every rank allocates
    larger ones; the old buffers are kept for two more exchanges for the same reason.
    """

    GROW_ALIGN = 1 << 21   # halves grow to 1.25x the need, rounded up to this many bytes

    def __init__(self, group=None, device: Optional[int] = None):
        import torch.distributed as dist
        from . import _culsh_core
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.h = _culsh_core.get_handle(device)
        self.capacity = 0      # bytes per half
        self.phase = 0         # half used by the next exchange
        self.local = None      # device address of my buffer (two halves)
        self.peers = []        # device addresses of every rank's buffer as mapped here
        self.retired = []      # [age, local, peers] of outgrown buffers that results may still use
        self.last_ms = {}      # host wall time of the steps of the last exchange (every step ends in a sync)

    def _unmap_and_free(self, sets):
        """Collective, two phases: every rank unmaps its peers' buffers, the group meets at a
        barrier, and only then each rank frees what it exported - a buffer must not be freed
        while another process still has it mapped.  If a rank failed on the way (the barrier
        raises), the exports are left to the driver at process exit rather than freed early."""
        import ctypes as C
        import torch.distributed as dist
        from . import _lib
        if not sets:
            return
        for local, peers in sets:
            for r, p in enumerate(peers):
                if r != self.rank and p:
                    _lib.check(self.h.lib.culsh_peer_close(self.h.ptr, C.c_void_p(p)))
        dist.barrier(self.group)   # all importers have unmapped
        for local, peers in sets:
            if local:
                _lib.check(self.h.lib.culsh_peer_free(self.h.ptr, C.c_void_p(local)))

    def close(self):
        """Collective.  Results obtained from this object must not be used afterwards."""
        import torch.distributed as dist
        dist.barrier(self.group)   # nobody is still writing or reading
        sets = [(loc, peers) for _, loc, peers in self.retired]
        if self.local or self.peers:
            sets.append((self.local, self.peers))
        self.retired, self.local, self.peers, self.capacity = [], None, [], 0
        self._unmap_and_free(sets)

    def _barrier(self):
        """One-word all-reduce: a barrier over the group on any backend."""
        import torch
        import torch.distributed as dist
        on_gpu = dist.get_backend(self.group) == "nccl"
        t = torch.zeros(1, dtype=torch.int64, device=f"cuda:{self.h.device}" if on_gpu else "cpu")
        dist.all_reduce(t, group=self.group)
        t.item()

    def _grow(self, need: int):
        """Collective (every rank calls it with the same `need`): allocate, export, map.  The
        outgrown buffers are retired, not freed: earlier results may still point into them."""
        import ctypes as C
        import torch.distributed as dist
        from . import _lib
        if self.local or self.peers:
            self.retired.append([0, self.local, self.peers])
        a = self.GROW_ALIGN
        cap = (int(need * 1.25) + a) // a * a
        ptr = C.c_void_p()
        hbuf = C.create_string_buffer(64)
        _lib.check(self.h.lib.culsh_peer_alloc(self.h.ptr, 2 * cap, C.byref(ptr), hbuf))
        self.local, self.capacity = ptr.value, cap
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(hbuf.raw), group=self.group)
        self.peers = []
        for r, hb in enumerate(handles):
            if r == self.rank:
                self.peers.append(self.local)
            else:
                q = C.c_void_p()
                _lib.check(self.h.lib.culsh_peer_open(self.h.ptr, hb, C.byref(q)))
                self.peers.append(q.value)

    def _all_counts(self, cand):
        """[world, n_queries] int64 device tensor of every rank's per-query candidate counts."""
        import torch
        import torch.distributed as dist
        _, cp, _ = cand.device_pointers()
        dev = f"cuda:{self.h.device}"
        nq = cand.n_queries
        mine = torch.as_tensor(_DeviceView(cp, nq, "<i8", cand), device=dev)
        if dist.get_backend(self.group) == "nccl":
            out = torch.empty(self.world * nq, dtype=torch.int64, device=dev)
            dist.all_gather_into_tensor(out, mine, group=self.group)
            return out
        parts = [torch.empty(nq, dtype=torch.int64) for _ in range(self.world)]
        dist.all_gather(parts, mine.cpu(), group=self.group)
        return torch.cat(parts).to(dev)

    def exchange(self, cand, row_bases: List[int]):
        """Returns (Candidates of my query slice with global row ids, (q_lo, q_hi)).  Collective:
        every rank passes the result of the same queries over its own rows."""
        import ctypes as C
        import torch
        from . import _culsh_core, _lib
        import time
        nq = cand.n_queries
        lib, hp = self.h.lib, self.h.ptr
        lo, hi = shard_bounds(nq, self.world, self.rank)
        t0 = time.perf_counter()
        # outgrown buffers: results that pointed into them have expired two exchanges later
        for entry in self.retired:
            entry[0] += 1
        expired = [(loc, peers) for age, loc, peers in self.retired if age > 2]
        self.retired = [e for e in self.retired if e[0] <= 2]
        self._unmap_and_free(expired)
        # the all-gather is also the point after which the half about to be written is free:
        # every rank has entered this exchange, so results of the exchange before last are dead
        counts_all = self._all_counts(cand)
        dstpos = torch.empty(max(nq, 1), dtype=torch.int64, device=counts_all.device)
        totals = (C.c_uint64 * self.world)()
        out = C.c_void_p()
        torch.cuda.synchronize(counts_all.device)
        t1 = time.perf_counter()
        _lib.check(lib.culsh_exchange_plan(hp, self.world, self.rank, nq, counts_all.data_ptr(),
                                           dstpos.data_ptr(), totals, C.byref(out)))
        merged = _culsh_core.Candidates(out, self.h)
        need = 4 * max(int(t) for t in totals)
        if need > self.capacity:      # the totals are the same on every rank: same decision everywhere
            self._grow(max(need, 256))
        t2 = time.perf_counter()
        shift = self.phase * self.capacity
        recv = (C.c_void_p * self.world)(*[C.c_void_p(p + shift) for p in self.peers])
        ip, _, op = cand.device_pointers()
        _lib.check(lib.culsh_exchange_push(hp, self.world, self.rank, nq, ip or None, op, dstpos.data_ptr(), recv,
                                           int(row_bases[self.rank]), int(cand.n_total_candidates)))
        t3 = time.perf_counter()
        self._barrier()               # every rank's stores have landed
        t4 = time.perf_counter()
        self.last_ms = {"counts_all_gather": (t1 - t0) * 1e3, "plan": (t2 - t1) * 1e3, "push": (t3 - t2) * 1e3,
                        "barrier": (t4 - t3) * 1e3, "pushed_bytes": 4 * int(cand.n_total_candidates)}
        merged._attach(self.local + shift, int(totals[self.rank]), keepalive=self)
        self.phase ^= 1
        return merged, (lo, hi)


def all_gather_rows(X, group=None):
    """Every rank's row block, concatenated in rank order, on every rank.

    NumPy arrays travel as objects (any backend); torch tensors are padded to the longest block
    and gathered with one all_gather_into_tensor on their own device (NCCL for CUDA tensors).
    Returns (X_all, rows_per_rank).
    """
    import numpy as np
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    if isinstance(X, np.ndarray):
        parts = [None] * world
        dist.all_gather_object(parts, X, group=group)
        return np.concatenate(parts, axis=0), [int(p.shape[0]) for p in parts]
    rows = [None] * world
    dist.all_gather_object(rows, int(X.shape[0]), group=group)
    longest = max(rows)
    block = X if X.shape[0] == longest else torch.cat(
        [X, X.new_zeros((longest - X.shape[0],) + tuple(X.shape[1:]))])
    out = X.new_empty((world * longest,) + tuple(X.shape[1:]))
    dist.all_gather_into_tensor(out, block.contiguous(), group=group)
    if all(r == longest for r in rows):
        return out, rows
    return torch.cat([out[j * longest:j * longest + r] for j, r in enumerate(rows)]), rows


def all_gather_row_keys(index, group=None, device=None):
    """Packed keys of every shard's rows, [L][n_all][key_words] int32 on this rank's device, rows in
    rank order; returns (keys_all, rows_per_rank).  Every shard writes the keys of its own rows
    (`index.row_keys`), one padded all_gather_into_tensor (NCCL) moves them."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    L, nw, n_local = index.n_hash_tables, index.key_words, index.n_samples
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    rows = [None] * world
    dist.all_gather_object(rows, int(n_local), group=group)
    longest = max(rows)
    block = torch.zeros((L, longest, nw), dtype=torch.int32, device=dev) if n_local < longest else \
        torch.empty((L, longest, nw), dtype=torch.int32, device=dev)
    if n_local == longest:
        index.row_keys(block.data_ptr())
    else:
        mine = torch.empty((L, n_local, nw), dtype=torch.int32, device=dev)
        index.row_keys(mine.data_ptr())
        block[:, :n_local] = mine
    gathered = torch.empty((world, L, longest, nw), dtype=torch.int32, device=dev)
    dist.all_gather_into_tensor(gathered, block, group=group)
    keys_all = torch.empty((L, sum(rows), nw), dtype=torch.int32, device=dev)
    base = 0
    for j, r in enumerate(rows):
        keys_all[:, base:base + r] = gathered[j, :, :r]
        base += r
    return keys_all, rows


def fit_query_sharded(estimator, X_local, exchange: "PeerExchange", batch_size: Optional[int] = None,
                      group=None, ship: Optional[str] = None):
    """Self-join over a row-sharded data set (upstream: single-GPU fit_query, core/fit_query.cuh:30-55).

    `estimator` is an unfitted RPLSH / PStableLSH object built with the same arguments (seed
    included) on every rank; `X_local` is this rank's row block (blocks in rank order form the
    data set, every block as long as the first except possibly the last ones, as shard_bounds
    cuts them).  Every rank fits its block, then every rank asks its shard for the neighbours of
    EVERY row, and the peer exchange hands each rank the merged candidate lists of its own rows
    with global row ids.  Returns (Candidates, (row_lo, row_hi)).

    What travels between the shards (`ship`): "keys" - the packed signatures of the rows, taken
    from the fitted index, so that every row is hashed once, by its own shard (RPLSH on CUDA
    tensors: a signature bit means the same on every shard) - or "rows" - the rows themselves,
    hashed again by every shard (PStableLSH, whose shards may narrow their key elements
    differently; NumPy inputs).  Default: "keys" where it applies.
    """
    import numpy as np
    model = estimator.fit(X_local)
    keys_ok = (type(estimator).__name__ == "RPLSH" and not isinstance(X_local, np.ndarray)
               and getattr(X_local, "is_cuda", False))
    if ship is None:
        ship = "keys" if keys_ok else "rows"
    if ship == "keys":
        if not keys_ok:
            raise ValueError("signatures can be shipped for RPLSH on CUDA tensors only")
        keys_all, rows = all_gather_row_keys(model.index, group, X_local.device)
        cand = model._core.query_keys(keys_all.data_ptr(), int(keys_all.shape[1]), model.index)
        del keys_all
    else:
        X_all, rows = all_gather_rows(X_local, group)
        cand = model.query(X_all, batch_size=batch_size)
    bases = [0]
    for r in rows[:-1]:
        bases.append(bases[-1] + r)
    merged, (lo, hi) = exchange.exchange(cand, bases)
    me = exchange.rank
    if (lo, hi) != (bases[me], bases[me] + rows[me]):
        raise ValueError("row blocks must be cut as shard_bounds(n_rows, world, rank) cuts them")
    return merged, (lo, hi)
