"""Host-side logic of the row-sharded path with two gloo ranks on CPU: row partition, the
exchange of per-shard CSR results to the root, and the union identity (checked with the
oracle's merge, the CUDA merge kernel has its own GPU test)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from culsh_b200 import sharded
from oracle import oracle


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rng = np.random.RandomState(5)
        n, nq, L, k = 1001, 48, 4, 2
        sig = rng.randint(-2, 3, size=(n, L * k)).astype(np.int32)
        qsig = sig[rng.randint(0, n, size=nq)]
        lo, hi = sharded.shard_bounds(n, world, rank)
        ind, off, cnt = oracle.query_index(oracle.fit_index(sig[lo:hi], L, k), qsig)
        got = sharded.exchange_to_root(torch.from_numpy(ind.copy()),
                                       torch.from_numpy(off.astype(np.int64)), dst=0)
        if rank == 0:
            idx_list, off_list = got
            res = [(i.numpy(), o.numpy().astype(np.uint64), np.diff(o.numpy()).astype(np.uint64))
                   for i, o in zip(idx_list, off_list)]
            bases = [sharded.shard_bounds(n, world, r)[0] for r in range(world)]
            merged = oracle.merge_shard_candidates(res, bases)
            want = oracle.query_index(oracle.fit_index(sig, L, k), qsig)
            ok = all(np.array_equal(a, b) for a, b in zip(merged, want))
            with open(out_path, "w") as f:
                f.write("ok" if ok else "mismatch")
        else:
            assert got is None
    finally:
        dist.destroy_process_group()


def test_shard_bounds_cover_all_rows():
    for n, w in [(10, 3), (1000, 8), (7, 8), (16, 4)]:
        spans = [sharded.shard_bounds(n, w, r) for r in range(w)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        for a, b in zip(spans, spans[1:]):
            assert a[1] == b[0]


@pytest.mark.timeout(120)
def test_two_rank_exchange_and_union(tmp_path):
    out = str(tmp_path / "result.txt")
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert open(out).read() == "ok"


def _gather_worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, d = 11, 3  # ragged: 6 rows on rank 0, 5 on rank 1
        X = np.arange(n * d, dtype=np.float32).reshape(n, d)
        lo, hi = sharded.shard_bounds(n, world, rank)
        a, rows_a = sharded.all_gather_rows(X[lo:hi])
        b, rows_b = sharded.all_gather_rows(torch.from_numpy(X[lo:hi].copy()))
        ok = (np.array_equal(a, X) and np.array_equal(b.numpy(), X) and rows_a == rows_b == [6, 5])
        with open(f"{out_path}.{rank}", "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_all_gather_rows_numpy_and_tensor_ragged(tmp_path):
    out = str(tmp_path / "gather")
    mp.spawn(_gather_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert open(out + ".0").read() == "ok" and open(out + ".1").read() == "ok"
