"""Peer-memory shard exchange: two processes share ONE GPU (CUDA IPC works between processes on
the same device), gloo carries the handles and barriers, and each rank's merge kernel reads
the other rank's per-shard CSR through the mapped pointer.  The union over both query slices
must equal the unsharded result."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.cuda.set_device(0)
        import culsh_b200
        from culsh_b200 import sharded
        rng = np.random.RandomState(77)
        n, d, L, k, nq = 6000, 16, 6, 6, 201
        reps = (57, nq, 33, nq)  # both halves of the buffer are reused; the second call has to grow it
        X = rng.randn(n, d).astype(np.float32)
        Q = X[rng.randint(0, n, nq)] + 0.01 * rng.randn(nq, d).astype(np.float32)
        sharded.PeerExchange.GROW_ALIGN = 256  # small results must still outgrow the first buffer
        ex = sharded.PeerExchange(device=0)
        bases = [sharded.shard_bounds(n, world, r)[0] for r in range(world)]
        lo, hi = sharded.shard_bounds(n, world, rank)
        model = culsh_b200.RPLSH(L, k, seed=13).fit(X[lo:hi])
        for rep, nqq in enumerate(reps):
            cand = model.query(Q[:nqq])
            merged, (q_lo, q_hi) = ex.exchange(cand, bases)
            np.savez(os.path.join(out_dir, f"r{rank}_{rep}.npz"), idx=merged.get_indices(),
                     off=merged.get_offsets(), q_lo=q_lo, q_hi=q_hi)
        if rank == 0:
            whole = culsh_b200.RPLSH(L, k, seed=13).fit(X)
            for rep, nqq in enumerate(reps):
                w = whole.query(Q[:nqq])
                np.savez(os.path.join(out_dir, f"whole_{rep}.npz"), idx=w.get_indices(), off=w.get_offsets())
        # sharded self-join: every rank ends with the fit_query lists of its own rows
        est = culsh_b200.PStableLSH(5, 3, window_size=2, seed=4)
        fq, (r_lo, r_hi) = sharded.fit_query_sharded(est, X[lo:hi], ex, batch_size=1500)
        np.savez(os.path.join(out_dir, f"fq{rank}.npz"), idx=fq.get_indices(), off=fq.get_offsets(),
                 r_lo=r_lo, r_hi=r_hi)
        if rank == 0:
            w = culsh_b200.PStableLSH(5, 3, window_size=2, seed=4).fit_query(X)
            np.savez(os.path.join(out_dir, "fq_whole.npz"), idx=w.get_indices(), off=w.get_offsets())
        ex.close()
    finally:
        dist.destroy_process_group()


def test_peer_exchange_two_processes_one_gpu(tmp_path):
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for rep in range(4):
        w = np.load(tmp_path / f"whole_{rep}.npz")
        woff = w["off"].astype(np.int64)
        for r in range(world):
            g = np.load(tmp_path / f"r{r}_{rep}.npz")
            q_lo, q_hi = int(g["q_lo"]), int(g["q_hi"])
            off = g["off"].astype(np.int64)
            assert len(off) == q_hi - q_lo + 1
            assert np.array_equal(off, woff[q_lo:q_hi + 1] - woff[q_lo])
            assert np.array_equal(g["idx"], w["idx"][woff[q_lo]:woff[q_hi]])
    w = np.load(tmp_path / "fq_whole.npz")
    woff = w["off"].astype(np.int64)
    covered = 0
    for r in range(world):
        g = np.load(tmp_path / f"fq{r}.npz")
        r_lo, r_hi = int(g["r_lo"]), int(g["r_hi"])
        assert r_lo == covered
        covered = r_hi
        assert np.array_equal(g["off"].astype(np.int64), woff[r_lo:r_hi + 1] - woff[r_lo])
        assert np.array_equal(g["idx"], w["idx"][woff[r_lo]:woff[r_hi]])
    assert covered == len(woff) - 1


def _nccl_worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    try:
        import culsh_b200
        from culsh_b200 import sharded
        rng = np.random.RandomState(5)
        n, d, L, k = 9001, 24, 6, 10  # ragged split: 4501 + 4500 rows
        X = rng.randn(n, d).astype(np.float32)
        lo, hi = sharded.shard_bounds(n, world, rank)
        Xd = torch.from_numpy(X[lo:hi]).cuda(rank)
        ex = sharded.PeerExchange(device=rank)
        # default for RPLSH on CUDA tensors: the shards ship packed signatures, not rows
        fq, (r_lo, r_hi) = sharded.fit_query_sharded(culsh_b200.RPLSH(L, k, seed=9), Xd, ex)
        np.savez(os.path.join(out_dir, f"n{rank}.npz"), idx=fq.get_indices(), off=fq.get_offsets(),
                 r_lo=r_lo, r_hi=r_hi)
        fr, (q_lo, q_hi) = sharded.fit_query_sharded(culsh_b200.RPLSH(L, k, seed=9), Xd, ex, batch_size=2000,
                                                      ship="rows")
        assert (q_lo, q_hi) == (r_lo, r_hi)
        assert np.array_equal(fr.get_indices(), fq.get_indices())
        assert np.array_equal(fr.get_offsets(), fq.get_offsets())
        if rank == 0:
            w = culsh_b200.RPLSH(L, k, seed=9).fit_query(X)
            np.savez(os.path.join(out_dir, "n_whole.npz"), idx=w.get_indices(), off=w.get_offsets())
        ex.close()
    finally:
        dist.destroy_process_group()


def test_fit_query_sharded_two_gpus_nccl(tmp_path):
    """Real peers: one process per GPU, NCCL for the row all-gather and the barriers, CUDA IPC
    mappings across two devices for the exchange."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_nccl_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    w = np.load(tmp_path / "n_whole.npz")
    woff = w["off"].astype(np.int64)
    covered = 0
    for r in range(world):
        g = np.load(tmp_path / f"n{r}.npz")
        r_lo, r_hi = int(g["r_lo"]), int(g["r_hi"])
        assert r_lo == covered
        covered = r_hi
        assert np.array_equal(g["off"].astype(np.int64), woff[r_lo:r_hi + 1] - woff[r_lo])
        assert np.array_equal(g["idx"], w["idx"][woff[r_lo]:woff[r_hi]])
    assert covered == len(woff) - 1
