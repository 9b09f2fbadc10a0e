"""The allocation-free shard merge against the allocating one, through the C ABI.

Collected last on purpose (file name), so that a run that stops at the first failure has
already run every other test.  Two calls in a row with different shard layouts check that
whatever the first call left in the library's fixed scratch array does not leak into the
second."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _shard_results(culsh, X, Q, shards, L, k, seed):
    n = len(X)
    per = -(-n // shards)
    keep, ip, op, bases = [], [], [], []
    for r in range(shards):
        lo, hi = r * per, min(n, (r + 1) * per)
        c = culsh.RPLSH(L, k, seed=seed).fit(X[lo:hi]).query(Q)
        keep.append(c)
        a, _, o = c.device_pointers()
        ip.append(a)
        op.append(o)
        bases.append(lo)
    return keep, ip, op, bases


def test_noalloc_merge_matches_allocating_merge_twice_in_a_row():
    import torch
    import culsh_b200
    from culsh_b200 import _culsh_core as cc

    rng = np.random.RandomState(2024)
    n, d, L, k = 5000, 16, 6, 6
    X = rng.randn(n, d).astype(np.float32)
    for call, (shards, nq) in enumerate([(5, 300), (3, 77)]):
        Q = X[rng.randint(0, n, nq)] + 0.01 * rng.randn(nq, d).astype(np.float32)
        keep, ip, op, bases = _shard_results(culsh_b200, X, Q, shards, L, k, seed=17)
        want = cc.merge_shard_candidates(ip, op, bases, nq)
        cap = int(want.n_total_candidates) + 13
        out_idx = torch.full((cap,), -7, dtype=torch.int32, device="cuda")
        out_cnt = torch.zeros(nq, dtype=torch.int64, device="cuda")
        out_off = torch.zeros(nq + 1, dtype=torch.int64, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        total = cc.merge_shard_candidates_into(ip, op, bases, nq, out_idx.data_ptr(), cap,
                                               out_cnt.data_ptr(), out_off.data_ptr())
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        assert total == want.n_total_candidates, f"call {call}"
        assert np.array_equal(out_idx[:total].cpu().numpy(), want.get_indices())
        assert np.array_equal(out_cnt.cpu().numpy().astype(np.uint64), want.get_counts())
        assert np.array_equal(out_off.cpu().numpy().astype(np.uint64), want.get_offsets())
        assert bool((out_idx[total:] == -7).all()), "wrote past the merged result"


def test_noalloc_merge_rejects_oversize_and_short_outputs():
    import torch
    import culsh_b200
    from culsh_b200 import _culsh_core as cc

    rng = np.random.RandomState(7)
    X = rng.randn(600, 8).astype(np.float32)
    Q = X[:40]
    keep, ip, op, bases = _shard_results(culsh_b200, X, Q, 2, 4, 4, seed=3)
    out_cnt = torch.zeros(40, dtype=torch.int64, device="cuda")
    out_off = torch.zeros(41, dtype=torch.int64, device="cuda")
    tiny = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(RuntimeError, match="holds 1 ids"):
        cc.merge_shard_candidates_into(ip, op, bases, 40, tiny.data_ptr(), 1, out_cnt.data_ptr(),
                                       out_off.data_ptr())
    with pytest.raises(RuntimeError, match="at most 64 shards"):
        cc.merge_shard_candidates_into(ip * 40, op * 40, bases * 40, 40, tiny.data_ptr(), 1,
                                       out_cnt.data_ptr(), out_off.data_ptr())
    with pytest.raises(RuntimeError, match="at most 4194304 queries"):
        cc.merge_shard_candidates_into(ip, op, bases, (1 << 22) + 1, tiny.data_ptr(), 1,
                                       out_cnt.data_ptr(), out_off.data_ptr())


def test_noalloc_merge_at_the_shard_limit_with_many_queries():
    """64 shards (the limit) and 300,000 queries (several tiles of the offset scan, whose block
    sums live in the fixed scratch array), on synthetic per-shard lists; the device's free
    memory must be the same before and after the call."""
    import torch
    from culsh_b200 import _culsh_core as cc

    shards, nq, rows_per_shard = 64, 300_000, 1000
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    keep, ip, op, bases = [], [], [], []
    for r in range(shards):
        cnt = torch.randint(0, 4, (nq,), device="cuda", generator=g)
        off = torch.zeros(nq + 1, dtype=torch.int64, device="cuda")
        off[1:] = torch.cumsum(cnt, 0)
        # ascending local ids inside every list: position in the list + a per-query start
        start = torch.randint(0, rows_per_shard - 4, (nq,), device="cuda", generator=g)
        q_of = torch.repeat_interleave(torch.arange(nq, device="cuda"), cnt)
        idx = (start[q_of] + torch.arange(q_of.numel(), device="cuda") - off[:-1][q_of]).to(torch.int32)
        keep.append((idx, off))
        ip.append(idx.data_ptr())
        op.append(off.data_ptr())
        bases.append(r * rows_per_shard)
    torch.cuda.synchronize()
    want = cc.merge_shard_candidates(ip, op, bases, nq)
    cap = int(want.n_total_candidates)
    out_idx = torch.empty(cap, dtype=torch.int32, device="cuda")
    out_cnt = torch.zeros(nq, dtype=torch.int64, device="cuda")
    out_off = torch.zeros(nq + 1, dtype=torch.int64, device="cuda")
    for call in range(2):
        out_idx.fill_(-1)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        total = cc.merge_shard_candidates_into(ip, op, bases, nq, out_idx.data_ptr(), cap,
                                               out_cnt.data_ptr(), out_off.data_ptr())
        assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
        assert total == cap, f"call {call}"
        assert np.array_equal(out_idx.cpu().numpy(), want.get_indices())
        assert np.array_equal(out_off.cpu().numpy().astype(np.uint64), want.get_offsets())
        assert np.array_equal(out_cnt.cpu().numpy().astype(np.uint64), want.get_counts())
