"""Parity of the CUDA path (through the C ABI) with the CPU oracle on the same seeded inputs.

Bars: integer stages (MinHash signatures, every index array, candidate CSR) bit-exact;
dense signatures bit-exact except elements whose pre-quantisation value lies within 1e-5
(relative) of the sign / floor boundary - those are counted and must stay rare.
"""
import os

import numpy as np
import pytest
import scipy.sparse as sp

from oracle import oracle

pytestmark = pytest.mark.gpu

REL_BAND = 1e-5  # tolerance stated by the target: relative distance to the quantisation boundary


@pytest.fixture(scope="module")
def eng():
    import culsh_b200
    from culsh_b200 import _culsh_core
    return culsh_b200, _culsh_core


def _sig_matrix(sig_lnk):
    """[L][n][k] -> [n][L*k] (oracle layout)."""
    L, n, k = sig_lnk.shape
    return np.ascontiguousarray(sig_lnk.transpose(1, 0, 2)).reshape(n, L * k)


def _index_row_signatures(index, fam):
    """[n][L*k] signatures recovered from a fitted index (bucket signature of every member)."""
    n, L, s = index.n_samples, index.n_hash_tables, index.sig_nbytes
    bco = index.get_bucket_candidate_offsets().astype(np.int64)
    bs = index.get_bucket_signatures().reshape(-1, s)
    cand = index.get_candidate_indices()
    bucket_of_item = np.repeat(np.arange(len(bco) - 1), np.diff(bco))
    raw = np.empty((L, n, s), dtype=np.uint8)
    raw[np.arange(len(cand)) // n, cand] = bs[bucket_of_item]
    elem = np.uint8 if fam == "rplsh" else np.int32
    return np.ascontiguousarray(raw.transpose(1, 0, 2)).view(elem).reshape(n, -1)


def _assert_index_equals_oracle(index, sig_nH, L, k):
    want = oracle.fit_index(sig_nH, L, k)
    assert index.n_total_buckets == want.n_total_buckets
    assert np.array_equal(index.get_table_bucket_offsets(), want.table_bucket_offsets)
    assert np.array_equal(index.get_bucket_candidate_offsets(), want.bucket_candidate_offsets)
    assert np.array_equal(index.get_bucket_signatures(), want.bucket_signatures)
    assert np.array_equal(index.get_candidate_indices(), want.candidate_indices)
    return want


def _assert_candidates_equal(cand, want):
    indices, offsets, counts = want
    assert cand.n_queries == len(counts)
    assert np.array_equal(cand.get_offsets(), offsets)
    assert np.array_equal(cand.get_counts(), counts)
    assert np.array_equal(cand.get_indices(), indices)
    assert cand.n_total_candidates == len(indices)


# ------------------------------------------------------------------------------------------
# RPLSH
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("n,d,L,k", [(3000, 32, 8, 12), (1000, 100, 32, 16), (777, 33, 3, 20),
                                     (5000, 16, 4, 2), (257, 7, 2, 40)])
def test_rplsh_fit_query_parity(eng, dtype, n, d, L, k):
    culsh, core_mod = eng
    rng = np.random.RandomState(n + d)
    X = rng.randn(n, d).astype(dtype)
    Q = np.concatenate([X[:40] + 0.01 * rng.randn(40, d), rng.randn(25, d)]).astype(dtype)
    model = culsh.RPLSH(L, k, seed=7).fit(X)
    ix = model.index
    P = ix.get_projection_matrix().reshape(L * k, d)
    assert P.dtype == dtype

    core = core_mod.RPLSHCore(L, k, 7)
    sig = _sig_matrix(core.hash(X, ix))
    near = oracle.rplsh_near_boundary(X, P, REL_BAND)
    want_sig = oracle.rplsh_signatures(X, P)
    assert np.array_equal(sig[~near], want_sig[~near])
    assert near.mean() < 1e-3

    _assert_index_equals_oracle(ix, sig, L, k)
    qsig = _sig_matrix(core.hash(Q, ix))
    qnear = oracle.rplsh_near_boundary(Q, P, REL_BAND)
    assert np.array_equal(qsig[~qnear], oracle.rplsh_signatures(Q, P)[~qnear])
    oidx = oracle.fit_index(sig, L, k)
    _assert_candidates_equal(model.query(Q), oracle.query_index(oidx, qsig))


def test_rplsh_fit_query_self_join_and_batches(eng):
    culsh, _ = eng
    rng = np.random.RandomState(0)
    X = rng.randn(2000, 24).astype(np.float32)
    lsh = culsh.RPLSH(6, 10, seed=3)
    a = lsh.fit_query(X)
    model = lsh.fit(X)
    b = model.query(X)
    for f in ("get_indices", "get_offsets", "get_counts"):
        assert np.array_equal(getattr(a, f)(), getattr(b, f)())
    off = a.get_offsets().astype(np.int64)
    ind = a.get_indices()
    for q in range(0, 2000, 97):  # every row is its own candidate
        seg = ind[off[q]:off[q + 1]]
        assert q in seg and np.all(np.diff(seg) > 0)
    for bs in (10, 333, 1999, 2000, 5000):
        c = model.query(X, batch_size=bs)
        for f in ("get_indices", "get_offsets", "get_counts"):
            assert np.array_equal(getattr(c, f)(), getattr(b, f)())
    c = lsh.fit_query(X, batch_size=500)
    assert np.array_equal(c.get_indices(), b.get_indices())


def test_count_pass_bounds_feed_the_warp_path(eng):
    """From 2^22 (query, table) pairs on, the count pass keeps the list bounds it reads and the warp
    dedupe path takes them from there; smaller batches fetch them through the bucket ids.  Both
    ways, and the self-join, must give the same CSR."""
    culsh, _ = eng
    rng = np.random.RandomState(17)
    n, d, L, k = 140_000, 16, 32, 22
    X = rng.randn(n, d).astype(np.float32)
    lsh = culsh.RPLSH(L, k, seed=5)
    model = lsh.fit(X)
    whole = model.query(X)                       # 4.48 M pairs in one batch
    parts = model.query(X, batch_size=50_000)    # 1.6 M pairs per batch
    joined = lsh.fit_query(X)
    for f in ("get_indices", "get_offsets", "get_counts"):
        assert np.array_equal(getattr(whole, f)(), getattr(parts, f)())
        assert np.array_equal(getattr(whole, f)(), getattr(joined, f)())
    counts = whole.get_counts().astype(np.int64)
    assert counts.min() >= 1 and (counts <= 256).mean() > 0.5  # the warp path carries most of this case


def test_rplsh_zero_rows_take_the_sign_bit_rule(eng):
    """x.p == +0.0 hashes to 1 (sign bit clear), as upstream's kernel; upstream's Python oracle
    (x > 0) would give 0."""
    culsh, core_mod = eng
    X = np.zeros((64, 8), dtype=np.float32)
    X[1::2] = np.random.RandomState(1).randn(32, 8)
    model = culsh.RPLSH(2, 8, seed=1).fit(X)
    sig = core_mod.RPLSHCore(2, 8, 1).hash(X, model.index)
    assert np.all(sig[:, 0::2, :] == 1)
    cand = model.query(X[:2])
    off = cand.get_offsets()
    assert np.array_equal(cand.get_indices()[: int(off[1])], np.arange(0, 64, 2))


# ------------------------------------------------------------------------------------------
# PSLSH
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [np.float32, np.float64])
@pytest.mark.parametrize("n,d,L,k,w,scale", [(3000, 32, 8, 4, 4, 1.0), (1000, 100, 16, 8, 8, 1.0),
                                             (999, 18, 5, 3, 1, 30.0), (600, 10, 2, 2, 1, 5000.0),
                                             (500, 12, 4, 16, 4, 1.0)])
def test_pslsh_fit_query_parity(eng, dtype, n, d, L, k, w, scale):
    """scale 30 pushes hash values beyond int8, 5000 beyond int16 (key widening paths)."""
    culsh, core_mod = eng
    rng = np.random.RandomState(n + d + k)
    X = (scale * rng.randn(n, d)).astype(dtype)
    Q = np.concatenate([X[:30] + 0.01 * rng.randn(30, d), scale * rng.randn(20, d),
                        1e6 * rng.randn(5, d)]).astype(dtype)  # the last rows fall outside every bucket
    model = culsh.PStableLSH(L, k, window_size=w, seed=11).fit(X)
    ix = model.index
    P = ix.get_projection_matrix().reshape(L * k, d)
    b = ix.get_bias()
    assert np.all(b > 0) and np.all(b <= 1)

    core = core_mod.PSLSHCore(L, k, w, 11)
    sig = _sig_matrix(core.hash(X, ix))
    near = oracle.pslsh_near_boundary(X, P, b, REL_BAND)
    want = oracle.pslsh_signatures(X, P, b)
    assert np.array_equal(sig[~near], want[~near])
    if scale == 1.0:  # the band is relative to sum|x.p|: at large magnitudes it spans whole buckets
        assert near.mean() < 2e-3
    lo, hi = int(sig.min()), int(sig.max())
    expect_eb = 1 if (lo >= -128 and hi <= 127) else (2 if (lo >= -32768 and hi <= 32767) else 4)
    assert ix.elem_bytes == expect_eb  # narrowest element width that holds every indexed value

    _assert_index_equals_oracle(ix, sig, L, k)
    qsig = _sig_matrix(core.hash(Q, ix))
    _assert_candidates_equal(model.query(Q), oracle.query_index(oracle.fit_index(sig, L, k), qsig))


def test_large_tables_use_the_chunked_tile_scan(eng):
    """Tables of 512 tiles or more take the two-level tile scan of the radix sort (here 8-byte
    keys: 3072 items per tile, 554 tiles per table); index arrays must still equal the oracle's."""
    culsh, core_mod = eng
    rng = np.random.RandomState(91)
    n, d, L, k, w = 1_700_000, 4, 2, 6, 1
    X = rng.randn(n, d).astype(np.float32)
    model = culsh.PStableLSH(L, k, window_size=w, seed=21).fit(X)
    ix = model.index
    assert ix.elem_bytes == 1
    sig = _sig_matrix(core_mod.PSLSHCore(L, k, w, 21).hash(X, ix))
    oidx = _assert_index_equals_oracle(ix, sig, L, k)
    sel = rng.randint(0, n, 16)
    _assert_candidates_equal(model.query(X[sel]), oracle.query_index(oidx, sig[sel]))


def test_pslsh_consistency_and_auto_window(eng):
    culsh, _ = eng
    rng = np.random.RandomState(5)
    X = rng.randn(1500, 20).astype(np.float32)
    lsh = culsh.PStableLSH(8, 4, window_size=4, seed=2)
    a = lsh.fit_query(X)
    model = lsh.fit(X)
    b = model.query(X)
    for f in ("get_indices", "get_offsets", "get_counts"):
        assert np.array_equal(getattr(a, f)(), getattr(b, f)())
    for bs in (10, 50, 100):
        c = model.query(X[:300], batch_size=bs)
        d = model.query(X[:300])
        assert np.array_equal(c.get_indices(), d.get_indices())
        assert np.array_equal(c.get_offsets(), d.get_offsets())
    Xn = X / np.linalg.norm(X, axis=1, keepdims=True) * 100.0
    m = culsh.PStableLSH(4, 4, window_size="auto", seed=1).fit(Xn.astype(np.float32))
    assert m.window_size == 100 or m.window_size == 99  # python/tests/test_pslsh.py:243-255


def test_pslsh_compressed_sort_equals_plain_sort(eng, monkeypatch):
    """One-byte p-stable keys (up to eight hashes) whose values span at most 32 levels are sorted in
    compressed form (5 bits per hash); the index must be the one the sort of the plain keys builds
    (negative and non-negative hash values, odd and even numbers of hashes, one and two key words,
    more than one sort tile; sixteen hashes keep the plain sort); with five to eight hashes the
    compressed key and the row id travel packed in one 64-bit item."""
    culsh, _ = eng
    rng = np.random.RandomState(41)
    for n, d, L, k, w in [(20000, 24, 5, 8, 4), (9000, 16, 3, 3, 2), (5000, 32, 4, 16, 8), (7000, 12, 6, 5, 3)]:
        X = rng.randn(n, d).astype(np.float32)
        monkeypatch.delenv("CULSH_SORT_PLAIN_KEYS", raising=False)
        a = culsh.PStableLSH(L, k, window_size=w, seed=3).fit(X)
        monkeypatch.setenv("CULSH_SORT_PLAIN_KEYS", "1")
        b = culsh.PStableLSH(L, k, window_size=w, seed=3).fit(X)
        monkeypatch.delenv("CULSH_SORT_PLAIN_KEYS", raising=False)
        monkeypatch.setenv("CULSH_SORT_NO_PACK", "1")  # compressed, key and row id in separate arrays
        c = culsh.PStableLSH(L, k, window_size=w, seed=3).fit(X)
        monkeypatch.delenv("CULSH_SORT_NO_PACK", raising=False)
        assert a.index.elem_bytes == 1
        for g in ("get_candidate_indices", "get_bucket_signatures", "get_bucket_candidate_offsets",
                  "get_table_bucket_offsets"):
            assert np.array_equal(getattr(a.index, g)(), getattr(b.index, g)()), (g, n, k)
            assert np.array_equal(getattr(a.index, g)(), getattr(c.index, g)()), (g, n, k)
        sig = a.index.get_bucket_signatures().view(np.int32)
        assert sig.min() < 0 < sig.max()


def test_own_parameter_generator_equals_curand_host_api(eng, monkeypatch):
    """The single-launch XORWOW kernel must reproduce cuRAND's host API bit for bit: parameter
    counts below, at and above one round of the 4096 generator streams, a uniform call that starts
    in the middle of a round, MinHash's two consecutive integer calls (rplsh/hash.cuh:59-78,
    pslsh/hash.cuh:60-89, minhash/hash.cuh:26-54)."""
    culsh, core_mod = eng
    ones = {d: np.ones((4, d), np.float32) for d in (2, 6, 24, 128, 250)}
    tiny = sp.csr_matrix(np.array([[1, 1, 0, 0]], dtype=np.float32))
    handle_core = core_mod.RPLSHCore(1, 1, 0)  # every core of this thread shares one engine handle

    def params(host_api, fam, L, k, d, seed):
        if host_api:
            monkeypatch.setenv("CULSH_PARAMS_HOST_API", "1")
        else:
            monkeypatch.delenv("CULSH_PARAMS_HOST_API", raising=False)
        if fam == "rplsh":
            est = culsh.RPLSH(L, k, seed=seed)
        elif fam == "pslsh":
            est = culsh.PStableLSH(L, k, window_size=3, seed=seed)
        else:
            est = culsh.MinHashLSH(L, k, seed=seed)
        handle_core.set_param_cache(False)
        try:
            ix = est.fit(tiny if fam == "minhash" else ones[d]).index
        finally:
            handle_core.set_param_cache(True)
        if fam == "rplsh":
            return [ix.get_projection_matrix()]
        if fam == "pslsh":
            return [ix.get_projection_matrix(), ix.get_bias()]
        return [ix.get_hash_a(), ix.get_hash_b()]

    cases = [("rplsh", 1, 1, 2), ("rplsh", 3, 5, 6), ("rplsh", 16, 16, 24), ("rplsh", 32, 16, 128),
             ("rplsh", 48, 24, 250), ("pslsh", 1, 1, 2), ("pslsh", 7, 3, 6), ("pslsh", 16, 8, 128),
             ("pslsh", 80, 64, 24), ("pslsh", 100, 41, 6), ("minhash", 1, 1, 0), ("minhash", 32, 4, 0),
             ("minhash", 256, 16, 0), ("minhash", 625, 16, 0)]
    for fam, L, k, d in cases:
        for seed in (0, 42, 2**40 + 7):
            own = params(False, fam, L, k, d, seed)
            ref = params(True, fam, L, k, d, seed)
            for a, b in zip(own, ref):
                assert a.dtype == b.dtype and a.shape == b.shape
                assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), (fam, L, k, d, seed)


# ------------------------------------------------------------------------------------------
# MinHash
# ------------------------------------------------------------------------------------------
def _random_csr(rng, n, d, density):
    X = sp.random(n, d, density=density, format="csr", dtype=np.float32, random_state=rng)
    X.data[:] = 1.0
    X.sort_indices()
    return X


@pytest.mark.parametrize("n,d,L,k,density", [(1000, 100, 8, 4, 0.1), (1000, 100, 32, 8, 0.5),
                                             (500, 5000, 64, 16, 0.01), (300, 50, 3, 3, 0.2),
                                             (400, 1 << 20, 4, 2, 1e-5)])
def test_minhash_fit_query_parity(eng, n, d, L, k, density):
    culsh, core_mod = eng
    rng = np.random.RandomState(L * k)
    X = _random_csr(rng, n, d, density)
    Q = sp.vstack([X[:30], _random_csr(rng, 20, d, density)]).tocsr()
    Q.sort_indices()
    model = culsh.MinHashLSH(L, k, seed=9).fit(X)
    ix = model.index
    A, B = ix.get_hash_a(), ix.get_hash_b()
    assert np.all(A >= 1) and np.all(A < oracle.MINHASH_PRIME) and np.all(B < oracle.MINHASH_PRIME)

    core = core_mod.MinHashCore(L, k, 9)
    sig = _sig_matrix(core.hash(X.indices, X.indptr, n, ix))
    want = oracle.minhash_signatures(X.indices, X.indptr, A, B)
    assert np.array_equal(sig, want)  # integer stage: bit exact
    empty = np.flatnonzero(np.diff(X.indptr) == 0)
    if len(empty):
        assert np.all(sig[empty] == 0xFFFFFFFF)

    oidx = _assert_index_equals_oracle(ix, want, L, k)
    qsig = oracle.minhash_signatures(Q.indices, Q.indptr, A, B)
    _assert_candidates_equal(model.query(Q), oracle.query_index(oidx, qsig))
    a = culsh.MinHashLSH(L, k, seed=9).fit_query(X)
    b = model.query(X)
    assert np.array_equal(a.get_indices(), b.get_indices())
    assert np.array_equal(a.get_offsets(), b.get_offsets())


# ------------------------------------------------------------------------------------------
# Gather / dedupe paths and edge cases
# ------------------------------------------------------------------------------------------
def test_minhash_values_next_to_the_prime(eng):
    """Hash parameters chosen so that a*c + b lands in [p, 2^32 + 15) before the final reduction -
    the inputs for which the kernel's fast evaluation wraps and the row is evaluated again in full -
    and right below p, where it must not."""
    culsh, core_mod = eng
    p = oracle.MINHASH_PRIME
    L, k, d = 2, 4, 64
    A = np.array([1, 1, 2, 3, 1, 5, 7, 4294967290], dtype=np.uint32)
    B = np.array([p - 1, p - 3, p - 5, 5, 0, p - 2, p - 1, 17], dtype=np.uint32)
    rows = [[3, 10], [0], [1, 2, 3, 4, 5, 6, 7], [], [2, 40, 63], [1], list(range(0, 64, 3))]
    indptr = np.concatenate([[0], np.cumsum([len(r) for r in rows])]).astype(np.int32)
    indices = np.array([c for r in rows for c in r], dtype=np.int32)
    want = oracle.minhash_signatures(indices, indptr, A, B)
    # at least one evaluation per family of cases: wraps (sum >= p) and stays (sum < p)
    sums = A[None, :].astype(np.uint64) * indices[:, None].astype(np.uint64) + B[None, :].astype(np.uint64)
    assert ((sums >= p) & (sums < 2**32 + 15)).any() and (sums < p).any()
    oidx = oracle.fit_index(want, L, k)
    ix = core_mod.MinHashIndex.load(
        candidate_indices=oidx.candidate_indices, bucket_signatures=oidx.bucket_signatures,
        bucket_candidate_offsets=oidx.bucket_candidate_offsets, table_bucket_offsets=oidx.table_bucket_offsets,
        hash_a=A, hash_b=B, n_total_candidates=len(oidx.candidate_indices), n_total_buckets=oidx.n_total_buckets,
        n_hash_tables=L, n_hashes=k, sig_nbytes=oidx.sig_nbytes, n_features=d, seed=0)
    got = _sig_matrix(core_mod.MinHashCore(L, k, 0).hash(indices, indptr, len(rows), ix))
    assert np.array_equal(got, want)


def test_warp_path_sorts_up_to_1024_ids(eng):
    """One or two tables of ~700-row buckets: raw candidate counts on both sides of 512 (sixteen ids
    per lane of the warp's sort network) and of 1024 (thirty-two, the warp path's limit)."""
    culsh, core_mod = eng
    rng = np.random.RandomState(77)
    n, d = 45000, 10
    X = rng.randn(n, d).astype(np.float32)
    seen = np.zeros(3, bool)
    for L, k in ((1, 6), (2, 7)):
        model = culsh.RPLSH(L, k, seed=5).fit(X)
        core = core_mod.RPLSHCore(L, k, 5)
        sig = _sig_matrix(core.hash(X, model.index))
        sel = rng.randint(0, n, 96)
        want = oracle.query_index(oracle.fit_index(sig, L, k), sig[sel])
        raw = np.zeros(len(sel), np.int64)  # raw = sum of the matched buckets' sizes
        for t in range(L):
            keys = [bytes(r) for r in sig[:, t * k:(t + 1) * k]]
            sizes = {}
            for kk in keys:
                sizes[kk] = sizes.get(kk, 0) + 1
            raw += np.array([sizes[keys[i]] for i in sel])
        seen |= np.array([(raw <= 512).any(), ((raw > 512) & (raw <= 1024)).any(), (raw > 1024).any()])
        _assert_candidates_equal(model.query(X[sel]), want)
    assert seen.all(), seen


def test_large_buckets_use_the_bitmap_path(eng):
    """k = 2 sign bits -> four buckets per table of ~n/4 rows: raw candidate counts far above
    the warp path's limit; heavy cross-table duplication."""
    culsh, core_mod = eng
    rng = np.random.RandomState(42)
    n, d, L, k = 40000, 12, 6, 2
    X = rng.randn(n, d).astype(np.float32)
    model = culsh.RPLSH(L, k, seed=5).fit(X)
    core = core_mod.RPLSHCore(L, k, 5)
    sig = _sig_matrix(core.hash(X, model.index))
    Q = X[:16]
    _assert_candidates_equal(model.query(Q), oracle.query_index(oracle.fit_index(sig, L, k), sig[:16]))


def test_bitmap_windows_beyond_one_window(eng):
    """More rows than one shared-memory bitmap window covers (2^20 ids)."""
    culsh, core_mod = eng
    rng = np.random.RandomState(8)
    n, d, L, k = (1 << 20) + 300000, 8, 3, 3
    X = rng.randn(n, d).astype(np.float32)
    model = culsh.RPLSH(L, k, seed=6).fit(X)
    core = core_mod.RPLSHCore(L, k, 6)
    sig = _sig_matrix(core.hash(X, model.index))
    oidx = oracle.fit_index(sig, L, k)
    assert np.array_equal(model.index.get_candidate_indices(), oidx.candidate_indices)
    sel = [0, 5, n - 1, n // 2]
    _assert_candidates_equal(model.query(X[sel]), oracle.query_index(oidx, sig[sel]))


def test_sort_path_for_mid_sized_sets_on_a_large_index(eng):
    """More rows than two bitmap windows: candidate sets between the warp path's and the sort
    path's limits are merged by the shared-memory radix sort; larger ones by windowed bitmaps."""
    culsh, core_mod = eng
    rng = np.random.RandomState(21)
    n, d, L, k = 2_300_000, 8, 4, 16
    X = rng.randn(n, d).astype(np.float32)
    model = culsh.RPLSH(L, k, seed=8).fit(X)
    core = core_mod.RPLSHCore(L, k, 8)
    sig = _sig_matrix(core.hash(X, model.index))
    oidx = oracle.fit_index(sig, L, k)
    sel = rng.randint(0, n, 24)
    cand = model.query(X[sel])
    want = oracle.query_index(oidx, sig[sel])
    counts = want[2].astype(np.int64)
    assert ((counts > 1024) & (counts <= 8192)).mean() >= 0.15  # a good share takes the sort path
    _assert_candidates_equal(cand, want)
    # one-table, few-bit index on the same rows: sets far above the sort path's limit
    m2 = culsh.RPLSH(2, 3, seed=8).fit(X)
    sig2 = _sig_matrix(core_mod.RPLSHCore(2, 3, 8).hash(X, m2.index))
    _assert_candidates_equal(m2.query(X[sel[:3]]), oracle.query_index(oracle.fit_index(sig2, 2, 3), sig2[sel[:3]]))


@pytest.mark.parametrize("bits,stage,threads,slices,loads", [
    (None, None, None, None, None),  # defaults: one window at this size, ids stored straight into the CSR
    (131072, 0, 256, 1, 16),         # 3 windows, no stage, a warp's ids do not fit one batch of loads at 16
    (65536, 0, 512, 0, 4),           # 5 windows, no stage, second walk over the lists
    (8192, 256, 256, 1, 16),         # many windows (falls back to the windowed bitmap kernel)
    (65536, 256, 256, 1, 8),         # 5 windows, many copy-out chunks, precomputed slices
    (65536, 300, 512, 0, 4),         # the CTAs search their slices themselves
    (131072, 40960, 384, 0, 8),      # 3 windows, one chunk
    (1 << 20, 5632, 384, 1, 4),      # one window
])
def test_chained_dedupe_windows_chunks_and_slices(eng, monkeypatch, bits, stage, threads, slices, loads):
    """Query sets dominated by large candidate sets take the chained single-pass kernel; its window
    size, stage size, CTA size and slice source must not change the result."""
    culsh, core_mod = eng
    for name, v in (("CULSH_CHAIN_BITS", bits), ("CULSH_CHAIN_STAGE", stage), ("CULSH_CHAIN_THREADS", threads),
                    ("CULSH_CHAIN_SLICES", slices), ("CULSH_CHAIN_LOADS", loads)):
        if v is None:
            monkeypatch.delenv(name, raising=False)
        else:
            monkeypatch.setenv(name, str(v))
    rng = np.random.RandomState(33)
    n, d, L, k = 300_000, 8, 6, 5
    X = rng.randn(n, d).astype(np.float32)
    model = culsh.RPLSH(L, k, seed=12).fit(X)
    core = core_mod.RPLSHCore(L, k, 12)
    sig = _sig_matrix(core.hash(X, model.index))
    oidx = oracle.fit_index(sig, L, k)
    sel = np.concatenate([rng.randint(0, n, 40), [0, n - 1]])
    Q = X[sel].copy()
    Q[5] = 1e6 * np.sign(rng.randn(d)).astype(np.float32)  # most likely a rare signature
    sigq = _sig_matrix(core.hash(Q, model.index))
    want = oracle.query_index(oidx, sigq)
    assert (want[2].astype(np.int64) > 20000).mean() > 0.8  # large sets: ~n/32 rows per table
    _assert_candidates_equal(model.query(Q), want)


def test_query_by_row_keys_equals_fit_query(eng):
    """The packed keys an index reports for its own rows, fed back as queries, give the self-join
    of fit_query (the path a row-sharded self-join takes between shards); one- and two-word keys,
    sign bits and p-stable bytes."""
    import torch
    culsh, core_mod = eng
    rng = np.random.RandomState(17)
    n, d = 5000, 24
    X = rng.randn(n, d).astype(np.float32)
    X[100:140] = X[7]  # a larger bucket
    cases = [(culsh.RPLSH(6, 10, seed=3), core_mod.RPLSHCore(6, 10, 3)),
             (culsh.RPLSH(3, 40, seed=3), core_mod.RPLSHCore(3, 40, 3)),
             (culsh.PStableLSH(5, 6, window_size=2, seed=3), core_mod.PSLSHCore(5, 6, 2, 3))]
    for lsh, core in cases:
        model = lsh.fit(X)
        ix = model.index
        keys = torch.full((ix.n_hash_tables, n, ix.key_words), -1, dtype=torch.int32, device="cuda")
        ix.row_keys(keys.data_ptr())
        got = core.query_keys(keys.data_ptr(), n, ix)
        want = lsh.fit_query(X)
        assert np.array_equal(got.get_offsets(), want.get_offsets())
        assert np.array_equal(got.get_indices(), want.get_indices())
        assert np.array_equal(got.get_counts(), want.get_counts())
        sub = core.query_keys(keys[:, :0].contiguous().data_ptr(), 0, ix)
        assert sub.n_queries == 0


def test_trim_scratch_frees_and_recovers(eng):
    """The handle's grow-only temporaries and kept result blocks can be handed back to the device;
    the next call allocates what it needs again and returns the same result."""
    import torch
    culsh, core_mod = eng
    rng = np.random.RandomState(3)
    X = rng.randn(200_000, 16).astype(np.float32)
    lsh = culsh.RPLSH(8, 6, seed=2)
    core = core_mod.RPLSHCore(8, 6, 2)
    model = lsh.fit(X)
    first = model.query(X[:2000])
    idx, off = first.get_indices(), first.get_offsets()
    del first
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    core.trim_scratch(0)
    free_after = torch.cuda.mem_get_info()[0]
    assert free_after > free_before + (8 << 20)  # sort buffers of 1.6 M items alone are 12.8 MB
    again = model.query(X[:2000])
    assert np.array_equal(again.get_indices(), idx) and np.array_equal(again.get_offsets(), off)
    core.trim_scratch(1 << 40)  # nothing is that large: a no-op
    assert np.array_equal(lsh.fit(X).query(X[:2000]).get_offsets(), off)


def test_no_match_and_zero_queries(eng):
    culsh, _ = eng
    rng = np.random.RandomState(3)
    X = rng.randn(200, 16).astype(np.float32)
    model = culsh.PStableLSH(4, 8, window_size=1, seed=4).fit(X)
    far = (1000.0 + rng.randn(7, 16)).astype(np.float32)
    c = model.query(far)
    assert c.n_queries == 7 and c.n_total_candidates == 0
    assert np.array_equal(c.get_counts(), np.zeros(7, np.uint64))
    assert np.array_equal(c.get_offsets(), np.zeros(8, np.uint64))
    assert c.get_indices().shape == (0,)
    mixed = np.concatenate([far[:2], X[:3], far[2:4]])
    m = model.query(mixed)
    counts = m.get_counts()
    assert np.all(counts[[0, 1, 5, 6]] == 0) and np.all(counts[2:5] >= 1)
    z = model.query(np.zeros((0, 16), dtype=np.float32))
    assert z.n_queries == 0 and z.n_total_candidates == 0


def test_all_rows_identical_and_all_distinct(eng):
    culsh, _ = eng
    X = np.tile(np.arange(1, 9, dtype=np.float32), (300, 1))
    model = culsh.RPLSH(3, 5, seed=1).fit(X)
    assert model.index.n_total_buckets == 3
    c = model.query(X[:2])
    assert np.array_equal(c.get_indices(), np.concatenate([np.arange(300), np.arange(300)]))
    rng = np.random.RandomState(2)
    Y = rng.randn(64, 30).astype(np.float32)
    m2 = culsh.RPLSH(2, 60, seed=1).fit(Y)  # 60 bits: all rows distinct, two-word keys
    assert m2.index.n_total_buckets == 128 and m2.index.key_words == 2
    c2 = m2.query(Y)
    assert np.array_equal(c2.get_indices(), np.arange(64))


def test_errors_are_python_exceptions(eng):
    culsh, core_mod = eng
    X = np.random.RandomState(0).randn(50, 8)
    m32 = culsh.RPLSH(2, 4, seed=1).fit(X.astype(np.float32))
    with pytest.raises(RuntimeError, match="float32"):
        m32._core.query_double(X, 50, m32.index)
    with pytest.raises(ValueError):
        m32.query(np.zeros((3, 9), dtype=np.float32))
    with pytest.raises(TypeError):
        culsh.RPLSH(2, 4, seed=1).fit(X.astype(np.float16))
    with pytest.raises(ValueError):
        culsh.RPLSH(0, 4)
    with pytest.raises(RuntimeError, match="even"):
        culsh.RPLSH(1, 1, seed=1).fit(np.zeros((4, 3), dtype=np.float32))
    with pytest.raises(ValueError):
        Xs = sp.random(10, 10, density=0.5, format="csr")
        Xs.indices = Xs.indices.astype(np.int64)
        Xs.indptr = Xs.indptr.astype(np.int64)
        culsh.MinHashLSH(2, 2, seed=1).fit(Xs)


def test_device_inputs_match_host_inputs(eng, monkeypatch):
    import torch
    culsh, core_mod = eng
    rng = np.random.RandomState(12)
    X = rng.randn(3000, 48).astype(np.float32)
    Q = rng.randn(100, 48).astype(np.float32)
    mh = culsh.RPLSH(8, 8, seed=21).fit(X)
    md = culsh.RPLSH(8, 8, seed=21).fit(torch.from_numpy(X).cuda())
    assert np.array_equal(mh.index.get_candidate_indices(), md.index.get_candidate_indices())
    a = mh.query(Q)
    b = md.query(torch.from_numpy(Q).cuda())
    assert np.array_equal(a.get_indices(), b.get_indices())
    t = b.get_indices(as_torch=True)
    assert t.is_cuda and np.array_equal(t.cpu().numpy(), a.get_indices())
    # host input larger than one staging chunk (32 MiB): chunked copy/hash pipeline
    Xb = rng.randn(300000, 64).astype(np.float32)
    i1 = culsh.RPLSH(2, 16, seed=3).fit(Xb).index
    i2 = culsh.RPLSH(2, 16, seed=3).fit(torch.from_numpy(Xb).cuda()).index
    assert np.array_equal(i1.get_candidate_indices(), i2.get_candidate_indices())
    assert np.array_equal(i1.get_bucket_signatures(), i2.get_bucket_signatures())
    # host CSR larger than one staging chunk (chunks of 65,536 column ids here): rows streamed in
    # chunks, with empty rows at chunk borders and one row longer than a chunk
    monkeypatch.setenv("CULSH_CSR_CHUNK_NNZ", "65536")
    Xs = _random_csr(rng, 9000, 5000, 0.01).tolil()
    Xs[4000, :] = 0
    Xs[4001, :] = 0
    Xs = Xs.tocsr()
    long_row = sp.csr_matrix((np.ones(70000, np.float32), (np.zeros(70000, int), np.arange(70000))), shape=(1, 80000))
    Xs = sp.vstack([sp.csr_matrix((Xs.data, Xs.indices, Xs.indptr), shape=(9000, 80000)), long_row,
                    sp.csr_matrix((1, 80000), dtype=np.float32)]).tocsr()
    Xs.sort_indices()
    assert Xs.nnz > 4 * 65536
    mh = culsh.MinHashLSH(6, 3, seed=8).fit(Xs)
    xi = torch.from_numpy(Xs.indices.astype(np.int32)).cuda()
    xp = torch.from_numpy(Xs.indptr.astype(np.int32)).cuda()
    dev = core_mod.MinHashCore(6, 3, 8).fit(xi, xp, Xs.shape[0], Xs.shape[1])
    for g in ("get_candidate_indices", "get_bucket_signatures", "get_bucket_candidate_offsets"):
        assert np.array_equal(getattr(mh.index, g)(), getattr(dev, g)()), g
    a = mh.query(Xs[:300])
    b = core_mod.MinHashCore(6, 3, 8).query(xi[:int(Xs.indptr[300])], xp[:301], 300, dev)
    assert np.array_equal(a.get_indices(), b.get_indices())


# ------------------------------------------------------------------------------------------
# save / load and the upstream-oracle fixtures
# ------------------------------------------------------------------------------------------
def test_save_load_round_trip(eng, tmp_path):
    culsh, _ = eng
    rng = np.random.RandomState(1)
    X = rng.randn(800, 20).astype(np.float32)
    Q = X[:50]
    for make, cls in ((lambda: culsh.RPLSH(6, 9, seed=5), culsh.RPLSHModel),
                      (lambda: culsh.PStableLSH(6, 4, window_size=3, seed=5), culsh.PStableLSHModel)):
        m = make().fit(X)
        path = str(tmp_path / "m.npz")
        m.save(path)
        m2 = cls.load(path)
        for attr in ("n_hash_tables", "n_hashes", "n_features"):
            assert getattr(m, attr) == getattr(m2, attr)
        for g in ("get_candidate_indices", "get_bucket_signatures", "get_bucket_candidate_offsets",
                  "get_table_bucket_offsets", "get_projection_matrix"):
            assert np.array_equal(getattr(m.index, g)(), getattr(m2.index, g)())
        assert m.index.seed == m2.index.seed and m.index.sig_nbytes == m2.index.sig_nbytes
        assert np.array_equal(m.query(Q).get_indices(), m2.query(Q).get_indices())
    Xs = _random_csr(rng, 400, 200, 0.05)
    m = culsh.MinHashLSH(8, 3, seed=5).fit(Xs)
    path = str(tmp_path / "mh.npz")
    m.save(path)
    m2 = culsh.MinHashLSHModel.load(path)
    assert np.array_equal(m.index.get_hash_a(), m2.index.get_hash_a())
    assert np.array_equal(m.index.get_bucket_signatures(), m2.index.get_bucket_signatures())
    assert np.array_equal(m.query(Xs).get_indices(), m2.query(Xs).get_indices())


def _load_fixture_index(core_mod, g, family):
    L, k = int(g["L"]), int(g["k"])
    oidx = oracle.fit_index(g["sig_X"], L, k)
    common = dict(candidate_indices=oidx.candidate_indices, bucket_signatures=oidx.bucket_signatures,
                  bucket_candidate_offsets=oidx.bucket_candidate_offsets,
                  table_bucket_offsets=oidx.table_bucket_offsets,
                  n_total_candidates=len(oidx.candidate_indices), n_total_buckets=oidx.n_total_buckets,
                  n_hash_tables=L, n_hashes=k, sig_nbytes=oidx.sig_nbytes, seed=0)
    if family == "rplsh":
        return core_mod.RPLSHIndex.load_float(projection=g["P"], n_features=g["X"].shape[1], **common)
    if family == "pslsh":
        w = int(g["window"])
        return core_mod.PSLSHIndex.load_float(projection=(g["P"] / w).astype(np.float32),
                                              bias=(g["b"] / w).astype(np.float32),
                                              n_features=g["X"].shape[1], window_size=w, **common)
    return core_mod.MinHashIndex.load(hash_a=g["A"], hash_b=g["B"], n_features=int(g["n_features"]), **common)


def test_upstream_python_oracle_fixtures(eng, golden_dir):
    """Indexes built from the fixtures written by upstream's ref_lsh.py, queried by the CUDA
    path: candidate lists equal upstream's (dense families: for queries whose signatures have
    no element inside the rounding band)."""
    culsh, core_mod = eng
    g = np.load(os.path.join(golden_dir, "ref_lsh_minhash.npz"))
    ix = _load_fixture_index(core_mod, g, "minhash")
    core = core_mod.MinHashCore(int(g["L"]), int(g["k"]), 0)
    nq = len(g["Q_indptr"]) - 1
    sig = _sig_matrix(core.hash(g["Q_indices"], g["Q_indptr"], nq, ix))
    assert np.array_equal(sig, g["sig_Q"])
    c = core.query(g["Q_indices"], g["Q_indptr"], nq, ix)
    assert np.array_equal(c.get_offsets(), g["cand_offsets"])
    assert np.array_equal(c.get_indices(), g["cand_indices"])

    for fam, Core in (("rplsh", core_mod.RPLSHCore), ("pslsh", core_mod.PSLSHCore)):
        g = np.load(os.path.join(golden_dir, f"ref_lsh_{fam}.npz"))
        L, k = int(g["L"]), int(g["k"])
        ix = _load_fixture_index(core_mod, g, fam)
        core = Core(L, k, 0) if fam == "rplsh" else Core(L, k, int(g["window"]), 0)
        Q = g["Q"]
        sig = _sig_matrix(core.hash(Q, ix)).astype(np.int64)
        same = np.all(sig == g["sig_Q"].astype(np.int64), axis=1)
        assert same.mean() > 0.9
        c = core.query_float(Q, len(Q), ix)
        off, ind = c.get_offsets().astype(np.int64), c.get_indices()
        roff, rind = g["cand_offsets"].astype(np.int64), g["cand_indices"]
        for q in np.flatnonzero(same):
            assert np.array_equal(ind[off[q]:off[q + 1]], rind[roff[q]:roff[q + 1]])


def test_shard_merge_equals_unsharded(eng):
    import torch
    culsh, core_mod = eng
    rng = np.random.RandomState(77)
    n, d, L, k = 6000, 16, 6, 6
    X = rng.randn(n, d).astype(np.float32)
    Q = X[rng.randint(0, n, 200)] + 0.01 * rng.randn(200, d).astype(np.float32)
    whole = culsh.RPLSH(L, k, seed=13).fit(X).query(Q)
    for shards in (2, 3, 8):
        per = -(-n // shards)
        keep, ip, op, bases = [], [], [], []
        for r in range(shards):
            lo, hi = r * per, min(n, (r + 1) * per)
            c = culsh.RPLSH(L, k, seed=13).fit(X[lo:hi]).query(Q)
            keep.append(c)
            a, _, o = c.device_pointers()
            ip.append(a)
            op.append(o)
            bases.append(lo)
        merged = core_mod.merge_shard_candidates(ip, op, bases, len(Q))
        assert np.array_equal(merged.get_indices(), whole.get_indices())
        assert np.array_equal(merged.get_offsets(), whole.get_offsets())
        assert np.array_equal(merged.get_counts(), whole.get_counts())


# ------------------------------------------------------------------------------------------
# tensor-core projection (tcgen05 3xTF32) against the CUDA-core projection and the oracle
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("variant", [{"CULSH_TC_VARIANT": "0"}, {"CULSH_TC_VARIANT": "1"}, {"CULSH_TC_VARIANT": "3"},
                                     {"CULSH_TC_VARIANT": "0", "CULSH_TC_KBLK": "32"}],
                         ids=["operands_from_shared_memory", "x_from_tensor_memory", "x_from_tensor_memory_192_columns",
                              "wide_k_blocks"])
def test_tensor_core_projection_kernel_variants(variant):
    """Which tensor-core kernel projects a shape is decided once per process (by shape, or by
    CULSH_TC_VARIANT / CULSH_TC_KBLK), so every case below also runs in child processes that
    force each kernel onto all shapes."""
    import subprocess
    import sys
    if os.environ.get("CULSH_TC_CHILD") == "1":
        pytest.skip("already inside the child process")
    env = dict(os.environ, CULSH_TC_CHILD="1", **variant)
    res = subprocess.run([sys.executable, "-m", "pytest", os.path.abspath(__file__), "-q", "-x", "-m", "gpu",
                          "-p", "no:cacheprovider", "-k",
                          "test_tensor_core_projection and not kernel_variants"],
                         env=env, capture_output=True, text=True, timeout=900)
    tail = (res.stdout + res.stderr)[-2000:]
    assert res.returncode == 0, tail
    assert "11 passed" in res.stdout, tail


@pytest.mark.parametrize("fam,n,d,L,k", [("rplsh", 5000, 128, 32, 16), ("rplsh", 1000, 100, 8, 12),
                                         ("rplsh", 3333, 256, 48, 24), ("rplsh", 130, 64, 3, 40),
                                         # sign-bit packer: second half of a unit starting off a 16-column
                                         # boundary (36, 4, 10), one bit and 32 bits per key
                                         ("rplsh", 777, 48, 5, 12), ("rplsh", 500, 32, 7, 1),
                                         ("rplsh", 640, 40, 3, 5), ("rplsh", 900, 64, 3, 32),
                                         ("pslsh", 4097, 96, 16, 8), ("pslsh", 999, 32, 5, 3),
                                         ("pslsh", 2000, 128, 4, 16)])
@pytest.mark.parametrize("kblk", [int(os.environ.get("CULSH_TC_KBLK", "16"))])  # chosen per process
def test_tensor_core_projection(eng, fam, n, d, L, k, kblk):
    culsh, core_mod = eng
    rng = np.random.RandomState(n + d + L)
    X = rng.randn(n, d).astype(np.float32)
    X[: n // 4] = np.round(X[: n // 4] * (50 if fam == "rplsh" else 4))  # integer rows: zero-lo fast path
    if fam == "rplsh":
        lsh, core = culsh.RPLSH(L, k, seed=31), core_mod.RPLSHCore(L, k, 31)
    else:
        lsh, core = culsh.PStableLSH(L, k, window_size=4, seed=31), core_mod.PSLSHCore(L, k, 4, 31)
    try:
        core.set_projection_path(2)  # tensor cores required: an unsupported shape is an error
        model = lsh.fit(X)
        assert core.last_stats()["hash_path"] == 1
        sig_tc = _index_row_signatures(model.index, fam)  # what the tensor-core fit really stored
        core.set_projection_path(1)
        model_simt = lsh.fit(X)
        assert core.last_stats()["hash_path"] == 0
        sig_simt = _index_row_signatures(model_simt.index, fam)
    finally:
        core.set_projection_path(0)
    P = model.index.get_projection_matrix().reshape(L * k, d)
    if fam == "rplsh":
        near, want = oracle.rplsh_near_boundary(X, P, REL_BAND), oracle.rplsh_signatures(X, P)
    else:
        b = model.index.get_bias()
        near, want = oracle.pslsh_near_boundary(X, P, b, REL_BAND), oracle.pslsh_signatures(X, P, b)
    assert np.array_equal(sig_tc[~near], want[~near])
    assert np.array_equal(sig_simt[~near], want[~near])
    assert (sig_tc != sig_simt).mean() < 1e-4
    _assert_index_equals_oracle(model.index, sig_tc, L, k)
