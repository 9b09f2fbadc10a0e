"""The CPU oracle against fixtures produced by upstream's own Python oracle
(python/tests/ref_lsh.py) with injected hash parameters."""
import os

import numpy as np
import pytest

from oracle import oracle


def _load(golden_dir, name):
    return np.load(os.path.join(golden_dir, name))


def _check_index_against_ref(idx, g, L, elem_dtype):
    """Bucket membership of every table equals upstream's dict-of-lists index."""
    s = idx.sig_nbytes
    bs = idx.bucket_signatures.reshape(-1, s)
    for t in range(L):
        b0, b1 = idx.table_bucket_offsets[t], idx.table_bucket_offsets[t + 1]
        ours = {}
        for b in range(b0, b1):
            key = tuple(int(v) for v in bs[b].view(elem_dtype))
            lo, hi = idx.bucket_candidate_offsets[b], idx.bucket_candidate_offsets[b + 1]
            rows = idx.candidate_indices[lo:hi]
            assert np.all(np.diff(rows) > 0), "row ids must ascend inside a bucket"
            ours[key] = rows.tolist()
        ptr = g[f"bucket_ptr_t{t}"]
        rows = g[f"bucket_rows_t{t}"]
        sigs = g[f"bucket_sigs_t{t}"]
        theirs = {tuple(int(v) for v in sigs[i]): rows[ptr[i]:ptr[i + 1]].tolist()
                  for i in range(len(sigs))}
        assert ours == theirs
        # canonical order: unsigned byte-lexicographic over raw signature memory
        as_bytes = [bytes(bs[b]) for b in range(b0, b1)]
        assert as_bytes == sorted(as_bytes)


def _check_query_against_ref(idx, sig_q, g):
    indices, offsets, counts = oracle.query_index(idx, sig_q)
    assert np.array_equal(offsets, g["cand_offsets"])
    assert np.array_equal(indices, g["cand_indices"])
    assert np.array_equal(counts, np.diff(offsets.astype(np.int64)).astype(np.uint64))


def test_rplsh_oracle_matches_upstream_python_oracle(golden_dir):
    g = _load(golden_dir, "ref_lsh_rplsh.npz")
    L, k = int(g["L"]), int(g["k"])
    sig = oracle.rplsh_signatures(g["X"], g["P"])
    near = oracle.rplsh_near_boundary(g["X"], g["P"])
    # upstream's oracle uses (x > 0), the CUDA rule is "sign bit clear"; equal away from 0
    assert np.array_equal(sig[~near], g["sig_X"][~near])
    idx = oracle.fit_index(g["sig_X"], L, k)
    _check_index_against_ref(idx, g, L, np.uint8)
    _check_query_against_ref(idx, g["sig_Q"], g)


def test_pslsh_oracle_matches_upstream_python_oracle(golden_dir):
    g = _load(golden_dir, "ref_lsh_pslsh.npz")
    L, k, w = int(g["L"]), int(g["k"]), int(g["window"])
    Ps = (g["P"] / w).astype(np.float32)
    bs = (g["b"] / w).astype(np.float32)
    sig = oracle.pslsh_signatures(g["X"], Ps, bs)
    near = oracle.pslsh_near_boundary(g["X"], Ps, bs, rel=1e-5)
    assert np.array_equal(sig[~near], g["sig_X"][~near])
    assert near.mean() < 1e-3
    idx = oracle.fit_index(g["sig_X"], L, k)
    _check_index_against_ref(idx, g, L, np.int32)
    _check_query_against_ref(idx, g["sig_Q"], g)


def test_minhash_oracle_matches_upstream_python_oracle(golden_dir):
    g = _load(golden_dir, "ref_lsh_minhash.npz")
    L, k = int(g["L"]), int(g["k"])
    sig = oracle.minhash_signatures(g["X_indices"], g["X_indptr"], g["A"], g["B"])
    assert np.array_equal(sig, g["sig_X"])  # integer stage: bit exact
    sig_q = oracle.minhash_signatures(g["Q_indices"], g["Q_indptr"], g["A"], g["B"], chunk_nnz=7)
    assert np.array_equal(sig_q, g["sig_Q"])
    empty = np.flatnonzero(np.diff(g["X_indptr"]) == 0)
    assert len(empty) >= 2 and np.all(sig[empty] == 0xFFFFFFFF)
    idx = oracle.fit_index(sig, L, k)
    _check_index_against_ref(idx, g, L, np.uint32)
    _check_query_against_ref(idx, sig_q, g)


def test_fit_query_is_fit_then_query():
    rng = np.random.RandomState(0)
    sig = rng.randint(0, 3, size=(200, 12)).astype(np.int32)
    a = oracle.fit_query(sig, 4, 3)
    idx = oracle.fit_index(sig, 4, 3)
    b = oracle.query_index(idx, sig)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    # every row is its own candidate
    ind, off, _ = a
    for q in range(200):
        assert q in ind[int(off[q]):int(off[q + 1])]


def test_fast_packed_variant_equals_canonical():
    rng = np.random.RandomState(3)
    n, nq, L, k = 3000, 200, 5, 7
    bits = rng.randint(0, 2, size=(n, L * k)).astype(np.uint8)
    qbits = np.concatenate([bits[:100], rng.randint(0, 2, size=(nq - 100, L * k)).astype(np.uint8)])
    idx = oracle.fit_index(bits, L, k)
    want = oracle.query_index(idx, qbits)
    tables = oracle.fast_fit_packed(oracle.pack_bits_msb_first(bits, L, k))
    got = oracle.fast_query_packed(tables, oracle.pack_bits_msb_first(qbits, L, k))
    for x, y in zip(got, want):
        assert np.array_equal(x, y)
    # packed order == canonical bucket order
    for t in range(L):
        b0, b1 = idx.table_bucket_offsets[t], idx.table_bucket_offsets[t + 1]
        raw = idx.bucket_signatures.reshape(-1, k)[b0:b1]
        packed = oracle.pack_bits_msb_first(raw.reshape(-1, k), 1, k)[0]
        assert np.array_equal(packed, tables[t][0])


def test_shard_union_equals_unsharded():
    rng = np.random.RandomState(5)
    n, nq, L, k = 1000, 64, 4, 2
    sig = rng.randint(-2, 3, size=(n, L * k)).astype(np.int32)
    qsig = sig[rng.randint(0, n, size=nq)]
    want = oracle.query_index(oracle.fit_index(sig, L, k), qsig)
    for shards in (2, 3, 8):
        per = -(-n // shards)
        res, bases = [], []
        for r in range(shards):
            lo, hi = r * per, min(n, (r + 1) * per)
            res.append(oracle.query_index(oracle.fit_index(sig[lo:hi], L, k), qsig))
            bases.append(lo)
        got = oracle.merge_shard_candidates(res, bases)
        for x, y in zip(got, want):
            assert np.array_equal(x, y)
