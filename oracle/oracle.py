"""CPU restatement of cuLSH's hash -> bucket index -> lookup -> gather/dedupe -> CSR path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module; it is
the checker used by the tests, by the smoke check and by the benchmark's CPU-baseline
leg.  Every function cites the upstream cuLSH file:line whose behaviour it restates
(paths are relative to the upstream project root).

Parity status: the upstream test-suite holds no golden vectors for this path (its
tests compare recall statistics and three self-consistency identities), so this
restatement is pinned in two ways instead:
  * against upstream's own pure-Python oracle ``python/tests/ref_lsh.py`` run with
    injected hash parameters (fixtures under ``tests/golden/ref_lsh_*.npz``, made by
    ``tests/golden/make_ref_lsh_fixtures.py``);
  * against arrays captured from upstream's CUDA build on a B200
    (``tests/golden/ref_cuda_*.npz``, made by ``tests/golden/capture_ref_cuda.py``).

All index arrays use upstream's canonical layout:
  candidate_indices         int32 [n*L]   row ids grouped by (table, bucket), ascending in a bucket
  bucket_signatures         uint8 [B*s]   raw signature bytes of each bucket, s = k*sizeof(elem)
  bucket_candidate_offsets  int32 [B+1]
  table_bucket_offsets      int32 [L+1]
Buckets of one table are ordered by unsigned byte-lexicographic order of the raw
signature memory (core/fit.cuh:265-282, core/query.cuh:44-48).
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np

MINHASH_PRIME = 4294967291  # minhash/hash.cuh:17


# --------------------------------------------------------------------------------------
# Hash stages
# --------------------------------------------------------------------------------------
def rplsh_projection(X: np.ndarray, P: np.ndarray) -> np.ndarray:
    """X_hash = X . P^T in float64 (the exact value the fp32 GEMM approximates).

    rplsh/hash.cuh:107-120 (cublasSgemm, OP_T/OP_N, row-major result [n][H]).
    """
    return np.asarray(X, dtype=np.float64) @ np.asarray(P, dtype=np.float64).T


def rplsh_signatures(X: np.ndarray, P: np.ndarray) -> np.ndarray:
    """uint8 [n, H]: 1 where the fp32 projection's sign bit is clear.

    rplsh/hash.cuh:24-48: ``(float_as_uint(x) >> 31) ^ 1`` - so +0.0 -> 1, -0.0 -> 0,
    and a float64 projection is narrowed to float32 before the test.
    """
    v = rplsh_projection(X, P).astype(np.float32)
    return (~np.signbit(v)).astype(np.uint8)


def rplsh_near_boundary(X: np.ndarray, P: np.ndarray, rel: float = 1e-5) -> np.ndarray:
    """bool [n, H]: bits whose projection lies within ``rel`` (relative to sum |x_i p_i|)
    of the sign boundary; an fp32 GEMM with a different summation order may flip them."""
    X64 = np.asarray(X, dtype=np.float64)
    P64 = np.asarray(P, dtype=np.float64)
    v = X64 @ P64.T
    scale = np.abs(X64) @ np.abs(P64).T
    return np.abs(v) <= rel * scale


def pslsh_signatures(X: np.ndarray, P_scaled: np.ndarray, b: np.ndarray) -> np.ndarray:
    """int32 [n, H] = floor(fp(X . P_scaled^T) + b), add and floor in the input precision.

    pslsh/hash.cuh:26-47 (bias_floor_reorder_kernel) and :105-142; ``P_scaled`` is the
    projection already divided by the integer window (pslsh/hash.cuh:84-86) and ``b``
    is uniform in (0, 1].
    """
    dt = np.float64 if np.asarray(X).dtype == np.float64 else np.float32
    v = (np.asarray(X, dtype=np.float64) @ np.asarray(P_scaled, dtype=np.float64).T).astype(dt)
    return np.floor(v + np.asarray(b, dtype=dt)[None, :]).astype(np.int32)


def pslsh_near_boundary(X, P_scaled, b, rel: float = 1e-5) -> np.ndarray:
    """bool [n, H]: elements whose pre-floor value is within ``rel * max(1, sum|x p| + |b|)``
    of an integer."""
    X64 = np.asarray(X, dtype=np.float64)
    P64 = np.asarray(P_scaled, dtype=np.float64)
    b64 = np.asarray(b, dtype=np.float64)
    v = X64 @ P64.T + b64[None, :]
    scale = np.maximum(1.0, np.abs(X64) @ np.abs(P64).T + np.abs(b64)[None, :])
    return np.abs(v - np.rint(v)) <= rel * scale


def minhash_normalize(A_raw: np.ndarray, B_raw: np.ndarray):
    """A <- A mod (p-1) + 1, B <- B mod p.  minhash/hash.cuh:26-32."""
    A = (np.asarray(A_raw, dtype=np.uint64) % np.uint64(MINHASH_PRIME - 1)) + np.uint64(1)
    B = np.asarray(B_raw, dtype=np.uint64) % np.uint64(MINHASH_PRIME)
    return A.astype(np.uint32), B.astype(np.uint32)


def minhash_signatures(indices: np.ndarray, indptr: np.ndarray, A: np.ndarray, B: np.ndarray,
                       chunk_nnz: int = 1 << 18) -> np.ndarray:
    """uint32 [n, H] = min over the row's column ids c of (A[h]*c + B[h]) mod p; an empty
    row gives 0xFFFFFFFF.  minhash/hash.cuh:69-128 (64-bit multiply-add, % prime, min)."""
    indices = np.asarray(indices)
    indptr = np.asarray(indptr).astype(np.int64)
    n = len(indptr) - 1
    A64 = np.asarray(A, dtype=np.uint64)[None, :]
    B64 = np.asarray(B, dtype=np.uint64)[None, :]
    H = A64.shape[1]
    out = np.full((n, H), 0xFFFFFFFF, dtype=np.uint32)
    row = 0
    while row < n:
        # take a run of rows holding about chunk_nnz entries
        end = int(np.searchsorted(indptr, indptr[row] + chunk_nnz, side="right")) - 1
        end = min(max(end, row + 1), n)
        lo, hi = indptr[row], indptr[end]
        if hi > lo:
            cols = indices[lo:hi].astype(np.uint32).astype(np.uint64)[:, None]
            hv = ((A64 * cols + B64) % np.uint64(MINHASH_PRIME)).astype(np.uint32)
            starts = (indptr[row:end] - lo)
            nonempty = indptr[row + 1:end + 1] > indptr[row:end]
            if nonempty.any():
                red = np.minimum.reduceat(hv, starts[nonempty], axis=0)
                out[row:end][nonempty] = red
        row = end
    return out


# --------------------------------------------------------------------------------------
# Index build
# --------------------------------------------------------------------------------------
@dataclass
class OracleIndex:
    candidate_indices: np.ndarray
    bucket_signatures: np.ndarray
    bucket_candidate_offsets: np.ndarray
    table_bucket_offsets: np.ndarray
    n_hash_tables: int
    n_hashes: int
    sig_nbytes: int
    n_samples: int

    @property
    def n_total_buckets(self) -> int:
        return int(self.table_bucket_offsets[-1])


def table_signature_bytes(sig: np.ndarray, L: int, k: int) -> np.ndarray:
    """[n, H] elements (uint8 / int32 / uint32) -> uint8 [L, n, s] raw little-endian bytes,
    the table-major X_sig layout of core/fit.cuh:222-226."""
    sig = np.ascontiguousarray(sig)
    n = sig.shape[0]
    raw = sig.reshape(n, L, k).transpose(1, 0, 2)
    raw = np.ascontiguousarray(raw)
    return raw.view(np.uint8).reshape(L, n, k * sig.dtype.itemsize)


def _unique_rows_lex(rows: np.ndarray):
    """Unique rows of a uint8 matrix in unsigned lexicographic order + inverse map."""
    if rows.shape[0] == 0:
        return rows, np.zeros(0, dtype=np.int64)
    s = rows.shape[1]
    # big-endian packing into uint64 words keeps lexicographic order under tuple compare
    pad = (-s) % 8
    padded = np.pad(rows, ((0, 0), (0, pad))) if pad else rows
    words = np.ascontiguousarray(padded).view(">u8").astype(np.uint64)  # [n, W]
    order = np.lexsort(words.T[::-1])  # last key is primary -> reverse; lexsort is stable
    sw = words[order]
    new = np.ones(len(order), dtype=bool)
    new[1:] = np.any(sw[1:] != sw[:-1], axis=1)
    bucket_of_sorted = np.cumsum(new) - 1
    inverse = np.empty(len(order), dtype=np.int64)
    inverse[order] = bucket_of_sorted
    uniq = rows[order[new]]
    return uniq, inverse


def fit_index(sig: np.ndarray, L: int, k: int) -> OracleIndex:
    """core/fit.cuh:222-374: order all (table,row) items by table, then signature bytes
    (lexicographic, unsigned), then row id; mark bucket boundaries; emit the flat index."""
    raw = table_signature_bytes(sig, L, k)
    n = raw.shape[1]
    s = raw.shape[2]
    cand, sigs, offs, tbo = [], [], [], [0]
    base = 0
    for t in range(L):
        uniq, inv = _unique_rows_lex(raw[t])
        order = np.argsort(inv, kind="stable")  # row ids ascending inside a bucket
        counts = np.bincount(inv, minlength=len(uniq))
        starts = np.concatenate([[0], np.cumsum(counts)[:-1]]) if len(uniq) else np.zeros(0, int)
        cand.append(order.astype(np.int32))
        sigs.append(uniq.reshape(-1))
        offs.append((starts + base).astype(np.int32))
        base += n
        tbo.append(tbo[-1] + len(uniq))
    offs.append(np.array([n * L], dtype=np.int32))
    return OracleIndex(
        candidate_indices=np.concatenate(cand) if cand else np.zeros(0, np.int32),
        bucket_signatures=np.concatenate(sigs).astype(np.uint8) if sigs else np.zeros(0, np.uint8),
        bucket_candidate_offsets=np.concatenate(offs),
        table_bucket_offsets=np.asarray(tbo, dtype=np.int32),
        n_hash_tables=L, n_hashes=k, sig_nbytes=s, n_samples=n)


# --------------------------------------------------------------------------------------
# Query
# --------------------------------------------------------------------------------------
def find_matching_buckets(index: OracleIndex, qsig: np.ndarray) -> np.ndarray:
    """int32 [n_q, L]: bucket id holding the query's signature in each table, -1 if none.
    core/query.cuh:31-101 (binary search with unsigned byte-lexicographic compare)."""
    L, k, s = index.n_hash_tables, index.n_hashes, index.sig_nbytes
    qraw = table_signature_bytes(qsig, L, k)
    nq = qraw.shape[1]
    out = np.full((nq, L), -1, dtype=np.int32)
    bsig = index.bucket_signatures.reshape(-1, s)
    for t in range(L):
        b0, b1 = int(index.table_bucket_offsets[t]), int(index.table_bucket_offsets[t + 1])
        tb = bsig[b0:b1]
        stacked = np.concatenate([tb, qraw[t]], axis=0)
        _, inv = _unique_rows_lex(stacked)
        nb = b1 - b0
        owner = np.full(int(inv.max()) + 1 if len(inv) else 0, -1, dtype=np.int64)
        owner[inv[:nb]] = np.arange(nb) + b0
        out[:, t] = owner[inv[nb:]]
    return out


def query_from_matched_buckets(index: OracleIndex, matched: np.ndarray):
    """core/query.cuh:290-478: gather the matched buckets' members, per-query sort + unique.
    Returns (indices int32, offsets uint64 [n_q+1], counts uint64 [n_q])."""
    nq = matched.shape[0]
    bco = index.bucket_candidate_offsets.astype(np.int64)
    cand = index.candidate_indices
    pieces, counts = [], np.zeros(nq, dtype=np.uint64)
    for q in range(nq):
        m = matched[q]
        m = m[m >= 0]
        if len(m) == 0:
            continue
        rows = np.concatenate([cand[bco[b]:bco[b + 1]] for b in m])
        u = np.unique(rows)
        pieces.append(u.astype(np.int32))
        counts[q] = len(u)
    offsets = np.zeros(nq + 1, dtype=np.uint64)
    np.cumsum(counts, out=offsets[1:])
    indices = np.concatenate(pieces) if pieces else np.zeros(0, dtype=np.int32)
    return indices, offsets, counts


def query_index(index: OracleIndex, qsig: np.ndarray):
    """core/query.cuh:490-522."""
    return query_from_matched_buckets(index, find_matching_buckets(index, qsig))


def fit_query(sig: np.ndarray, L: int, k: int):
    """core/fit_query.cuh:30-55: every row queries the index built from the same rows."""
    index = fit_index(sig, L, k)
    return query_index(index, sig)


def merge_shard_candidates(shard_results, row_offsets):
    """Union of per-shard CSR results: shard r's local ids are shifted by row_offsets[r] and
    the per-query lists are concatenated in rank order (id ranges are disjoint and
    increasing, so the result is sorted and duplicate-free).  No upstream counterpart:
    upstream is single-GPU; the identity follows from core/fit.cuh:160-208."""
    nq = len(shard_results[0][2])
    counts = np.zeros(nq, dtype=np.uint64)
    for _, _, c in shard_results:
        counts += c
    offsets = np.zeros(nq + 1, dtype=np.uint64)
    np.cumsum(counts, out=offsets[1:])
    out = np.empty(int(offsets[-1]), dtype=np.int32)
    cursor = offsets[:-1].astype(np.int64).copy()
    for (idx, off, cnt), base in zip(shard_results, row_offsets):
        off = off.astype(np.int64)
        for q in range(nq):
            c = int(cnt[q])
            if c:
                out[cursor[q]:cursor[q] + c] = idx[off[q]:off[q] + c] + base
                cursor[q] += c
    return out, offsets, counts


# --------------------------------------------------------------------------------------
# Fast vectorised variant used as the timed CPU baseline (same results, bigger inputs)
# --------------------------------------------------------------------------------------
def pack_bits_msb_first(bits: np.ndarray, L: int, k: int) -> np.ndarray:
    """uint64 [L, n]: RPLSH signature bits packed with hash 0 as the most significant bit;
    numeric order of the packed word equals the byte-lexicographic order of the k raw
    0/1 bytes (k <= 64)."""
    n = bits.shape[0]
    b = bits.reshape(n, L, k).astype(np.uint64)
    w = (np.uint64(1) << np.arange(k - 1, -1, -1, dtype=np.uint64))
    return (b * w[None, None, :]).sum(axis=2).T.copy()


def fast_fit_packed(keys: np.ndarray):
    """keys uint64 [L, n] -> per-table (sorted unique keys, bucket starts, member rows)."""
    tables = []
    for t in range(keys.shape[0]):
        order = np.argsort(keys[t], kind="stable")
        sk = keys[t][order]
        head = np.ones(len(sk), dtype=bool)
        head[1:] = sk[1:] != sk[:-1]
        starts = np.flatnonzero(head)
        tables.append((sk[starts], np.append(starts, len(sk)), order.astype(np.int32)))
    return tables


def fast_query_packed(tables, qkeys: np.ndarray):
    """qkeys uint64 [L, n_q] -> CSR (indices, offsets, counts), sorted unique per query."""
    nq = qkeys.shape[1]
    per_q = [[] for _ in range(nq)]
    for t, (bk, starts, members) in enumerate(tables):
        pos = np.searchsorted(bk, qkeys[t])
        pos_c = np.minimum(pos, len(bk) - 1)
        hit = (pos < len(bk)) & (bk[pos_c] == qkeys[t])
        for q in np.flatnonzero(hit):
            p = pos[q]
            per_q[q].append(members[starts[p]:starts[p + 1]])
    counts = np.zeros(nq, dtype=np.uint64)
    pieces = []
    for q in range(nq):
        if per_q[q]:
            u = np.unique(np.concatenate(per_q[q]))
            pieces.append(u)
            counts[q] = len(u)
    offsets = np.zeros(nq + 1, dtype=np.uint64)
    np.cumsum(counts, out=offsets[1:])
    indices = np.concatenate(pieces).astype(np.int32) if pieces else np.zeros(0, np.int32)
    return indices, offsets, counts


def signature_keys(sig_x: np.ndarray, sig_q: np.ndarray, L: int, k: int):
    """(uint64 [L, n], uint64 [L, n_q]): one word per (table, row) such that two rows of a table
    have equal words exactly when their k signature elements are equal (bucket membership is
    an equality relation, core/fit.cuh:77-84, so any injective relabelling keeps the candidate
    sets).  Signatures of at most 8 bytes are packed directly; wider ones are numbered per
    table over the rows of both inputs."""
    n, nq = sig_x.shape[0], sig_q.shape[0]
    item = sig_x.dtype.itemsize
    both = np.concatenate([sig_x, sig_q.astype(sig_x.dtype, copy=False)], axis=0)
    both = np.ascontiguousarray(both.reshape(n + nq, L, k).transpose(1, 0, 2))  # [L, n+nq, k]
    out = np.empty((L, n + nq), dtype=np.uint64)
    if k * item <= 8:
        raw = both.view(np.uint8).reshape(L, n + nq, k * item)
        padded = np.zeros((L, n + nq, 8), dtype=np.uint8)
        padded[:, :, :k * item] = raw
        out[:] = padded.view(np.uint64).reshape(L, n + nq)
    else:
        rows = both.view(np.dtype((np.void, k * item))).reshape(L, n + nq)
        for t in range(L):
            _, inv = np.unique(rows[t], return_inverse=True)
            out[t] = inv.astype(np.uint64)
    return np.ascontiguousarray(out[:, :n]), np.ascontiguousarray(out[:, n:])
