"""Generate golden fixtures from upstream cuLSH's own pure-Python oracle.

Run in a checkout that has the upstream project next to it:

    python tests/golden/make_ref_lsh_fixtures.py /path/to/cuLSH

It imports ``python/tests/ref_lsh.py`` from the upstream tree UNCHANGED, subclasses its
three LSH classes only to inject explicit hash parameters (upstream draws them from
NumPy's global RNG, the CUDA code from cuRAND, so parameters have to be shared to compare
anything bit-for-bit), runs fit + query, and stores inputs, parameters and results as
small ``ref_lsh_<family>.npz`` files beside this script.

Stored per family:
  X / Q (dense) or X_indices, X_indptr, Q_indices, Q_indptr (CSR), n_features
  hash parameters (P | P_scaled, b, window | A, B), L, k
  sig_X, sig_Q            signatures produced by upstream's _hash ([n, L*k])
  cand_indices/offsets    upstream's query result as a CSR with every list sorted
  bucket_rows_t<j>/bucket_ptr_t<j>/bucket_sigs_t<j>  upstream's index of table j, buckets
                          in lexicographic order of the signature tuple (element-wise)
"""
import os
import sys

import numpy as np
import scipy.sparse as sp

if len(sys.argv) > 1:
    REF = sys.argv[1]
elif os.environ.get("CULSH_REFERENCE"):
    REF = os.environ["CULSH_REFERENCE"]
else:
    raise SystemExit("usage: make_ref_lsh_fixtures.py /path/to/cuLSH   (or set CULSH_REFERENCE)")
sys.path.insert(0, os.path.join(REF, "python", "tests"))
import ref_lsh  # noqa: E402  (upstream module, imported as-is)

OUT = os.path.dirname(os.path.abspath(__file__))


def _inject(cls, params):
    class Injected(cls):
        def _generate_hash_params(self, n_features, dtype):
            return params
    return Injected


def _csr_from_lists(lists):
    counts = np.array([len(c) for c in lists], dtype=np.uint64)
    offsets = np.zeros(len(lists) + 1, dtype=np.uint64)
    np.cumsum(counts, out=offsets[1:])
    flat = [np.sort(np.asarray(c, dtype=np.int32)) for c in lists if len(c)]
    idx = np.concatenate(flat) if flat else np.zeros(0, np.int32)
    return idx, offsets


def _dump_index(model, out):
    for j, table in enumerate(model.index):
        keys = sorted(table.keys())
        rows = [np.asarray(table[key], dtype=np.int32) for key in keys]
        ptr = np.zeros(len(keys) + 1, dtype=np.int64)
        np.cumsum([len(r) for r in rows], out=ptr[1:])
        out[f"bucket_rows_t{j}"] = np.concatenate(rows) if rows else np.zeros(0, np.int32)
        out[f"bucket_ptr_t{j}"] = ptr
        out[f"bucket_sigs_t{j}"] = np.asarray(keys, dtype=np.int64).reshape(len(keys), -1)


def make_rplsh():
    rng = np.random.RandomState(1234)
    n, nq, d, L, k = 400, 60, 24, 6, 5
    X = rng.randn(n, d).astype(np.float32)
    Q = np.concatenate([X[:20] + 0.05 * rng.randn(20, d).astype(np.float32),
                        rng.randn(nq - 20, d).astype(np.float32)])
    P = rng.randn(L * k, d).astype(np.float32)
    lsh = _inject(ref_lsh.RandomProjectionLSH, P)(L, k, seed=0)
    model = lsh.fit(X)
    cand = model.query(Q)
    out = dict(X=X, Q=Q, P=P, L=L, k=k,
               sig_X=lsh._hash(X, P).astype(np.uint8), sig_Q=lsh._hash(Q, P).astype(np.uint8))
    out["cand_indices"], out["cand_offsets"] = _csr_from_lists(cand)
    _dump_index(model, out)
    np.savez_compressed(os.path.join(OUT, "ref_lsh_rplsh.npz"), **out)


def make_pslsh():
    rng = np.random.RandomState(4321)
    n, nq, d, L, k, w = 500, 50, 16, 5, 3, 4
    X = rng.randn(n, d).astype(np.float32)
    Q = np.concatenate([X[:25] + 0.02 * rng.randn(25, d).astype(np.float32),
                        rng.randn(nq - 25, d).astype(np.float32)])
    P = rng.randn(L * k, d).astype(np.float32)
    b = rng.uniform(0, w, size=L * k).astype(np.float32)
    params = (P, b, np.array(w, dtype=np.float32))
    lsh = _inject(ref_lsh.PStableLSH, params)(L, k, window_size=w, seed=0)
    model = lsh.fit(X)
    cand = model.query(Q)
    out = dict(X=X, Q=Q, P=P, b=b, window=w, L=L, k=k,
               sig_X=lsh._hash(X, params), sig_Q=lsh._hash(Q, params))
    out["cand_indices"], out["cand_offsets"] = _csr_from_lists(cand)
    _dump_index(model, out)
    np.savez_compressed(os.path.join(OUT, "ref_lsh_pslsh.npz"), **out)


def make_minhash():
    rng = np.random.RandomState(99)
    n, nq, d, L, k = 300, 40, 500, 8, 2
    X = sp.random(n, d, density=0.04, format="csr", dtype=np.float32, random_state=rng)
    X.data[:] = 1.0
    X = sp.csr_matrix(X)
    # a few empty rows and duplicates exercise the sentinel and multi-member buckets
    lil = X.tolil()
    lil[5, :] = 0
    lil[17, :] = 0
    lil[30, :] = lil[31, :]
    X = sp.csr_matrix(lil)
    X.sort_indices()
    Q = sp.vstack([X[:20], sp.random(nq - 20, d, density=0.04, format="csr", dtype=np.float32,
                                     random_state=rng)]).tocsr()
    Q.data[:] = 1.0
    Q.sort_indices()
    A = rng.randint(1, ref_lsh.MINHASH_PRIME, size=L * k, dtype=np.uint64)
    B = rng.randint(0, ref_lsh.MINHASH_PRIME, size=L * k, dtype=np.uint64)
    lsh = _inject(ref_lsh.MinHashLSH, (A, B))(L, k, seed=0)
    model = lsh.fit(X)
    cand = model.query(Q)
    out = dict(X_indices=X.indices.astype(np.int32), X_indptr=X.indptr.astype(np.int32),
               Q_indices=Q.indices.astype(np.int32), Q_indptr=Q.indptr.astype(np.int32),
               n_features=d, A=A.astype(np.uint32), B=B.astype(np.uint32), L=L, k=k,
               sig_X=lsh._hash(X, (A, B)), sig_Q=lsh._hash(Q, (A, B)))
    out["cand_indices"], out["cand_offsets"] = _csr_from_lists(cand)
    _dump_index(model, out)
    np.savez_compressed(os.path.join(OUT, "ref_lsh_minhash.npz"), **out)


if __name__ == "__main__":
    make_rplsh()
    make_pslsh()
    make_minhash()
    print("wrote fixtures to", OUT)
