"""MinHash LSH (Jaccard) over CSR rows.  Same public behaviour as
python/culsh/minhash_lsh.py:14-311."""
from __future__ import annotations

from typing import Optional

import numpy as np
import scipy.sparse

from ._culsh_core import Candidates, MinHashCore, MinHashIndex
from .utils import get_array_info, resolve_seed


def _csr_arrays(X):
    """(indices, indptr) of a SciPy / cupyx CSR matrix as int32; values are ignored.  Index
    arrays that are not int32 are rejected like upstream's ensure_int32_indices
    (minhash_lsh.py:300-311)."""
    if scipy.sparse.issparse(X):
        if not scipy.sparse.isspmatrix_csr(X):
            X = scipy.sparse.csr_matrix(X)
    elif not type(X).__module__.startswith("cupyx.scipy.sparse"):
        raise TypeError("MinHashLSH expects a scipy.sparse or cupyx.scipy.sparse CSR matrix")
    indices, indptr = X.indices, X.indptr
    if indices.dtype != np.int32 or indptr.dtype != np.int32:
        raise ValueError(
            f"CSR indices/indptr must be int32, got {indices.dtype}/{indptr.dtype} "
            "(the matrix is too large for 32-bit indexing)")
    return indices, indptr


class MinHashLSH:
    """``n_hash_tables`` tables of ``n_hashes`` min-wise hashes (universal hashing of column
    ids modulo the prime 4294967291)."""

    def __init__(self, n_hash_tables: int, n_hashes: int, seed: Optional[int] = None):
        if n_hash_tables <= 0:
            raise ValueError("n_hash_tables must be positive")
        if n_hashes <= 0:
            raise ValueError("n_hashes must be positive")
        self._n_hash_tables = n_hash_tables
        self._n_hashes = n_hashes
        self._seed = resolve_seed(seed)

    n_hash_tables = property(lambda self: self._n_hash_tables)
    n_hashes = property(lambda self: self._n_hashes)
    seed = property(lambda self: self._seed)

    def fit(self, X) -> "MinHashLSHModel":
        n, d, _ = get_array_info(X)
        indices, indptr = _csr_arrays(X)
        core = MinHashCore(self._n_hash_tables, self._n_hashes, self._seed)
        index = core.fit(indices, indptr, n, d)
        return MinHashLSHModel(self._n_hash_tables, self._n_hashes, d, core, index)

    def fit_query(self, X) -> Candidates:
        n, d, _ = get_array_info(X)
        indices, indptr = _csr_arrays(X)
        core = MinHashCore(self._n_hash_tables, self._n_hashes, self._seed)
        return core.fit_query(indices, indptr, n, d)


class MinHashLSHModel:
    def __init__(self, n_hash_tables: int, n_hashes: int, n_features: int, core: MinHashCore,
                 index: MinHashIndex):
        self._n_hash_tables = n_hash_tables
        self._n_hashes = n_hashes
        self._n_features = n_features
        self._core = core
        self._index = index

    n_hash_tables = property(lambda self: self._n_hash_tables)
    n_hashes = property(lambda self: self._n_hashes)
    n_features = property(lambda self: self._n_features)
    index = property(lambda self: self._index)

    def query(self, Q) -> Candidates:
        n_q, d, _ = get_array_info(Q)
        if d != self._n_features:
            raise ValueError(f"Query features ({d}) != fitted features ({self._n_features})")
        indices, indptr = _csr_arrays(Q)
        return self._core.query(indices, indptr, n_q, self._index)

    def save(self, path: str) -> None:
        """npz with upstream's keys and array layout (minhash_lsh.py:240-255)."""
        ix = self._index
        np.savez_compressed(
            path,
            n_hash_tables=self._n_hash_tables, n_hashes=self._n_hashes, n_features=self._n_features,
            n_total_candidates=ix.n_total_candidates, n_total_buckets=ix.n_total_buckets,
            seed=ix.seed, sig_nbytes=ix.sig_nbytes,
            candidate_indices=ix.get_candidate_indices(),
            bucket_signatures=ix.get_bucket_signatures(),
            bucket_candidate_offsets=ix.get_bucket_candidate_offsets(),
            table_bucket_offsets=ix.get_table_bucket_offsets(),
            hash_a=ix.get_hash_a(), hash_b=ix.get_hash_b(),
        )

    @classmethod
    def load(cls, path: str) -> "MinHashLSHModel":
        data = np.load(path)
        core = MinHashCore(int(data["n_hash_tables"]), int(data["n_hashes"]), int(data["seed"]))
        index = MinHashIndex.load(
            candidate_indices=data["candidate_indices"], bucket_signatures=data["bucket_signatures"],
            bucket_candidate_offsets=data["bucket_candidate_offsets"],
            table_bucket_offsets=data["table_bucket_offsets"],
            hash_a=data["hash_a"], hash_b=data["hash_b"],
            n_total_candidates=int(data["n_total_candidates"]),
            n_total_buckets=int(data["n_total_buckets"]), n_hash_tables=int(data["n_hash_tables"]),
            n_hashes=int(data["n_hashes"]), sig_nbytes=int(data["sig_nbytes"]),
            n_features=int(data["n_features"]), seed=int(data["seed"]))
        return cls(int(data["n_hash_tables"]), int(data["n_hashes"]), int(data["n_features"]), core, index)
