"""Random-projection LSH (cosine).  Same public behaviour as python/culsh/rp_lsh.py:14-320."""
from __future__ import annotations

from typing import Optional

import numpy as np

from ._culsh_core import Candidates, RPLSHCore, RPLSHIndex
from .utils import ensure_engine_array, get_array_info, resolve_seed


def _check_counts(n_hash_tables, n_hashes):
    if n_hash_tables <= 0:
        raise ValueError("n_hash_tables must be positive")
    if n_hashes <= 0:
        raise ValueError("n_hashes must be positive")


class RPLSH:
    """Sign-of-random-projection hashing: ``n_hash_tables`` tables (OR-amplification) of
    ``n_hashes`` sign bits each (AND-amplification).  ``seed=None`` draws a random seed."""

    def __init__(self, n_hash_tables: int, n_hashes: int, seed: Optional[int] = None):
        _check_counts(n_hash_tables, n_hashes)
        self._n_hash_tables = n_hash_tables
        self._n_hashes = n_hashes
        self._seed = resolve_seed(seed)

    n_hash_tables = property(lambda self: self._n_hash_tables)
    n_hashes = property(lambda self: self._n_hashes)
    seed = property(lambda self: self._seed)

    def _core(self):
        return RPLSHCore(self._n_hash_tables, self._n_hashes, self._seed)

    def fit(self, X) -> "RPLSHModel":
        """Build the index over the rows of X (NumPy, CuPy or torch; float32 or float64)."""
        n, d, dtype = get_array_info(X)
        X = ensure_engine_array(X)
        core = self._core()
        if dtype == np.float32:
            index = core.fit_float(X, n, d)
        elif dtype == np.float64:
            index = core.fit_double(X, n, d)
        else:
            raise TypeError(f"Unsupported dtype: {dtype}. Supported dtypes are float32, float64.")
        return RPLSHModel(self._n_hash_tables, self._n_hashes, d, core, index)

    def fit_query(self, X, batch_size: Optional[int] = None) -> Candidates:
        """Index X and query it with its own rows (every row is its own candidate).  With
        ``batch_size`` this is fit(X) followed by a batched query(X), as upstream
        (rp_lsh.py:145-147)."""
        if batch_size is not None:
            return self.fit(X).query(X, batch_size=batch_size)
        n, d, dtype = get_array_info(X)
        X = ensure_engine_array(X)
        core = self._core()
        if dtype == np.float32:
            return core.fit_query_float(X, n, d)
        if dtype == np.float64:
            return core.fit_query_double(X, n, d)
        raise TypeError(f"Unsupported dtype: {dtype}. Supported dtypes are float32, float64.")


class RPLSHModel:
    """Fitted RPLSH index plus the core that queries it."""

    def __init__(self, n_hash_tables: int, n_hashes: int, n_features: int, core: RPLSHCore,
                 index: RPLSHIndex):
        self._n_hash_tables = n_hash_tables
        self._n_hashes = n_hashes
        self._n_features = n_features
        self._core = core
        self._index = index

    n_hash_tables = property(lambda self: self._n_hash_tables)
    n_hashes = property(lambda self: self._n_hashes)
    n_features = property(lambda self: self._n_features)
    index = property(lambda self: self._index)

    def query(self, Q, batch_size: Optional[int] = None) -> Candidates:
        n_q, d, dtype = get_array_info(Q)
        Q = ensure_engine_array(Q)
        if d != self._n_features:
            raise ValueError(f"Query features ({d}) != fitted features ({self._n_features})")
        if dtype == np.float32:
            return self._core.query_float(Q, n_q, self._index, batch_size)
        if dtype == np.float64:
            return self._core.query_double(Q, n_q, self._index, batch_size)
        raise TypeError(f"Unsupported dtype: {dtype}. Use float32 or float64.")

    def save(self, path: str) -> None:
        """npz with upstream's keys and array layout (rp_lsh.py:259-274), so files written by
        either implementation load in the other."""
        ix = self._index
        np.savez_compressed(
            path,
            n_hash_tables=self._n_hash_tables, n_hashes=self._n_hashes, n_features=self._n_features,
            n_total_candidates=ix.n_total_candidates, n_total_buckets=ix.n_total_buckets,
            seed=ix.seed, sig_nbytes=ix.sig_nbytes, is_double=ix.is_double,
            candidate_indices=ix.get_candidate_indices(),
            bucket_signatures=ix.get_bucket_signatures(),
            bucket_candidate_offsets=ix.get_bucket_candidate_offsets(),
            table_bucket_offsets=ix.get_table_bucket_offsets(),
            projection=ix.get_projection_matrix(),
        )

    @classmethod
    def load(cls, path: str) -> "RPLSHModel":
        data = np.load(path)
        core = RPLSHCore(int(data["n_hash_tables"]), int(data["n_hashes"]), int(data["seed"]))
        kwargs = dict(
            candidate_indices=data["candidate_indices"], bucket_signatures=data["bucket_signatures"],
            bucket_candidate_offsets=data["bucket_candidate_offsets"],
            table_bucket_offsets=data["table_bucket_offsets"], projection=data["projection"],
            n_total_candidates=int(data["n_total_candidates"]),
            n_total_buckets=int(data["n_total_buckets"]), n_hash_tables=int(data["n_hash_tables"]),
            n_hashes=int(data["n_hashes"]), sig_nbytes=int(data["sig_nbytes"]),
            n_features=int(data["n_features"]), seed=int(data["seed"]))
        index = RPLSHIndex.load_double(**kwargs) if data["is_double"] else RPLSHIndex.load_float(**kwargs)
        return cls(int(data["n_hash_tables"]), int(data["n_hashes"]), int(data["n_features"]), core, index)
