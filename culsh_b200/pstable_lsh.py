"""p-stable LSH (Euclidean).  Same public behaviour as python/culsh/pstable_lsh.py:14-396."""
from __future__ import annotations

from typing import Literal, Optional, Union

import numpy as np

from ._culsh_core import Candidates, PSLSHCore, PSLSHIndex
from .utils import ensure_engine_array, get_array_info, get_logger, is_device_array, resolve_seed


class PStableLSH:
    """h(x) = floor((x.p + b) / w) with Gaussian p: ``n_hash_tables`` tables of ``n_hashes``
    such values.  ``window_size`` is an integer bucket width, or "auto" to take
    max(1, int(mean row norm)) of (a sample of) the data at fit time."""

    def __init__(self, n_hash_tables: int, n_hashes: int,
                 window_size: Union[int, Literal["auto"]] = "auto", seed: Optional[int] = None):
        if n_hash_tables <= 0:
            raise ValueError("n_hash_tables must be positive")
        if n_hashes <= 0:
            raise ValueError("n_hashes must be positive")
        if window_size != "auto" and window_size <= 0:
            raise ValueError("window_size must be positive")
        self._n_hash_tables = n_hash_tables
        self._n_hashes = n_hashes
        self._window_size = window_size
        self._seed = resolve_seed(seed)
        self._logger = get_logger(self)

    n_hash_tables = property(lambda self: self._n_hash_tables)
    n_hashes = property(lambda self: self._n_hashes)
    window_size = property(lambda self: self._window_size)
    seed = property(lambda self: self._seed)

    def _resolve_window(self, X) -> int:
        if self._window_size != "auto":
            return int(self._window_size)
        w = self._estimate_window_size(X)
        self._logger.info(f"Using estimated window size: {w}")
        return w

    def fit(self, X) -> "PStableLSHModel":
        n, d, dtype = get_array_info(X)
        X = ensure_engine_array(X)
        w = self._resolve_window(X)
        core = PSLSHCore(self._n_hash_tables, self._n_hashes, w, self._seed)
        if dtype == np.float32:
            index = core.fit_float(X, n, d)
        elif dtype == np.float64:
            index = core.fit_double(X, n, d)
        else:
            raise TypeError(f"Unsupported dtype: {dtype}. Supported dtypes are float32, float64.")
        return PStableLSHModel(self._n_hash_tables, self._n_hashes, w, d, core, index)

    def fit_query(self, X, batch_size: Optional[int] = None) -> Candidates:
        if batch_size is not None:  # pstable_lsh.py:167-169
            return self.fit(X).query(X, batch_size=batch_size)
        n, d, dtype = get_array_info(X)
        X = ensure_engine_array(X)
        w = self._resolve_window(X)
        core = PSLSHCore(self._n_hash_tables, self._n_hashes, w, self._seed)
        if dtype == np.float32:
            return core.fit_query_float(X, n, d)
        if dtype == np.float64:
            return core.fit_query_double(X, n, d)
        raise TypeError(f"Unsupported dtype: {dtype}. Supported dtypes are float32, float64.")

    @staticmethod
    def _estimate_window_size(X, scale_factor: float = 1.0, max_samples: int = 10000) -> int:
        """Mean L2 norm of up to ``max_samples`` rows (an unseeded sample without replacement
        when there are more), divided by ``scale_factor``, truncated, at least 1
        (pstable_lsh.py:191-223)."""
        n = len(X)
        if is_device_array(X):
            if type(X).__module__.startswith("torch"):
                import torch
                xs = X[torch.randperm(n, device=X.device)[:max_samples]] if n > max_samples else X
                mean = float(torch.linalg.norm(xs.double(), dim=1).mean())
            else:
                import cupy as cp
                xs = X[cp.random.choice(n, max_samples, replace=False)] if n > max_samples else X
                mean = float(cp.linalg.norm(xs, axis=1).mean())
        else:
            xs = X[np.random.choice(n, max_samples, replace=False)] if n > max_samples else X
            mean = float(np.linalg.norm(xs, axis=1).mean())
        return max(1, int(mean / scale_factor))


class PStableLSHModel:
    def __init__(self, n_hash_tables: int, n_hashes: int, window_size: int, n_features: int,
                 core: PSLSHCore, index: PSLSHIndex):
        self._n_hash_tables = n_hash_tables
        self._n_hashes = n_hashes
        self._window_size = window_size
        self._n_features = n_features
        self._core = core
        self._index = index

    n_hash_tables = property(lambda self: self._n_hash_tables)
    n_hashes = property(lambda self: self._n_hashes)
    window_size = property(lambda self: self._window_size)
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
        """npz with upstream's keys and array layout (pstable_lsh.py:330-347)."""
        ix = self._index
        np.savez_compressed(
            path,
            n_hash_tables=self._n_hash_tables, n_hashes=self._n_hashes,
            window_size=self._window_size, n_features=self._n_features,
            n_total_candidates=ix.n_total_candidates, n_total_buckets=ix.n_total_buckets,
            seed=ix.seed, sig_nbytes=ix.sig_nbytes, is_double=ix.is_double,
            candidate_indices=ix.get_candidate_indices(),
            bucket_signatures=ix.get_bucket_signatures(),
            bucket_candidate_offsets=ix.get_bucket_candidate_offsets(),
            table_bucket_offsets=ix.get_table_bucket_offsets(),
            projection=ix.get_projection_matrix(), bias=ix.get_bias(),
        )

    @classmethod
    def load(cls, path: str) -> "PStableLSHModel":
        data = np.load(path)
        w = int(data["window_size"])
        core = PSLSHCore(int(data["n_hash_tables"]), int(data["n_hashes"]), w, int(data["seed"]))
        kwargs = dict(
            candidate_indices=data["candidate_indices"], bucket_signatures=data["bucket_signatures"],
            bucket_candidate_offsets=data["bucket_candidate_offsets"],
            table_bucket_offsets=data["table_bucket_offsets"], projection=data["projection"],
            bias=data["bias"], n_total_candidates=int(data["n_total_candidates"]),
            n_total_buckets=int(data["n_total_buckets"]), n_hash_tables=int(data["n_hash_tables"]),
            n_hashes=int(data["n_hashes"]), sig_nbytes=int(data["sig_nbytes"]),
            n_features=int(data["n_features"]), seed=int(data["seed"]), window_size=w)
        index = PSLSHIndex.load_double(**kwargs) if data["is_double"] else PSLSHIndex.load_float(**kwargs)
        return cls(int(data["n_hash_tables"]), int(data["n_hashes"]), w, int(data["n_features"]), core, index)
