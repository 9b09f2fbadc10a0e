"""Drop-in for upstream's pybind11 module ``culsh._culsh_core`` on top of the C ABI.

Class and method names, argument meaning and error behaviour follow
python/csrc/bindings.cu:481-588 (stubs: python/culsh/_culsh_core.pyi:22-301):
``RPLSHCore / PSLSHCore / MinHashCore`` (fit / query / fit_query entry points),
``RPLSHIndex / PSLSHIndex / MinHashIndex`` (properties, getters, loaders) and
``Candidates`` (``get_indices / get_counts / get_offsets``).

Array arguments may be NumPy arrays (host memory: the library stages them itself) or any
object exposing ``__cuda_array_interface__`` (CuPy, torch CUDA tensors: the raw device
pointer is borrowed for the duration of the call, as in
python/csrc/common/array_utils.cuh:17-28).
"""
from __future__ import annotations

import ctypes as C
import threading
from typing import Optional

import numpy as np

from . import _lib

RPLSH, PSLSH, MINHASH = 0, 1, 2

_handles = threading.local()


def _current_device() -> int:
    import sys
    torch = sys.modules.get("torch")
    if torch is not None and torch.cuda.is_available() and torch.cuda.is_initialized():
        return int(torch.cuda.current_device())
    cupy = sys.modules.get("cupy")
    if cupy is not None:
        try:
            return int(cupy.cuda.Device().id)
        except Exception:  # pragma: no cover
            pass
    return 0


class _Handle:
    """One engine handle (stream + scratch) per (thread, device); shared by the Core objects."""

    def __init__(self, device: int):
        self.lib = _lib.load()
        self.ptr = C.c_void_p()
        self.device = device
        _lib.check(self.lib.culsh_create(device, C.byref(self.ptr)))

    def __del__(self):
        try:
            if self.ptr:
                self.lib.culsh_destroy(self.ptr)
        except Exception:  # interpreter shutdown
            pass

    def stats(self) -> dict:
        s = _lib.Stats()
        _lib.check(self.lib.culsh_get_stats(self.ptr, C.byref(s)))
        return {name: getattr(s, name) for name, _ in s._fields_}


def get_handle(device: Optional[int] = None) -> _Handle:
    device = _current_device() if device is None else int(device)
    cache = getattr(_handles, "cache", None)
    if cache is None:
        cache = _handles.cache = {}
    h = cache.get(device)
    if h is None:
        h = cache[device] = _Handle(device)
    return h


def _pointer(obj, dtype=None):
    """(address, keepalive) of a host or device array."""
    if obj is None:
        return None, None
    if hasattr(obj, "__cuda_array_interface__"):
        iface = obj.__cuda_array_interface__
        if iface.get("strides") is not None:
            raise ValueError("device array must be C-contiguous")
        return int(iface["data"][0]), obj
    if type(obj).__module__.startswith("torch"):
        if obj.is_cuda:
            if not obj.is_contiguous():
                raise ValueError("device array must be C-contiguous")
            return int(obj.data_ptr()), obj
        obj = obj.detach().numpy()
    arr = np.ascontiguousarray(obj, dtype=dtype)
    return int(arr.ctypes.data), arr


def _is_device_obj(obj) -> bool:
    if hasattr(obj, "__cuda_array_interface__"):
        return True
    return type(obj).__module__.startswith("torch") and bool(getattr(obj, "is_cuda", False))


class _PinnedBlock:
    """A page-locked host block lent to one NumPy result array; it goes back to the pool when
    the last view of that array dies."""

    def __init__(self, pool, ptr, cap):
        self._pool, self.ptr, self.cap = pool, ptr, cap
        self.__array_interface__ = {"shape": (cap,), "typestr": "|u1", "data": (ptr, False), "version": 3}

    def __del__(self):
        try:
            self._pool._release(self.ptr, self.cap)
        except Exception:  # interpreter shutdown
            pass


class _PinnedPool:
    """Recycles page-locked blocks for large result arrays, so that steady-state getters copy
    device -> pinned host memory at full PCIe rate instead of into fresh pageable pages.
    CULSH_PINNED_POOL_MB bounds the bytes kept idle (default 2048, 0 disables pinning)."""
    MIN_BYTES = 1 << 20

    def __init__(self):
        import os
        self.limit = int(os.environ.get("CULSH_PINNED_POOL_MB", "2048")) << 20
        self.free = []  # (cap, ptr)
        self.idle = 0
        self.lock = threading.Lock()

    def acquire(self, nbytes):
        if self.limit <= 0 or nbytes < self.MIN_BYTES:
            return None
        with self.lock:
            best = None
            for i, (cap, ptr) in enumerate(self.free):
                if nbytes <= cap <= 2 * nbytes and (best is None or cap < self.free[best][0]):
                    best = i
            if best is not None:
                cap, ptr = self.free.pop(best)
                self.idle -= cap
                return _PinnedBlock(self, ptr, cap)
        cap = (nbytes + (1 << 20) - 1) >> 20 << 20
        out = C.c_void_p()
        if _lib.load().culsh_host_alloc(cap, C.byref(out)) != 0:
            return None  # fall back to pageable memory
        return _PinnedBlock(self, out.value, cap)

    def _release(self, ptr, cap):
        with self.lock:
            if self.idle + cap <= self.limit:
                self.free.append((cap, ptr))
                self.idle += cap
                return
        _lib.load().culsh_host_free(C.c_void_p(ptr))


_pinned_pool = _PinnedPool()


def _alloc_out(n, dtype, as_cupy=False, as_torch=False, device=0):
    if as_cupy:
        import cupy as cp  # upstream imports cupy lazily too (bindings.cu:272)
        arr = cp.empty(int(n), dtype=dtype)
        return arr, int(arr.data.ptr)
    if as_torch:
        import torch
        tdt = {np.dtype(np.int32): torch.int32, np.dtype(np.uint64): torch.uint64,
               np.dtype(np.uint8): torch.uint8, np.dtype(np.uint32): torch.uint32,
               np.dtype(np.float32): torch.float32, np.dtype(np.float64): torch.float64}[np.dtype(dtype)]
        arr = torch.empty(int(n), dtype=tdt, device=f"cuda:{device}")
        return arr, int(arr.data_ptr())
    nbytes = int(n) * np.dtype(dtype).itemsize
    block = _pinned_pool.acquire(nbytes)
    if block is not None:
        arr = np.asarray(block)[:nbytes].view(dtype)  # arr.base chain keeps the block alive
        return arr, int(block.ptr)
    arr = np.empty(int(n), dtype=dtype)
    return arr, int(arr.ctypes.data)


class Candidates:
    """CSR result of a query: core::Candidates (core/candidates.cuh:14-137) behind the getters of
    bindings.cu:268-338.  ``indices`` are int32 row ids, sorted ascending and unique inside
    each query; ``offsets`` (uint64, n_queries+1) is their exclusive scan; ``counts`` uint64."""

    def __init__(self, ptr: C.c_void_p, handle: _Handle):
        self._ptr = ptr
        self._h = handle
        n = C.c_int32()
        t = C.c_uint64()
        e = C.c_int32()
        _lib.check(handle.lib.culsh_candidates_get_meta(ptr, C.byref(n), C.byref(t), C.byref(e)))
        self._n_queries, self._total, self._empty = int(n.value), int(t.value), bool(e.value)

    def __del__(self):
        try:
            if self._ptr:
                self._h.lib.culsh_candidates_free(self._ptr)
                self._ptr = None
        except Exception:
            pass

    def empty(self) -> bool:
        return self._empty

    @property
    def n_queries(self) -> int:
        return self._n_queries

    @property
    def n_total_candidates(self) -> int:
        return self._total

    def _get(self, fn, n, dtype, as_cupy, as_torch):
        if self._empty:
            n = 0
        arr, addr = _alloc_out(n, dtype, as_cupy, as_torch, self._h.device)
        if n:
            _lib.check(fn(self._ptr, addr))
        return arr

    def get_indices(self, as_cupy: bool = False, as_torch: bool = False):
        return self._get(self._h.lib.culsh_candidates_get_indices, self._total, np.int32, as_cupy, as_torch)

    def get_counts(self, as_cupy: bool = False, as_torch: bool = False):
        return self._get(self._h.lib.culsh_candidates_get_counts, self._n_queries, np.uint64, as_cupy, as_torch)

    def get_offsets(self, as_cupy: bool = False, as_torch: bool = False):
        return self._get(self._h.lib.culsh_candidates_get_offsets, self._n_queries + 1, np.uint64, as_cupy, as_torch)

    def _attach(self, indices_ptr: int, total: int, keepalive=None):
        """Point this result at an id array it does not own (the receive buffer of a shard
        exchange); `keepalive` is held as long as this object lives."""
        _lib.check(self._h.lib.culsh_candidates_attach_indices(self._ptr, indices_ptr or None, int(total)))
        self._total = int(total)
        self._empty = False
        self._keepalive = keepalive

    def device_pointers(self):
        """(indices, counts, offsets) raw device addresses, borrowed from this object."""
        a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
        _lib.check(self._h.lib.culsh_candidates_device_ptrs(self._ptr, C.byref(a), C.byref(b), C.byref(c)))
        return a.value or 0, b.value or 0, c.value or 0


class _IndexBase:
    """Common part of RPLSHIndex / PSLSHIndex / MinHashIndex (bind_core_index_properties,
    bindings.cu:381-404)."""
    _family = -1

    def __init__(self, ptr: C.c_void_p, handle: _Handle):
        self._ptr = ptr
        self._h = handle
        m = _lib.IndexMeta()
        _lib.check(handle.lib.culsh_index_get_meta(ptr, C.byref(m)))
        self._m = m

    def __del__(self):
        try:
            if self._ptr:
                self._h.lib.culsh_index_free(self._ptr)
                self._ptr = None
        except Exception:
            pass

    def empty(self) -> bool:
        return self._ptr is None

    def size_bytes(self) -> int:
        return int(self._m.size_bytes)

    n_total_candidates = property(lambda self: int(self._m.n_total_candidates))
    n_total_buckets = property(lambda self: int(self._m.n_total_buckets))
    n_hash_tables = property(lambda self: int(self._m.n_hash_tables))
    n_hashes = property(lambda self: int(self._m.n_hashes))
    sig_nbytes = property(lambda self: int(self._m.sig_nbytes))
    n_features = property(lambda self: int(self._m.n_features))
    seed = property(lambda self: int(self._m.seed))
    # extras (no upstream counterpart): the engine's internal key layout
    n_samples = property(lambda self: int(self._m.n_samples))
    key_words = property(lambda self: int(self._m.key_words))
    elem_bytes = property(lambda self: int(self._m.elem_bytes))

    def row_keys(self, out_ptr: int):
        """Write the packed key of every indexed row, [L][n_samples][key_words] uint32 in row
        order, to device memory at `out_ptr`."""
        _lib.check(self._h.lib.culsh_index_row_keys(self._h.ptr, self._ptr, out_ptr))

    def _copy(self, fn, n, dtype):
        arr = np.empty(int(n), dtype=dtype)
        if n:
            _lib.check(fn(self._ptr, int(arr.ctypes.data)))
        return arr

    def get_candidate_indices(self) -> np.ndarray:
        return self._copy(self._h.lib.culsh_index_get_candidate_indices, self.n_total_candidates, np.int32)

    def get_bucket_signatures(self) -> np.ndarray:
        return self._copy(self._h.lib.culsh_index_get_bucket_signatures,
                          self.n_total_buckets * self.sig_nbytes, np.uint8)

    def get_bucket_candidate_offsets(self) -> np.ndarray:
        return self._copy(self._h.lib.culsh_index_get_bucket_candidate_offsets, self.n_total_buckets + 1, np.int32)

    def get_table_bucket_offsets(self) -> np.ndarray:
        return self._copy(self._h.lib.culsh_index_get_table_bucket_offsets, self.n_hash_tables + 1, np.int32)

    @classmethod
    def _load(cls, is_double, candidate_indices, bucket_signatures, bucket_candidate_offsets,
              table_bucket_offsets, param0, param1, n_total_candidates, n_total_buckets,
              n_hash_tables, n_hashes, sig_nbytes, n_features, seed, window_size=0, pdtype=None):
        h = get_handle()
        keep = []

        def p(a, dt):
            addr, k = _pointer(a, dt)
            keep.append(k)
            return addr

        out = C.c_void_p()
        _lib.check(h.lib.culsh_index_load(
            h.ptr, cls._family, int(bool(is_double)),
            p(candidate_indices, np.int32), p(bucket_signatures, np.uint8),
            p(bucket_candidate_offsets, np.int32), p(table_bucket_offsets, np.int32),
            p(param0, pdtype), p(param1, pdtype) if param1 is not None else None,
            int(n_total_candidates), int(n_total_buckets), int(n_hash_tables), int(n_hashes),
            int(sig_nbytes), int(n_features), int(window_size), int(seed), C.byref(out)))
        return cls(out, h)


class RPLSHIndex(_IndexBase):
    _family = RPLSH
    is_double = property(lambda self: bool(self._m.is_double))

    def get_projection_matrix(self) -> np.ndarray:
        n = self.n_hash_tables * self.n_hashes * self.n_features
        return self._copy(self._h.lib.culsh_index_get_projection, n,
                          np.float64 if self.is_double else np.float32)

    @classmethod
    def load_float(cls, candidate_indices, bucket_signatures, bucket_candidate_offsets,
                   table_bucket_offsets, projection, n_total_candidates, n_total_buckets,
                   n_hash_tables, n_hashes, sig_nbytes, n_features, seed):
        return cls._load(False, candidate_indices, bucket_signatures, bucket_candidate_offsets,
                         table_bucket_offsets, projection, None, n_total_candidates, n_total_buckets,
                         n_hash_tables, n_hashes, sig_nbytes, n_features, seed, pdtype=np.float32)

    @classmethod
    def load_double(cls, candidate_indices, bucket_signatures, bucket_candidate_offsets,
                    table_bucket_offsets, projection, n_total_candidates, n_total_buckets,
                    n_hash_tables, n_hashes, sig_nbytes, n_features, seed):
        return cls._load(True, candidate_indices, bucket_signatures, bucket_candidate_offsets,
                         table_bucket_offsets, projection, None, n_total_candidates, n_total_buckets,
                         n_hash_tables, n_hashes, sig_nbytes, n_features, seed, pdtype=np.float64)


class PSLSHIndex(_IndexBase):
    _family = PSLSH
    is_double = property(lambda self: bool(self._m.is_double))
    window_size = property(lambda self: int(self._m.window_size))

    def get_projection_matrix(self) -> np.ndarray:
        n = self.n_hash_tables * self.n_hashes * self.n_features
        return self._copy(self._h.lib.culsh_index_get_projection, n,
                          np.float64 if self.is_double else np.float32)

    def get_bias(self) -> np.ndarray:
        return self._copy(self._h.lib.culsh_index_get_bias, self.n_hash_tables * self.n_hashes,
                          np.float64 if self.is_double else np.float32)

    @classmethod
    def load_float(cls, candidate_indices, bucket_signatures, bucket_candidate_offsets,
                   table_bucket_offsets, projection, bias, n_total_candidates, n_total_buckets,
                   n_hash_tables, n_hashes, sig_nbytes, n_features, seed, window_size=0):
        return cls._load(False, candidate_indices, bucket_signatures, bucket_candidate_offsets,
                         table_bucket_offsets, projection, bias, n_total_candidates, n_total_buckets,
                         n_hash_tables, n_hashes, sig_nbytes, n_features, seed, window_size, np.float32)

    @classmethod
    def load_double(cls, candidate_indices, bucket_signatures, bucket_candidate_offsets,
                    table_bucket_offsets, projection, bias, n_total_candidates, n_total_buckets,
                    n_hash_tables, n_hashes, sig_nbytes, n_features, seed, window_size=0):
        return cls._load(True, candidate_indices, bucket_signatures, bucket_candidate_offsets,
                         table_bucket_offsets, projection, bias, n_total_candidates, n_total_buckets,
                         n_hash_tables, n_hashes, sig_nbytes, n_features, seed, window_size, np.float64)


class MinHashIndex(_IndexBase):
    _family = MINHASH

    def get_hash_a(self) -> np.ndarray:
        return self._copy(self._h.lib.culsh_index_get_hash_a, self.n_hash_tables * self.n_hashes, np.uint32)

    def get_hash_b(self) -> np.ndarray:
        return self._copy(self._h.lib.culsh_index_get_hash_b, self.n_hash_tables * self.n_hashes, np.uint32)

    @classmethod
    def load(cls, candidate_indices, bucket_signatures, bucket_candidate_offsets,
             table_bucket_offsets, hash_a, hash_b, n_total_candidates, n_total_buckets,
             n_hash_tables, n_hashes, sig_nbytes, n_features, seed):
        return cls._load(False, candidate_indices, bucket_signatures, bucket_candidate_offsets,
                         table_bucket_offsets, hash_a, hash_b, n_total_candidates, n_total_buckets,
                         n_hash_tables, n_hashes, sig_nbytes, n_features, seed, pdtype=np.uint32)


class _CoreBase:
    def __init__(self, n_hash_tables: int, n_hashes: int, seed: int = 42):
        self._L, self._k, self._seed = int(n_hash_tables), int(n_hashes), int(seed)
        self._h = get_handle()

    n_hash_tables = property(lambda self: self._L)
    n_hashes = property(lambda self: self._k)
    seed = property(lambda self: self._seed)

    def last_stats(self) -> dict:
        """Per-stage figures of the last call (extension; see culsh_stats)."""
        return self._h.stats()

    def set_profiling(self, enabled: bool):
        _lib.check(self._h.lib.culsh_set_profiling(self._h.ptr, int(bool(enabled))))

    def set_param_cache(self, enabled: bool):
        """False: every fit generates its hash parameters again (upstream's behaviour) instead
        of reusing the set this handle made for the same (family, shape, seed)."""
        _lib.check(self._h.lib.culsh_set_param_cache(self._h.ptr, int(bool(enabled))))

    def query_keys(self, keys_ptr: int, n_queries: int, index) -> Candidates:
        """Candidates for queries given as packed keys on the device ([L][n_queries][key_words]
        uint32 in the index's own key layout, e.g. another shard's `index.row_keys`): lookup,
        gather and dedupe without hashing."""
        out = C.c_void_p()
        _lib.check(self._h.lib.culsh_index_query_keys(self._h.ptr, index._ptr, keys_ptr, int(n_queries),
                                                      C.byref(out)))
        return Candidates(out, self._h)

    def trim_scratch(self, keep_bytes: int = 0):
        """Free the engine's grow-only temporaries and kept result blocks larger than
        `keep_bytes` (they are allocated again when next needed)."""
        _lib.check(self._h.lib.culsh_trim_scratch(self._h.ptr, int(keep_bytes)))

    def set_projection_path(self, path: int):
        _lib.check(self._h.lib.culsh_set_projection_path(self._h.ptr, int(path)))


def _batch(batch_size: Optional[int]) -> int:
    return -1 if batch_size is None else int(batch_size)


class RPLSHCore(_CoreBase):
    """RPLSHCore of bindings.cu:25-116."""

    def _fit(self, fn, X, n, d, dtype):
        addr, keep = _pointer(X, dtype)
        out = C.c_void_p()
        _lib.check(fn(self._h.ptr, addr, int(n), int(d), self._L, self._k, self._seed, C.byref(out)))
        return out

    def fit_float(self, X, n_samples, n_features) -> RPLSHIndex:
        return RPLSHIndex(self._fit(self._h.lib.culsh_rplsh_fit_f32, X, n_samples, n_features, np.float32), self._h)

    def fit_double(self, X, n_samples, n_features) -> RPLSHIndex:
        return RPLSHIndex(self._fit(self._h.lib.culsh_rplsh_fit_f64, X, n_samples, n_features, np.float64), self._h)

    def _query(self, fn, Q, n, index, batch_size, dtype):
        addr, keep = _pointer(Q, dtype)
        out = C.c_void_p()
        _lib.check(fn(self._h.ptr, addr, int(n), index._ptr, _batch(batch_size), C.byref(out)))
        return Candidates(out, self._h)

    def query_float(self, Q, n_queries, index: RPLSHIndex, batch_size: Optional[int] = None) -> Candidates:
        return self._query(self._h.lib.culsh_rplsh_query_f32, Q, n_queries, index, batch_size, np.float32)

    def query_double(self, Q, n_queries, index: RPLSHIndex, batch_size: Optional[int] = None) -> Candidates:
        return self._query(self._h.lib.culsh_rplsh_query_f64, Q, n_queries, index, batch_size, np.float64)

    def fit_query_float(self, X, n_samples, n_features) -> Candidates:
        return Candidates(self._fit(self._h.lib.culsh_rplsh_fit_query_f32, X, n_samples, n_features, np.float32), self._h)

    def fit_query_double(self, X, n_samples, n_features) -> Candidates:
        return Candidates(self._fit(self._h.lib.culsh_rplsh_fit_query_f64, X, n_samples, n_features, np.float64), self._h)

    def hash(self, X, index: RPLSHIndex) -> np.ndarray:
        """uint8 [L][n][k] signatures of X under the index's projections (diagnostic)."""
        n = X.shape[0]
        addr, keep = _pointer(X, np.float64 if index.is_double else np.float32)
        out = np.empty((index.n_hash_tables, n, index.n_hashes), dtype=np.uint8)
        _lib.check(self._h.lib.culsh_index_hash_dense(self._h.ptr, index._ptr, addr, int(n), int(out.ctypes.data)))
        return out


class PSLSHCore(_CoreBase):
    """PSLSHCore of bindings.cu:171-265."""

    def __init__(self, n_hash_tables: int, n_hashes: int, window_size: int, seed: int = 42):
        super().__init__(n_hash_tables, n_hashes, seed)
        self._w = int(window_size)

    window_size = property(lambda self: self._w)

    def _fit(self, fn, X, n, d, dtype):
        addr, keep = _pointer(X, dtype)
        out = C.c_void_p()
        _lib.check(fn(self._h.ptr, addr, int(n), int(d), self._L, self._k, self._w, self._seed, C.byref(out)))
        return out

    def fit_float(self, X, n_samples, n_features) -> PSLSHIndex:
        return PSLSHIndex(self._fit(self._h.lib.culsh_pslsh_fit_f32, X, n_samples, n_features, np.float32), self._h)

    def fit_double(self, X, n_samples, n_features) -> PSLSHIndex:
        return PSLSHIndex(self._fit(self._h.lib.culsh_pslsh_fit_f64, X, n_samples, n_features, np.float64), self._h)

    def _query(self, fn, Q, n, index, batch_size, dtype):
        addr, keep = _pointer(Q, dtype)
        out = C.c_void_p()
        _lib.check(fn(self._h.ptr, addr, int(n), index._ptr, _batch(batch_size), C.byref(out)))
        return Candidates(out, self._h)

    def query_float(self, Q, n_queries, index: PSLSHIndex, batch_size: Optional[int] = None) -> Candidates:
        return self._query(self._h.lib.culsh_pslsh_query_f32, Q, n_queries, index, batch_size, np.float32)

    def query_double(self, Q, n_queries, index: PSLSHIndex, batch_size: Optional[int] = None) -> Candidates:
        return self._query(self._h.lib.culsh_pslsh_query_f64, Q, n_queries, index, batch_size, np.float64)

    def fit_query_float(self, X, n_samples, n_features) -> Candidates:
        return Candidates(self._fit(self._h.lib.culsh_pslsh_fit_query_f32, X, n_samples, n_features, np.float32), self._h)

    def fit_query_double(self, X, n_samples, n_features) -> Candidates:
        return Candidates(self._fit(self._h.lib.culsh_pslsh_fit_query_f64, X, n_samples, n_features, np.float64), self._h)

    def hash(self, X, index: PSLSHIndex) -> np.ndarray:
        """int32 [L][n][k] signatures of X under the index's projections and biases (diagnostic)."""
        n = X.shape[0]
        addr, keep = _pointer(X, np.float64 if index.is_double else np.float32)
        out = np.empty((index.n_hash_tables, n, index.n_hashes), dtype=np.int32)
        _lib.check(self._h.lib.culsh_index_hash_dense(self._h.ptr, index._ptr, addr, int(n), int(out.ctypes.data)))
        return out


class MinHashCore(_CoreBase):
    """MinHashCore of bindings.cu:119-168 (int32 CSR indices / indptr)."""

    def fit(self, indices, indptr, n_samples, n_features) -> MinHashIndex:
        a, k1 = _pointer(indices, np.int32)
        b, k2 = _pointer(indptr, np.int32)
        out = C.c_void_p()
        _lib.check(self._h.lib.culsh_minhash_fit(self._h.ptr, a, b, int(n_samples), int(n_features),
                                                 self._L, self._k, self._seed, C.byref(out)))
        return MinHashIndex(out, self._h)

    def query(self, indices, indptr, n_queries, index: MinHashIndex) -> Candidates:
        a, k1 = _pointer(indices, np.int32)
        b, k2 = _pointer(indptr, np.int32)
        out = C.c_void_p()
        _lib.check(self._h.lib.culsh_minhash_query(self._h.ptr, a, b, int(n_queries), index._ptr, C.byref(out)))
        return Candidates(out, self._h)

    def fit_query(self, indices, indptr, n_samples, n_features) -> Candidates:
        a, k1 = _pointer(indices, np.int32)
        b, k2 = _pointer(indptr, np.int32)
        out = C.c_void_p()
        _lib.check(self._h.lib.culsh_minhash_fit_query(self._h.ptr, a, b, int(n_samples), int(n_features),
                                                       self._L, self._k, self._seed, C.byref(out)))
        return Candidates(out, self._h)

    def hash(self, indices, indptr, n_rows, index: MinHashIndex) -> np.ndarray:
        """uint32 [L][n][k] MinHash signatures under the index's (A, B) (diagnostic)."""
        a, k1 = _pointer(indices, np.int32)
        b, k2 = _pointer(indptr, np.int32)
        out = np.empty((index.n_hash_tables, int(n_rows), index.n_hashes), dtype=np.uint32)
        _lib.check(self._h.lib.culsh_index_hash_csr(self._h.ptr, index._ptr, a, b, int(n_rows), int(out.ctypes.data)))
        return out


def merge_shard_candidates(shard_indices_ptrs, shard_offsets_ptrs, row_base, n_queries,
                           device: Optional[int] = None) -> Candidates:
    """Interleave per-shard CSR results (device pointers on one GPU) into one CSR with global ids."""
    h = get_handle(device)
    R = len(shard_indices_ptrs)
    idx = (C.c_void_p * R)(*[C.c_void_p(int(p)) for p in shard_indices_ptrs])
    off = (C.c_void_p * R)(*[C.c_void_p(int(p)) for p in shard_offsets_ptrs])
    base = (C.c_int64 * R)(*[int(b) for b in row_base])
    out = C.c_void_p()
    _lib.check(h.lib.culsh_merge_shard_candidates(h.ptr, R, int(n_queries), idx, off, base, C.byref(out)))
    return Candidates(out, h)


def merge_shard_candidates_into(shard_indices_ptrs, shard_offsets_ptrs, row_base, n_queries,
                                out_indices_ptr, out_capacity, out_counts_ptr, out_offsets_ptr,
                                device: Optional[int] = None) -> int:
    """Allocation-free form of :func:`merge_shard_candidates` for hosts that may not allocate
    device memory at merge time (the framework owns the whole device, or cudaMalloc's implicit
    synchronisation is not acceptable there): the caller supplies the three result arrays as
    device addresses and gets the merged id count back.  At most 64 shards and 4,194,304
    queries; calls that overlap on one GPU must be serialised (they share a small fixed
    scratch array inside the library)."""
    h = get_handle(device)
    R = len(shard_indices_ptrs)
    idx = (C.c_void_p * R)(*[C.c_void_p(int(p)) for p in shard_indices_ptrs])
    off = (C.c_void_p * R)(*[C.c_void_p(int(p)) for p in shard_offsets_ptrs])
    base = (C.c_int64 * R)(*[int(b) for b in row_base])
    total = C.c_uint64(0)
    _lib.check(h.lib.culsh_merge_shard_candidates_noalloc(
        h.ptr, R, int(n_queries), idx, off, base, int(out_indices_ptr) or None, int(out_capacity),
        int(out_counts_ptr), int(out_offsets_ptr), C.byref(total)))
    return int(total.value)
