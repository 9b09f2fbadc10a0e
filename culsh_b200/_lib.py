"""ctypes loader for libculsh_b200.so (the C ABI declared in include/culsh_b200.h).

There is no CPU fallback: if the library is missing or cannot be loaded the import of the
product layer fails loudly.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libculsh_b200.so")

c_i32p = C.POINTER(C.c_int32)
c_u64p = C.POINTER(C.c_uint64)


class IndexMeta(C.Structure):
    _fields_ = [
        ("family", C.c_int32), ("n_total_candidates", C.c_int32), ("n_total_buckets", C.c_int32),
        ("n_hash_tables", C.c_int32), ("n_hashes", C.c_int32), ("sig_nbytes", C.c_int32),
        ("n_features", C.c_int32), ("is_double", C.c_int32), ("window_size", C.c_int32),
        ("n_samples", C.c_int32), ("key_words", C.c_int32), ("elem_bytes", C.c_int32),
        ("seed", C.c_uint64), ("size_bytes", C.c_uint64),
    ]


class Stats(C.Structure):
    _fields_ = [
        ("hash_ms", C.c_float), ("sort_ms", C.c_float), ("build_ms", C.c_float),
        ("lookup_ms", C.c_float), ("gather_ms", C.c_float), ("total_ms", C.c_float),
        ("scatter_ms", C.c_float), ("dedupe_ms", C.c_float),
        ("params_ms", C.c_float), ("hash_lo_fraction", C.c_float),
        ("n_items", C.c_uint64), ("n_buckets", C.c_uint64), ("raw_candidates", C.c_uint64),
        ("unique_candidates", C.c_uint64),
        ("sort_passes", C.c_int32), ("key_words", C.c_int32), ("elem_bytes", C.c_int32),
        ("hash_path", C.c_int32), ("launches", C.c_int32), ("reserved1", C.c_int32),
    ]


VP = C.c_void_p
I = C.c_int
U64 = C.c_uint64
PP = C.POINTER(C.c_void_p)

# name -> argtypes (every function returns int unless listed in _VOID / _CHARP)
SIGNATURES = {
    "culsh_create": [I, PP],
    "culsh_destroy": [VP],
    "culsh_get_stats": [VP, C.POINTER(Stats)],
    "culsh_set_profiling": [VP, I],
    "culsh_set_param_cache": [VP, I],
    "culsh_trim_scratch": [VP, U64],
    "culsh_set_projection_path": [VP, I],
    "culsh_rplsh_fit_f32": [VP, VP, I, I, I, I, U64, PP],
    "culsh_rplsh_fit_f64": [VP, VP, I, I, I, I, U64, PP],
    "culsh_rplsh_query_f32": [VP, VP, I, VP, I, PP],
    "culsh_rplsh_query_f64": [VP, VP, I, VP, I, PP],
    "culsh_rplsh_fit_query_f32": [VP, VP, I, I, I, I, U64, PP],
    "culsh_rplsh_fit_query_f64": [VP, VP, I, I, I, I, U64, PP],
    "culsh_pslsh_fit_f32": [VP, VP, I, I, I, I, I, U64, PP],
    "culsh_pslsh_fit_f64": [VP, VP, I, I, I, I, I, U64, PP],
    "culsh_pslsh_query_f32": [VP, VP, I, VP, I, PP],
    "culsh_pslsh_query_f64": [VP, VP, I, VP, I, PP],
    "culsh_pslsh_fit_query_f32": [VP, VP, I, I, I, I, I, U64, PP],
    "culsh_pslsh_fit_query_f64": [VP, VP, I, I, I, I, I, U64, PP],
    "culsh_minhash_fit": [VP, VP, VP, I, I, I, I, U64, PP],
    "culsh_minhash_query": [VP, VP, VP, I, VP, PP],
    "culsh_minhash_fit_query": [VP, VP, VP, I, I, I, I, U64, PP],
    "culsh_index_hash_dense": [VP, VP, VP, I, VP],
    "culsh_index_hash_csr": [VP, VP, VP, VP, I, VP],
    "culsh_index_get_meta": [VP, C.POINTER(IndexMeta)],
    "culsh_index_get_candidate_indices": [VP, VP],
    "culsh_index_get_bucket_signatures": [VP, VP],
    "culsh_index_get_bucket_candidate_offsets": [VP, VP],
    "culsh_index_get_table_bucket_offsets": [VP, VP],
    "culsh_index_get_projection": [VP, VP],
    "culsh_index_get_bias": [VP, VP],
    "culsh_index_get_hash_a": [VP, VP],
    "culsh_index_get_hash_b": [VP, VP],
    "culsh_index_load": [VP, I, I, VP, VP, VP, VP, VP, VP, I, I, I, I, I, I, I, U64, PP],
    "culsh_candidates_get_meta": [VP, C.POINTER(C.c_int32), C.POINTER(C.c_uint64), C.POINTER(C.c_int32)],
    "culsh_candidates_get_indices": [VP, VP],
    "culsh_candidates_get_counts": [VP, VP],
    "culsh_candidates_get_offsets": [VP, VP],
    "culsh_candidates_device_ptrs": [VP, PP, PP, PP],
    "culsh_peer_alloc": [VP, C.c_size_t, PP, C.c_char_p],
    "culsh_peer_free": [VP, VP],
    "culsh_peer_open": [VP, C.c_char_p, PP],
    "culsh_peer_close": [VP, VP],
    "culsh_device_copy": [VP, VP, VP, C.c_size_t],
    "culsh_host_alloc": [C.c_size_t, PP],
    "culsh_host_free": [VP],
    "culsh_merge_shard_candidates": [VP, I, I, PP, PP, C.POINTER(C.c_int64), PP],
    "culsh_exchange_plan": [VP, I, I, I, VP, VP, C.POINTER(C.c_uint64), PP],
    "culsh_index_row_keys": [VP, VP, VP],
    "culsh_index_query_keys": [VP, VP, VP, I, PP],
    "culsh_exchange_push": [VP, I, I, I, VP, VP, VP, PP, C.c_int64, U64],
    "culsh_candidates_attach_indices": [VP, VP, U64],
    "culsh_merge_shard_candidates_noalloc": [VP, I, I, PP, PP, C.POINTER(C.c_int64), VP, U64, VP, VP,
                                             C.POINTER(C.c_uint64)],
}
_VOID = {"culsh_index_free": [VP], "culsh_candidates_free": [VP]}
_CHARP = {"culsh_last_error": []}

ALL_SYMBOLS = sorted(list(SIGNATURES) + list(_VOID) + list(_CHARP))

_lib = None


def load():
    """Load the shared library once; raise if it is missing (no fallback path exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m culsh_b200.build` "
            "(needs nvcc; the engine has no CPU fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, args in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = C.c_int
    for name, args in _VOID.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = None
    lib.culsh_last_error.argtypes = []
    lib.culsh_last_error.restype = C.c_char_p
    _lib = lib
    return lib


def check(status: int):
    """Map a non-zero status to the exception upstream's binding would raise
    (std::runtime_error -> RuntimeError, python/csrc/common/cuda_utils.cuh:11-25)."""
    if status == 0:
        return
    msg = load().culsh_last_error().decode("utf-8", "replace")
    if status == -3:
        raise MemoryError(msg)
    raise RuntimeError(msg)
