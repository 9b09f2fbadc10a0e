/*
 * culsh_b200 - C ABI of the B200-native LSH engine (hash -> bucket index -> lookup ->
 * gather/dedupe -> CSR) that stands in for cuLSH's pybind11 module `culsh._culsh_core`.
 *
 * Upstream has no C ABI: its Python layer binds C++ classes with pybind11
 * (python/csrc/bindings.cu:481-588).  Each entry point below names the upstream
 * class method / C++ function it replaces (paths relative to the upstream project root).
 *
 * Conventions
 *  - Every function returns 0 on success, a negative culsh_status otherwise; the text of
 *    the last failure is available from culsh_last_error() (thread-local).  Nothing calls
 *    exit() and no CUDA error is ignored (upstream: core/utils.cuh:10-52).
 *  - Array arguments are plain pointers.  An input or output pointer may live on the
 *    device of the handle OR in host memory (pageable or pinned); the library finds out
 *    with cudaPointerGetAttributes and stages host data itself.  Upstream only takes
 *    device pointers (python/csrc/common/array_utils.cuh:17-28) and leaves the
 *    host->device copy to CuPy in the Python layer (python/culsh/utils.py:34-53).
 *  - Dense inputs are C-contiguous row-major [n][d]; CSR inputs are int32 indices/indptr.
 *  - Every call is synchronous: it returns after its work on the handle's stream has
 *    finished (upstream: synchronize() after each method, bindings.cu:41,51,68,...).
 *  - Objects are not thread-safe; use one handle per host thread.
 */
#ifndef CULSH_B200_H
#define CULSH_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum culsh_status {
    CULSH_OK = 0,
    CULSH_ERR_INVALID = -1,    /* bad argument (shape, dtype mismatch, null pointer)        */
    CULSH_ERR_CUDA = -2,       /* a CUDA runtime / cuRAND call failed                       */
    CULSH_ERR_ALLOC = -3,      /* device or host allocation failed                          */
    CULSH_ERR_INTERNAL = -4,   /* a kernel reported a failed self-check (e.g. a bounded wait
                                  ran out); the context stays usable                        */
    CULSH_ERR_UNSUPPORTED = -5 /* limits: n*L >= 2^31, n_hashes too wide for one CTA, ...   */
} culsh_status;

typedef enum culsh_family {
    CULSH_RPLSH = 0,  /* random projection, cosine; signature element uint8 0/1 */
    CULSH_PSLSH = 1,  /* p-stable, Euclidean; signature element int32            */
    CULSH_MINHASH = 2 /* MinHash, Jaccard; signature element uint32              */
} culsh_family;

/* Opaque objects. */
typedef struct culsh_handle culsh_handle;         /* replaces CUDAResourceManager, python/csrc/common/cuda_utils.cuh:30-61 */
typedef struct culsh_index culsh_index;           /* replaces rplsh::Index / pslsh::Index / minhash::Index (+ core::Index, core/index.cuh:12-195) */
typedef struct culsh_candidates culsh_candidates; /* replaces core::Candidates, core/candidates.cuh:14-137 */

/* Mirror of the read-only properties bound in bindings.cu:381-404 (+ is_double, window). */
typedef struct culsh_index_meta {
    int32_t family;             /* culsh_family */
    int32_t n_total_candidates; /* n_samples * n_hash_tables */
    int32_t n_total_buckets;
    int32_t n_hash_tables;
    int32_t n_hashes;
    int32_t sig_nbytes;         /* upstream's raw signature width: k*1 (RPLSH) or k*4 */
    int32_t n_features;
    int32_t is_double;          /* dense families: parameters stored as float64 */
    int32_t window_size;        /* PSLSH only, else 0 */
    int32_t n_samples;
    int32_t key_words;          /* internal packed key width in 32-bit words */
    int32_t elem_bytes;         /* internal bytes kept per signature element */
    uint64_t seed;
    uint64_t size_bytes;        /* core/index.cuh:148-165 + family parameters, upstream layout */
} culsh_index_meta;

/* Per-stage figures of the last fit / query on a handle (device time from CUDA events). */
typedef struct culsh_stats {
    float hash_ms, sort_ms, build_ms, lookup_ms, gather_ms, total_ms;
    float scatter_ms; /* the scatter launch of the last radix pass alone */
    float dedupe_ms;  /* the dedupe launch (chained or bitmap kernel) of the query batches alone */
    float params_ms;  /* fit: host wall time of the hash-parameter generation (0 on a cache hit) */
    float hash_lo_fraction; /* tensor-core projection with profiling on: share of the K-blocks whose rows had
                               a non-zero low part, i.e. that issued three MMAs instead of two */
    uint64_t n_items, n_buckets, raw_candidates, unique_candidates;
    int32_t sort_passes, key_words, elem_bytes, hash_path; /* hash_path: 0 SIMT, 1 tcgen05 */
    int32_t launches;  /* kernels of this library launched by the call */
    int32_t reserved1;
} culsh_stats;

/* ---- handle -------------------------------------------------------------------------- */
/* CUDAResourceManager(): one stream per object (python/csrc/common/cuda_utils.cuh:36-39). */
int culsh_create(int device, culsh_handle** out);
int culsh_destroy(culsh_handle* h);
const char* culsh_last_error(void);
int culsh_get_stats(const culsh_handle* h, culsh_stats* out);
/* 1 = time stages with CUDA events (adds a few event records per call). Default 0. */
int culsh_set_profiling(culsh_handle* h, int enabled);
/* 1 (default) = hash parameters generated on this handle are kept and reused by later fits
 * with the same (family, shape, window, dtype, seed); 0 = every fit generates them again,
 * as upstream does (rplsh/hash.cuh:59-78, pslsh/hash.cuh:60-89, minhash/hash.cuh:42-54). */
int culsh_set_param_cache(culsh_handle* h, int enabled);
/* Temporaries live in per-handle device buffers that only grow (after a 10M-row self-join:
 * 5.7 GB) and released result blocks are kept for reuse; this frees every such buffer larger
 * than keep_bytes (0 = all of them).  Waits for the handle's streams; the next call that needs
 * a buffer allocates it again.  No upstream counterpart (upstream allocates and frees its
 * temporaries inside every call, core/fit.cuh:160-252, core/query.cuh:290-478). */
int culsh_trim_scratch(culsh_handle* h, uint64_t keep_bytes);
/* Force the projection path: 0 auto, 1 SIMT fp32/fp64 kernel, 2 tcgen05 3xTF32 kernel. */
int culsh_set_projection_path(culsh_handle* h, int path);

/* ---- RPLSH: RPLSHCore, bindings.cu:25-116; rplsh/rplsh.cu:18-226 ---------------------- */
/* RPLSHCore.fit_float / fit_double  -> rplsh::fit (rplsh.cu:18-84). */
int culsh_rplsh_fit_f32(culsh_handle* h, const float* X, int n_samples, int n_features,
                        int n_hash_tables, int n_hashes, uint64_t seed, culsh_index** out);
int culsh_rplsh_fit_f64(culsh_handle* h, const double* X, int n_samples, int n_features,
                        int n_hash_tables, int n_hashes, uint64_t seed, culsh_index** out);
/* RPLSHCore.query_float / query_double -> rplsh::query / query_batched (rplsh.cu:86-128,
 * 188-226).  batch_size <= 0 means "not given".  A dtype that differs from the index's is
 * CULSH_ERR_INVALID (bindings.cu:58-60,75-77). */
int culsh_rplsh_query_f32(culsh_handle* h, const float* Q, int n_queries, const culsh_index* index,
                          int batch_size, culsh_candidates** out);
int culsh_rplsh_query_f64(culsh_handle* h, const double* Q, int n_queries, const culsh_index* index,
                          int batch_size, culsh_candidates** out);
/* RPLSHCore.fit_query_float / fit_query_double -> rplsh::fit_query (rplsh.cu:130-186). */
int culsh_rplsh_fit_query_f32(culsh_handle* h, const float* X, int n_samples, int n_features,
                              int n_hash_tables, int n_hashes, uint64_t seed, culsh_candidates** out);
int culsh_rplsh_fit_query_f64(culsh_handle* h, const double* X, int n_samples, int n_features,
                              int n_hash_tables, int n_hashes, uint64_t seed, culsh_candidates** out);

/* ---- PSLSH: PSLSHCore, bindings.cu:171-265; pslsh/pslsh.cu:18-242 --------------------- */
int culsh_pslsh_fit_f32(culsh_handle* h, const float* X, int n_samples, int n_features,
                        int n_hash_tables, int n_hashes, int window_size, uint64_t seed,
                        culsh_index** out);
int culsh_pslsh_fit_f64(culsh_handle* h, const double* X, int n_samples, int n_features,
                        int n_hash_tables, int n_hashes, int window_size, uint64_t seed,
                        culsh_index** out);
int culsh_pslsh_query_f32(culsh_handle* h, const float* Q, int n_queries, const culsh_index* index,
                          int batch_size, culsh_candidates** out);
int culsh_pslsh_query_f64(culsh_handle* h, const double* Q, int n_queries, const culsh_index* index,
                          int batch_size, culsh_candidates** out);
int culsh_pslsh_fit_query_f32(culsh_handle* h, const float* X, int n_samples, int n_features,
                              int n_hash_tables, int n_hashes, int window_size, uint64_t seed,
                              culsh_candidates** out);
int culsh_pslsh_fit_query_f64(culsh_handle* h, const double* X, int n_samples, int n_features,
                              int n_hash_tables, int n_hashes, int window_size, uint64_t seed,
                              culsh_candidates** out);

/* ---- MinHash: MinHashCore, bindings.cu:119-168; minhash/minhash.cu:19-102 ------------- */
/* indices: int32 [nnz] column ids, indptr: int32 [n+1]; nnz = indptr[n]. */
int culsh_minhash_fit(culsh_handle* h, const int32_t* indices, const int32_t* indptr, int n_samples,
                      int n_features, int n_hash_tables, int n_hashes, uint64_t seed,
                      culsh_index** out);
int culsh_minhash_query(culsh_handle* h, const int32_t* indices, const int32_t* indptr,
                        int n_queries, const culsh_index* index, culsh_candidates** out);
int culsh_minhash_fit_query(culsh_handle* h, const int32_t* indices, const int32_t* indptr,
                            int n_samples, int n_features, int n_hash_tables, int n_hashes,
                            uint64_t seed, culsh_candidates** out);

/* ---- packed keys in and out (extension; no upstream counterpart: upstream's self-join,
 *      core/fit_query.cuh:30-55, is single-GPU).  A row-sharded self-join ships the rows' packed
 *      signatures between the shards instead of the rows, so every row is hashed once.
 *   culsh_index_row_keys: packed key of every indexed row in row order, device memory,
 *     [n_hash_tables][n_samples][key_words] uint32 (key_words from culsh_index_get_meta).
 *   culsh_index_query_keys: candidates for n_queries queries given as such keys (device,
 *     [n_hash_tables][n_queries][key_words], same family, shape, seed and key layout as the
 *     index): lookup + gather + dedupe, no hashing. -------------------------------------- */
int culsh_index_row_keys(culsh_handle* h, const culsh_index* index, uint32_t* keys_out);
int culsh_index_query_keys(culsh_handle* h, const culsh_index* index, const uint32_t* keys, int n_queries,
                           culsh_candidates** out);

/* ---- signatures only (diagnostic; upstream keeps X_sig internal: rplsh/hash.cuh:93-129,
 *      pslsh/hash.cuh:105-142, minhash/hash.cuh:142-155).  `sig_out` receives upstream's
 *      table-major raw layout [L][n][k] of uint8 / int32 / uint32, host or device. -------- */
int culsh_index_hash_dense(culsh_handle* h, const culsh_index* index, const void* X, int n_rows,
                           void* sig_out);
int culsh_index_hash_csr(culsh_handle* h, const culsh_index* index, const int32_t* indices,
                         const int32_t* indptr, int n_rows, void* sig_out);

/* ---- Index: getters bindings.cu:341-404, loaders bindings.cu:407-476 ------------------ */
int culsh_index_get_meta(const culsh_index* index, culsh_index_meta* out);
/* Each getter copies into dst (host or device): sizes are n_total_candidates, B*sig_nbytes,
 * B+1 and L+1 elements.  Arrays are produced in upstream's canonical layout. */
int culsh_index_get_candidate_indices(const culsh_index* index, int32_t* dst);
int culsh_index_get_bucket_signatures(const culsh_index* index, uint8_t* dst);
int culsh_index_get_bucket_candidate_offsets(const culsh_index* index, int32_t* dst);
int culsh_index_get_table_bucket_offsets(const culsh_index* index, int32_t* dst);
/* get_projection_matrix (H*d), get_bias (H): element type follows is_double.
 * get_hash_a / get_hash_b (H uint32). */
int culsh_index_get_projection(const culsh_index* index, void* dst);
int culsh_index_get_bias(const culsh_index* index, void* dst);
int culsh_index_get_hash_a(const culsh_index* index, uint32_t* dst);
int culsh_index_get_hash_b(const culsh_index* index, uint32_t* dst);
/* RPLSHIndex.load_float/load_double, PSLSHIndex.load_*, MinHashIndex.load: rebuild an
 * index from arrays in upstream's layout (as written by Model.save, e.g.
 * python/culsh/rp_lsh.py:259-274).  param0 = projection | hash_a, param1 = bias | hash_b
 * (NULL for RPLSH). */
int culsh_index_load(culsh_handle* h, int family, int is_double, const int32_t* candidate_indices,
                     const uint8_t* bucket_signatures, const int32_t* bucket_candidate_offsets,
                     const int32_t* table_bucket_offsets, const void* param0, const void* param1,
                     int n_total_candidates, int n_total_buckets, int n_hash_tables, int n_hashes,
                     int sig_nbytes, int n_features, int window_size, uint64_t seed,
                     culsh_index** out);
void culsh_index_free(culsh_index* index);

/* ---- Candidates: getters bindings.cu:268-338 ------------------------------------------ */
int culsh_candidates_get_meta(const culsh_candidates* c, int32_t* n_queries,
                              uint64_t* n_total_candidates, int32_t* is_empty);
/* dst holds n_total_candidates int32 / n_queries uint64 / n_queries+1 uint64; host or device. */
int culsh_candidates_get_indices(const culsh_candidates* c, int32_t* dst);
int culsh_candidates_get_counts(const culsh_candidates* c, uint64_t* dst);
int culsh_candidates_get_offsets(const culsh_candidates* c, uint64_t* dst);
/* Device pointers of the result (borrowed; valid until culsh_candidates_free). */
int culsh_candidates_device_ptrs(const culsh_candidates* c, const int32_t** indices,
                                 const uint64_t** counts, const uint64_t** offsets);
void culsh_candidates_free(culsh_candidates* c);

/* ---- pinned host buffers for results --------------------------------------------------- */
/* Upstream's getters copy into freshly allocated pageable NumPy memory (bindings.cu:268-338),
 * which caps the device->host read of a large CSR at a few GB/s.  These two calls let a
 * binding keep a pool of page-locked blocks for result arrays (culsh_b200/_culsh_core.py does). */
int culsh_host_alloc(size_t bytes, void** out);
int culsh_host_free(void* p);

/* ---- row-sharded indexes (no upstream counterpart: upstream is single-GPU) ------------- */
/* Interleave R per-shard CSR results that were produced for the same queries into one CSR
 * with global row ids: shard r's ids are shifted by row_base[r]; per query the shard lists
 * are concatenated in shard order.  All shard arrays are device pointers on the handle's
 * device (gathered there by the caller, e.g. with NCCL). */
int culsh_merge_shard_candidates(culsh_handle* h, int n_shards, int n_queries,
                                 const int32_t* const* shard_indices,
                                 const uint64_t* const* shard_offsets, const int64_t* row_base,
                                 culsh_candidates** out);

/* Push form of the exchange between R ranks that answered the same n_queries queries over
 * their own row shards (no upstream counterpart).  Rank j owns the queries [j*per, (j+1)*per),
 * per = ceil(n_queries / R), and ends up with their merged lists.
 *   culsh_exchange_plan: from the per-query unique counts of all ranks (counts_all, device,
 *     [R][n_queries], e.g. all-gathered) compute where this rank's list of every query starts
 *     inside its owner's merged id array (dstpos, device, n_queries), the id count of every
 *     slice (slice_totals, host, R) and a result object for this rank's slice that holds the
 *     merged counts and offsets but no ids yet.
 *   culsh_exchange_push: store this rank's lists (indices / offsets, device, local row ids),
 *     shifted by row_base, at dstpos inside recv[owner] - device pointers, peer memory for the
 *     other ranks (culsh_peer_open), each with room for its slice total.  The queries are
 *     visited so that every rank deals its stores evenly over all owners at any moment (the
 *     order depends on rank), which keeps every NVLink ingress equally loaded.  Returns when
 *     the stores have been issued and the stream is idle; the owners may read after a barrier.
 *   culsh_candidates_attach_indices: point a result object at an id array it does not own
 *     (the owner's receive buffer, which must outlive it). */
int culsh_exchange_plan(culsh_handle* h, int n_ranks, int rank, int n_queries, const uint64_t* counts_all,
                        uint64_t* dstpos, uint64_t* slice_totals, culsh_candidates** out);
int culsh_exchange_push(culsh_handle* h, int n_ranks, int rank, int n_queries, const int32_t* indices,
                        const uint64_t* offsets, const uint64_t* dstpos, void* const* recv, int64_t row_base,
                        uint64_t total);
int culsh_candidates_attach_indices(culsh_candidates* c, const int32_t* indices, uint64_t total);

/* Peer-memory plumbing for the row-sharded exchange (no upstream counterpart).  A rank exports
 * a plain device allocation to the other processes of the box; peers map it and the merge
 * kernel of culsh_merge_shard_candidates then reads their per-shard CSR arrays directly over
 * NVLink with ordinary loads (no staging copy, no collective library on the data path).
 * `handle` is the 64-byte cudaIpcMemHandle_t. */
int culsh_peer_alloc(culsh_handle* h, size_t bytes, void** dptr, unsigned char handle[64]);
int culsh_peer_free(culsh_handle* h, void* dptr);
int culsh_peer_open(culsh_handle* h, const unsigned char handle[64], void** dptr);
int culsh_peer_close(culsh_handle* h, void* dptr);
/* dst (device, this handle's device) <- src (device) on the handle's stream, then wait. */
int culsh_device_copy(culsh_handle* h, void* dst, const void* src, size_t bytes);

/* Same merge for callers that must not allocate (no counterpart in the reference).
 *
 * Some hosts of this library cannot call cudaMalloc at the point where shard results are
 * merged: a serving process whose framework has already claimed the whole device for its own
 * caching allocator, a latency-critical loop where the implicit device synchronisation of
 * cudaMalloc / cudaFree is not acceptable, or code that runs under a fixed memory budget
 * audited at start-up.  This variant therefore takes every result array from the caller and
 * keeps its only temporaries - the per-shard pointer / row-base tables and the block sums of
 * the offset scan - in a 32 KB array that is a fixed part of the library image (each GPU that
 * loads the library holds those 32 KB until the process exits).  It calls no cudaMalloc,
 * cudaFree or other allocating routine.
 *
 *   out_indices  device, room for out_capacity ids (may be NULL when the result is empty)
 *   out_counts   device, n_queries uint64
 *   out_offsets  device, n_queries + 1 uint64
 *   total_out    host; receives the merged id count, also when out_capacity is too small
 *                (the call then fails with CULSH_ERR_INVALID and writes no ids)
 *
 * Limits: at most 64 shards and 4,194,304 queries per call; more is CULSH_ERR_UNSUPPORTED.
 * The first call on a device looks the array's device address up once (with that device
 * current); make that first call before starting any stream capture.  All calls on a device
 * share the array and it keeps whatever the previous call left there - every word a call
 * reads is written earlier in the same call, so nothing needs clearing - which also means
 * two calls that overlap on the same GPU (different handles or threads) race on it: serialise
 * them.  The shard arrays are device pointers on the handle's device, as for
 * culsh_merge_shard_candidates; the three tables themselves are host arrays. */
int culsh_merge_shard_candidates_noalloc(culsh_handle* h, int n_shards, int n_queries,
                                         const int32_t* const* shard_indices,
                                         const uint64_t* const* shard_offsets, const int64_t* row_base,
                                         int32_t* out_indices, uint64_t out_capacity,
                                         uint64_t* out_counts, uint64_t* out_offsets,
                                         uint64_t* total_out);

#ifdef __cplusplus
}
#endif
#endif /* CULSH_B200_H */
