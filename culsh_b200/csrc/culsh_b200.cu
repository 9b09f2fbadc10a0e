// Host orchestration and the C ABI of the engine (see include/culsh_b200.h).
#include "common.cuh"
#include "index_build.cuh"
#include "minhash.cuh"
#include "project_simt.cuh"
#include "project_tc.cuh"
#include "query.cuh"
#include "radix_sort.cuh"

#include <algorithm>
#include <chrono>
#include <cstdlib>

using namespace culsh_b200;

// -----------------------------------------------------------------------------------------
// Objects behind the opaque pointers
// -----------------------------------------------------------------------------------------
struct culsh_handle {
    CtxPtr ctx;
};

// Hash parameters of an index; immutable once generated, so indexes built on one handle with
// the same (family, shape, window, dtype, seed) share one set.
struct ParamSet {
    DevBuf<uint8_t> p0;       // projection (float/double [H][d]) | hash A (uint32 [H])
    DevBuf<uint8_t> p1;       // bias (float/double [H])          | hash B (uint32 [H])
    DevBuf<uint8_t> p_split;  // tensor-core path: hi/lo split of the projection
};

struct culsh_index {
    CtxPtr ctx;
    KeySpec ks;
    int family = 0, n = 0, d = 0, L = 0, k = 0, window = 0, is_double = 0;
    uint64_t seed = 0;
    int n_buckets = 0;
    DevBuf<int32_t> cand;            // [n*L]   row ids grouped by (table, bucket)
    DevBuf<uint32_t> bucket_keys;    // [B][NW] packed signatures, sorted inside a table
    DevBuf<int32_t> bucket_offsets;  // [B+1]
    DevBuf<int32_t> table_offsets;   // [L+1]
    std::shared_ptr<ParamSet> params = std::make_shared<ParamSet>();  // may be shared between indexes
};

struct culsh_candidates {
    CtxPtr ctx;
    int n_queries = 0;
    uint64_t total = 0;
    DevBuf<int32_t> indices;
    DevBuf<uint64_t> counts;
    DevBuf<uint64_t> offsets;
    bool empty() const { return !indices.p && !counts.p && !offsets.p; }
};

namespace {

thread_local std::string g_last_error;

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return CULSH_OK;
    } catch (const Error& e) {
        g_last_error = e.what();
        return e.status;
    } catch (const std::bad_alloc&) {
        g_last_error = "host allocation failed";
        return CULSH_ERR_ALLOC;
    } catch (const std::exception& e) {
        g_last_error = e.what();
        return CULSH_ERR_INTERNAL;
    }
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        CU_CHECK(cudaGetDevice(&prev));
        if (prev != dev) CU_CHECK(cudaSetDevice(dev));
        else prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

struct StageTimer {
    const CtxPtr& c;
    int next = 0;
    explicit StageTimer(const CtxPtr& ctx) : c(ctx) {}
    void mark() {
        if (c->profiling && next < 7) cudaEventRecord(c->ev[next++], c->stream);
    }
    float last_scatter() const {  // ev_pass[] are recorded by the sort driver
        float ms = 0.f;
        if (c->profiling) cudaEventElapsedTime(&ms, c->ev_pass[0], c->ev_pass[1]);
        return ms;
    }
    float between(int a, int b) const {
        float ms = 0.f;
        if (c->profiling && b < next) cudaEventElapsedTime(&ms, c->ev[a], c->ev[b]);
        return ms;
    }
};

// Optional host-side trace (CULSH_TRACE=1): wall-clock of host steps, printed to stderr.
struct HostTrace {
    bool on;
    std::chrono::steady_clock::time_point t;
    HostTrace() : on(getenv("CULSH_TRACE") != nullptr), t(std::chrono::steady_clock::now()) {}
    void lap(const char* what) {
        if (!on) return;
        auto now = std::chrono::steady_clock::now();
        uint64_t reserved = 0, used = 0;
        int dev = 0;
        cudaGetDevice(&dev);
        cudaMemPool_t pool;
        if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
            cudaMemPoolGetAttribute(pool, cudaMemPoolAttrReservedMemCurrent, &reserved);
            cudaMemPoolGetAttribute(pool, cudaMemPoolAttrUsedMemCurrent, &used);
        }
        fprintf(stderr, "[culsh trace] %-28s %9.1f us   pool reserved %7.1f MB used %7.1f MB\n", what,
                std::chrono::duration<double, std::micro>(now - t).count(), reserved / 1048576.0,
                used / 1048576.0);
        t = std::chrono::steady_clock::now();
    }
};

inline long env_long_early(const char* name, long dflt) {
    const char* e = getenv(name);
    return e && *e ? atol(e) : dflt;
}

void reset_error_word(const CtxPtr& c) {
    CU_CHECK(cudaMemsetAsync(c->d_error, 0, sizeof(int), c->stream));
}

int read_error_word(const CtxPtr& c) {
    int e = 0;
    read_words(c, c->d_error, sizeof(int), &e);
    return e;
}

void check_error_word(int e) {
    if (e & DEV_ERR_LOOKBACK_TIMEOUT)
        fail(CULSH_ERR_INTERNAL, "radix sort: a bounded wait on a preceding tile ran out");
    if (e & DEV_ERR_MBAR_TIMEOUT)
        fail(CULSH_ERR_INTERNAL, "projection: a bounded wait on a copy/MMA barrier ran out");
    if (e & DEV_ERR_RANGE) fail(CULSH_ERR_INTERNAL, "a kernel skipped an out-of-range index");
}

// -----------------------------------------------------------------------------------------
// Hash parameters.  Same cuRAND calls in the same order as upstream so that a seed means
// the same hash functions: XORWOW (CURAND_RNG_PSEUDO_DEFAULT), default ordering,
//   RPLSH   : GenerateNormal[Double](H*d)                      rplsh/hash.cuh:59-78
//   PSLSH   : GenerateNormal[Double](H*d), GenerateUniform[Double](H), P /= int w
//                                                               pslsh/hash.cuh:60-89
//   MinHash : Generate(A,H), Generate(B,H), A%(p-1)+1, B%p      minhash/hash.cuh:26-54
// -----------------------------------------------------------------------------------------
template <typename T>
__global__ void scale_by_int_kernel(T* p, size_t n, int w) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = p[i] / w;  // T / int, as upstream's thrust placeholder expression
}

__global__ void minhash_normalize_kernel(uint32_t* A, uint32_t* B, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        A[i] = (A[i] % (MINHASH_PRIME - 1u)) + 1u;
        B[i] = B[i] % MINHASH_PRIME;
    }
}

// Own generator kernel for the single-precision and integer parameter sets.  cuRAND's host
// API with the XORWOW generator in its default ordering runs 4096 independent streams -
// stream t is curand_init(seed, subsequence t, offset 0) of the device API - and deals the
// output round-robin: 32-bit element e of a generator's life comes from stream e mod 4096
// (its next draw), a normal pair p (outputs 2p, 2p + 1) is the next curand_normal2 of stream
// p mod 4096, and a call that follows continues at the element after the last pair, every
// stream going on from its own state.  One launch replaces the host API's seeding launch,
// generation launches and the scaling / normalisation kernels (0.17 ms of host and device time
// per fit); equality with the host API's output is what the parameter parity tests check.
constexpr int XW_STREAMS = 4096;
constexpr int XW_BLOCK = 32;

__global__ void __launch_bounds__(XW_BLOCK)
xorwow_dense_params_kernel(unsigned long long seed, float* __restrict__ normals, size_t n_pairs, int w,
                           float* __restrict__ uniforms, int n_unif) {
    const int t = blockIdx.x * XW_BLOCK + threadIdx.x;
    curandStateXORWOW_t st;
    curand_init(seed, (unsigned long long)t, 0ull, &st);
    float2* out2 = reinterpret_cast<float2*>(normals);
    for (size_t p = (size_t)t; p < n_pairs; p += XW_STREAMS) {
        float2 v = curand_normal2(&st);
        if (w) { v.x = v.x / w; v.y = v.y / w; }  // float / int, pslsh/hash.cuh:84-88
        out2[p] = v;
    }
    // the uniform call continues at element n_pairs of the round-robin
    const int first = (int)(n_pairs % XW_STREAMS);
    for (int j = (t - first + XW_STREAMS) % XW_STREAMS; j < n_unif; j += XW_STREAMS)
        uniforms[j] = curand_uniform(&st);
}

__global__ void __launch_bounds__(XW_BLOCK)
xorwow_minhash_params_kernel(unsigned long long seed, uint32_t* __restrict__ A, uint32_t* __restrict__ B, int H) {
    const int t = blockIdx.x * XW_BLOCK + threadIdx.x;
    curandStateXORWOW_t st;
    curand_init(seed, (unsigned long long)t, 0ull, &st);
    for (int e = t; e < 2 * H; e += XW_STREAMS) {  // two consecutive calls of H elements
        const uint32_t v = curand(&st);
        if (e < H) A[e] = (v % (MINHASH_PRIME - 1u)) + 1u;  // minhash/hash.cuh:44-53
        else B[e - H] = v % MINHASH_PRIME;
    }
}

// The handle keeps one XORWOW generator for its lifetime (creating one allocates device
// memory and synchronises the device); a call re-seeds it, which restarts the sequence at
// offset 0 exactly as a freshly created generator would.
curandGenerator_t seeded_generator(const CtxPtr& c, uint64_t seed) {
    if (!c->curand) {
        curandGenerator_t g = nullptr;
        CURAND_CHECK(curandCreateGenerator(&g, CURAND_RNG_PSEUDO_DEFAULT));
        curandStatus_t st = curandSetStream(g, c->stream);
        if (st != CURAND_STATUS_SUCCESS) {
            curandDestroyGenerator(g);
            fail(CULSH_ERR_CUDA, "cuRAND generator setup failed: status %d", (int)st);
        }
        c->curand = g;
    }
    CURAND_CHECK(curandSetPseudoRandomGeneratorSeed(c->curand, seed));
    CURAND_CHECK(curandSetGeneratorOffset(c->curand, 0ull));
    return c->curand;
}

// CULSH_PARAMS_HOST_API=1 routes every parameter set through cuRAND's host API (the tests compare
// the two); double-precision sets always take it.
inline bool own_generator() {
    const char* e = getenv("CULSH_PARAMS_HOST_API");
    return !(e && *e && atoi(e) != 0);
}

void generate_params_uncached(culsh_index& ix);

void prepare_tc_split(culsh_index& ix);

// Parameters + (fp32 dense families) the hi/lo split of the projection for the tensor-core
// kernel.  last_params_ms is the host wall time of the generation (0 on a cache hit).
void generate_params(culsh_index& ix) {
    const CtxPtr& c = ix.ctx;
    c->last_params_ms = 0.f;
    ParamKey key{ix.family, ix.L * ix.k, ix.family == CULSH_MINHASH ? 0 : ix.d, ix.window, ix.is_double, ix.seed};
    if (c->param_cache_enabled) {
        auto it = c->param_cache.find(key);
        if (it != c->param_cache.end()) {
            ix.params = std::static_pointer_cast<ParamSet>(it->second);
            return;
        }
    }
    const auto t0 = std::chrono::steady_clock::now();
    HostTrace tr;
    generate_params_uncached(ix);
    tr.lap("params: cuRAND calls issued");
    prepare_tc_split(ix);
    CU_CHECK(cudaStreamSynchronize(c->stream));
    tr.lap("params: split + sync");
    c->last_params_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (c->param_cache_enabled) {
        if (c->param_cache.size() >= 16) c->param_cache.clear();
        c->param_cache[key] = ix.params;
    }
}

void generate_params_uncached(culsh_index& ix) {
    const CtxPtr& c = ix.ctx;
    const int H = ix.L * ix.k;
    ix.params = std::make_shared<ParamSet>();
    if (ix.family == CULSH_MINHASH) {
        ix.params->p0.alloc(c, sizeof(uint32_t) * H);
        ix.params->p1.alloc(c, sizeof(uint32_t) * H);
        if (own_generator()) {
            xorwow_minhash_params_kernel<<<XW_STREAMS / XW_BLOCK, XW_BLOCK, 0, c->stream>>>(
                ix.seed, reinterpret_cast<uint32_t*>(ix.params->p0.p), reinterpret_cast<uint32_t*>(ix.params->p1.p), H);
            KERNEL_CHECK();
            return;
        }
        struct { curandGenerator_t g; } gen{seeded_generator(c, ix.seed)};
        CURAND_CHECK(curandGenerate(gen.g, reinterpret_cast<uint32_t*>(ix.params->p0.p), H));
        CURAND_CHECK(curandGenerate(gen.g, reinterpret_cast<uint32_t*>(ix.params->p1.p), H));
        minhash_normalize_kernel<<<(unsigned)ceil_div(H, 256), 256, 0, c->stream>>>(
            reinterpret_cast<uint32_t*>(ix.params->p0.p), reinterpret_cast<uint32_t*>(ix.params->p1.p), H);
        KERNEL_CHECK();
        return;
    }
    const size_t pn = (size_t)H * ix.d;
    if (pn % 2 != 0)
        fail(CULSH_ERR_INVALID,
             "n_hash_tables*n_hashes*n_features = %zu must be even (cuRAND normal generation)", pn);
    const size_t esz = ix.is_double ? 8 : 4;
    ix.params->p0.alloc(c, esz * pn);
    if (!ix.is_double && own_generator()) {
        const bool ps = ix.family == CULSH_PSLSH;
        if (ps) ix.params->p1.alloc(c, esz * H);
        xorwow_dense_params_kernel<<<XW_STREAMS / XW_BLOCK, XW_BLOCK, 0, c->stream>>>(
            ix.seed, reinterpret_cast<float*>(ix.params->p0.p), pn / 2, ps ? ix.window : 0,
            ps ? reinterpret_cast<float*>(ix.params->p1.p) : nullptr, ps ? H : 0);
        KERNEL_CHECK();
        return;
    }
    struct { curandGenerator_t g; } gen{seeded_generator(c, ix.seed)};
    if (ix.is_double)
        CURAND_CHECK(curandGenerateNormalDouble(gen.g, reinterpret_cast<double*>(ix.params->p0.p), pn, 0.0, 1.0));
    else
        CURAND_CHECK(curandGenerateNormal(gen.g, reinterpret_cast<float*>(ix.params->p0.p), pn, 0.0f, 1.0f));
    if (ix.family == CULSH_PSLSH) {
        ix.params->p1.alloc(c, esz * H);
        if (ix.is_double) {
            CURAND_CHECK(curandGenerateUniformDouble(gen.g, reinterpret_cast<double*>(ix.params->p1.p), H));
            scale_by_int_kernel<double><<<(unsigned)ceil_div(pn, 256), 256, 0, c->stream>>>(
                reinterpret_cast<double*>(ix.params->p0.p), pn, ix.window);
        } else {
            CURAND_CHECK(curandGenerateUniform(gen.g, reinterpret_cast<float*>(ix.params->p1.p), H));
            scale_by_int_kernel<float><<<(unsigned)ceil_div(pn, 256), 256, 0, c->stream>>>(
                reinterpret_cast<float*>(ix.params->p0.p), pn, ix.window);
        }
        KERNEL_CHECK();
    }
}

// -----------------------------------------------------------------------------------------
// Hash stage drivers
// -----------------------------------------------------------------------------------------
// Hash dense rows (host or device memory) into keys[L][n_total][NW] at row_offset.
template <typename T>
void hash_dense(const culsh_index& ix, const KeySpec& ks, const T* X, int n, uint32_t* keys,
                uint8_t* ovf_rows, int n_total, int row_offset, bool allow_fallback = false) {
    const CtxPtr& c = ix.ctx;
    if (n == 0) return;
    const T* P = reinterpret_cast<const T*>(ix.params->p0.p);
    const T* bias = reinterpret_cast<const T*>(ix.params->p1.p);
    auto launch = [&](cudaStream_t s, const T* Xd, int rows, int off) {
        bool tc = false;
        if (std::is_same<T, float>::value && c->projection_path != 1)
            tc = launch_project_tc(c, s, ix.family, reinterpret_cast<const float*>(Xd),
                                   reinterpret_cast<const float*>(P), ix.params->p_split.p,
                                   reinterpret_cast<const float*>(bias), rows, ix.d, ix.L, ix.k, ks,
                                   keys, ovf_rows, off, n_total);
        if (!tc) {
            if (c->projection_path == 2 && !allow_fallback)
                fail(CULSH_ERR_UNSUPPORTED, "tensor-core projection path is not available for this shape");
            launch_project_simt<T>(c, s, ix.family, Xd, P, bias, rows, ix.d, ix.L, ix.k, ks, keys,
                                   ovf_rows, off, n_total);
        }
        c->stats.hash_path = tc ? 1 : 0;
    };
    if (is_device_pointer(X)) {
        launch(c->stream, X, n, row_offset);
        return;
    }
    // Host input: stream it through two device staging buffers so the copy of chunk i+1
    // overlaps the hashing of chunk i.
    const size_t row_bytes = sizeof(T) * (size_t)ix.d;
    size_t chunk_rows = std::max<size_t>(1024, (size_t)(32u << 20) / row_bytes);
    chunk_rows = std::min<size_t>(chunk_rows, (size_t)n);
    chunk_rows = (chunk_rows + 127) / 128 * 128;
    Scratch<uint8_t> stage[2];
    stage[0].reserve(c, SL_STAGE0, chunk_rows * row_bytes);
    stage[1].reserve(c, SL_STAGE1, chunk_rows * row_bytes);
    // the staging buffers were allocated on the main stream: order the copy stream after it
    CU_CHECK(cudaEventRecord(c->chunk_free[0], c->stream));
    CU_CHECK(cudaEventRecord(c->chunk_free[1], c->stream));
    int slot = 0;
    for (size_t r0 = 0; r0 < (size_t)n; r0 += chunk_rows, slot ^= 1) {
        const int rows = (int)std::min(chunk_rows, (size_t)n - r0);
        CU_CHECK(cudaStreamWaitEvent(c->copy_stream, c->chunk_free[slot], 0));
        CU_CHECK(cudaMemcpyAsync(stage[slot].p, reinterpret_cast<const uint8_t*>(X) + r0 * row_bytes,
                                 rows * row_bytes, cudaMemcpyHostToDevice, c->copy_stream));
        CU_CHECK(cudaEventRecord(c->copy_done[slot], c->copy_stream));
        CU_CHECK(cudaStreamWaitEvent(c->stream, c->copy_done[slot], 0));
        launch(c->stream, reinterpret_cast<const T*>(stage[slot].p), rows, row_offset + (int)r0);
        CU_CHECK(cudaEventRecord(c->chunk_free[slot], c->stream));
    }
}

// CSR rows (host or device) -> keys.  When both arrays are host memory the rows are streamed in
// chunks of about 32 MB of column ids through two pairs of device staging buffers, so that the
// copy of chunk i+1 overlaps the hashing of chunk i; a chunk's indptr entries keep their
// absolute values and the kernel is handed the staging address minus the chunk's first entry,
// so nothing has to be rebased.
void hash_csr(const culsh_index& ix, const KeySpec& ks, const int32_t* indices, const int32_t* indptr,
              int n, uint32_t* keys, int n_total, int row_offset) {
    const CtxPtr& c = ix.ctx;
    if (n == 0) return;
    const uint32_t* A = reinterpret_cast<const uint32_t*>(ix.params->p0.p);
    const uint32_t* B = reinterpret_cast<const uint32_t*>(ix.params->p1.p);
    const bool ptr_host = !is_device_pointer(indptr), idx_host = !is_device_pointer(indices);
    if (ptr_host && idx_host) {
        const int64_t nnz = indptr[n];
        if (nnz < 0) fail(CULSH_ERR_INVALID, "indptr[n] is negative");
        if (nnz > 0 && !indices) fail(CULSH_ERR_INVALID, "indices is null");
        const int64_t chunk_nnz = std::max<int64_t>(1 << 16, env_long_early("CULSH_CSR_CHUNK_NNZ", 8 << 20));
        // chunk boundaries: rows [r0, r1) with at most chunk_nnz entries (one row at least)
        std::vector<int> cuts{0};
        while (cuts.back() < n) {
            const int r0 = cuts.back();
            const int32_t* hi = std::upper_bound(indptr + r0 + 1, indptr + n + 1, (int32_t)std::min<int64_t>(
                                                     (int64_t)indptr[r0] + chunk_nnz, INT32_MAX));
            int r1 = (int)(hi - indptr) - 1;
            cuts.push_back(std::min(n, std::max(r1, r0 + 1)));
        }
        size_t max_rows = 0, max_nnz = 0;
        for (size_t i = 0; i + 1 < cuts.size(); ++i) {
            max_rows = std::max<size_t>(max_rows, (size_t)(cuts[i + 1] - cuts[i]));
            max_nnz = std::max<size_t>(max_nnz, (size_t)(indptr[cuts[i + 1]] - indptr[cuts[i]]));
        }
        Scratch<int32_t> st_idx[2], st_ptr[2];
        st_idx[0].reserve(c, SL_STAGE0, std::max<size_t>(max_nnz, 1));
        st_idx[1].reserve(c, SL_STAGE1, std::max<size_t>(max_nnz, 1));
        st_ptr[0].reserve(c, SL_CSR_INDPTR, max_rows + 1);
        st_ptr[1].reserve(c, SL_CSR_INDICES, max_rows + 1);
        CU_CHECK(cudaEventRecord(c->chunk_free[0], c->stream));
        CU_CHECK(cudaEventRecord(c->chunk_free[1], c->stream));
        int slot = 0;
        for (size_t i = 0; i + 1 < cuts.size(); ++i, slot ^= 1) {
            const int r0 = cuts[i], rows = cuts[i + 1] - r0;
            const int64_t e0 = indptr[r0], cnt = indptr[r0 + rows] - e0;
            if (cnt < 0) fail(CULSH_ERR_INVALID, "indptr is not ascending");
            CU_CHECK(cudaStreamWaitEvent(c->copy_stream, c->chunk_free[slot], 0));
            CU_CHECK(cudaMemcpyAsync(st_ptr[slot].p, indptr + r0, sizeof(int32_t) * ((size_t)rows + 1),
                                     cudaMemcpyHostToDevice, c->copy_stream));
            if (cnt)
                CU_CHECK(cudaMemcpyAsync(st_idx[slot].p, indices + e0, sizeof(int32_t) * (size_t)cnt,
                                         cudaMemcpyHostToDevice, c->copy_stream));
            CU_CHECK(cudaEventRecord(c->copy_done[slot], c->copy_stream));
            CU_CHECK(cudaStreamWaitEvent(c->stream, c->copy_done[slot], 0));
            // entry e of the chunk sits at st_idx[e - e0]: the kernel indexes with absolute values
            const int32_t* shifted = reinterpret_cast<const int32_t*>(
                reinterpret_cast<uintptr_t>(st_idx[slot].p) - (uintptr_t)e0 * sizeof(int32_t));
            launch_minhash(c, c->stream, shifted, st_ptr[slot].p, A, B, rows, ix.L, ix.k, ks, keys, n_total,
                           row_offset + r0);
            CU_CHECK(cudaEventRecord(c->chunk_free[slot], c->stream));
        }
        return;
    }
    Scratch<int32_t> d_indptr, d_indices;
    const int32_t* ip = indptr;
    const int32_t* ii = indices;
    if (ptr_host) {
        d_indptr.reserve(c, SL_CSR_INDPTR, (size_t)n + 1);
        CU_CHECK(cudaMemcpyAsync(d_indptr.p, indptr, sizeof(int32_t) * ((size_t)n + 1),
                                 cudaMemcpyHostToDevice, c->stream));
        ip = d_indptr.p;
    }
    if (idx_host) {
        int32_t nnz = 0;
        read_words(c, indptr + n, sizeof(int32_t), &nnz);  // indptr is on the device here
        if (nnz < 0) fail(CULSH_ERR_INVALID, "indptr[n] is negative");
        if (nnz > 0 && !indices) fail(CULSH_ERR_INVALID, "indices is null");
        d_indices.reserve(c, SL_CSR_INDICES, (size_t)nnz);
        if (nnz)
            CU_CHECK(cudaMemcpyAsync(d_indices.p, indices, sizeof(int32_t) * (size_t)nnz,
                                     cudaMemcpyHostToDevice, c->stream));
        ii = d_indices.p;
    }
    launch_minhash(c, c->stream, ii, ip, A, B, n, ix.L, ix.k, ks, keys, n_total, row_offset);
    // staging buffers are released in stream order after the kernel
}

// -----------------------------------------------------------------------------------------
// Index build from hashed keys
// -----------------------------------------------------------------------------------------
struct SortBuffers {
    Scratch<uint32_t> keys[2];
    uint32_t* vals[2] = {nullptr, nullptr};
    DevBuf<uint32_t> vals_out;   // receives the sorted row ids: becomes the index's candidate array
    Scratch<uint32_t> vals_tmp;
    Scratch<uint32_t> tile_hist;
    int final_buf = 0;
    // p-stable keys of one byte per hash (up to eight) may be sorted in compressed form
    static bool may_compress(const KeySpec& ks) {
        return ks.family == CULSH_PSLSH && ks.elem_bytes == 1 && ks.key_words <= 2 && ks.key_bytes >= 2;
    }
    void alloc(const CtxPtr& c, size_t items, const KeySpec& ks, int n, int L) {
        keys[0].reserve(c, SL_KEYS0, items * ks.key_words);
        keys[1].reserve(c, SL_KEYS1, items * ks.key_words);
        vals_out.alloc(c, items);
        vals_tmp.reserve(c, SL_VALS, items);
        tile_hist.reserve(c, SL_STATUS, radix_sort_tile_words(n, L, ks.key_words));
    }
    // one buffer flip per radix pass: the last pass must write the row ids into vals_out
    void set_passes(int passes) {
        final_buf = passes & 1;
        vals[final_buf] = vals_out.p;
        vals[final_buf ^ 1] = vals_tmp.p;
    }
};

// Sort + bucket construction.  On return ix holds cand/bucket arrays; if want_i2b the
// (row, table) -> bucket map is filled.  Returns the device error word read at the one
// host synchronisation of the build.
int build_index(culsh_index& ix, SortBuffers& sb, Scratch<int32_t>* item_to_bucket, StageTimer& tm) {
    const CtxPtr& c = ix.ctx;
    const int n = ix.n, L = ix.L, NW = ix.ks.key_words;
    HostTrace tr;
    // compressed sort (5 bits per hash) when the hash values span at most 32 levels
    bool compressed = false;
    KeyComp kc{0u, 0u};
    if (SortBuffers::may_compress(ix.ks) && !getenv("CULSH_SORT_PLAIN_KEYS")) {
        static const uint32_t init[2] = {0u, 256u};
        Scratch<uint32_t> range(c, SL_MISC1, 2);
        CU_CHECK(cudaMemcpyAsync(range.p, init, sizeof(init), cudaMemcpyHostToDevice, c->stream));
        const size_t n_words = (size_t)n * L * NW;
        key_byte_range_kernel<<<(unsigned)std::min<size_t>(ceil_div(n_words, 1024), (size_t)c->sm_count * 16), 256, 0,
                                c->stream>>>(sb.keys[0].p, n_words, range.p);
        KERNEL_CHECK();
        uint32_t r[2] = {0, 256};
        read_words(c, range.p, sizeof(r), r);
        const uint32_t n_pos = r[0] + 1, n_neg = 256 - r[1];
        if (n_pos + n_neg <= 32 && radix_sort_passes(ix.ks.key_bytes, true) < ix.ks.key_bytes) {
            compressed = true;
            kc.n_pos = n_pos;
            kc.sub = n_neg ? r[1] - n_pos : 0u;
        }
    }
    const int passes = radix_sort_passes(ix.ks.key_bytes, compressed);
    sb.set_passes(passes);
    uint32_t* kp[2] = {sb.keys[0].p, sb.keys[1].p};
    uint32_t* vp[2] = {sb.vals[0], sb.vals[1]};
    int cur = radix_sort_tables(c, NW, kp, vp, n, L, ix.ks.key_bytes, sb.tile_hist.p, compressed, kc);
    tm.mark();
    const int tpt = (int)ceil_div(n, IB_TILE);
    const size_t n_tiles = (size_t)tpt * L;
    Scratch<uint32_t> tile_heads(c, SL_TILE_HEADS, n_tiles), tile_base(c, SL_TILE_BASE, n_tiles + 1),
        scratch(c, SL_SCAN, scan_scratch_elems(n_tiles) * 2);
    CULSH_DISPATCH_NW(NW, launch_bucket_count<NW>(c->stream, kp[cur], n, L, tile_heads.p));
    exclusive_scan<uint32_t, uint32_t>(c->stream, tile_heads.p, n_tiles, tile_base.p, scratch.p);
    // the one host round trip of the build: bucket total + self-check word
    uint32_t B = 0;
    int err = 0;
    CU_CHECK(cudaMemcpyAsync(c->pinned, tile_base.p + n_tiles, sizeof(uint32_t), cudaMemcpyDeviceToHost, c->stream));
    CU_CHECK(cudaMemcpyAsync(c->pinned + 1, c->d_error, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    CU_CHECK(cudaStreamSynchronize(c->stream));
    std::memcpy(&B, c->pinned, sizeof(uint32_t));
    std::memcpy(&err, c->pinned + 1, sizeof(int));
    if (err) return err;
    tr.lap("sort+count+scan+sync");
    ix.n_buckets = (int)B;
    ix.bucket_keys.alloc(c, (size_t)B * NW);
    ix.bucket_offsets.alloc(c, (size_t)B + 1);
    ix.table_offsets.alloc(c, (size_t)L + 1);
    Scratch<int32_t> i2b_tm;  // (table, row) -> bucket, transposed to (row, table) below
    if (item_to_bucket) {
        item_to_bucket->reserve(c, SL_I2B, (size_t)n * L);
        i2b_tm.reserve(c, SL_I2B_TM, (size_t)n * L);
    }
    tr.lap("alloc bucket arrays");
    CULSH_DISPATCH_NW(NW, launch_bucket_write<NW>(c->stream, kp[cur], vp[cur], n, L, tile_base.p,
                                                  ix.bucket_keys.p, ix.bucket_offsets.p,
                                                  ix.table_offsets.p, i2b_tm.p));
    if (item_to_bucket) {
        dim3 grid((unsigned)ceil_div(n, 32), (unsigned)ceil_div(L, 32));
        transpose_table_major_kernel<<<grid, 256, 0, c->stream>>>(i2b_tm.p, n, L, item_to_bucket->p);
        KERNEL_CHECK();
    }
    // the sorted row ids are the candidate array: adopt the buffer
    static_assert(sizeof(int32_t) == sizeof(uint32_t), "");
    if (cur != sb.final_buf) fail(CULSH_ERR_INTERNAL, "radix sort ended in the scratch buffer");
    DevBuf<uint32_t>& v = sb.vals_out;
    ix.cand.p = reinterpret_cast<int32_t*>(v.p);
    ix.cand.n = v.n;
    ix.cand.ctx = v.ctx;
    ix.cand.big_cap = v.big_cap;
    v.p = nullptr;
    v.n = 0;
    v.big_cap = 0;
    tm.mark();
    c->stats.n_items = (uint64_t)n * L;
    c->stats.n_buckets = B;
    c->stats.sort_passes = passes;
    c->stats.key_words = NW;
    c->stats.elem_bytes = ix.ks.elem_bytes;
    return 0;
}

void validate_shape(int n, int d, int L, int k) {
    if (n <= 0) fail(CULSH_ERR_INVALID, "n_samples must be positive");
    if (d <= 0) fail(CULSH_ERR_INVALID, "n_features must be positive");
    if (L <= 0) fail(CULSH_ERR_INVALID, "n_hash_tables must be positive");
    if (k <= 0) fail(CULSH_ERR_INVALID, "n_hashes must be positive");
    if ((uint64_t)n * (uint64_t)L >= (1ull << 31))
        fail(CULSH_ERR_UNSUPPORTED, "n_samples * n_hash_tables must be below 2^31");
    if (n >= (1 << 30)) fail(CULSH_ERR_UNSUPPORTED, "n_samples must be below 2^30");
}

// Hash + sort + build.  `hash_fn(ks, keys)` fills the key array for a given key layout.
template <typename HashFn>
void fit_common(culsh_index& ix, HashFn&& hash_fn, Scratch<int32_t>* item_to_bucket) {
    const CtxPtr& c = ix.ctx;
    c->stats = culsh_stats{};
    c->stats.params_ms = c->last_params_ms;
    launch_counter() = 0;
    int eb = ix.family == CULSH_PSLSH ? 1 : (ix.family == CULSH_MINHASH ? 4 : 0);
    const size_t items = (size_t)ix.n * ix.L;
    while (true) {
        ix.ks = make_key_spec(ix.family, ix.k, eb);
        if (ix.ks.key_words < 0)
            fail(CULSH_ERR_UNSUPPORTED, "signature of %d hashes x %d bytes exceeds the 64-byte key limit",
                 ix.k, std::max(1, eb));
        StageTimer tm(c);
        SortBuffers sb;
        sb.alloc(c, items, ix.ks, ix.n, ix.L);
        reset_error_word(c);
        if (c->profiling) CU_CHECK(cudaMemsetAsync(c->d_mma, 0, 2 * sizeof(unsigned long long), c->stream));
        tm.mark();
        hash_fn(ix.ks, sb.keys[0].p);
        tm.mark();
        int err = build_index(ix, sb, item_to_bucket, tm);
        if (err & DEV_ERR_NARROW_OVERFLOW) {  // p-stable values do not fit: widen and redo
            if (eb >= 4) fail(CULSH_ERR_INTERNAL, "overflow reported at full width");
            eb *= 2;
            continue;
        }
        check_error_word(err);
        CU_CHECK(cudaStreamSynchronize(c->stream));  // the stage events must have completed
        c->stats.hash_ms = tm.between(0, 1);
        c->stats.sort_ms = tm.between(1, 2);
        c->stats.scatter_ms = tm.last_scatter();
        c->stats.build_ms = tm.between(2, 3);
        c->stats.total_ms = tm.between(0, 3);
        if (c->profiling && c->stats.hash_path == 1) {
            unsigned long long mma[2] = {0, 0};
            read_words(c, c->d_mma, sizeof(mma), mma);
            c->stats.hash_lo_fraction = mma[0] ? (float)((double)mma[1] / (double)mma[0]) : 0.f;
        }
        break;
    }
}

// -----------------------------------------------------------------------------------------
// Query from matched bucket ids (matched[q*L + t])
// -----------------------------------------------------------------------------------------
int bitmap_window_bits(const CtxPtr& c, int n_rows) {
    size_t fixed = bitmap_smem_bytes(0) + 1024;
    // a multiple of 4096 bits: the emission walks the window in 128-word groups
    size_t max_bits = ((c->smem_optin > fixed ? c->smem_optin - fixed : 0) * 8) / 4096 * 4096;
    size_t want = ((size_t)n_rows + 4095) / 4096 * 4096;
    static const size_t cap_bits = [] { const char* e = getenv("CULSH_BITMAP_BITS"); return e ? (size_t)atol(e) : ((size_t)1 << 20); }();
    size_t cap = std::min<size_t>(max_bits, cap_bits);
    return (int)std::min(want, cap);
}

// Tuning knobs of the chained kernel, read from the environment at every call (tests vary them):
//   CULSH_CHAIN_BITS    rows per window (default 344,064: bitmap and prefixes of three CTAs fit
//                       one SM); the row range is cut into the fewest such windows, each a
//                       multiple of 4096 rows
//   CULSH_CHAIN_STAGE   ids staged in shared memory per copy-out chunk; 0 (default) = no stage,
//                       every id is stored straight at its CSR position (measured on 1M rows x
//                       10k queries: 1.22 ms against 1.29 ms with a 5120-id stage and the 253,952-row
//                       windows that then fit)
//   CULSH_CHAIN_THREADS threads per CTA: 256, 384 (default) or 512
//   CULSH_CHAIN_LOADS   loads in flight per lane in the list walks: 4, 8 or 16 (default)
//   CULSH_CHAIN_SLICES  0 = CTAs search their list slices themselves (default 1: precomputed)
constexpr int CHAIN_MAX_WINDOWS = 8;
inline long env_long(const char* name, long dflt) {
    const char* e = getenv(name);
    return e && *e ? atol(e) : dflt;
}
int chain_window_bits(int n_rows, int* n_win) {
    const size_t cap_bits = std::max<size_t>(4096, (size_t)env_long("CULSH_CHAIN_BITS", 344064) / 4096 * 4096);
    const size_t n = (size_t)std::max(n_rows, 1);
    const size_t wins = ceil_div(n, cap_bits);
    *n_win = (int)std::min<size_t>(wins, 1u << 20);
    return (int)(ceil_div(ceil_div(n, wins), (size_t)4096) * 4096);
}

void query_from_matched(const culsh_index& ix, const int32_t* matched, int n_q, culsh_candidates& out,
                        StageTimer& tm) {
    const CtxPtr& c = ix.ctx;
    cudaStream_t s = c->stream;
    const int L = ix.L;
    HostTrace tr;
    bool dedupe_timed = false;
    out.ctx = c;
    out.n_queries = n_q;
    out.counts.alloc(c, (size_t)n_q);
    out.offsets.alloc(c, (size_t)n_q + 1);
    Scratch<uint64_t> raw_cnt(c, SL_RAW_CNT, n_q), raw_off(c, SL_RAW_OFF, (size_t)n_q + 1),
        scratch(c, SL_SCAN, scan_scratch_elems(n_q));
    Scratch<uint32_t> big_list(c, SL_BIG_LIST, 2 * (size_t)n_q), n_big(c, SL_NBIG, 2);
    uint32_t* mid_list = big_list.p + n_q;
    const int wbits = bitmap_window_bits(c, ix.n);
    // with more rows than two bitmap windows, mid-sized candidate sets are sorted in shared memory
    const int mid_max = (size_t)ix.n > 2 * (size_t)wbits ? MID_MAX : 0;
    CU_CHECK(cudaMemsetAsync(n_big.p, 0, 2 * sizeof(uint32_t), s));
    // The count pass keeps the list bounds it reads for the warp path (one coalesced read there
    // instead of two dependent scattered ones), when the table is worth it and fits 8 GB.
    Scratch<int2> bounds;
    const size_t pairs = (size_t)n_q * L;
    if (pairs >= ((size_t)1 << 22) && pairs <= ((size_t)1 << 30)) bounds.reserve(c, SL_BOUNDS, pairs);
    raw_count_kernel<<<(unsigned)ceil_div(n_q, 256), 256, 0, s>>>(matched, ix.bucket_offsets.p, n_q, L,
                                                                 raw_cnt.p, big_list.p, mid_list, n_big.p,
                                                                 mid_max, bounds.p);
    KERNEL_CHECK();
    exclusive_scan<uint64_t, uint64_t>(s, raw_cnt.p, n_q, raw_off.p, scratch.p);
    uint64_t raw_total = 0;
    uint32_t nb = 0, nm = 0;
    CU_CHECK(cudaMemcpyAsync(c->pinned, raw_off.p + n_q, sizeof(uint64_t), cudaMemcpyDeviceToHost, s));
    CU_CHECK(cudaMemcpyAsync(c->pinned + 1, n_big.p, 2 * sizeof(uint32_t), cudaMemcpyDeviceToHost, s));
    CU_CHECK(cudaStreamSynchronize(s));
    std::memcpy(&raw_total, c->pinned, sizeof(uint64_t));
    std::memcpy(&nb, c->pinned + 1, sizeof(uint32_t));
    std::memcpy(&nm, reinterpret_cast<const char*>(c->pinned + 1) + sizeof(uint32_t), sizeof(uint32_t));
    tr.lap("count+scan+sync");
    c->stats.raw_candidates += raw_total;
    if (raw_total == 0) {
        CU_CHECK(cudaMemsetAsync(out.counts.p, 0, out.counts.bytes(), s));
        CU_CHECK(cudaMemsetAsync(out.offsets.p, 0, out.offsets.bytes(), s));
        out.total = 0;
        CU_CHECK(cudaStreamSynchronize(s));
        return;
    }
    // Single pass (ids emitted at their final CSR position, no compaction) when most queries have
    // large candidate sets and the row range is a few chain windows; otherwise scratch + compaction.
    int n_win = 1;
    const int cbits = chain_window_bits(ix.n, &n_win);
    const long stage_env = env_long("CULSH_CHAIN_STAGE", 0);
    const int stage_ids = stage_env == 0 ? 0 : (int)std::min<long>(40960, std::max<long>(256, stage_env));
    const bool chained = n_win <= CHAIN_MAX_WINDOWS && L <= CW_MAX_L && (size_t)nb * 2 >= (size_t)n_q &&
                         (uint64_t)n_q * (uint64_t)n_win < (1ull << 31) &&
                         chain_window_smem_bytes(cbits, stage_ids) + 1024 <= c->smem_optin;
    const uint32_t n_other = (uint32_t)n_q - nb - nm;  // queries on the warp path (incl. empty ones)
    // Scratch copy of the ids of the queries that do not take the chained kernel (warp / sort
    // paths write it, indexed by raw offsets); the chained kernel reads it only for those, so a
    // query set that is all large sets (the 1M-row benchmark: 743 MB) needs none.
    Scratch<int32_t> tmp;
    if (!(chained && n_other == 0 && nm == 0)) tmp.reserve(c, SL_TMP, raw_total);
    tr.lap("alloc tmp");
    if (n_other) {
        size_t blocks = std::min<size_t>(ceil_div(n_q, SM_WARPS), (size_t)c->sm_count * 16);
        dedupe_small_kernel<<<(unsigned)blocks, SM_THREADS, 0, s>>>(
            matched, ix.bucket_offsets.p, ix.cand.p, raw_cnt.p, raw_off.p, n_q, L, tmp.p, out.counts.p, bounds.p);
        KERNEL_CHECK();
    }
    if (nm) {
        int id_bytes = 1;
        while (id_bytes < 4 && ((uint64_t)ix.n - 1) >> (8 * id_bytes)) ++id_bytes;
        size_t smem = sort_path_smem_bytes();
        CU_CHECK(cudaFuncSetAttribute(dedupe_sort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        dedupe_sort_kernel<<<nm, MS_THREADS, smem, s>>>(mid_list, matched, ix.bucket_offsets.p, ix.cand.p,
                                                       raw_cnt.p, raw_off.p, L, id_bytes, tmp.p, out.counts.p);
        KERNEL_CHECK();
    }
    if (chained) {
        out.indices.alloc(c, raw_total);  // capacity: the unique total is not known yet
        const size_t n_tk = (size_t)n_q * n_win;
        Scratch<unsigned long long> status(c, SL_CHAIN, n_tk + 1);
        uint32_t* ticket = reinterpret_cast<uint32_t*>(status.p + n_tk);
        CU_CHECK(cudaMemsetAsync(status.p, 0, sizeof(unsigned long long) * (n_tk + 1), s));
        // list slices per window, precomputed when the table is small enough (<= 256 MB)
        Scratch<int2> slices;
        if (env_long("CULSH_CHAIN_SLICES", 1) && n_win > 1 && n_tk * (size_t)L <= ((size_t)32 << 20)) {
            slices.reserve(c, SL_SLICES, n_tk * (size_t)L);
            slice_lists_kernel<<<(unsigned)ceil_div(n_tk * (size_t)L, 256), 256, 0, s>>>(
                matched, ix.bucket_offsets.p, ix.cand.p, raw_cnt.p, n_q, L, cbits, n_win, mid_max, slices.p);
            KERNEL_CHECK();
        }
        auto launch = [&](auto nt_tag, auto mk_tag) {
            constexpr int NT = decltype(nt_tag)::value;
            constexpr int MK = decltype(mk_tag)::value;
            const size_t smem = chain_window_smem_bytes(cbits, stage_ids);
            CU_CHECK(cudaFuncSetAttribute(dedupe_chained_rank_kernel<NT, MK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            CU_CHECK(cudaFuncSetAttribute(dedupe_chained_rank_kernel<NT, MK>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
            dedupe_chained_rank_kernel<NT, MK><<<(unsigned)n_tk, NT, smem, s>>>(
                matched, ix.bucket_offsets.p, ix.cand.p, raw_cnt.p, raw_off.p, n_q, L, ix.n, cbits, n_win, stage_ids,
                mid_max, slices.p, tmp.p, status.p, ticket, out.indices.p, out.counts.p, out.offsets.p, c->d_error);
        };
        const long cw_threads = env_long("CULSH_CHAIN_THREADS", 384);
        const long cw_mk = env_long("CULSH_CHAIN_LOADS", 16);
        if (c->profiling) cudaEventRecord(c->ev_dedupe[0], s);
        auto with_loads = [&](auto nt_tag) {
            if (cw_mk == 4) launch(nt_tag, std::integral_constant<int, 4>{});
            else if (cw_mk == 8) launch(nt_tag, std::integral_constant<int, 8>{});
            else launch(nt_tag, std::integral_constant<int, 16>{});
        };
        if (cw_threads == 512) with_loads(std::integral_constant<int, 512>{});
        else if (cw_threads == 256) with_loads(std::integral_constant<int, 256>{});
        else with_loads(std::integral_constant<int, 384>{});
        KERNEL_CHECK();
        if (c->profiling) { cudaEventRecord(c->ev_dedupe[1], s); dedupe_timed = true; }
        if (n_win > 1) {
            counts_from_offsets_kernel<<<(unsigned)ceil_div(n_q, 256), 256, 0, s>>>(out.offsets.p, n_q, out.counts.p);
            KERNEL_CHECK();
        }
        uint64_t total = 0;
        read_words(c, out.offsets.p + n_q, sizeof(uint64_t), &total);
        tr.lap("chained dedupe+sync");
        out.total = total;
        c->stats.unique_candidates += total;
        if (total == 0) {
            out.indices.release();
        } else if (total * 4 < raw_total * 3) {  // much smaller than the capacity: keep an exact copy
            DevBuf<int32_t> exact(c, total);
            CU_CHECK(cudaMemcpyAsync(exact.p, out.indices.p, sizeof(int32_t) * total, cudaMemcpyDeviceToDevice, s));
            out.indices = std::move(exact);
        }
    } else {
        if (nb) {
            size_t smem = bitmap_smem_bytes(wbits);
            CU_CHECK(cudaFuncSetAttribute(dedupe_bitmap_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            if (c->profiling) cudaEventRecord(c->ev_dedupe[0], s);
            dedupe_bitmap_kernel<<<nb, BM_THREADS, smem, s>>>(big_list.p, matched, ix.bucket_offsets.p,
                                                              ix.cand.p, raw_off.p, L, ix.n, wbits, tmp.p,
                                                              out.counts.p);
            KERNEL_CHECK();
            if (c->profiling) { cudaEventRecord(c->ev_dedupe[1], s); dedupe_timed = true; }
        }
        exclusive_scan<uint64_t, uint64_t>(s, out.counts.p, n_q, out.offsets.p, scratch.p);
        uint64_t total = 0;
        read_words(c, out.offsets.p + n_q, sizeof(uint64_t), &total);
        tr.lap("dedupe+scan+sync");
        out.total = total;
        c->stats.unique_candidates += total;
        if (total) {
            out.indices.alloc(c, total);
            tr.lap("alloc indices");
            size_t blocks = std::min<size_t>(ceil_div((size_t)n_q * 32, 256), (size_t)c->sm_count * 32);
            compact_small_kernel<<<(unsigned)blocks, 256, 0, s>>>(tmp.p, raw_cnt.p, raw_off.p, out.counts.p,
                                                                 out.offsets.p, n_q, out.indices.p);
            KERNEL_CHECK();
            if (nb) {
                compact_big_kernel<<<nb, 256, 0, s>>>(big_list.p, tmp.p, raw_off.p, out.counts.p,
                                                      out.offsets.p, out.indices.p);
                KERNEL_CHECK();
            }
            if (nm) {
                compact_big_kernel<<<nm, 256, 0, s>>>(mid_list, tmp.p, raw_off.p, out.counts.p,
                                                      out.offsets.p, out.indices.p);
                KERNEL_CHECK();
            }
        }
    }
    tm.mark();
    CU_CHECK(cudaStreamSynchronize(s));
    if (dedupe_timed) {
        float ms = 0.f;
        cudaEventElapsedTime(&ms, c->ev_dedupe[0], c->ev_dedupe[1]);
        c->stats.dedupe_ms += ms;
    }
    tr.lap("compact+sync");
}

// Hash a batch of queries, look the buckets up, gather + dedupe.
template <typename HashFn>
void query_batch(const culsh_index& ix, int n_q, HashFn&& hash_fn, culsh_candidates& out) {
    const CtxPtr& c = ix.ctx;
    const int NW = ix.ks.key_words;
    StageTimer tm(c);
    const size_t pairs = (size_t)n_q * ix.L;
    Scratch<uint32_t> qkeys(c, SL_QKEYS, pairs * NW);
    Scratch<uint8_t> ovf;
    if (ix.family == CULSH_PSLSH && ix.ks.elem_bytes < 4) ovf.reserve(c, SL_QOVF, pairs);
    Scratch<int32_t> matched(c, SL_MATCHED, pairs);
    tm.mark();
    hash_fn(ix.ks, qkeys.p, ovf.p);
    tm.mark();
    CULSH_DISPATCH_NW(NW, (lookup_kernel<NW><<<(unsigned)ceil_div(pairs, 256), 256, 0, c->stream>>>(
                              qkeys.p, ovf.p, n_q, ix.L, ix.bucket_keys.p, ix.table_offsets.p, matched.p)));
    KERNEL_CHECK();
    tm.mark();
    query_from_matched(ix, matched.p, n_q, out, tm);
    c->stats.hash_ms += tm.between(0, 1);
    c->stats.lookup_ms += tm.between(1, 2);
    c->stats.gather_ms += tm.between(2, 3);
    c->stats.total_ms += tm.between(0, 3);
}

// Concatenate batch results (linear, once): replaces the per-batch Candidates::merge of
// core/candidates.cuh:139-197.
void concat_candidates(const CtxPtr& c, std::vector<std::unique_ptr<culsh_candidates>>& parts,
                       culsh_candidates& out) {
    int nq = 0;
    uint64_t total = 0;
    for (auto& p : parts) { nq += p->n_queries; total += p->total; }
    out.ctx = c;
    out.n_queries = nq;
    out.total = total;
    out.counts.alloc(c, nq);
    out.offsets.alloc(c, (size_t)nq + 1);
    if (total) out.indices.alloc(c, total);
    int q0 = 0;
    uint64_t base = 0;
    for (auto& p : parts) {
        if (p->n_queries == 0) continue;
        CU_CHECK(cudaMemcpyAsync(out.counts.p + q0, p->counts.p, sizeof(uint64_t) * p->n_queries,
                                 cudaMemcpyDeviceToDevice, c->stream));
        size_t m = (size_t)p->n_queries + 1;
        shift_offsets_kernel<<<(unsigned)ceil_div(m, 256), 256, 0, c->stream>>>(p->offsets.p, m, base,
                                                                              out.offsets.p + q0);
        KERNEL_CHECK();
        if (p->total)
            CU_CHECK(cudaMemcpyAsync(out.indices.p + base, p->indices.p, sizeof(int32_t) * p->total,
                                     cudaMemcpyDeviceToDevice, c->stream));
        q0 += p->n_queries;
        base += p->total;
    }
    CU_CHECK(cudaStreamSynchronize(c->stream));
}

void empty_result(const CtxPtr& c, culsh_candidates& out) {
    out.ctx = c;
    out.n_queries = 0;
    out.total = 0;
    out.counts.alloc(c, 1);  // non-null so the object is not "empty" in upstream's sense
    out.offsets.alloc(c, 1);
    CU_CHECK(cudaMemsetAsync(out.offsets.p, 0, sizeof(uint64_t), c->stream));
    CU_CHECK(cudaStreamSynchronize(c->stream));
}

// -----------------------------------------------------------------------------------------
// Family front ends
// -----------------------------------------------------------------------------------------
void prepare_tc_split(culsh_index& ix) {
    if (ix.family == CULSH_MINHASH || ix.is_double || ix.params->p_split.p) return;
    prepare_project_tc(ix.ctx, reinterpret_cast<const float*>(ix.params->p0.p), ix.L * ix.k, ix.d, ix.L, ix.k, ix.params->p_split);
}

template <typename T>
std::unique_ptr<culsh_index> new_dense_index(culsh_handle* h, int family, int n, int d, int L, int k,
                                             int window, uint64_t seed) {
    validate_shape(n, d, L, k);
    if (family == CULSH_PSLSH && window <= 0) fail(CULSH_ERR_INVALID, "window_size must be positive");
    auto ix = std::make_unique<culsh_index>();
    ix->ctx = h->ctx;
    ix->family = family;
    ix->n = n; ix->d = d; ix->L = L; ix->k = k;
    ix->window = family == CULSH_PSLSH ? window : 0;
    ix->is_double = std::is_same<T, double>::value ? 1 : 0;
    ix->seed = seed;
    generate_params(*ix);
    prepare_tc_split(*ix);
    return ix;
}

template <typename T>
void fit_dense(culsh_handle* h, int family, const T* X, int n, int d, int L, int k, int window,
               uint64_t seed, culsh_index** out) {
    if (!h || !out) fail(CULSH_ERR_INVALID, "null handle or output pointer");
    if (!X) fail(CULSH_ERR_INVALID, "X is null");
    DeviceGuard g(h->ctx->device);
    auto ix = new_dense_index<T>(h, family, n, d, L, k, window, seed);
    fit_common(*ix, [&](const KeySpec& ks, uint32_t* keys) {
        hash_dense<T>(*ix, ks, X, n, keys, nullptr, n, 0);
    }, nullptr);
    CU_CHECK(cudaStreamSynchronize(h->ctx->stream));
    *out = ix.release();
}

template <typename T>
void fit_query_dense(culsh_handle* h, int family, const T* X, int n, int d, int L, int k, int window,
                     uint64_t seed, culsh_candidates** out) {
    if (!h || !out) fail(CULSH_ERR_INVALID, "null handle or output pointer");
    if (!X) fail(CULSH_ERR_INVALID, "X is null");
    DeviceGuard g(h->ctx->device);
    auto ix = new_dense_index<T>(h, family, n, d, L, k, window, seed);
    Scratch<int32_t> i2b;
    fit_common(*ix, [&](const KeySpec& ks, uint32_t* keys) {
        hash_dense<T>(*ix, ks, X, n, keys, nullptr, n, 0);
    }, &i2b);
    auto res = std::make_unique<culsh_candidates>();
    StageTimer tm(h->ctx);
    tm.mark();
    query_from_matched(*ix, i2b.p, n, *res, tm);
    h->ctx->stats.gather_ms = tm.between(0, 1);
    check_error_word(read_error_word(h->ctx));  // the gather's bounded waits report here
    *out = res.release();
}

template <typename T>
void query_dense(culsh_handle* h, int family, const T* Q, int n_q, const culsh_index* ix,
                 int batch_size, culsh_candidates** out) {
    if (!h || !out || !ix) fail(CULSH_ERR_INVALID, "null handle, index or output pointer");
    if (ix->family != family) fail(CULSH_ERR_INVALID, "index belongs to another LSH family");
    if (ix->ctx->device != h->ctx->device) fail(CULSH_ERR_INVALID, "index lives on another device");
    const bool want_double = std::is_same<T, double>::value;
    if (ix->is_double && !want_double)
        fail(CULSH_ERR_INVALID, "Index was fitted with float64, but query is float32");
    if (!ix->is_double && want_double)
        fail(CULSH_ERR_INVALID, "Index was fitted with float32, but query is float64");
    if (n_q < 0) fail(CULSH_ERR_INVALID, "n_queries must not be negative");
    DeviceGuard g(h->ctx->device);
    const CtxPtr& c = ix->ctx;
    c->stats = culsh_stats{};
    launch_counter() = 0;
    auto res = std::make_unique<culsh_candidates>();
    if (n_q == 0) {
        empty_result(c, *res);
        *out = res.release();
        return;
    }
    if (!Q) fail(CULSH_ERR_INVALID, "Q is null");
    if ((uint64_t)n_q * ix->L >= (1ull << 31) && (batch_size <= 0 || batch_size >= n_q))
        fail(CULSH_ERR_UNSUPPORTED, "n_queries * n_hash_tables must be below 2^31 per batch");
    reset_error_word(c);
    auto run = [&](const T* Qb, int nb, culsh_candidates& dst) {
        query_batch(*ix, nb, [&](const KeySpec& ks, uint32_t* keys, uint8_t* ovf) {
            hash_dense<T>(*ix, ks, Qb, nb, keys, ovf, nb, 0);
        }, dst);
    };
    if (batch_size <= 0 || batch_size >= n_q) {  // rplsh.cu:190-192
        run(Q, n_q, *res);
    } else {
        std::vector<std::unique_ptr<culsh_candidates>> parts;
        for (int s0 = 0; s0 < n_q; s0 += batch_size) {
            int nb = std::min(batch_size, n_q - s0);
            parts.emplace_back(new culsh_candidates());
            run(Q + (size_t)s0 * ix->d, nb, *parts.back());
        }
        concat_candidates(c, parts, *res);
    }
    check_error_word(read_error_word(c));
    *out = res.release();
}

std::unique_ptr<culsh_index> new_minhash_index(culsh_handle* h, int n, int d, int L, int k, uint64_t seed) {
    validate_shape(n, std::max(d, 1), L, k);
    auto ix = std::make_unique<culsh_index>();
    ix->ctx = h->ctx;
    ix->family = CULSH_MINHASH;
    ix->n = n; ix->d = d; ix->L = L; ix->k = k;
    ix->seed = seed;
    generate_params(*ix);
    return ix;
}


}  // namespace

// =========================================================================================
// C ABI
// =========================================================================================
extern "C" {

const char* culsh_last_error(void) { return g_last_error.c_str(); }

int culsh_create(int device, culsh_handle** out) {
    return guarded([&] {
        if (!out) fail(CULSH_ERR_INVALID, "out is null");
        int count = 0;
        CU_CHECK(cudaGetDeviceCount(&count));
        if (device < 0 || device >= count) fail(CULSH_ERR_INVALID, "no CUDA device %d (have %d)", device, count);
        DeviceGuard g(device);
        auto c = std::make_shared<Ctx>();
        c->device = device;
        CU_CHECK(cudaStreamCreate(&c->stream));  // blocking stream, as upstream (cuda_utils.cuh:38)
        CU_CHECK(cudaStreamCreateWithFlags(&c->copy_stream, cudaStreamNonBlocking));
        for (auto& e : c->ev) CU_CHECK(cudaEventCreate(&e));
        for (auto& e : c->ev_pass) CU_CHECK(cudaEventCreate(&e));
        for (auto& e : c->ev_dedupe) CU_CHECK(cudaEventCreate(&e));
        for (auto& e : c->copy_done) CU_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        for (auto& e : c->chunk_free) CU_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        CU_CHECK(cudaMallocHost(&c->pinned, 64 * sizeof(uint64_t)));
        CU_CHECK(cudaMalloc(&c->d_error, sizeof(int)));
        CU_CHECK(cudaMemset(c->d_error, 0, sizeof(int)));
        CU_CHECK(cudaMalloc(&c->d_mma, 2 * sizeof(unsigned long long)));
        CU_CHECK(cudaMemset(c->d_mma, 0, 2 * sizeof(unsigned long long)));
        cudaDeviceProp prop{};
        CU_CHECK(cudaGetDeviceProperties(&prop, device));
        c->sm_count = prop.multiProcessorCount;
        c->smem_optin = prop.sharedMemPerBlockOptin;
        // keep freed blocks in the stream-ordered pool instead of returning them to the driver
        cudaMemPool_t pool;
        CU_CHECK(cudaDeviceGetDefaultMemPool(&pool, device));
        uint64_t thresh = UINT64_MAX;
        CU_CHECK(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thresh));
        auto h = new culsh_handle();
        h->ctx = c;
        *out = h;
    });
}

int culsh_destroy(culsh_handle* h) {
    return guarded([&] {
        if (h) h->ctx->param_cache.clear();  // the cached sets hold references to the context
        delete h;
    });
}

int culsh_get_stats(const culsh_handle* h, culsh_stats* out) {
    return guarded([&] {
        if (!h || !out) fail(CULSH_ERR_INVALID, "null argument");
        *out = h->ctx->stats;
        out->launches = launch_counter();
    });
}

int culsh_set_profiling(culsh_handle* h, int enabled) {
    return guarded([&] {
        if (!h) fail(CULSH_ERR_INVALID, "null handle");
        h->ctx->profiling = enabled != 0;
    });
}

int culsh_set_param_cache(culsh_handle* h, int enabled) {
    return guarded([&] {
        if (!h) fail(CULSH_ERR_INVALID, "null handle");
        h->ctx->param_cache_enabled = enabled != 0;
        if (!enabled) h->ctx->param_cache.clear();
    });
}

int culsh_trim_scratch(culsh_handle* h, uint64_t keep_bytes) {
    return guarded([&] {
        if (!h) fail(CULSH_ERR_INVALID, "null handle");
        const CtxPtr& c = h->ctx;
        DeviceGuard g(c->device);
        CU_CHECK(cudaStreamSynchronize(c->stream));
        CU_CHECK(cudaStreamSynchronize(c->copy_stream));
        for (int i = 0; i < SL_COUNT; ++i) {
            if (c->slot_ptr[i] && c->slot_cap[i] > keep_bytes) {
                CU_CHECK(cudaFree(c->slot_ptr[i]));
                c->slot_ptr[i] = nullptr;
                c->slot_cap[i] = 0;
            }
        }
        for (auto it = c->big_free.begin(); it != c->big_free.end();) {
            if (it->cap > keep_bytes) {
                c->big_free_bytes -= it->cap;
                CU_CHECK(cudaFree(it->p));
                it = c->big_free.erase(it);
            } else {
                ++it;
            }
        }
    });
}

int culsh_set_projection_path(culsh_handle* h, int path) {
    return guarded([&] {
        if (!h) fail(CULSH_ERR_INVALID, "null handle");
        if (path < 0 || path > 2) fail(CULSH_ERR_INVALID, "path must be 0, 1 or 2");
        h->ctx->projection_path = path;
    });
}

// ---- RPLSH ------------------------------------------------------------------------------
int culsh_rplsh_fit_f32(culsh_handle* h, const float* X, int n, int d, int L, int k, uint64_t seed,
                        culsh_index** out) {
    return guarded([&] { fit_dense<float>(h, CULSH_RPLSH, X, n, d, L, k, 0, seed, out); });
}
int culsh_rplsh_fit_f64(culsh_handle* h, const double* X, int n, int d, int L, int k, uint64_t seed,
                        culsh_index** out) {
    return guarded([&] { fit_dense<double>(h, CULSH_RPLSH, X, n, d, L, k, 0, seed, out); });
}
int culsh_rplsh_query_f32(culsh_handle* h, const float* Q, int n_q, const culsh_index* ix, int batch,
                          culsh_candidates** out) {
    return guarded([&] { query_dense<float>(h, CULSH_RPLSH, Q, n_q, ix, batch, out); });
}
int culsh_rplsh_query_f64(culsh_handle* h, const double* Q, int n_q, const culsh_index* ix, int batch,
                          culsh_candidates** out) {
    return guarded([&] { query_dense<double>(h, CULSH_RPLSH, Q, n_q, ix, batch, out); });
}
int culsh_rplsh_fit_query_f32(culsh_handle* h, const float* X, int n, int d, int L, int k,
                              uint64_t seed, culsh_candidates** out) {
    return guarded([&] { fit_query_dense<float>(h, CULSH_RPLSH, X, n, d, L, k, 0, seed, out); });
}
int culsh_rplsh_fit_query_f64(culsh_handle* h, const double* X, int n, int d, int L, int k,
                              uint64_t seed, culsh_candidates** out) {
    return guarded([&] { fit_query_dense<double>(h, CULSH_RPLSH, X, n, d, L, k, 0, seed, out); });
}

// ---- PSLSH ------------------------------------------------------------------------------
int culsh_pslsh_fit_f32(culsh_handle* h, const float* X, int n, int d, int L, int k, int w,
                        uint64_t seed, culsh_index** out) {
    return guarded([&] { fit_dense<float>(h, CULSH_PSLSH, X, n, d, L, k, w, seed, out); });
}
int culsh_pslsh_fit_f64(culsh_handle* h, const double* X, int n, int d, int L, int k, int w,
                        uint64_t seed, culsh_index** out) {
    return guarded([&] { fit_dense<double>(h, CULSH_PSLSH, X, n, d, L, k, w, seed, out); });
}
int culsh_pslsh_query_f32(culsh_handle* h, const float* Q, int n_q, const culsh_index* ix, int batch,
                          culsh_candidates** out) {
    return guarded([&] { query_dense<float>(h, CULSH_PSLSH, Q, n_q, ix, batch, out); });
}
int culsh_pslsh_query_f64(culsh_handle* h, const double* Q, int n_q, const culsh_index* ix, int batch,
                          culsh_candidates** out) {
    return guarded([&] { query_dense<double>(h, CULSH_PSLSH, Q, n_q, ix, batch, out); });
}
int culsh_pslsh_fit_query_f32(culsh_handle* h, const float* X, int n, int d, int L, int k, int w,
                              uint64_t seed, culsh_candidates** out) {
    return guarded([&] { fit_query_dense<float>(h, CULSH_PSLSH, X, n, d, L, k, w, seed, out); });
}
int culsh_pslsh_fit_query_f64(culsh_handle* h, const double* X, int n, int d, int L, int k, int w,
                              uint64_t seed, culsh_candidates** out) {
    return guarded([&] { fit_query_dense<double>(h, CULSH_PSLSH, X, n, d, L, k, w, seed, out); });
}

// ---- MinHash ----------------------------------------------------------------------------
int culsh_minhash_fit(culsh_handle* h, const int32_t* indices, const int32_t* indptr, int n, int d,
                      int L, int k, uint64_t seed, culsh_index** out) {
    return guarded([&] {
        if (!h || !out) fail(CULSH_ERR_INVALID, "null handle or output pointer");
        if (!indptr) fail(CULSH_ERR_INVALID, "indptr is null");
        DeviceGuard g(h->ctx->device);
        auto ix = new_minhash_index(h, n, d, L, k, seed);
        fit_common(*ix, [&](const KeySpec& ks, uint32_t* keys) {
            hash_csr(*ix, ks, indices, indptr, n, keys, n, 0);
        }, nullptr);
        CU_CHECK(cudaStreamSynchronize(h->ctx->stream));
        *out = ix.release();
    });
}

int culsh_minhash_query(culsh_handle* h, const int32_t* indices, const int32_t* indptr, int n_q,
                        const culsh_index* ix, culsh_candidates** out) {
    return guarded([&] {
        if (!h || !out || !ix) fail(CULSH_ERR_INVALID, "null handle, index or output pointer");
        if (ix->family != CULSH_MINHASH) fail(CULSH_ERR_INVALID, "index belongs to another LSH family");
        if (n_q < 0) fail(CULSH_ERR_INVALID, "n_queries must not be negative");
        DeviceGuard g(h->ctx->device);
        const CtxPtr& c = ix->ctx;
        c->stats = culsh_stats{};
        launch_counter() = 0;
        auto res = std::make_unique<culsh_candidates>();
        if (n_q == 0) {
            empty_result(c, *res);
            *out = res.release();
            return;
        }
        if (!indptr) fail(CULSH_ERR_INVALID, "indptr is null");
        if ((uint64_t)n_q * ix->L >= (1ull << 31))
            fail(CULSH_ERR_UNSUPPORTED, "n_queries * n_hash_tables must be below 2^31");
        reset_error_word(c);
        query_batch(*ix, n_q, [&](const KeySpec& ks, uint32_t* keys, uint8_t*) {
            hash_csr(*ix, ks, indices, indptr, n_q, keys, n_q, 0);
        }, *res);
        check_error_word(read_error_word(c));
        *out = res.release();
    });
}

int culsh_minhash_fit_query(culsh_handle* h, const int32_t* indices, const int32_t* indptr, int n,
                            int d, int L, int k, uint64_t seed, culsh_candidates** out) {
    return guarded([&] {
        if (!h || !out) fail(CULSH_ERR_INVALID, "null handle or output pointer");
        if (!indptr) fail(CULSH_ERR_INVALID, "indptr is null");
        DeviceGuard g(h->ctx->device);
        auto ix = new_minhash_index(h, n, d, L, k, seed);
        Scratch<int32_t> i2b;
        fit_common(*ix, [&](const KeySpec& ks, uint32_t* keys) {
            hash_csr(*ix, ks, indices, indptr, n, keys, n, 0);
        }, &i2b);
        auto res = std::make_unique<culsh_candidates>();
        StageTimer tm(h->ctx);
        tm.mark();
        query_from_matched(*ix, i2b.p, n, *res, tm);
        h->ctx->stats.gather_ms = tm.between(0, 1);
        check_error_word(read_error_word(h->ctx));  // the gather's bounded waits report here
        *out = res.release();
    });
}

// ---- signatures only --------------------------------------------------------------------
static void unpack_and_copy(const CtxPtr& c, const uint32_t* keys, size_t count, const KeySpec& ks,
                            void* dst) {
    Scratch<uint8_t> raw(c, SL_MISC0, count * ks.sig_nbytes);
    unpack_keys_kernel<<<(unsigned)ceil_div(count, 256), 256, 0, c->stream>>>(
        keys, count, ks.family, ks.n_hashes, ks.key_words, ks.elem_bytes, raw.p);
    KERNEL_CHECK();
    copy_out(c, dst, raw.p, raw.bytes());
}

int culsh_index_hash_dense(culsh_handle* h, const culsh_index* ix, const void* X, int n_rows,
                           void* sig_out) {
    return guarded([&] {
        if (!h || !ix || !X || !sig_out) fail(CULSH_ERR_INVALID, "null argument");
        if (ix->family == CULSH_MINHASH) fail(CULSH_ERR_INVALID, "use culsh_index_hash_csr for MinHash");
        if (n_rows <= 0) fail(CULSH_ERR_INVALID, "n_rows must be positive");
        DeviceGuard g(h->ctx->device);
        const CtxPtr& c = ix->ctx;
        KeySpec ks = make_key_spec(ix->family, ix->k, 4);  // full-width elements: nothing saturates
        if (ks.key_words < 0) fail(CULSH_ERR_UNSUPPORTED, "signature wider than 64 bytes");
        size_t items = (size_t)n_rows * ix->L;
        Scratch<uint32_t> keys(c, SL_KEYS0, items * ks.key_words);
        if (ix->is_double)
            hash_dense<double>(*ix, ks, static_cast<const double*>(X), n_rows, keys.p, nullptr, n_rows, 0, true);
        else
            hash_dense<float>(*ix, ks, static_cast<const float*>(X), n_rows, keys.p, nullptr, n_rows, 0, true);
        unpack_and_copy(c, keys.p, items, ks, sig_out);
    });
}

int culsh_index_hash_csr(culsh_handle* h, const culsh_index* ix, const int32_t* indices,
                         const int32_t* indptr, int n_rows, void* sig_out) {
    return guarded([&] {
        if (!h || !ix || !indptr || !sig_out) fail(CULSH_ERR_INVALID, "null argument");
        if (ix->family != CULSH_MINHASH) fail(CULSH_ERR_INVALID, "index is not a MinHash index");
        if (n_rows <= 0) fail(CULSH_ERR_INVALID, "n_rows must be positive");
        DeviceGuard g(h->ctx->device);
        const CtxPtr& c = ix->ctx;
        size_t items = (size_t)n_rows * ix->L;
        Scratch<uint32_t> keys(c, SL_KEYS0, items * ix->ks.key_words);
        hash_csr(*ix, ix->ks, indices, indptr, n_rows, keys.p, n_rows, 0);
        unpack_and_copy(c, keys.p, items, ix->ks, sig_out);
    });
}

// ---- packed keys in and out: the sharded self-join ships signatures, not rows -------------
int culsh_index_row_keys(culsh_handle* h, const culsh_index* ix, uint32_t* keys_out) {
    return guarded([&] {
        if (!h || !ix || !keys_out) fail(CULSH_ERR_INVALID, "null argument");
        if (!is_device_pointer(keys_out)) fail(CULSH_ERR_INVALID, "keys_out must be device memory");
        DeviceGuard g(h->ctx->device);
        const CtxPtr& c = ix->ctx;
        if (ix->n_buckets > 0) {
            CULSH_DISPATCH_NW(ix->ks.key_words,
                              (row_keys_kernel<NW><<<(unsigned)ceil_div(ix->n_buckets, 256), 256, 0, c->stream>>>(
                                  ix->bucket_keys.p, ix->bucket_offsets.p, ix->cand.p, ix->n_buckets, ix->n, keys_out)));
            KERNEL_CHECK();
        }
        CU_CHECK(cudaStreamSynchronize(c->stream));
    });
}

int culsh_index_query_keys(culsh_handle* h, const culsh_index* ix, const uint32_t* keys, int n_q,
                           culsh_candidates** out) {
    return guarded([&] {
        if (!h || !ix || !out) fail(CULSH_ERR_INVALID, "null handle, index or output pointer");
        if (ix->ctx->device != h->ctx->device) fail(CULSH_ERR_INVALID, "index lives on another device");
        if (n_q < 0) fail(CULSH_ERR_INVALID, "n_queries must not be negative");
        DeviceGuard g(h->ctx->device);
        const CtxPtr& c = ix->ctx;
        c->stats = culsh_stats{};
        launch_counter() = 0;
        auto res = std::make_unique<culsh_candidates>();
        if (n_q == 0) {
            empty_result(c, *res);
            *out = res.release();
            return;
        }
        if (!keys || !is_device_pointer(keys)) fail(CULSH_ERR_INVALID, "keys must be device memory");
        if ((uint64_t)n_q * ix->L >= (1ull << 31))
            fail(CULSH_ERR_UNSUPPORTED, "n_queries * n_hash_tables must be below 2^31 per call");
        reset_error_word(c);
        const int NW = ix->ks.key_words;
        const size_t pairs = (size_t)n_q * ix->L;
        StageTimer tm(c);
        Scratch<int32_t> matched(c, SL_MATCHED, pairs);
        tm.mark();
        CULSH_DISPATCH_NW(NW, (lookup_kernel<NW><<<(unsigned)ceil_div(pairs, 256), 256, 0, c->stream>>>(
                                  keys, nullptr, n_q, ix->L, ix->bucket_keys.p, ix->table_offsets.p, matched.p)));
        KERNEL_CHECK();
        tm.mark();
        query_from_matched(*ix, matched.p, n_q, *res, tm);
        c->stats.lookup_ms = tm.between(0, 1);
        c->stats.gather_ms = tm.between(1, 2);
        c->stats.total_ms = tm.between(0, 2);
        check_error_word(read_error_word(c));
        c->stats.launches = launch_counter();
        *out = res.release();
    });
}

// ---- Index getters / loaders ------------------------------------------------------------
int culsh_index_get_meta(const culsh_index* ix, culsh_index_meta* m) {
    return guarded([&] {
        if (!ix || !m) fail(CULSH_ERR_INVALID, "null argument");
        std::memset(m, 0, sizeof(*m));
        m->family = ix->family;
        m->n_total_candidates = (int32_t)((size_t)ix->n * ix->L);
        m->n_total_buckets = ix->n_buckets;
        m->n_hash_tables = ix->L;
        m->n_hashes = ix->k;
        m->sig_nbytes = ix->ks.sig_nbytes;
        m->n_features = ix->d;
        m->is_double = ix->is_double;
        m->window_size = ix->window;
        m->n_samples = ix->n;
        m->key_words = ix->ks.key_words;
        m->elem_bytes = ix->ks.elem_bytes;
        m->seed = ix->seed;
        // core/index.cuh:148-165 plus the family parameters (rplsh/index.cuh, pslsh/index.cuh,
        // minhash/index.cuh size_bytes), in upstream's layout
        uint64_t sz = ((uint64_t)ix->n_buckets + 1) * 4 + ((uint64_t)ix->L + 1) * 4 +
                      (uint64_t)ix->n_buckets * ix->ks.sig_nbytes + (uint64_t)ix->n * ix->L * 4;
        sz += ix->params->p0.bytes() + ix->params->p1.bytes();
        m->size_bytes = sz;
    });
}

int culsh_index_get_candidate_indices(const culsh_index* ix, int32_t* dst) {
    return guarded([&] {
        if (!ix) fail(CULSH_ERR_INVALID, "null index");
        DeviceGuard g(ix->ctx->device);
        copy_out(ix->ctx, dst, ix->cand.p, ix->cand.bytes());
    });
}
int culsh_index_get_bucket_signatures(const culsh_index* ix, uint8_t* dst) {
    return guarded([&] {
        if (!ix) fail(CULSH_ERR_INVALID, "null index");
        DeviceGuard g(ix->ctx->device);
        if (ix->n_buckets) unpack_and_copy(ix->ctx, ix->bucket_keys.p, (size_t)ix->n_buckets, ix->ks, dst);
    });
}
int culsh_index_get_bucket_candidate_offsets(const culsh_index* ix, int32_t* dst) {
    return guarded([&] {
        if (!ix) fail(CULSH_ERR_INVALID, "null index");
        DeviceGuard g(ix->ctx->device);
        copy_out(ix->ctx, dst, ix->bucket_offsets.p, ix->bucket_offsets.bytes());
    });
}
int culsh_index_get_table_bucket_offsets(const culsh_index* ix, int32_t* dst) {
    return guarded([&] {
        if (!ix) fail(CULSH_ERR_INVALID, "null index");
        DeviceGuard g(ix->ctx->device);
        copy_out(ix->ctx, dst, ix->table_offsets.p, ix->table_offsets.bytes());
    });
}
int culsh_index_get_projection(const culsh_index* ix, void* dst) {
    return guarded([&] {
        if (!ix) fail(CULSH_ERR_INVALID, "null index");
        if (ix->family == CULSH_MINHASH) fail(CULSH_ERR_INVALID, "MinHash index has no projection");
        DeviceGuard g(ix->ctx->device);
        copy_out(ix->ctx, dst, ix->params->p0.p, ix->params->p0.bytes());
    });
}
int culsh_index_get_bias(const culsh_index* ix, void* dst) {
    return guarded([&] {
        if (!ix) fail(CULSH_ERR_INVALID, "null index");
        if (ix->family != CULSH_PSLSH) fail(CULSH_ERR_INVALID, "only a p-stable index has a bias");
        DeviceGuard g(ix->ctx->device);
        copy_out(ix->ctx, dst, ix->params->p1.p, ix->params->p1.bytes());
    });
}
int culsh_index_get_hash_a(const culsh_index* ix, uint32_t* dst) {
    return guarded([&] {
        if (!ix) fail(CULSH_ERR_INVALID, "null index");
        if (ix->family != CULSH_MINHASH) fail(CULSH_ERR_INVALID, "not a MinHash index");
        DeviceGuard g(ix->ctx->device);
        copy_out(ix->ctx, dst, ix->params->p0.p, ix->params->p0.bytes());
    });
}
int culsh_index_get_hash_b(const culsh_index* ix, uint32_t* dst) {
    return guarded([&] {
        if (!ix) fail(CULSH_ERR_INVALID, "null index");
        if (ix->family != CULSH_MINHASH) fail(CULSH_ERR_INVALID, "not a MinHash index");
        DeviceGuard g(ix->ctx->device);
        copy_out(ix->ctx, dst, ix->params->p1.p, ix->params->p1.bytes());
    });
}

int culsh_index_load(culsh_handle* h, int family, int is_double, const int32_t* candidate_indices,
                     const uint8_t* bucket_signatures, const int32_t* bucket_candidate_offsets,
                     const int32_t* table_bucket_offsets, const void* param0, const void* param1,
                     int n_total_candidates, int n_total_buckets, int L, int k, int sig_nbytes,
                     int n_features, int window_size, uint64_t seed, culsh_index** out) {
    return guarded([&] {
        if (!h || !out) fail(CULSH_ERR_INVALID, "null handle or output pointer");
        if (family < CULSH_RPLSH || family > CULSH_MINHASH) fail(CULSH_ERR_INVALID, "unknown family");
        if (L <= 0 || k <= 0 || n_total_candidates <= 0 || n_total_buckets <= 0)
            fail(CULSH_ERR_INVALID, "index dimensions must be positive");
        if (n_total_candidates % L != 0)
            fail(CULSH_ERR_INVALID, "n_total_candidates is not a multiple of n_hash_tables");
        const int expect_sig = family == CULSH_RPLSH ? k : 4 * k;
        if (sig_nbytes != expect_sig)
            fail(CULSH_ERR_INVALID, "sig_nbytes=%d does not match n_hashes=%d for this family", sig_nbytes, k);
        if (!candidate_indices || !bucket_signatures || !bucket_candidate_offsets ||
            !table_bucket_offsets || !param0)
            fail(CULSH_ERR_INVALID, "null array");
        if (family != CULSH_RPLSH && !param1) fail(CULSH_ERR_INVALID, "second parameter array is null");
        if (family != CULSH_MINHASH && n_features <= 0) fail(CULSH_ERR_INVALID, "n_features must be positive");
        DeviceGuard g(h->ctx->device);
        const CtxPtr& c = h->ctx;
        cudaStream_t s = c->stream;
        auto ix = std::make_unique<culsh_index>();
        ix->ctx = c;
        ix->family = family;
        ix->L = L; ix->k = k; ix->d = n_features;
        ix->n = n_total_candidates / L;
        ix->window = family == CULSH_PSLSH ? window_size : 0;
        ix->is_double = family == CULSH_MINHASH ? 0 : (is_double ? 1 : 0);
        ix->seed = seed;
        ix->n_buckets = n_total_buckets;
        const size_t B = (size_t)n_total_buckets;
        ix->cand.alloc(c, (size_t)n_total_candidates);
        ix->bucket_offsets.alloc(c, B + 1);
        ix->table_offsets.alloc(c, (size_t)L + 1);
        CU_CHECK(cudaMemcpyAsync(ix->cand.p, candidate_indices, ix->cand.bytes(), cudaMemcpyDefault, s));
        CU_CHECK(cudaMemcpyAsync(ix->bucket_offsets.p, bucket_candidate_offsets, ix->bucket_offsets.bytes(), cudaMemcpyDefault, s));
        CU_CHECK(cudaMemcpyAsync(ix->table_offsets.p, table_bucket_offsets, ix->table_offsets.bytes(), cudaMemcpyDefault, s));
        const int H = L * k;
        if (family == CULSH_MINHASH) {
            ix->params->p0.alloc(c, sizeof(uint32_t) * H);
            ix->params->p1.alloc(c, sizeof(uint32_t) * H);
        } else {
            const size_t esz = ix->is_double ? 8 : 4;
            ix->params->p0.alloc(c, esz * H * n_features);
            if (family == CULSH_PSLSH) ix->params->p1.alloc(c, esz * H);
        }
        CU_CHECK(cudaMemcpyAsync(ix->params->p0.p, param0, ix->params->p0.bytes(), cudaMemcpyDefault, s));
        if (ix->params->p1.n) CU_CHECK(cudaMemcpyAsync(ix->params->p1.p, param1, ix->params->p1.bytes(), cudaMemcpyDefault, s));
        // raw signatures -> packed keys (p-stable: narrowest element width that holds them)
        Scratch<uint8_t> raw(c, SL_MISC0, B * sig_nbytes);
        CU_CHECK(cudaMemcpyAsync(raw.p, bucket_signatures, raw.bytes(), cudaMemcpyDefault, s));
        int eb = family == CULSH_MINHASH ? 4 : 0;
        if (family == CULSH_PSLSH) {
            Scratch<int> width(c, SL_MISC1, 1);
            int one = 1;
            CU_CHECK(cudaMemcpyAsync(width.p, &one, sizeof(int), cudaMemcpyHostToDevice, s));
            size_t cnt = B * k;
            pslsh_width_kernel<<<(unsigned)ceil_div(cnt, 256), 256, 0, s>>>(
                reinterpret_cast<const int32_t*>(raw.p), cnt, width.p);
            KERNEL_CHECK();
            read_words(c, width.p, sizeof(int), &eb);
            while (eb < 4 && round_key_words(k * eb) < 0) eb *= 2;
        }
        ix->ks = make_key_spec(family, k, eb);
        if (ix->ks.key_words < 0) fail(CULSH_ERR_UNSUPPORTED, "signature wider than the 64-byte key limit");
        ix->bucket_keys.alloc(c, B * ix->ks.key_words);
        pack_keys_kernel<<<(unsigned)ceil_div(B, 256), 256, 0, s>>>(raw.p, B, family, k, ix->ks.key_words,
                                                                   ix->ks.elem_bytes, ix->bucket_keys.p);
        KERNEL_CHECK();
        prepare_tc_split(*ix);
        CU_CHECK(cudaStreamSynchronize(s));
        *out = ix.release();
    });
}

void culsh_index_free(culsh_index* ix) {
    if (!ix) return;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(ix->ctx->device);
    delete ix;
    if (prev >= 0) cudaSetDevice(prev);
}

// ---- Candidates -------------------------------------------------------------------------
int culsh_candidates_get_meta(const culsh_candidates* c, int32_t* n_queries, uint64_t* total,
                              int32_t* is_empty) {
    return guarded([&] {
        if (!c) fail(CULSH_ERR_INVALID, "null candidates");
        if (n_queries) *n_queries = c->n_queries;
        if (total) *total = c->total;
        if (is_empty) *is_empty = c->empty() ? 1 : 0;
    });
}
int culsh_candidates_get_indices(const culsh_candidates* c, int32_t* dst) {
    return guarded([&] {
        if (!c) fail(CULSH_ERR_INVALID, "null candidates");
        DeviceGuard g(c->ctx->device);
        copy_out(c->ctx, dst, c->indices.p, sizeof(int32_t) * c->total);
    });
}
int culsh_candidates_get_counts(const culsh_candidates* c, uint64_t* dst) {
    return guarded([&] {
        if (!c) fail(CULSH_ERR_INVALID, "null candidates");
        DeviceGuard g(c->ctx->device);
        copy_out(c->ctx, dst, c->counts.p, sizeof(uint64_t) * (size_t)c->n_queries);
    });
}
int culsh_candidates_get_offsets(const culsh_candidates* c, uint64_t* dst) {
    return guarded([&] {
        if (!c) fail(CULSH_ERR_INVALID, "null candidates");
        DeviceGuard g(c->ctx->device);
        copy_out(c->ctx, dst, c->offsets.p, sizeof(uint64_t) * ((size_t)c->n_queries + 1));
    });
}
int culsh_candidates_device_ptrs(const culsh_candidates* c, const int32_t** indices,
                                 const uint64_t** counts, const uint64_t** offsets) {
    return guarded([&] {
        if (!c) fail(CULSH_ERR_INVALID, "null candidates");
        if (indices) *indices = c->indices.p;
        if (counts) *counts = c->counts.p;
        if (offsets) *offsets = c->offsets.p;
    });
}
void culsh_candidates_free(culsh_candidates* c) {
    if (!c) return;
    int prev = -1;
    cudaGetDevice(&prev);
    if (c->ctx) cudaSetDevice(c->ctx->device);
    delete c;
    if (prev >= 0) cudaSetDevice(prev);
}

// ---- pinned host buffers ----------------------------------------------------------------
int culsh_host_alloc(size_t bytes, void** out) {
    return guarded([&] {
        if (!out || bytes == 0) fail(CULSH_ERR_INVALID, "bad argument");
        void* p = nullptr;
        cudaError_t e = cudaHostAlloc(&p, bytes, cudaHostAllocPortable);
        if (e != cudaSuccess) {
            cudaGetLastError();
            fail(CULSH_ERR_ALLOC, "pinned host allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        }
        *out = p;
    });
}

int culsh_host_free(void* p) {
    return guarded([&] {
        if (p) CU_CHECK(cudaFreeHost(p));
    });
}

// ---- peer memory ------------------------------------------------------------------------
int culsh_peer_alloc(culsh_handle* h, size_t bytes, void** dptr, unsigned char handle[64]) {
    return guarded([&] {
        if (!h || !dptr || !handle || bytes == 0) fail(CULSH_ERR_INVALID, "bad argument");
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
        DeviceGuard g(h->ctx->device);
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, bytes);
        if (e != cudaSuccess) {
            cudaGetLastError();
            fail(CULSH_ERR_ALLOC, "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        }
        cudaIpcMemHandle_t ih;
        e = cudaIpcGetMemHandle(&ih, p);
        if (e != cudaSuccess) {
            cudaFree(p);
            cudaGetLastError();
            fail(CULSH_ERR_CUDA, "cudaIpcGetMemHandle failed: %s", cudaGetErrorString(e));
        }
        std::memcpy(handle, &ih, 64);
        *dptr = p;
    });
}

int culsh_peer_free(culsh_handle* h, void* dptr) {
    return guarded([&] {
        if (!h) fail(CULSH_ERR_INVALID, "null handle");
        DeviceGuard g(h->ctx->device);
        if (dptr) CU_CHECK(cudaFree(dptr));
    });
}

int culsh_peer_open(culsh_handle* h, const unsigned char handle[64], void** dptr) {
    return guarded([&] {
        if (!h || !handle || !dptr) fail(CULSH_ERR_INVALID, "bad argument");
        DeviceGuard g(h->ctx->device);
        cudaIpcMemHandle_t ih;
        std::memcpy(&ih, handle, 64);
        void* p = nullptr;
        CU_CHECK(cudaIpcOpenMemHandle(&p, ih, cudaIpcMemLazyEnablePeerAccess));
        *dptr = p;
    });
}

int culsh_peer_close(culsh_handle* h, void* dptr) {
    return guarded([&] {
        if (!h) fail(CULSH_ERR_INVALID, "null handle");
        DeviceGuard g(h->ctx->device);
        if (dptr) CU_CHECK(cudaIpcCloseMemHandle(dptr));
    });
}

int culsh_device_copy(culsh_handle* h, void* dst, const void* src, size_t bytes) {
    return guarded([&] {
        if (!h) fail(CULSH_ERR_INVALID, "null handle");
        if (bytes == 0) return;
        if (!dst || !src) fail(CULSH_ERR_INVALID, "null pointer");
        DeviceGuard g(h->ctx->device);
        CU_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, h->ctx->stream));
        CU_CHECK(cudaStreamSynchronize(h->ctx->stream));
    });
}

// ---- shard merge ------------------------------------------------------------------------
int culsh_merge_shard_candidates(culsh_handle* h, int n_shards, int n_q,
                                 const int32_t* const* shard_indices,
                                 const uint64_t* const* shard_offsets, const int64_t* row_base,
                                 culsh_candidates** out) {
    return guarded([&] {
        if (!h || !out || !shard_indices || !shard_offsets || !row_base)
            fail(CULSH_ERR_INVALID, "null argument");
        if (n_shards <= 0 || n_q < 0) fail(CULSH_ERR_INVALID, "bad shard or query count");
        DeviceGuard g(h->ctx->device);
        const CtxPtr& c = h->ctx;
        cudaStream_t s = c->stream;
        HostTrace tr;
        auto res = std::make_unique<culsh_candidates>();
        if (n_q == 0) {
            empty_result(c, *res);
            *out = res.release();
            return;
        }
        Scratch<const int32_t*> d_idx(c, SL_MISC0, n_shards);
        Scratch<const uint64_t*> d_off(c, SL_MISC1, n_shards);
        Scratch<int64_t> d_base(c, SL_MISC2, n_shards);
        CU_CHECK(cudaMemcpyAsync(d_idx.p, shard_indices, sizeof(void*) * n_shards, cudaMemcpyHostToDevice, s));
        CU_CHECK(cudaMemcpyAsync(d_off.p, shard_offsets, sizeof(void*) * n_shards, cudaMemcpyHostToDevice, s));
        CU_CHECK(cudaMemcpyAsync(d_base.p, row_base, sizeof(int64_t) * n_shards, cudaMemcpyHostToDevice, s));
        res->ctx = c;
        res->n_queries = n_q;
        res->counts.alloc(c, n_q);
        res->offsets.alloc(c, (size_t)n_q + 1);
        Scratch<uint64_t> scratch(c, SL_SCAN, scan_scratch_elems(n_q));
        shard_counts_kernel<<<(unsigned)ceil_div(n_q, 256), 256, 0, s>>>(d_off.p, n_shards, n_q, res->counts.p);
        KERNEL_CHECK();
        exclusive_scan<uint64_t, uint64_t>(s, res->counts.p, n_q, res->offsets.p, scratch.p);
        uint64_t total = 0;
        read_words(c, res->offsets.p + n_q, sizeof(uint64_t), &total);
        tr.lap("merge: tables+counts+scan+sync");
        res->total = total;
        if (total) {
            res->indices.alloc(c, total);
            tr.lap("merge: alloc indices");
            if (total / (uint64_t)n_q >= 512) {  // long lists: a CTA per query
                size_t blocks = std::min<size_t>((size_t)n_q, (size_t)c->sm_count * 8);
                shard_interleave_kernel<<<(unsigned)blocks, 256, 0, s>>>(d_idx.p, d_off.p, d_base.p, n_shards,
                                                                        n_q, res->offsets.p, res->indices.p);
            } else {
                size_t blocks = std::min<size_t>(ceil_div((size_t)n_q * 32, 256), (size_t)c->sm_count * 32);
                shard_interleave_small_kernel<<<(unsigned)blocks, 256, 0, s>>>(
                    d_idx.p, d_off.p, d_base.p, n_shards, n_q, res->offsets.p, res->indices.p);
            }
            KERNEL_CHECK();
        }
        CU_CHECK(cudaStreamSynchronize(s));
        tr.lap("merge: interleave+sync");
        *out = res.release();
    });
}

// ---- shard exchange, push form -----------------------------------------------------------
int culsh_exchange_plan(culsh_handle* h, int n_ranks, int rank, int n_q, const uint64_t* counts_all,
                        uint64_t* dstpos, uint64_t* slice_totals, culsh_candidates** out) {
    return guarded([&] {
        if (!h || !counts_all || !dstpos || !slice_totals || !out) fail(CULSH_ERR_INVALID, "null argument");
        if (n_ranks <= 0 || n_ranks > 64 || rank < 0 || rank >= n_ranks || n_q <= 0)
            fail(CULSH_ERR_INVALID, "bad rank, rank count (1..64) or query count");
        DeviceGuard g(h->ctx->device);
        const CtxPtr& c = h->ctx;
        cudaStream_t s = c->stream;
        const int per = (int)ceil_div(n_q, n_ranks);
        const int my_lo = std::min(n_q, rank * per), my_hi = std::min(n_q, my_lo + per);
        auto res = std::make_unique<culsh_candidates>();
        res->ctx = c;
        res->n_queries = my_hi - my_lo;
        res->counts.alloc(c, (size_t)std::max(1, my_hi - my_lo));
        res->offsets.alloc(c, (size_t)(my_hi - my_lo) + 1);
        Scratch<uint64_t> merged(c, SL_RAW_CNT, n_q), before(c, SL_MISC0, n_q), S(c, SL_RAW_OFF, (size_t)n_q + 1),
            scratch(c, SL_SCAN, scan_scratch_elems(n_q)), totals(c, SL_MISC1, n_ranks);
        exchange_counts_kernel<<<(unsigned)ceil_div(n_q, 256), 256, 0, s>>>(counts_all, n_ranks, rank, n_q, merged.p, before.p);
        KERNEL_CHECK();
        exclusive_scan<uint64_t, uint64_t>(s, merged.p, n_q, S.p, scratch.p);
        exchange_positions_kernel<<<(unsigned)ceil_div((size_t)std::max(n_q + 1, n_ranks), 256), 256, 0, s>>>(
            S.p, merged.p, before.p, n_q, per, n_ranks, my_lo, my_hi, dstpos, res->counts.p, res->offsets.p, totals.p);
        KERNEL_CHECK();
        read_words(c, totals.p, sizeof(uint64_t) * n_ranks, slice_totals);
        res->total = slice_totals[rank];
        *out = res.release();
    });
}

int culsh_exchange_push(culsh_handle* h, int n_ranks, int rank, int n_q, const int32_t* indices, const uint64_t* offsets,
                        const uint64_t* dstpos, void* const* recv, int64_t row_base, uint64_t total) {
    return guarded([&] {
        if (!h || !offsets || !dstpos || !recv) fail(CULSH_ERR_INVALID, "null argument");
        if (n_ranks <= 0 || n_ranks > 64 || rank < 0 || rank >= n_ranks || n_q <= 0)
            fail(CULSH_ERR_INVALID, "bad rank count (1..64), rank or query count");
        DeviceGuard g(h->ctx->device);
        const CtxPtr& c = h->ctx;
        cudaStream_t s = c->stream;
        if (total) {
            if (!indices) fail(CULSH_ERR_INVALID, "indices is null");
            Scratch<int32_t*> d_recv(c, SL_MISC2, n_ranks);
            CU_CHECK(cudaMemcpyAsync(d_recv.p, recv, sizeof(void*) * n_ranks, cudaMemcpyHostToDevice, s));
            const int per = (int)ceil_div(n_q, n_ranks);
            if (total / (uint64_t)n_q >= 512) {
                size_t blocks = std::min<size_t>((size_t)n_q, (size_t)c->sm_count * 8);
                shard_push_kernel<<<(unsigned)blocks, 256, 0, s>>>(indices, offsets, dstpos, d_recv.p, per, n_q, n_ranks, rank, (int32_t)row_base);
            } else {
                size_t blocks = std::min<size_t>(ceil_div((size_t)n_q * 32, 256), (size_t)c->sm_count * 32);
                shard_push_small_kernel<<<(unsigned)blocks, 256, 0, s>>>(indices, offsets, dstpos, d_recv.p, per, n_q, n_ranks, rank, (int32_t)row_base);
            }
            KERNEL_CHECK();
        }
        CU_CHECK(cudaStreamSynchronize(s));
    });
}

int culsh_candidates_attach_indices(culsh_candidates* cd, const int32_t* indices, uint64_t total) {
    return guarded([&] {
        if (!cd) fail(CULSH_ERR_INVALID, "null candidates");
        if (total && !indices) fail(CULSH_ERR_INVALID, "indices is null");
        cd->indices.release();
        cd->indices.p = const_cast<int32_t*>(indices);  // borrowed: no context, so release() frees nothing
        cd->indices.n = total;
        cd->indices.ctx = nullptr;
        cd->total = total;
    });
}

// ---- shard merge without any allocation -------------------------------------------------
// Scratch of the allocation-free merge: the three per-shard tables (pointers and row bases)
// and the block sums of the offset scan.  It is a fixed part of the module image, so every
// GPU that loads the library carries these 32 KB until the process exits.
constexpr int NOALLOC_MAX_SHARDS = 64;
constexpr int NOALLOC_MAX_QUERIES = 1 << 22;
constexpr size_t NOALLOC_TABLE_BYTES = 512;  // one table: 64 entries of 8 bytes
constexpr size_t NOALLOC_SCAN_OFFSET = 2048;
constexpr size_t NOALLOC_SCRATCH_BYTES = 32768;
static_assert(NOALLOC_SCAN_OFFSET + (NOALLOC_MAX_QUERIES / SCAN_TILE + 2) * sizeof(uint64_t) <= NOALLOC_SCRATCH_BYTES,
              "scan block sums must fit the static scratch");
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];
static void* g_noalloc_scratch_addr[64] = {};  // device address of the array, per device ordinal

int culsh_merge_shard_candidates_noalloc(culsh_handle* h, int n_shards, int n_q,
                                         const int32_t* const* shard_indices,
                                         const uint64_t* const* shard_offsets, const int64_t* row_base,
                                         int32_t* out_indices, uint64_t out_capacity, uint64_t* out_counts,
                                         uint64_t* out_offsets, uint64_t* total_out) {
    return guarded([&] {
        if (!h || !shard_indices || !shard_offsets || !row_base || !out_counts || !out_offsets || !total_out)
            fail(CULSH_ERR_INVALID, "null argument");
        if (n_shards <= 0 || n_q < 0) fail(CULSH_ERR_INVALID, "bad shard or query count");
        if (n_shards > NOALLOC_MAX_SHARDS)
            fail(CULSH_ERR_UNSUPPORTED, "allocation-free merge takes at most %d shards (got %d)",
                 NOALLOC_MAX_SHARDS, n_shards);
        if (n_q > NOALLOC_MAX_QUERIES)
            fail(CULSH_ERR_UNSUPPORTED, "allocation-free merge takes at most %d queries (got %d)",
                 NOALLOC_MAX_QUERIES, n_q);
        const CtxPtr& c = h->ctx;
        if (c->device < 0 || c->device >= 64) fail(CULSH_ERR_UNSUPPORTED, "device ordinal out of range");
        DeviceGuard g(c->device);
        cudaStream_t s = c->stream;
        // Set-up, once per device and with that device current: in host code the array's name is
        // only a handle for the runtime, the kernels need its address in device memory.
        if (!g_noalloc_scratch_addr[c->device]) {
            void* addr = nullptr;
            CU_CHECK(cudaGetSymbolAddress(&addr, g_noalloc_scratch));
            g_noalloc_scratch_addr[c->device] = addr;
        }
        unsigned char* base = static_cast<unsigned char*>(g_noalloc_scratch_addr[c->device]);
        *total_out = 0;
        if (n_q == 0) {
            CU_CHECK(cudaMemsetAsync(out_offsets, 0, sizeof(uint64_t), s));
            CU_CHECK(cudaStreamSynchronize(s));
            return;
        }
        auto** d_idx = reinterpret_cast<const int32_t**>(base);
        auto** d_off = reinterpret_cast<const uint64_t**>(base + NOALLOC_TABLE_BYTES);
        auto* d_base = reinterpret_cast<int64_t*>(base + 2 * NOALLOC_TABLE_BYTES);
        auto* d_sums = reinterpret_cast<uint64_t*>(base + NOALLOC_SCAN_OFFSET);
        // every scratch word read below is written first by these copies or by the scan's own
        // reduce step, so nothing has to be cleared between calls
        CU_CHECK(cudaMemcpyAsync(d_idx, shard_indices, sizeof(void*) * n_shards, cudaMemcpyHostToDevice, s));
        CU_CHECK(cudaMemcpyAsync(d_off, shard_offsets, sizeof(void*) * n_shards, cudaMemcpyHostToDevice, s));
        CU_CHECK(cudaMemcpyAsync(d_base, row_base, sizeof(int64_t) * n_shards, cudaMemcpyHostToDevice, s));
        shard_counts_kernel<<<(unsigned)ceil_div(n_q, 256), 256, 0, s>>>(d_off, n_shards, n_q, out_counts);
        KERNEL_CHECK();
        exclusive_scan<uint64_t, uint64_t>(s, out_counts, n_q, out_offsets, d_sums);
        uint64_t total = 0;
        read_words(c, out_offsets + n_q, sizeof(uint64_t), &total);
        *total_out = total;
        if (total > out_capacity)
            fail(CULSH_ERR_INVALID, "out_indices holds %llu ids but the merged result has %llu",
                 (unsigned long long)out_capacity, (unsigned long long)total);
        if (total) {
            if (!out_indices) fail(CULSH_ERR_INVALID, "out_indices is null");
            size_t blocks = std::min<size_t>(ceil_div((size_t)n_q * 32, 256), (size_t)c->sm_count * 32);
            shard_interleave_small_kernel<<<(unsigned)blocks, 256, 0, s>>>(d_idx, d_off, d_base, n_shards, n_q,
                                                                          out_offsets, out_indices);
            KERNEL_CHECK();
        }
        CU_CHECK(cudaStreamSynchronize(s));
    });
}

}  // extern "C"
