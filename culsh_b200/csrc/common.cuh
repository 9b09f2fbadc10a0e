// Shared host/device helpers: error plumbing, the per-handle context, stream-ordered
// buffers and the key layout description.
#pragma once

#include <cuda_runtime.h>
#include <curand.h>
#include <curand_kernel.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

#include "../../include/culsh_b200.h"

namespace culsh_b200 {

// ---------------------------------------------------------------------------------------
// Errors: host code throws Error, the C ABI catches it and returns the status code.
// ---------------------------------------------------------------------------------------
struct Error : public std::runtime_error {
    int status;
    Error(int s, const std::string& m) : std::runtime_error(m), status(s) {}
};

[[noreturn]] inline void fail(int status, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    throw Error(status, buf);
}

#define CU_CHECK(call)                                                                      \
    do {                                                                                    \
        cudaError_t e__ = (call);                                                           \
        if (e__ != cudaSuccess)                                                             \
            ::culsh_b200::fail(e__ == cudaErrorMemoryAllocation ? CULSH_ERR_ALLOC           \
                                                                : CULSH_ERR_CUDA,           \
                               "%s failed: %s (%s:%d)", #call, cudaGetErrorString(e__),     \
                               __FILE__, __LINE__);                                         \
    } while (0)

#define CURAND_CHECK(call)                                                                  \
    do {                                                                                    \
        curandStatus_t s__ = (call);                                                        \
        if (s__ != CURAND_STATUS_SUCCESS)                                                   \
            ::culsh_b200::fail(CULSH_ERR_CUDA, "%s failed: curand status %d (%s:%d)", #call, \
                               (int)s__, __FILE__, __LINE__);                               \
    } while (0)

// counts this library's kernel launches (reported per call in culsh_stats.launches)
inline int& launch_counter() {
    static thread_local int n = 0;
    return n;
}
#define KERNEL_CHECK()                     \
    do {                                   \
        ++::culsh_b200::launch_counter();  \
        CU_CHECK(cudaGetLastError());      \
    } while (0)

inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------------------------------
// Key layout.  A signature of one (row, table) is held as NW 32-bit words, word 0 most
// significant, so that comparing the words as unsigned integers in order equals the
// unsigned byte-lexicographic order of upstream's raw signature memory
// (core/fit.cuh:265-282, core/query.cuh:44-48):
//   RPLSH   : k sign bits, hash 0 as the most significant bit, right-aligned.
//   PSLSH   : for each hash its low `elem_bytes` bytes in little-endian order (the
//             remaining bytes of the int32 are sign extension, so they never decide a
//             comparison once every stored value fits the narrow width).
//   MinHash : bswap32 of each uint32 hash (elem_bytes = 4).
// key_bytes counts the significant bytes (the radix passes); unused leading bytes are 0.
// ---------------------------------------------------------------------------------------
struct KeySpec {
    int family = 0;
    int n_hashes = 0;
    int elem_bytes = 0;  // RPLSH: 0 (bit-packed)
    int key_bytes = 0;
    int key_words = 0;   // NW, one of 1, 2, 4, 8, 16
    int sig_nbytes = 0;  // upstream's raw width
};

inline int round_key_words(int bytes) {
    int w = (bytes + 3) / 4;
    if (w <= 1) return 1;
    if (w <= 2) return 2;
    if (w <= 4) return 4;
    if (w <= 8) return 8;
    if (w <= 16) return 16;
    return -1;
}

inline KeySpec make_key_spec(int family, int k, int elem_bytes) {
    KeySpec s;
    s.family = family;
    s.n_hashes = k;
    if (family == CULSH_RPLSH) {
        s.elem_bytes = 0;
        s.key_bytes = (k + 7) / 8;
        s.sig_nbytes = k;
    } else {
        s.elem_bytes = (family == CULSH_MINHASH) ? 4 : elem_bytes;
        s.key_bytes = k * s.elem_bytes;
        s.sig_nbytes = k * 4;
    }
    s.key_words = round_key_words(s.key_bytes);
    return s;
}

// ---------------------------------------------------------------------------------------
// Context behind a handle: device, stream, a pinned scratch block for small D2H reads,
// staging buffers for host inputs, cached hash parameters.
// ---------------------------------------------------------------------------------------
struct ParamKey {
    int family, H, d, window, is_double;
    uint64_t seed;
    bool operator<(const ParamKey& o) const {
        return std::tie(family, H, d, window, is_double, seed) <
               std::tie(o.family, o.H, o.d, o.window, o.is_double, o.seed);
    }
};

// Scratch slots: every temporary of the pipeline has its own grow-only device buffer that
// lives as long as the handle, so steady-state calls allocate nothing for temporaries and
// the stream-ordered pool only ever sees the (repeating) sizes of results.
enum ScratchSlot {
    SL_STAGE0, SL_STAGE1, SL_CSR_INDPTR, SL_CSR_INDICES, SL_KEYS0, SL_KEYS1, SL_VALS, SL_GHIST,
    SL_STATUS, SL_COUNTER, SL_TILE_HEADS, SL_TILE_BASE, SL_SCAN, SL_RAW_CNT, SL_RAW_OFF,
    SL_BIG_LIST, SL_NBIG, SL_TMP, SL_QKEYS, SL_QOVF, SL_MATCHED, SL_I2B, SL_MISC0, SL_MISC1,
    SL_MISC2, SL_CHAIN, SL_SLICES, SL_I2B_TM, SL_BOUNDS, SL_COUNT
};

struct Ctx {
    int device = 0;
    // hash parameters already generated on this handle (they depend only on the key): the
    // cuRAND generator set-up costs more than a tenth of a 1M-row fit
    std::map<ParamKey, std::shared_ptr<void>> param_cache;
    bool param_cache_enabled = true;
    float last_params_ms = 0.f;       // host wall time of the last parameter generation (0: cache hit)
    curandGenerator_t curand = nullptr;  // created on first use, re-seeded per parameter set
    void* slot_ptr[SL_COUNT] = {};
    size_t slot_cap[SL_COUNT] = {};
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t ev[8] = {};
    cudaEvent_t ev_pass[2] = {};      // around the scatter launch of the last radix pass
    cudaEvent_t ev_dedupe[2] = {};    // around the chained / bitmap dedupe launch of the last query batch
    cudaEvent_t copy_done[2] = {};
    cudaEvent_t chunk_free[2] = {};
    uint64_t* pinned = nullptr;       // 64 x u64 words of pinned host memory
    int* d_error = nullptr;           // device-side self-check word
    unsigned long long* d_mma = nullptr;  // tensor-core projection: K-blocks issued / with the low-part MMA
    bool profiling = false;
    int projection_path = 0;
    culsh_stats stats{};
    int sm_count = 148;
    size_t smem_optin = 0;
    // Large result / index blocks (>= BIG_BLOCK_MIN bytes) that were released: kept here and handed
    // out again by size instead of going through the stream-ordered pool, where small short-lived
    // allocations between two large ones fragment the reserve and send the next large request
    // to the driver (milliseconds once peers have the device mapped).
    struct BigBlock { void* p; size_t cap; };
    std::vector<BigBlock> big_free;
    size_t big_free_bytes = 0;

    ~Ctx() {
        cudaSetDevice(device);
        if (stream) cudaStreamSynchronize(stream);
        if (curand) curandDestroyGenerator(curand);
        for (auto& e : ev) if (e) cudaEventDestroy(e);
        for (auto& e : ev_pass) if (e) cudaEventDestroy(e);
        for (auto& e : ev_dedupe) if (e) cudaEventDestroy(e);
        for (auto& e : copy_done) if (e) cudaEventDestroy(e);
        for (auto& e : chunk_free) if (e) cudaEventDestroy(e);
        if (copy_stream) cudaStreamSynchronize(copy_stream);
        for (auto& q : slot_ptr) if (q) cudaFree(q);
        for (auto& b : big_free) cudaFree(b.p);
        if (pinned) cudaFreeHost(pinned);
        if (d_error) cudaFree(d_error);
        if (d_mma) cudaFree(d_mma);
        if (copy_stream) cudaStreamDestroy(copy_stream);
        if (stream) cudaStreamDestroy(stream);
    }
};
using CtxPtr = std::shared_ptr<Ctx>;

constexpr size_t BIG_BLOCK_MIN = (size_t)32 << 20;       // requests from this size on use the block list
constexpr size_t BIG_BLOCK_KEEP = (size_t)16 << 30;      // at most this many released bytes are kept
constexpr size_t BIG_BLOCK_KEEP_COUNT = 8;

// Takes a released block that fits (no more than twice the request), else allocates one.
inline void* big_block_alloc(Ctx& c, size_t bytes, size_t* cap_out) {
    size_t best = c.big_free.size();
    for (size_t i = 0; i < c.big_free.size(); ++i) {
        const size_t cap = c.big_free[i].cap;
        if (cap >= bytes && cap <= 2 * bytes && (best == c.big_free.size() || cap < c.big_free[best].cap)) best = i;
    }
    if (best < c.big_free.size()) {
        Ctx::BigBlock b = c.big_free[best];
        c.big_free.erase(c.big_free.begin() + (long)best);
        c.big_free_bytes -= b.cap;
        *cap_out = b.cap;
        return b.p;
    }
    const size_t cap = (bytes + ((size_t)2 << 20) - 1) & ~(((size_t)2 << 20) - 1);
    void* q = nullptr;
    cudaError_t e = cudaMalloc(&q, cap);
    if (e != cudaSuccess && !c.big_free.empty()) {  // give the kept blocks back and try once more
        cudaGetLastError();
        for (auto& b : c.big_free) cudaFree(b.p);
        c.big_free.clear();
        c.big_free_bytes = 0;
        e = cudaMalloc(&q, cap);
    }
    if (e != cudaSuccess) {
        cudaGetLastError();
        fail(CULSH_ERR_ALLOC, "device allocation of %zu bytes failed: %s", cap, cudaGetErrorString(e));
    }
    *cap_out = cap;
    return q;
}

// The block may still be in use by work queued on the handle's stream; whoever takes it next
// uses it on the same stream, so the order of the stream protects it.  Blocks beyond the keep
// limits go back to the driver (oldest first; cudaFree waits for the device).
inline void big_block_release(Ctx& c, void* p, size_t cap) {
    c.big_free.push_back(Ctx::BigBlock{p, cap});
    c.big_free_bytes += cap;
    while (c.big_free.size() > BIG_BLOCK_KEEP_COUNT || c.big_free_bytes > BIG_BLOCK_KEEP) {
        Ctx::BigBlock b = c.big_free.front();
        c.big_free.erase(c.big_free.begin());
        c.big_free_bytes -= b.cap;
        cudaFree(b.p);
    }
}

// Device buffer owned by a result or index object: small ones come from the stream-ordered
// pool (cudaMallocAsync on the context's stream; the pool keeps freed blocks, so steady-state
// calls do not reach the driver allocator), large ones from the handle's block list.
template <typename T>
struct DevBuf {
    T* p = nullptr;
    size_t n = 0;
    CtxPtr ctx;
    size_t big_cap = 0;  // non-zero: a block of the handle's block list with this capacity
    DevBuf() = default;
    DevBuf(const CtxPtr& c, size_t count) { alloc(c, count); }
    DevBuf(const DevBuf&) = delete;
    DevBuf& operator=(const DevBuf&) = delete;
    DevBuf(DevBuf&& o) noexcept : p(o.p), n(o.n), ctx(std::move(o.ctx)), big_cap(o.big_cap) {
        o.p = nullptr; o.n = 0; o.big_cap = 0;
    }
    DevBuf& operator=(DevBuf&& o) noexcept {
        if (this != &o) {
            release();
            p = o.p; n = o.n; ctx = std::move(o.ctx); big_cap = o.big_cap;
            o.p = nullptr; o.n = 0; o.big_cap = 0;
        }
        return *this;
    }
    ~DevBuf() { release(); }
    void alloc(const CtxPtr& c, size_t count) {
        release();
        ctx = c;
        n = count;
        if (count == 0) return;
        const size_t bytes = count * sizeof(T);
        if (bytes >= BIG_BLOCK_MIN) {
            p = static_cast<T*>(big_block_alloc(*c, bytes, &big_cap));
            return;
        }
        void* q = nullptr;
        cudaError_t e = cudaMallocAsync(&q, bytes, c->stream);
        if (e != cudaSuccess) {
            cudaGetLastError();
            fail(CULSH_ERR_ALLOC, "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
        }
        p = static_cast<T*>(q);
    }
    void release() {
        if (p && ctx) {
            int cur = -1;
            cudaGetDevice(&cur);
            if (cur != ctx->device) cudaSetDevice(ctx->device);
            if (big_cap) big_block_release(*ctx, p, big_cap);
            else cudaFreeAsync(p, ctx->stream);
            if (cur != ctx->device && cur >= 0) cudaSetDevice(cur);
        }
        p = nullptr;
        n = 0;
        big_cap = 0;
    }
    size_t bytes() const { return n * sizeof(T); }
};

// Temporary in a scratch slot of the handle (see ScratchSlot).  Two live Scratch objects must
// not share a slot.  Growing a slot waits for the handle's streams, frees the old block and
// allocates the new size; contents are not preserved.
template <typename T>
struct Scratch {
    T* p = nullptr;
    size_t n = 0;
    Scratch() = default;
    Scratch(const CtxPtr& c, ScratchSlot slot, size_t count) { reserve(c, slot, count); }
    void reserve(const CtxPtr& c, ScratchSlot slot, size_t count) {
        n = count;
        const size_t need = count * sizeof(T);
        if (need > c->slot_cap[slot]) {
            CU_CHECK(cudaStreamSynchronize(c->stream));
            CU_CHECK(cudaStreamSynchronize(c->copy_stream));
            if (c->slot_ptr[slot]) CU_CHECK(cudaFree(c->slot_ptr[slot]));
            c->slot_ptr[slot] = nullptr;
            c->slot_cap[slot] = 0;
            const size_t cap = (need + 255) / 256 * 256;
            void* q = nullptr;
            cudaError_t e = cudaMalloc(&q, cap);
            if (e != cudaSuccess) {
                cudaGetLastError();
                fail(CULSH_ERR_ALLOC, "device allocation of %zu bytes failed: %s", cap, cudaGetErrorString(e));
            }
            c->slot_ptr[slot] = q;
            c->slot_cap[slot] = cap;
        }
        p = count ? static_cast<T*>(c->slot_ptr[slot]) : nullptr;
    }
    size_t bytes() const { return n * sizeof(T); }
};

inline bool is_device_pointer(const void* p) {
    if (!p) return false;
    cudaPointerAttributes a{};
    cudaError_t e = cudaPointerGetAttributes(&a, p);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

// Copy device -> (host | device) destination and wait.
inline void copy_out(const CtxPtr& c, void* dst, const void* src_dev, size_t bytes) {
    if (bytes == 0) return;
    if (!dst) fail(CULSH_ERR_INVALID, "destination pointer is null");
    CU_CHECK(cudaMemcpyAsync(dst, src_dev, bytes, cudaMemcpyDefault, c->stream));
    CU_CHECK(cudaStreamSynchronize(c->stream));
}

// Read up to 64 u64 words from device memory through the pinned scratch block.
inline void read_words(const CtxPtr& c, const void* src_dev, size_t bytes, void* host_out) {
    if (bytes > 64 * sizeof(uint64_t)) fail(CULSH_ERR_INTERNAL, "read_words: too large");
    CU_CHECK(cudaMemcpyAsync(c->pinned, src_dev, bytes, cudaMemcpyDeviceToHost, c->stream));
    CU_CHECK(cudaStreamSynchronize(c->stream));
    std::memcpy(host_out, c->pinned, bytes);
}

// Device-side self-check word: kernels OR a code into it instead of trapping.
enum DeviceErrorBits : int {
    DEV_ERR_LOOKBACK_TIMEOUT = 1,  // a bounded wait on another tile's status ran out
    DEV_ERR_NARROW_OVERFLOW = 2,   // a p-stable hash value does not fit the narrow key width
    DEV_ERR_MBAR_TIMEOUT = 4,      // a bounded mbarrier wait ran out (tensor-core projection)
    DEV_ERR_RANGE = 8              // an index outside its array was skipped
};

}  // namespace culsh_b200
