// Per-table stable LSD radix sort of (packed key, row id) pairs, all tables in one launch
// per 8-bit digit.  Replaces upstream's loop of extract_byte_key_kernel +
// cub::DeviceRadixSort::SortPairs per signature byte plus the table-id pass
// (core/fit.cuh:254-282): here the packed key travels with the row id, so no pass gathers
// signature bytes at random, tables never mix (a tile belongs to one table), and a pass
// reads and writes each pair exactly once (single-sweep scatter whose tile prefixes come
// from a decoupled look-back over the preceding tiles of the same table).
//
// Every wait on another tile's status word is bounded: when it runs out the kernel records
// DEV_ERR_LOOKBACK_TIMEOUT in the handle's error word and carries on to completion; the
// host then reports CULSH_ERR_INTERNAL.
#pragma once

#include "common.cuh"

namespace culsh_b200 {

constexpr int RS_THREADS = 256;
constexpr int RS_WARPS = RS_THREADS / 32;

template <int NW>
struct SortCfg {
    static constexpr int IPT = NW <= 4 ? 16 : (NW == 8 ? 8 : 4);  // items per thread
    static constexpr int TILE = RS_THREADS * IPT;
    static constexpr size_t SMEM =
        sizeof(uint32_t) * ((size_t)TILE * NW + TILE + RS_WARPS * 256 + 256 + 256 + 32);
};

inline int sort_tile_items(int NW) {
    switch (NW) {
        case 1: return SortCfg<1>::TILE;
        case 2: return SortCfg<2>::TILE;
        case 4: return SortCfg<4>::TILE;
        case 8: return SortCfg<8>::TILE;
        default: return SortCfg<16>::TILE;
    }
}

// Byte p of a key (p = 0 least significant): word NW-1-p/4, shift 8*(p%4).
template <int NW>
__device__ __forceinline__ uint32_t key_digit(const uint32_t* key, int p) {
    const int sel = NW - 1 - (p >> 2);
    uint32_t word = key[0];
#pragma unroll
    for (int w = 1; w < NW; ++w)  // select chain keeps the key in registers
        if (w == sel) word = key[w];
    return (word >> (8 * (p & 3))) & 0xFFu;
}

template <int NW>
__device__ __forceinline__ void load_key(const uint32_t* __restrict__ src, uint32_t* k) {
    if (NW == 1) {
        k[0] = src[0];
    } else if (NW == 2) {
        uint2 v = *reinterpret_cast<const uint2*>(src);
        k[0] = v.x; k[1] = v.y;
    } else {
#pragma unroll
        for (int i = 0; i < NW / 4; ++i) {
            uint4 v = reinterpret_cast<const uint4*>(src)[i];
            k[4 * i] = v.x; k[4 * i + 1] = v.y; k[4 * i + 2] = v.z; k[4 * i + 3] = v.w;
        }
    }
}

template <int NW>
__device__ __forceinline__ void store_key(uint32_t* __restrict__ dst, const uint32_t* k) {
    if (NW == 1) {
        dst[0] = k[0];
    } else if (NW == 2) {
        *reinterpret_cast<uint2*>(dst) = make_uint2(k[0], k[1]);
    } else {
#pragma unroll
        for (int i = 0; i < NW / 4; ++i)
            reinterpret_cast<uint4*>(dst)[i] =
                make_uint4(k[4 * i], k[4 * i + 1], k[4 * i + 2], k[4 * i + 3]);
    }
}

// ---------------------------------------------------------------------------------------
// Digit histograms of every byte position, one read of the keys.
// ghist layout: [L][KB][256].
// ---------------------------------------------------------------------------------------
constexpr int RS_HIST_CHUNK = 16384;

template <int NW>
__global__ void __launch_bounds__(RS_THREADS)
radix_hist_kernel(const uint32_t* __restrict__ keys, int n, int KB, uint32_t* __restrict__ ghist) {
    extern __shared__ uint32_t sh_hist[];  // [KB][256]
    const int t = blockIdx.y;
    for (int i = threadIdx.x; i < KB * 256; i += RS_THREADS) sh_hist[i] = 0;
    __syncthreads();
    const int begin = blockIdx.x * RS_HIST_CHUNK;
    const int end = min(n, begin + RS_HIST_CHUNK);
    const int n_words = (KB + 3) / 4;
    for (int i = begin + threadIdx.x; i < end; i += RS_THREADS) {
        const uint32_t* kp = keys + ((size_t)t * n + i) * NW;
        for (int w = 0; w < n_words; ++w) {
            const uint32_t word = kp[NW - 1 - w];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int p = w * 4 + b;
                if (p < KB) atomicAdd(&sh_hist[p * 256 + ((word >> (8 * b)) & 0xFFu)], 1u);
            }
        }
    }
    __syncthreads();
    uint32_t* g = ghist + (size_t)t * KB * 256;
    for (int i = threadIdx.x; i < KB * 256; i += RS_THREADS) {
        uint32_t v = sh_hist[i];
        if (v) atomicAdd(&g[i], v);
    }
}

// In-place exclusive scan of each 256-bin histogram: one block per (table, byte).
__global__ void __launch_bounds__(256) radix_bin_prefix_kernel(uint32_t* __restrict__ ghist) {
    __shared__ uint32_t warp_tot[8];
    uint32_t* h = ghist + (size_t)blockIdx.x * 256;
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    uint32_t v = h[threadIdx.x];
    uint32_t inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += x;
    }
    if (lane == 31) warp_tot[w] = inc;
    __syncthreads();
    uint32_t base = 0;
    for (int i = 0; i < w; ++i) base += warp_tot[i];
    h[threadIdx.x] = base + inc - v;
}

// ---------------------------------------------------------------------------------------
// One scatter pass on byte `p`.
// ---------------------------------------------------------------------------------------
constexpr uint32_t RS_FLAG_AGG = 1u << 30;
constexpr uint32_t RS_FLAG_INC = 2u << 30;
constexpr uint32_t RS_VAL_MASK = (1u << 30) - 1;
constexpr int RS_SPIN_LIMIT = 1 << 22;

__device__ __forceinline__ uint32_t ld_volatile_u32(const uint32_t* p) {
    return *reinterpret_cast<const volatile uint32_t*>(p);
}
__device__ __forceinline__ void st_volatile_u32(uint32_t* p, uint32_t v) {
    *reinterpret_cast<volatile uint32_t*>(p) = v;
}

template <int NW, bool FIRST>
__global__ void __launch_bounds__(RS_THREADS)
radix_pass_kernel(const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                  uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out, int n,
                  int tiles_per_table, int p, int KB, const uint32_t* __restrict__ gbase,
                  uint32_t* __restrict__ status, uint32_t* __restrict__ tile_counter,
                  int* __restrict__ d_error) {
    using Cfg = SortCfg<NW>;
    constexpr int IPT = Cfg::IPT;
    constexpr int TILE = Cfg::TILE;
    extern __shared__ __align__(16) uint32_t smem[];
    uint32_t* s_keys = smem;                       // [TILE][NW]
    uint32_t* s_vals = s_keys + (size_t)TILE * NW; // [TILE]
    uint32_t* s_whist = s_vals + TILE;             // [RS_WARPS][256]
    uint32_t* s_gdst = s_whist + RS_WARPS * 256;   // [256] global dst of local position 0 of a bin
    uint32_t* s_binstart = s_gdst + 256;           // [256]
    uint32_t* s_misc = s_binstart + 256;           // [32]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_misc[0] = atomicAdd(tile_counter, 1u);
    for (int i = tid; i < RS_WARPS * 256; i += RS_THREADS) s_whist[i] = 0;
    __syncthreads();
    const uint32_t tile = s_misc[0];
    const int t = tile / tiles_per_table;
    const int lt = tile - t * tiles_per_table;
    const int item0 = lt * TILE;
    const int count = min(TILE, n - item0);
    const size_t base = (size_t)t * n + item0;
    const uint32_t my_gbase = gbase[((size_t)t * KB + p) * 256 + tid];  // needed late: fetch early

    // ---- load (all loads in flight together), then rank inside the warp ---------------
    uint32_t key[IPT][NW];
    uint32_t val[IPT];
    uint16_t rank[IPT];
    uint16_t dig[IPT];
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
        const int li = warp * (32 * IPT) + i * 32 + lane;
        if (li < count) {
            load_key<NW>(keys_in + (base + li) * NW, key[i]);
            val[i] = FIRST ? (uint32_t)(item0 + li) : vals_in[base + li];
        } else {
#pragma unroll
            for (int w = 0; w < NW; ++w) key[i][w] = 0;
            val[i] = 0;
        }
    }
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
        const int li = warp * (32 * IPT) + i * 32 + lane;
        const bool valid = li < count;
        const uint32_t d = valid ? key_digit<NW>(key[i], p) : 0x100u;
        const uint32_t peers = __match_any_sync(0xFFFFFFFFu, d);
        const uint32_t below = __popc(peers & ((1u << lane) - 1));
        uint32_t old = valid ? s_whist[warp * 256 + d] : 0u;
        __syncwarp();
        if (valid && below == 0) s_whist[warp * 256 + d] = old + __popc(peers);
        __syncwarp();
        rank[i] = (uint16_t)(old + below);
        dig[i] = (uint16_t)d;
    }
    __syncthreads();

    // ---- per-bin: warp offsets, tile count, look-back --------------------------------
    uint32_t cnt = 0;
    {
        const int b = tid;
#pragma unroll
        for (int w = 0; w < RS_WARPS; ++w) {
            uint32_t x = s_whist[w * 256 + b];
            s_whist[w * 256 + b] = cnt;
            cnt += x;
        }
    }
    // publish as early as possible so later tiles can move on
    uint32_t* my_status = status + (size_t)tile * 256 + tid;
    if (lt == 0) st_volatile_u32(my_status, RS_FLAG_INC | cnt);
    else st_volatile_u32(my_status, RS_FLAG_AGG | cnt);

    // block exclusive scan of cnt over the 256 bins
    uint32_t inc = cnt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        uint32_t x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += x;
    }
    if (lane == 31) s_misc[1 + warp] = inc;
    __syncthreads();
    uint32_t wbase = 0;
    for (int i = 0; i < warp; ++i) wbase += s_misc[1 + i];
    const uint32_t binstart = wbase + inc - cnt;

    uint32_t excl = 0;
    if (lt != 0) {
        // Walk back over the preceding tiles of this table, eight status words per round so
        // their latencies overlap; stop at the first tile that published an inclusive prefix.
        int j = (int)tile - 1;
        const int first = (int)tile - lt;
        bool timed_out = false, done = false;
        while (!done && !timed_out) {
            uint32_t sv[8];
            const int avail = min(8, j - first + 1);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                sv[u] = u < avail ? ld_volatile_u32(status + (size_t)(j - u) * 256 + tid) : 0u;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (u < avail && !done && !timed_out) {
                    uint32_t s = sv[u];
                    if ((s >> 30) == 0) {
                        const uint32_t* sp = status + (size_t)(j - u) * 256 + tid;
                        int spins = 0;
                        while ((s >> 30) == 0) {
                            if (++spins > RS_SPIN_LIMIT) { timed_out = true; break; }
                            if (spins > 32) __nanosleep(40);
                            s = ld_volatile_u32(sp);
                        }
                    }
                    if (!timed_out) {
                        excl += s & RS_VAL_MASK;
                        if ((s >> 30) == 2u || j - u == first) done = true;
                    }
                }
            }
            j -= 8;
        }
        if (timed_out) atomicOr(d_error, DEV_ERR_LOOKBACK_TIMEOUT);
        st_volatile_u32(my_status, RS_FLAG_INC | ((excl + cnt) & RS_VAL_MASK));
    }
    s_binstart[tid] = binstart;
    s_gdst[tid] = (uint32_t)((size_t)t * n) + my_gbase + excl - binstart;
    __syncthreads();

    // ---- reorder inside shared memory ------------------------------------------------
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
        const uint32_t d = dig[i];
        if (d < 256u) {
            const uint32_t pos = s_binstart[d] + s_whist[warp * 256 + d] + rank[i];
#pragma unroll
            for (int w = 0; w < NW; ++w) s_keys[(size_t)pos * NW + w] = key[i][w];
            s_vals[pos] = val[i];
        }
    }
    __syncthreads();

    // ---- coalesced runs out ----------------------------------------------------------
    for (int pos = tid; pos < count; pos += RS_THREADS) {
        uint32_t kk[NW];
#pragma unroll
        for (int w = 0; w < NW; ++w) kk[w] = s_keys[(size_t)pos * NW + w];
        const uint32_t d = key_digit<NW>(kk, p);
        const uint32_t g = s_gdst[d] + (uint32_t)pos;
        store_key<NW>(keys_out + (size_t)g * NW, kk);
        vals_out[g] = s_vals[pos];
    }
}

// ---------------------------------------------------------------------------------------
// Host driver.  keys[0]/vals[0] hold the input (vals[0] is never read: the first pass
// takes the row id from the position); returns which buffer (0/1) holds the result.
// ---------------------------------------------------------------------------------------
template <int NW>
inline int radix_sort_tables_nw(const CtxPtr& c, uint32_t* keys[2], uint32_t* vals[2], int n, int L,
                                int KB, uint32_t* ghist, uint32_t* status, uint32_t* tile_counter) {
    using Cfg = SortCfg<NW>;
    cudaStream_t s = c->stream;
    const int tiles_per_table = (int)ceil_div(n, Cfg::TILE);
    const size_t total_tiles = (size_t)tiles_per_table * L;
    CU_CHECK(cudaMemsetAsync(ghist, 0, sizeof(uint32_t) * (size_t)L * KB * 256, s));
    dim3 hgrid((unsigned)ceil_div(n, RS_HIST_CHUNK), (unsigned)L);
    const size_t hist_smem = sizeof(uint32_t) * KB * 256;
    if (hist_smem > 48 * 1024)
        CU_CHECK(cudaFuncSetAttribute(radix_hist_kernel<NW>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)hist_smem));
    radix_hist_kernel<NW><<<hgrid, RS_THREADS, hist_smem, s>>>(keys[0], n, KB, ghist);
    KERNEL_CHECK();
    radix_bin_prefix_kernel<<<(unsigned)(L * KB), 256, 0, s>>>(ghist);
    KERNEL_CHECK();
    if (c->profiling) cudaEventRecord(c->ev[7], s);  // start of the scatter passes
    auto k_first = radix_pass_kernel<NW, true>;
    auto k_next = radix_pass_kernel<NW, false>;
    CU_CHECK(cudaFuncSetAttribute(k_first, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM));
    CU_CHECK(cudaFuncSetAttribute(k_next, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM));
    int cur = 0;
    for (int p = 0; p < KB; ++p) {
        CU_CHECK(cudaMemsetAsync(status, 0, sizeof(uint32_t) * total_tiles * 256, s));
        CU_CHECK(cudaMemsetAsync(tile_counter, 0, sizeof(uint32_t), s));
        if (p == 0)
            k_first<<<(unsigned)total_tiles, RS_THREADS, Cfg::SMEM, s>>>(
                keys[cur], vals[cur], keys[cur ^ 1], vals[cur ^ 1], n, tiles_per_table, p, KB, ghist,
                status, tile_counter, c->d_error);
        else
            k_next<<<(unsigned)total_tiles, RS_THREADS, Cfg::SMEM, s>>>(
                keys[cur], vals[cur], keys[cur ^ 1], vals[cur ^ 1], n, tiles_per_table, p, KB, ghist,
                status, tile_counter, c->d_error);
        KERNEL_CHECK();
        cur ^= 1;
    }
    return cur;
}

inline size_t radix_sort_status_words(int n, int L, int NW) {
    return ceil_div(n, sort_tile_items(NW)) * (size_t)L * 256;
}

inline int radix_sort_tables(const CtxPtr& c, int NW, uint32_t* keys[2], uint32_t* vals[2], int n,
                             int L, int KB, uint32_t* ghist, uint32_t* status,
                             uint32_t* tile_counter) {
    switch (NW) {
        case 1: return radix_sort_tables_nw<1>(c, keys, vals, n, L, KB, ghist, status, tile_counter);
        case 2: return radix_sort_tables_nw<2>(c, keys, vals, n, L, KB, ghist, status, tile_counter);
        case 4: return radix_sort_tables_nw<4>(c, keys, vals, n, L, KB, ghist, status, tile_counter);
        case 8: return radix_sort_tables_nw<8>(c, keys, vals, n, L, KB, ghist, status, tile_counter);
        case 16: return radix_sort_tables_nw<16>(c, keys, vals, n, L, KB, ghist, status, tile_counter);
    }
    fail(CULSH_ERR_UNSUPPORTED, "unsupported key width: %d words", NW);
}

// ---------------------------------------------------------------------------------------
// Device-wide exclusive scan (three phases).  out has n+1 elements: out[n] = total.
// ---------------------------------------------------------------------------------------
constexpr int SCAN_THREADS = 256;
constexpr int SCAN_IPT = 8;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_IPT;

template <typename TOut>
__device__ __forceinline__ TOut block_exclusive_scan(TOut v, TOut* s_warp, TOut& total) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    TOut inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        TOut x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += x;
    }
    __syncthreads();  // protect s_warp reuse between calls
    if (lane == 31) s_warp[w] = inc;
    __syncthreads();
    TOut base = 0, tot = 0;
    const int nw = blockDim.x >> 5;
    for (int i = 0; i < nw; ++i) {
        TOut x = s_warp[i];
        if (i < w) base += x;
        tot += x;
    }
    total = tot;
    return base + inc - v;
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_reduce_kernel(const TIn* __restrict__ in, size_t n, TOut* __restrict__ block_sums) {
    __shared__ TOut s_warp[32];
    size_t base = (size_t)blockIdx.x * SCAN_TILE;
    TOut sum = 0;
    for (int i = 0; i < SCAN_IPT; ++i) {
        size_t idx = base + (size_t)i * SCAN_THREADS + threadIdx.x;
        if (idx < n) sum += (TOut)in[idx];
    }
    TOut total;
    block_exclusive_scan<TOut>(sum, s_warp, total);
    if (threadIdx.x == 0) block_sums[blockIdx.x] = total;
}

template <typename TOut>
__global__ void __launch_bounds__(1024)
scan_block_sums_kernel(TOut* __restrict__ block_sums, size_t n_blocks, TOut* __restrict__ total_out) {
    __shared__ TOut s_warp[32];
    TOut carry = 0;
    for (size_t base = 0; base < n_blocks; base += 1024) {
        size_t idx = base + threadIdx.x;
        TOut v = idx < n_blocks ? block_sums[idx] : TOut(0);
        TOut total;
        TOut ex = block_exclusive_scan<TOut>(v, s_warp, total);
        if (idx < n_blocks) block_sums[idx] = carry + ex;
        carry += total;
    }
    if (threadIdx.x == 0 && total_out) *total_out = carry;
}

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(SCAN_THREADS)
scan_apply_kernel(const TIn* __restrict__ in, size_t n, const TOut* __restrict__ block_sums,
                  TOut* __restrict__ out) {
    __shared__ TOut s_warp[32];
    const size_t base = (size_t)blockIdx.x * SCAN_TILE + (size_t)threadIdx.x * SCAN_IPT;
    TOut v[SCAN_IPT];
    TOut sum = 0;
#pragma unroll
    for (int i = 0; i < SCAN_IPT; ++i) {
        size_t idx = base + i;
        v[i] = idx < n ? (TOut)in[idx] : TOut(0);
        sum += v[i];
    }
    TOut total;
    TOut ex = block_exclusive_scan<TOut>(sum, s_warp, total) + block_sums[blockIdx.x];
#pragma unroll
    for (int i = 0; i < SCAN_IPT; ++i) {
        size_t idx = base + i;
        if (idx < n) out[idx] = ex;
        ex += v[i];
    }
}

// scratch must hold ceil(n / SCAN_TILE) TOut elements.  out[n] receives the total.
template <typename TIn, typename TOut>
inline void exclusive_scan(cudaStream_t s, const TIn* in, size_t n, TOut* out, TOut* scratch) {
    if (n == 0) {
        CU_CHECK(cudaMemsetAsync(out, 0, sizeof(TOut), s));
        return;
    }
    size_t n_blocks = ceil_div(n, SCAN_TILE);
    scan_reduce_kernel<TIn, TOut><<<(unsigned)n_blocks, SCAN_THREADS, 0, s>>>(in, n, scratch);
    KERNEL_CHECK();
    scan_block_sums_kernel<TOut><<<1, 1024, 0, s>>>(scratch, n_blocks, out + n);
    KERNEL_CHECK();
    scan_apply_kernel<TIn, TOut><<<(unsigned)n_blocks, SCAN_THREADS, 0, s>>>(in, n, scratch, out);
    KERNEL_CHECK();
}

inline size_t scan_scratch_elems(size_t n) { return ceil_div(n, SCAN_TILE) + 1; }

}  // namespace culsh_b200
