// Bucket boundaries and offsets from the sorted (key, row) pairs.  Replaces
// mark_boundaries_kernel + ExclusiveSum + Select::Flagged + build_final_index_kernel
// (core/fit.cuh:97-208, 285-363).  The sorted keys sit next to each other, so a boundary
// is a compare of two adjacent keys (no gather of signatures through the permutation),
// the sorted row ids already are all_candidate_indices, and one count pass + one write
// pass produce bucket keys, bucket offsets, table offsets and (for fit_query) the
// (row, table) -> bucket map.
#pragma once

#include "common.cuh"
#include "radix_sort.cuh"

namespace culsh_b200 {

constexpr int IB_THREADS = 256;
constexpr int IB_IPT = 8;
constexpr int IB_TILE = IB_THREADS * IB_IPT;

template <int NW>
__device__ __forceinline__ bool keys_differ(const uint32_t* __restrict__ a,
                                            const uint32_t* __restrict__ b) {
    bool d = false;
#pragma unroll
    for (int w = 0; w < NW; ++w) d |= a[w] != b[w];
    return d;
}

// heads per tile; a tile covers IB_TILE consecutive items of one table
template <int NW>
__global__ void __launch_bounds__(IB_THREADS)
bucket_count_kernel(const uint32_t* __restrict__ keys, int n, int tiles_per_table,
                    uint32_t* __restrict__ tile_heads) {
    __shared__ uint32_t s_warp[32];
    const int t = blockIdx.x / tiles_per_table;
    const int lt = blockIdx.x - t * tiles_per_table;
    const size_t tbase = (size_t)t * n;
    uint32_t c = 0;
#pragma unroll
    for (int i = 0; i < IB_IPT; ++i) {
        int li = lt * IB_TILE + i * IB_THREADS + threadIdx.x;
        if (li < n) {
            bool head = li == 0 ||
                        keys_differ<NW>(keys + (tbase + li) * NW, keys + (tbase + li - 1) * NW);
            c += head ? 1u : 0u;
        }
    }
    uint32_t total;
    block_exclusive_scan<uint32_t>(c, s_warp, total);
    if (threadIdx.x == 0) tile_heads[blockIdx.x] = total;
}

// tile_base: exclusive scan of tile_heads (tile_base[n_tiles] = B).
// Items are visited in warp-coalesced order twice: the first sweep records the head flags of
// the tile as one ballot word per 32 consecutive items, a prefix over those words then gives
// every item its bucket id, and the second sweep writes bucket keys / offsets (consecutive
// heads -> consecutive addresses) and the optional (table, row) -> bucket map [L][n].
template <int NW>
__global__ void __launch_bounds__(IB_THREADS)
bucket_write_kernel(const uint32_t* __restrict__ keys, const uint32_t* __restrict__ rows, int n,
                    int L, int tiles_per_table, const uint32_t* __restrict__ tile_base,
                    uint32_t n_tiles, uint32_t* __restrict__ bucket_keys,
                    int32_t* __restrict__ bucket_offsets, int32_t* __restrict__ table_offsets,
                    int32_t* __restrict__ item_to_bucket) {
    constexpr int WORDS = IB_TILE / 32;
    __shared__ uint32_t s_bits[WORDS];
    __shared__ uint32_t s_pref[WORDS];
    const int t = blockIdx.x / tiles_per_table;
    const int lt = blockIdx.x - t * tiles_per_table;
    const size_t tbase = (size_t)t * n;
    const int lane = threadIdx.x & 31;
    const uint32_t base_bucket = tile_base[blockIdx.x];
#pragma unroll
    for (int i = 0; i < IB_IPT; ++i) {
        const int local = i * IB_THREADS + threadIdx.x;
        const int li = lt * IB_TILE + local;
        bool head = false;
        if (li < n)
            head = li == 0 || keys_differ<NW>(keys + (tbase + li) * NW, keys + (tbase + li - 1) * NW);
        const uint32_t word = __ballot_sync(0xFFFFFFFFu, head);
        if (lane == 0) s_bits[local >> 5] = word;
    }
    __syncthreads();
    if (threadIdx.x < 32) {  // exclusive prefix of the pop-counts of the WORDS ballot words
        uint32_t run = 0;
        for (int w0 = 0; w0 < WORDS; w0 += 32) {
            const uint32_t c = __popc(s_bits[w0 + lane]);
            uint32_t inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                if (lane >= o) inc += x;
            }
            s_pref[w0 + lane] = run + inc - c;
            run += __shfl_sync(0xFFFFFFFFu, inc, 31);
        }
    }
    __syncthreads();
    if (lt == 0 && threadIdx.x == 0) table_offsets[t] = (int32_t)base_bucket;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        uint32_t B = tile_base[n_tiles];
        table_offsets[L] = (int32_t)B;
        bucket_offsets[B] = (int32_t)((size_t)n * L);
    }
#pragma unroll
    for (int i = 0; i < IB_IPT; ++i) {
        const int local = i * IB_THREADS + threadIdx.x;
        const int li = lt * IB_TILE + local;
        if (li >= n) continue;
        const uint32_t word = s_bits[local >> 5];
        const bool head = (word >> lane) & 1u;
        // heads up to and including this item, minus one = bucket of the item
        const uint32_t bid = base_bucket + s_pref[local >> 5] + __popc(word & (0xFFFFFFFFu >> (31 - lane))) - 1u;
        if (head) {
            const uint32_t* kp = keys + (tbase + li) * NW;
            uint32_t kk[NW];
            load_key<NW>(kp, kk);
            store_key<NW>(bucket_keys + (size_t)bid * NW, kk);
            bucket_offsets[bid] = (int32_t)(tbase + li);
        }
        // table-major: the writes of one table stay inside its n*4-byte strip, which the L2 merges
        // into full lines (row-major would touch a separate sector per item)
        if (item_to_bucket) item_to_bucket[tbase + rows[tbase + li]] = (int32_t)bid;
    }
}

template <int NW>
inline void launch_bucket_count(cudaStream_t s, const uint32_t* keys, int n, int L,
                                uint32_t* tile_heads) {
    int tpt = (int)ceil_div(n, IB_TILE);
    bucket_count_kernel<NW><<<(unsigned)((size_t)tpt * L), IB_THREADS, 0, s>>>(keys, n, tpt, tile_heads);
    KERNEL_CHECK();
}

template <int NW>
inline void launch_bucket_write(cudaStream_t s, const uint32_t* keys, const uint32_t* rows, int n,
                                int L, const uint32_t* tile_base, uint32_t* bucket_keys,
                                int32_t* bucket_offsets, int32_t* table_offsets,
                                int32_t* item_to_bucket) {
    int tpt = (int)ceil_div(n, IB_TILE);
    uint32_t n_tiles = (uint32_t)((size_t)tpt * L);
    bucket_write_kernel<NW><<<n_tiles, IB_THREADS, 0, s>>>(keys, rows, n, L, tpt, tile_base, n_tiles,
                                                          bucket_keys, bucket_offsets, table_offsets,
                                                          item_to_bucket);
    KERNEL_CHECK();
}

// [L][n] -> [n][L]: 32 x 32 tiles through shared memory, coalesced on both sides.
__global__ void __launch_bounds__(256)
transpose_table_major_kernel(const int32_t* __restrict__ src, int n, int L, int32_t* __restrict__ dst) {
    __shared__ int32_t tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const size_t row0 = (size_t)blockIdx.x * 32;
    const int t0 = blockIdx.y * 32;
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
        const int t = t0 + j;
        const size_t row = row0 + tx;
        if (t < L && row < (size_t)n) tile[j][tx] = src[(size_t)t * n + row];
    }
    __syncthreads();
#pragma unroll
    for (int j = ty; j < 32; j += 8) {
        const size_t row = row0 + j;
        const int t = t0 + tx;
        if (row < (size_t)n && t < L) dst[row * L + t] = tile[tx][j];
    }
}

#define CULSH_DISPATCH_NW(NWVAL, ...)                                         \
    switch (NWVAL) {                                                          \
        case 1: { constexpr int NW = 1; __VA_ARGS__; } break;                 \
        case 2: { constexpr int NW = 2; __VA_ARGS__; } break;                 \
        case 4: { constexpr int NW = 4; __VA_ARGS__; } break;                 \
        case 8: { constexpr int NW = 8; __VA_ARGS__; } break;                 \
        case 16: { constexpr int NW = 16; __VA_ARGS__; } break;               \
        default: ::culsh_b200::fail(CULSH_ERR_UNSUPPORTED, "unsupported key width"); \
    }

// ---------------------------------------------------------------------------------------
// Conversions between packed keys and upstream's raw signature bytes.
// ---------------------------------------------------------------------------------------
// raw: [count][sig_nbytes] (uint8 0/1 per hash, or little-endian int32/uint32 per hash)
__global__ void unpack_keys_kernel(const uint32_t* __restrict__ keys, size_t count, int family,
                                   int k, int NW, int elem_bytes, uint8_t* __restrict__ raw) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const uint32_t* key = keys + i * NW;
    if (family == CULSH_RPLSH) {
        uint8_t* dst = raw + i * k;
        for (int j = 0; j < k; ++j) {
            int pos = k - 1 - j;
            dst[j] = (uint8_t)((key[NW - 1 - (pos >> 5)] >> (pos & 31)) & 1u);
        }
    } else {
        int32_t* dst = reinterpret_cast<int32_t*>(raw + i * (size_t)k * 4);
        const int pad = NW * 4 - k * elem_bytes;
        for (int j = 0; j < k; ++j) {
            uint32_t v = 0;
            for (int c = 0; c < elem_bytes; ++c) {
                int bp = pad + j * elem_bytes + c;  // big-endian byte position in the key
                uint32_t byte = (key[bp >> 2] >> (24 - 8 * (bp & 3))) & 0xFFu;
                v |= byte << (8 * c);
            }
            if (family == CULSH_PSLSH && elem_bytes < 4) {  // sign-extend
                int sh = 32 - 8 * elem_bytes;
                v = (uint32_t)(((int32_t)(v << sh)) >> sh);
            }
            dst[j] = (int32_t)v;
        }
    }
}

// Largest |value| bucket of raw int32 signatures needs: 1, 2 or 4 bytes (p-stable load).
__global__ void pslsh_width_kernel(const int32_t* __restrict__ raw, size_t count, int* __restrict__ width) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    int w = 1;
    if (i < count) {
        int v = raw[i];
        if (v < -32768 || v > 32767) w = 4;
        else if (v < -128 || v > 127) w = 2;
    }
    w = max(w, __shfl_xor_sync(0xFFFFFFFFu, w, 16));
    w = max(w, __shfl_xor_sync(0xFFFFFFFFu, w, 8));
    w = max(w, __shfl_xor_sync(0xFFFFFFFFu, w, 4));
    w = max(w, __shfl_xor_sync(0xFFFFFFFFu, w, 2));
    w = max(w, __shfl_xor_sync(0xFFFFFFFFu, w, 1));
    if ((threadIdx.x & 31) == 0 && w > 1) atomicMax(width, w);
}

__global__ void pack_keys_kernel(const uint8_t* __restrict__ raw, size_t count, int family, int k,
                                 int NW, int elem_bytes, uint32_t* __restrict__ keys) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    uint32_t* key = keys + i * NW;
    for (int w = 0; w < NW; ++w) key[w] = 0;
    if (family == CULSH_RPLSH) {
        const uint8_t* src = raw + i * k;
        for (int j = 0; j < k; ++j) {
            int pos = k - 1 - j;
            if (src[j]) key[NW - 1 - (pos >> 5)] |= 1u << (pos & 31);
        }
    } else {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(raw + i * (size_t)k * 4);
        const int pad = NW * 4 - k * elem_bytes;
        for (int j = 0; j < k; ++j) {
            uint32_t v = src[j];
            for (int c = 0; c < elem_bytes; ++c) {
                int bp = pad + j * elem_bytes + c;
                key[bp >> 2] |= ((v >> (8 * c)) & 0xFFu) << (24 - 8 * (bp & 3));
            }
        }
    }
}

// Packed key of every indexed row, in row order: out[(t * n + row) * NW + w] = key of the bucket
// that holds `row` in table t.  One thread per bucket walks the bucket's rows (buckets of an LSH
// index are short); the stores of a table stay inside its n * NW words.
template <int NW>
__global__ void __launch_bounds__(256)
row_keys_kernel(const uint32_t* __restrict__ bucket_keys, const int32_t* __restrict__ bucket_offsets,
                const int32_t* __restrict__ cand, int n_buckets, int n, uint32_t* __restrict__ out) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_buckets) return;
    uint32_t key[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) key[w] = bucket_keys[(size_t)b * NW + w];
    const int lo = bucket_offsets[b], hi = bucket_offsets[b + 1];
    if (lo >= hi) return;
    const size_t table_base = (size_t)(lo / n) * (size_t)n;  // a bucket lies inside one table
    for (int p = lo; p < hi; ++p) {
        uint32_t* dst = out + (table_base + (size_t)cand[p]) * NW;
#pragma unroll
        for (int w = 0; w < NW; ++w) dst[w] = key[w];
    }
}

}  // namespace culsh_b200
