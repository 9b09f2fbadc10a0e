// Per-table stable LSD radix sort of (packed key, row id) pairs, all tables in one launch
// per 8-bit digit.  Replaces upstream's loop of extract_byte_key_kernel +
// cub::DeviceRadixSort::SortPairs per signature byte plus the table-id pass
// (core/fit.cuh:254-282): here the packed key travels with the row id, so no pass gathers
// signature bytes at random, and tables never mix (a tile belongs to one table).  A pass is
// three launches - tile histograms, a per-table scan that turns them into destination
// offsets, and the stable scatter - so no CTA ever waits on another one: a chained
// look-back between tiles was measured to cost more than the extra 4 bytes per item that
// the histogram read adds at this bandwidth.
//
// P-stable keys of one byte per hash (at most eight hashes) whose values span at most 32 levels
// are sorted in COMPRESSED form: the first pass replaces every key byte by its 5-bit rank among
// the values in use and packs the ranks (hash 0 most significant), the passes in between see a
// key of 5 bits per hash - 5 passes instead of 8 for eight hashes -, and the last pass writes the
// original bytes back.  The rank keeps the unsigned order of the byte (non-negative values
// first, then the negative ones, two's complement bytes 128..255), so the sorted order is the
// one a byte-per-pass sort of the original keys gives.  When such a key takes two words (five to
// eight hashes: at most 40 bits compressed) and the table has at most 2^24 rows, the compressed
// key and the row id travel PACKED in one 64-bit item (key << 24 | id) between the first and the
// last pass: 8 bytes per item instead of 12 and no separate id array in the passes in between.
#pragma once

#include "common.cuh"

namespace culsh_b200 {

constexpr int RS_THREADS = 256;
#ifndef RS_MIN_BLOCKS
#define RS_MIN_BLOCKS 3
#endif
constexpr int RS_WARPS = RS_THREADS / 32;

template <int NW>
struct SortCfg {
    // items per thread: fewer for wide keys so that the tile's keys stay in registers at an
    // occupancy of 2-3 CTAs per SM
    static constexpr int IPT = NW == 1 ? 16 : (NW == 2 ? 12 : (NW == 4 ? 8 : (NW == 8 ? 4 : 2)));
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
// Compressed form of one-byte-per-hash keys (NW = 1 or 2).  rank(u) = u for a byte below 128
// (n_pos such values in use: 0 .. n_pos-1), u - sub for a byte from 128 up, with
// sub = smallest negative byte - n_pos; every rank is below 32.
// ---------------------------------------------------------------------------------------
struct KeyComp {
    uint32_t sub;    // see above
    uint32_t n_pos;  // ranks below n_pos are non-negative values
};

__device__ __forceinline__ uint32_t comp_word(uint32_t w, uint32_t sub) {  // 4 bytes -> 20 bits
    const uint32_t neg = (w >> 7) & 0x01010101u;
    uint32_t c = w - neg * sub;                                   // four ranks, one per byte
    c = (c & 0x001F001Fu) | ((c & 0x1F001F00u) >> 3);             // two 10-bit fields
    return (c & 0x3FFu) | ((c >> 6) & 0xFFC00u);
}
__device__ __forceinline__ uint32_t decomp_word(uint32_t c20, KeyComp kc) {  // 20 bits -> 4 bytes
    uint32_t c = (c20 & 0x3FFu) | ((c20 & 0xFFC00u) << 6);
    c = (c & 0x001F001Fu) | ((c << 3) & 0x1F001F00u);
    uint32_t w = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const uint32_t r = (c >> (8 * b)) & 0xFFu;
        w |= (r + (r >= kc.n_pos ? kc.sub : 0u)) << (8 * b);
    }
    return w;
}
template <int NW>
__device__ __forceinline__ void comp_key(uint32_t* k, uint32_t sub) {
    if (NW == 1) {
        k[0] = comp_word(k[0], sub);
    } else {
        const uint64_t v = ((uint64_t)comp_word(k[0], sub) << 20) | comp_word(k[1], sub);
        k[0] = (uint32_t)(v >> 32);
        k[1] = (uint32_t)v;
    }
}
template <int NW>
__device__ __forceinline__ void decomp_key(uint32_t* k, KeyComp kc) {
    if (NW == 1) {
        k[0] = decomp_word(k[0], kc);
    } else {
        const uint64_t v = ((uint64_t)k[0] << 32) | k[1];
        k[0] = decomp_word((uint32_t)(v >> 20) & 0xFFFFFu, kc);
        k[1] = decomp_word((uint32_t)v & 0xFFFFFu, kc);
    }
}

// ---------------------------------------------------------------------------------------
// Pass step 1: digit histogram of every tile (a tile is TILE consecutive items of one
// table).  tile_hist layout: [tile][256].
// ---------------------------------------------------------------------------------------
template <int NW, bool COMP0>
__global__ void __launch_bounds__(RS_THREADS)
radix_tile_hist_kernel(const uint32_t* __restrict__ keys, int n, int tiles_per_table, int p, uint32_t sub,
                       uint32_t* __restrict__ tile_hist) {
    using Cfg = SortCfg<NW>;
    __shared__ uint32_t s_hist[256];
    const int tile = blockIdx.x;
    const int t = tile / tiles_per_table;
    const int lt = tile - t * tiles_per_table;
    const int item0 = lt * Cfg::TILE;
    const int count = min(Cfg::TILE, n - item0);
    const uint32_t* base = keys + ((size_t)t * n + item0) * NW + (NW - 1 - (p >> 2));
    const int shift = 8 * (p & 3);
    s_hist[threadIdx.x] = 0;
    __syncthreads();
    if (COMP0) {  // p == 0 of a compressed sort: the digit is the low byte of the compressed key
        const uint32_t* last = keys + ((size_t)t * n + item0) * NW + (NW - 1);
#pragma unroll 4
        for (int i = threadIdx.x; i < count; i += RS_THREADS)
            atomicAdd(&s_hist[comp_word(last[(size_t)i * NW], sub) & 0xFFu], 1u);
    } else {
#pragma unroll 4
        for (int i = threadIdx.x; i < count; i += RS_THREADS)
            atomicAdd(&s_hist[(base[(size_t)i * NW] >> shift) & 0xFFu], 1u);
    }
    __syncthreads();
    tile_hist[(size_t)tile * 256 + threadIdx.x] = s_hist[threadIdx.x];
}

// ---------------------------------------------------------------------------------------
// Pass step 2: one block per table turns the tile histograms into the offset (inside the
// table) at which each tile's run of each digit starts:
//   off[tile][d] = sum over d' < d of total[d'] + sum over earlier tiles of hist[tile'][d].
// 1024 threads = 4 tile segments x 256 digits.
// ---------------------------------------------------------------------------------------
constexpr int RS_SCAN_THREADS = 1024;
constexpr int RS_SCAN_SEGS = RS_SCAN_THREADS / 256;

__global__ void __launch_bounds__(RS_SCAN_THREADS)
radix_tile_scan_kernel(uint32_t* __restrict__ tile_hist, int tiles_per_table) {
    __shared__ uint32_t s_seg[RS_SCAN_SEGS][256];
    __shared__ uint32_t s_base[256];
    __shared__ uint32_t s_warp[8];
    const int d = threadIdx.x & 255, seg = threadIdx.x >> 8;
    uint32_t* h = tile_hist + (size_t)blockIdx.x * tiles_per_table * 256 + d;
    const int per_seg = (tiles_per_table + RS_SCAN_SEGS - 1) / RS_SCAN_SEGS;
    const int i0 = seg * per_seg, i1 = min(tiles_per_table, i0 + per_seg);
    uint32_t sum = 0;
#pragma unroll 8
    for (int i = i0; i < i1; ++i) sum += h[(size_t)i * 256];
    s_seg[seg][d] = sum;
    __syncthreads();
    if (seg == 0) {  // exclusive scan of the digit totals over the 256 digits
        uint32_t tot = 0;
#pragma unroll
        for (int g = 0; g < RS_SCAN_SEGS; ++g) tot += s_seg[g][d];
        const int lane = d & 31, w = d >> 5;
        uint32_t inc = tot;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            uint32_t x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += x;
        }
        if (lane == 31) s_warp[w] = inc;
        s_base[d] = inc - tot;  // exclusive inside the warp; the warp bases are added below
    }
    __syncthreads();
    uint32_t run = s_base[d];
    for (int w = 0; w < (d >> 5); ++w) run += s_warp[w];
    for (int g = 0; g < seg; ++g) run += s_seg[g][d];
#pragma unroll 8
    for (int i = i0; i < i1; ++i) {
        uint32_t x = h[(size_t)i * 256];
        h[(size_t)i * 256] = run;
        run += x;
    }
}

// Tables with many tiles: one block per (table, chunk of RS_CHUNK_TILES tiles) scans its chunk
// on its own (exclusive prefix over the chunk's tiles per digit, chunk totals on the side), a
// second tiny launch turns the chunk totals into chunk bases (digit prefix + earlier chunks), and
// the scatter adds the base of its chunk.  With one block per table the scan of a 10M-row table
// (2441 tiles) ran on 48 SMs for 1.2 ms per pass.
constexpr int RS_CHUNK_TILES = 256;
constexpr int RS_CHUNK_MIN_TILES = 512;  // tables with fewer tiles keep the single-launch scan

__global__ void __launch_bounds__(RS_SCAN_THREADS)
radix_tile_scan_chunk_kernel(uint32_t* __restrict__ tile_hist, int tiles_per_table, int n_chunks,
                             uint32_t* __restrict__ chunk_tot /* [table][chunk][256] */) {
    __shared__ uint32_t s_seg[RS_SCAN_SEGS][256];
    const int d = threadIdx.x & 255, seg = threadIdx.x >> 8;
    const int table = blockIdx.x / n_chunks, chunk = blockIdx.x - table * n_chunks;
    const int t_begin = chunk * RS_CHUNK_TILES, t_end = min(tiles_per_table, t_begin + RS_CHUNK_TILES);
    uint32_t* h = tile_hist + (size_t)table * tiles_per_table * 256 + d;
    const int per_seg = (t_end - t_begin + RS_SCAN_SEGS - 1) / RS_SCAN_SEGS;
    const int i0 = t_begin + seg * per_seg, i1 = min(t_end, i0 + per_seg);
    uint32_t sum = 0;
#pragma unroll 8
    for (int i = i0; i < i1; ++i) sum += h[(size_t)i * 256];
    s_seg[seg][d] = sum;
    __syncthreads();
    uint32_t run = 0, tot = 0;
#pragma unroll
    for (int g = 0; g < RS_SCAN_SEGS; ++g) {
        const uint32_t x = s_seg[g][d];
        if (g < seg) run += x;
        tot += x;
    }
    if (seg == 0) chunk_tot[(size_t)blockIdx.x * 256 + d] = tot;
#pragma unroll 8
    for (int i = i0; i < i1; ++i) {
        const uint32_t x = h[(size_t)i * 256];
        h[(size_t)i * 256] = run;
        run += x;
    }
}

// one block of 256 threads per table: chunk_tot -> chunk bases, in place
__global__ void __launch_bounds__(256)
radix_chunk_base_kernel(uint32_t* __restrict__ chunk_tot, int n_chunks) {
    __shared__ uint32_t s_warp[8];
    const int d = threadIdx.x, lane = d & 31, w = d >> 5;
    uint32_t* ct = chunk_tot + (size_t)blockIdx.x * n_chunks * 256 + d;
    uint32_t tot = 0;
    for (int c = 0; c < n_chunks; ++c) tot += ct[(size_t)c * 256];
    uint32_t inc = tot;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += x;
    }
    if (lane == 31) s_warp[w] = inc;
    __syncthreads();
    uint32_t run = inc - tot;
    for (int i = 0; i < w; ++i) run += s_warp[i];
    for (int c = 0; c < n_chunks; ++c) {
        const uint32_t x = ct[(size_t)c * 256];
        ct[(size_t)c * 256] = run;
        run += x;
    }
}

// ---------------------------------------------------------------------------------------
// Pass step 3: stable scatter of one tile on byte `p`.
// ---------------------------------------------------------------------------------------
// COMP: 0 plain keys; 1 first pass of a compressed sort (keys are compressed as they are
// loaded); 2 its last pass (the original bytes are written back).
// PACK (NW = 2, compressed): items are (compressed key << 24 | row id); the digit of pass p is
// byte p + 3 of the item, ids are neither loaded nor stored except by the last pass.
constexpr int RS_PACK_ID_BITS = 24;

template <int NW, bool FIRST, int COMP, bool PACK = false>
__global__ void __launch_bounds__(RS_THREADS, (NW <= 2 ? 4 : RS_MIN_BLOCKS))
radix_scatter_kernel(const uint32_t* __restrict__ keys_in, const uint32_t* __restrict__ vals_in,
                     uint32_t* __restrict__ keys_out, uint32_t* __restrict__ vals_out, int n,
                     int tiles_per_table, int p, KeyComp kc, const uint32_t* __restrict__ tile_off,
                     const uint32_t* __restrict__ chunk_base /* or null */, int n_chunks) {
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
    const int tile = blockIdx.x;
    const int t = tile / tiles_per_table;
    const int lt = tile - t * tiles_per_table;
    const int item0 = lt * TILE;
    const int count = min(TILE, n - item0);
    const size_t base = (size_t)t * n + item0;
    const int pd = PACK ? p + 3 : p;  // byte of the item that holds this pass's digit
    // needed late: fetched early, and summed only where used (an add here would stall the warp on
    // both loads before the key loads are issued)
    const uint32_t my_off = tile_off[(size_t)tile * 256 + tid];
    const uint32_t my_base = chunk_base ? chunk_base[((size_t)t * n_chunks + lt / RS_CHUNK_TILES) * 256 + tid] : 0u;
    for (int i = tid; i < RS_WARPS * 256; i += RS_THREADS) s_whist[i] = 0;

    // ---- load (all loads in flight together) ------------------------------------------
    uint32_t key[IPT][NW];
    uint32_t val[IPT];
    uint16_t rank[IPT];
    uint16_t dig[IPT];
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
        const int li = warp * (32 * IPT) + i * 32 + lane;
        if (li < count) {
            load_key<NW>(keys_in + (base + li) * NW, key[i]);
            if (COMP == 1) comp_key<NW>(key[i], kc.sub);
            if constexpr (PACK) {
                if (COMP == 1) {  // (40-bit compressed key) << 24 | row id
                    key[i][0] = (key[i][0] << RS_PACK_ID_BITS) | (key[i][NW - 1] >> (32 - RS_PACK_ID_BITS));
                    key[i][NW - 1] = (key[i][NW - 1] << RS_PACK_ID_BITS) | (uint32_t)(item0 + li);
                }
                val[i] = 0;
            } else {
                val[i] = FIRST ? (uint32_t)(item0 + li) : vals_in[base + li];
            }
        } else {
#pragma unroll
            for (int w = 0; w < NW; ++w) key[i][w] = 0;
            val[i] = 0;
        }
    }
    __syncthreads();
    // ---- rank inside the warp: lanes holding the same digit elect their lowest lane, which
    // bumps the warp's counter once; lane order inside the group keeps the sort stable ----
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
        const int li = warp * (32 * IPT) + i * 32 + lane;
        const bool valid = li < count;
        const uint32_t d = valid ? key_digit<NW>(key[i], pd) : 0x100u;
        // lanes with the same digit.  For one-word keys and for packed items the kernel is bound by
        // the latency of the shared-memory / match pipeline, and nine ballots (digit bits +
        // validity) are cheaper than match.any (packed 12.5M-row shard: 0.55 ms less over the first
        // four passes; the last pass, which also unpacks, is 0.35 ms faster with match.any and keeps
        // it); wider keys are bandwidth-bound and take the shorter instruction.
        uint32_t peers;
        if constexpr (NW == 1 || (PACK && COMP != 2)) {
            peers = count == TILE ? 0xFFFFFFFFu : __ballot_sync(0xFFFFFFFFu, valid);
            if (!valid) peers = ~peers;
#pragma unroll
            for (int b = 0; b < 8; ++b) {
                const bool bit = (d >> b) & 1u;
                const uint32_t m = __ballot_sync(0xFFFFFFFFu, bit);
                peers &= bit ? m : ~m;
            }
        } else {
            peers = __match_any_sync(0xFFFFFFFFu, d);
        }
        const int leader = __ffs(peers) - 1;
        const uint32_t below = __popc(peers & ((1u << lane) - 1));
        uint32_t old = 0;
        if (valid && lane == leader) old = atomicAdd(&s_whist[warp * 256 + d], (uint32_t)__popc(peers));
        old = __shfl_sync(0xFFFFFFFFu, old, leader);
        rank[i] = (uint16_t)(old + below);
        dig[i] = (uint16_t)d;
    }
    __syncthreads();

    // ---- per bin: exclusive offsets of the warps, tile count, start inside the tile ----
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
    s_binstart[tid] = binstart;
    s_gdst[tid] = (uint32_t)((size_t)t * n) + my_off + my_base - binstart;
    __syncthreads();

    // ---- reorder inside shared memory ------------------------------------------------
#pragma unroll
    for (int i = 0; i < IPT; ++i) {
        const uint32_t d = dig[i];
        if (d < 256u) {
            const uint32_t pos = s_binstart[d] + s_whist[warp * 256 + d] + rank[i];
#pragma unroll
            for (int w = 0; w < NW; ++w) s_keys[(size_t)pos * NW + w] = key[i][w];
            if constexpr (!PACK) s_vals[pos] = val[i];
        }
    }
    __syncthreads();

    // ---- coalesced runs out ----------------------------------------------------------
    for (int pos = tid; pos < count; pos += RS_THREADS) {
        uint32_t kk[NW];
#pragma unroll
        for (int w = 0; w < NW; ++w) kk[w] = s_keys[(size_t)pos * NW + w];
        const uint32_t d = key_digit<NW>(kk, pd);
        const uint32_t g = s_gdst[d] + (uint32_t)pos;
        if constexpr (PACK) {
            if (COMP == 2) {  // unpack: id from the low bits, the key back to its two-word compressed form
                vals_out[g] = kk[NW - 1] & ((1u << RS_PACK_ID_BITS) - 1u);
                kk[NW - 1] = (kk[0] << (32 - RS_PACK_ID_BITS)) | (kk[NW - 1] >> RS_PACK_ID_BITS);
                kk[0] >>= RS_PACK_ID_BITS;
                decomp_key<NW>(kk, kc);
            }
            store_key<NW>(keys_out + (size_t)g * NW, kk);
        } else {
            if (COMP == 2) decomp_key<NW>(kk, kc);
            store_key<NW>(keys_out + (size_t)g * NW, kk);
            vals_out[g] = s_vals[pos];
        }
    }
}

// ---------------------------------------------------------------------------------------
// Range of the key bytes of p-stable keys with one byte per hash: out[0] = largest byte below
// 128 (largest non-negative hash value, 0 if none), out[1] = smallest byte from 128 up (the
// smallest negative value as an unsigned byte, 256 if none).  out must hold {0, 256} before.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
key_byte_range_kernel(const uint32_t* __restrict__ keys, size_t n_words, uint32_t* __restrict__ out) {
    uint32_t hi_pos = 0, lo_neg = 256;
    auto take = [&](uint32_t w) {
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const uint32_t u = (w >> (8 * b)) & 0xFFu;
            if (u < 128u) hi_pos = max(hi_pos, u); else lo_neg = min(lo_neg, u);
        }
    };
    const size_t n4 = n_words / 4;  // the key array starts on a 16-byte boundary
    const uint4* k4 = reinterpret_cast<const uint4*>(keys);
    const size_t stride = (size_t)gridDim.x * blockDim.x, first = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (size_t i = first; i < n4; i += stride) {
        const uint4 v = k4[i];
        take(v.x); take(v.y); take(v.z); take(v.w);
    }
    for (size_t i = 4 * n4 + first; i < n_words; i += stride) take(keys[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        hi_pos = max(hi_pos, __shfl_xor_sync(0xFFFFFFFFu, hi_pos, o));
        lo_neg = min(lo_neg, __shfl_xor_sync(0xFFFFFFFFu, lo_neg, o));
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMax(&out[0], hi_pos);
        atomicMin(&out[1], lo_neg);
    }
}

// ---------------------------------------------------------------------------------------
// Host driver.  keys[0]/vals[0] hold the input (vals[0] is never read: the first pass
// takes the row id from the position); after radix_sort_passes() passes the result is in
// buffer passes & 1.  tile_hist must hold radix_sort_tile_words(n, L, NW) words.
// `compressed` (NW <= 2 only): sort the 5-bit-per-byte form of the keys, see the top of the file.
// ---------------------------------------------------------------------------------------
inline int radix_sort_passes(int KB, bool compressed) { return compressed ? (5 * KB + 7) / 8 : KB; }

template <int NW>
inline int radix_sort_tables_nw(const CtxPtr& c, uint32_t* keys[2], uint32_t* vals[2], int n, int L,
                                int KB, uint32_t* tile_hist, bool compressed, KeyComp kc) {
    using Cfg = SortCfg<NW>;
    cudaStream_t s = c->stream;
    const int tiles_per_table = (int)ceil_div(n, Cfg::TILE);
    const size_t total_tiles = (size_t)tiles_per_table * L;
    constexpr bool CAN_COMP = NW <= 2;
    auto k_first = radix_scatter_kernel<NW, true, 0>;
    auto k_next = radix_scatter_kernel<NW, false, 0>;
    auto k_first_c = radix_scatter_kernel<NW, true, CAN_COMP ? 1 : 0>;
    auto k_last_c = radix_scatter_kernel<NW, false, CAN_COMP ? 2 : 0>;
    constexpr bool CAN_PACK = NW == 2;
    auto k_first_p = radix_scatter_kernel<NW, true, CAN_PACK ? 1 : 0, CAN_PACK>;
    auto k_next_p = radix_scatter_kernel<NW, false, 0, CAN_PACK>;
    auto k_last_p = radix_scatter_kernel<NW, false, CAN_PACK ? 2 : 0, CAN_PACK>;
    // CULSH_SORT_NO_PACK=1 keeps key and id apart in a compressed sort (the tests compare the two)
    const char* no_pack = getenv("CULSH_SORT_NO_PACK");
    const bool pack = compressed && CAN_PACK && n <= (1 << RS_PACK_ID_BITS) && !(no_pack && atoi(no_pack) != 0);
    for (auto k : {k_first, k_next, k_first_c, k_last_c, k_first_p, k_next_p, k_last_p})
        CU_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM));
    if (compressed && !CAN_COMP) fail(CULSH_ERR_INTERNAL, "compressed sort needs a key of at most two words");
    const bool chunked = tiles_per_table >= RS_CHUNK_MIN_TILES;
    const int n_chunks = chunked ? (int)ceil_div(tiles_per_table, RS_CHUNK_TILES) : 1;
    uint32_t* chunk_tot = tile_hist + total_tiles * 256;  // [L][n_chunks][256], behind the tile histograms
    const int passes = radix_sort_passes(KB, compressed);
    int cur = 0;
    for (int p = 0; p < passes; ++p) {
        if (compressed && p == 0)
            radix_tile_hist_kernel<NW, CAN_COMP><<<(unsigned)total_tiles, RS_THREADS, 0, s>>>(
                keys[cur], n, tiles_per_table, p, kc.sub, tile_hist);
        else
            radix_tile_hist_kernel<NW, false><<<(unsigned)total_tiles, RS_THREADS, 0, s>>>(
                keys[cur], n, tiles_per_table, pack ? p + 3 : p, 0u, tile_hist);
        KERNEL_CHECK();
        if (chunked) {
            radix_tile_scan_chunk_kernel<<<(unsigned)(L * n_chunks), RS_SCAN_THREADS, 0, s>>>(
                tile_hist, tiles_per_table, n_chunks, chunk_tot);
            KERNEL_CHECK();
            radix_chunk_base_kernel<<<(unsigned)L, 256, 0, s>>>(chunk_tot, n_chunks);
        } else {
            radix_tile_scan_kernel<<<(unsigned)L, RS_SCAN_THREADS, 0, s>>>(tile_hist, tiles_per_table);
        }
        KERNEL_CHECK();
        const bool last = p == passes - 1;
        if (last && c->profiling) cudaEventRecord(c->ev_pass[0], s);
        auto kern = p == 0 ? (compressed ? k_first_c : k_first) : (compressed && last ? k_last_c : k_next);
        if (pack) kern = p == 0 ? k_first_p : (last ? k_last_p : k_next_p);
        kern<<<(unsigned)total_tiles, RS_THREADS, Cfg::SMEM, s>>>(
            keys[cur], vals[cur], keys[cur ^ 1], vals[cur ^ 1], n, tiles_per_table, p, kc, tile_hist,
            chunked ? chunk_tot : nullptr, n_chunks);
        KERNEL_CHECK();
        if (last && c->profiling) cudaEventRecord(c->ev_pass[1], s);
        cur ^= 1;
    }
    return cur;
}

inline size_t radix_sort_tile_words(int n, int L, int NW) {
    const size_t tiles = ceil_div(n, sort_tile_items(NW));
    return (tiles + ceil_div(tiles, (size_t)RS_CHUNK_TILES)) * (size_t)L * 256;  // tile histograms + chunk totals
}

inline int radix_sort_tables(const CtxPtr& c, int NW, uint32_t* keys[2], uint32_t* vals[2], int n,
                             int L, int KB, uint32_t* tile_hist, bool compressed = false,
                             KeyComp kc = KeyComp{0u, 0u}) {
    switch (NW) {
        case 1: return radix_sort_tables_nw<1>(c, keys, vals, n, L, KB, tile_hist, compressed, kc);
        case 2: return radix_sort_tables_nw<2>(c, keys, vals, n, L, KB, tile_hist, compressed, kc);
        case 4: return radix_sort_tables_nw<4>(c, keys, vals, n, L, KB, tile_hist, compressed, kc);
        case 8: return radix_sort_tables_nw<8>(c, keys, vals, n, L, KB, tile_hist, compressed, kc);
        case 16: return radix_sort_tables_nw<16>(c, keys, vals, n, L, KB, tile_hist, compressed, kc);
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
