// Query side: bucket lookup, candidate gather and per-query cross-table dedupe, written
// into the CSR result.  Replaces find_matching_buckets_kernel (core/query.cuh:31-101) and
// query_from_matched_buckets (core/query.cuh:290-478): upstream materialises the raw
// candidates, runs a 32-bit segmented radix sort over them, flags/reduces/scans and
// compacts (about 15 passes over `raw` ints); here each query's bucket lists are merged
// on chip - a shared-memory bitmap over row ids for large candidate sets, a warp-level
// sort for small ones - and each list is read once and its unique ids written once.
#pragma once

#include "common.cuh"
#include "radix_sort.cuh"

namespace culsh_b200 {

// ---------------------------------------------------------------------------------------
// Lookup: one thread per (table, query); binary search over the table's sorted bucket keys.
// matched[q*L + t] = bucket id or -1 (same layout as upstream's matched_bucket_indices).
// ---------------------------------------------------------------------------------------
template <int NW>
__device__ __forceinline__ int compare_keys(const uint32_t* __restrict__ a,
                                            const uint32_t* __restrict__ b) {
#pragma unroll
    for (int w = 0; w < NW; ++w) {
        if (a[w] != b[w]) return a[w] < b[w] ? -1 : 1;
    }
    return 0;
}

template <int NW>
__global__ void __launch_bounds__(256)
lookup_kernel(const uint32_t* __restrict__ qkeys, const uint8_t* __restrict__ q_ovf, int n_q, int L,
              const uint32_t* __restrict__ bucket_keys, const int32_t* __restrict__ table_offsets,
              int32_t* __restrict__ matched) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_q * L) return;
    const int t = (int)(idx / n_q);
    const int q = (int)(idx - (size_t)t * n_q);
    uint32_t key[NW];
    load_key<NW>(qkeys + idx * NW, key);
    int lo = table_offsets[t], hi = table_offsets[t + 1] - 1;
    int found = -1;
    if (q_ovf && q_ovf[idx]) hi = lo - 1;  // value outside the index's narrow range: no bucket
    while (lo <= hi) {
        int mid = lo + ((hi - lo) >> 1);
        int c = compare_keys<NW>(key, bucket_keys + (size_t)mid * NW);
        if (c == 0) { found = mid; break; }
        if (c < 0) hi = mid - 1; else lo = mid + 1;
    }
    matched[(size_t)q * L + t] = found;
}

// ---------------------------------------------------------------------------------------
// Raw (pre-dedupe) candidate count per query; queries above the small-path limit are
// appended to big_list.
// ---------------------------------------------------------------------------------------
// largest raw count handled by the warp path (1024: 32 ids per lane in the sort network; with 512
// the queries of 513 - 1024 ids of a 12.5M-row shard took a CTA each on the sort path: 0.77 -> 0.50 ms
// per 10k queries, the 10M-row self-join, all below 512, is unchanged)
constexpr int SMALL_MAX = 1024;

constexpr int RC_BATCH = 8;  // sixteen measured no faster on the 10M-row self-join
// counters[0] = queries for the bitmap path (big_list), counters[1] = queries for the
// shared-memory sort path (mid_list; only used when mid_max > SMALL_MAX)
__global__ void __launch_bounds__(256)
raw_count_kernel(const int32_t* __restrict__ matched, const int32_t* __restrict__ bucket_offsets,
                 int n_q, int L, uint64_t* __restrict__ raw_cnt, uint32_t* __restrict__ big_list,
                 uint32_t* __restrict__ mid_list, uint32_t* __restrict__ counters, int mid_max,
                 int2* __restrict__ bounds /* or null: [n_q][L] list bounds for the warp path */) {
    int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= n_q) return;
    int2* bq = bounds ? bounds + (size_t)q * L : nullptr;
    // RC_BATCH tables at a time, branch-free, so that the dependent loads (bucket id -> bounds) of
    // different tables are in flight together
    uint64_t c = 0;
    const int32_t* mq = matched + (size_t)q * L;
    int t = 0;
    for (; t + RC_BATCH <= L; t += RC_BATCH) {
        int b[RC_BATCH], lo[RC_BATCH], hi[RC_BATCH];
#pragma unroll
        for (int j = 0; j < RC_BATCH; ++j) b[j] = mq[t + j];
#pragma unroll
        for (int j = 0; j < RC_BATCH; ++j) {
            const int bb = max(b[j], 0);
            lo[j] = bucket_offsets[bb];
            hi[j] = bucket_offsets[bb + 1];
        }
#pragma unroll
        for (int j = 0; j < RC_BATCH; ++j) {
            c += b[j] >= 0 ? (uint64_t)(hi[j] - lo[j]) : 0ull;
            if (bq) bq[t + j] = b[j] >= 0 ? make_int2(lo[j], hi[j]) : make_int2(0, 0);
        }
    }
    for (; t < L; ++t) {
        const int b = mq[t];
        int lo = 0, hi = 0;
        if (b >= 0) { lo = bucket_offsets[b]; hi = bucket_offsets[b + 1]; }
        c += (uint64_t)(hi - lo);
        if (bq) bq[t] = make_int2(lo, hi);
    }
    raw_cnt[q] = c;
    if (c > SMALL_MAX) {
        if (c <= (uint64_t)mid_max) mid_list[atomicAdd(&counters[1], 1u)] = (uint32_t)q;
        else big_list[atomicAdd(&counters[0], 1u)] = (uint32_t)q;
    }
}

// ---------------------------------------------------------------------------------------
// Small path: one warp per query, raw <= SMALL_MAX.  The ids are gathered into the warp's slice
// of shared memory, sorted in registers (bitonic, shuffles), made unique and compacted by
// ballots.  Output goes to tmp[raw_off[q] ...].
// ---------------------------------------------------------------------------------------
constexpr int SM_THREADS = 256;
constexpr int SM_WARPS = SM_THREADS / 32;

// Bitonic sort of 32*E ids held E per lane (position p = 32*e + lane lives in v[e] of `lane`),
// then adjacent-unique and ballot compaction to out[]; returns the number of unique ids.
// Exchanges at distance >= 32 stay inside a lane, shorter ones are one shuffle each; everything
// is unrolled at compile time, so the ids never leave registers.
template <int E>
__device__ __forceinline__ int warp_sort_unique(const int32_t* __restrict__ buf, int r, int lane,
                                                int32_t* __restrict__ out) {
    int32_t v[E];
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const int p = 32 * e + lane;
        v[e] = p < r ? buf[p] : 0x7FFFFFFF;
    }
#pragma unroll
    for (int ksz = 2; ksz <= 32 * E; ksz <<= 1) {
#pragma unroll
        for (int j = ksz >> 1; j > 0; j >>= 1) {
            if (j >= 32) {
                const int je = j >> 5;
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    if ((e & je) == 0) {
                        const bool up = ((32 * e + lane) & ksz) == 0;
                        const int32_t a = v[e], b = v[e | je];
                        const bool sw = (a > b) == up;
                        v[e] = sw ? b : a;
                        v[e | je] = sw ? a : b;
                    }
                }
            } else {
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    const bool up = ((32 * e + lane) & ksz) == 0;
                    const int32_t other = __shfl_xor_sync(0xFFFFFFFFu, v[e], j);
                    const bool keep_min = ((lane & j) == 0) == up;
                    v[e] = keep_min ? min(v[e], other) : max(v[e], other);
                }
            }
        }
    }
    int written = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        int32_t prev = __shfl_up_sync(0xFFFFFFFFu, v[e], 1);
        if (e > 0) {
            const int32_t last = __shfl_sync(0xFFFFFFFFu, v[e - 1], 31);
            if (lane == 0) prev = last;
        }
        const int p = 32 * e + lane;
        const bool keep = p < r && (p == 0 || prev != v[e]);
        const uint32_t mask = __ballot_sync(0xFFFFFFFFu, keep);
        if (keep) out[written + __popc(mask & ((1u << lane) - 1))] = v[e];
        written += __popc(mask);
    }
    return written;
}

__global__ void __launch_bounds__(SM_THREADS)
dedupe_small_kernel(const int32_t* __restrict__ matched, const int32_t* __restrict__ bucket_offsets,
                    const int32_t* __restrict__ cand, const uint64_t* __restrict__ raw_cnt,
                    const uint64_t* __restrict__ raw_off, int n_q, int L, int32_t* __restrict__ tmp,
                    uint64_t* __restrict__ uniq_cnt,
                    const int2* __restrict__ bounds /* or null: list bounds kept by raw_count_kernel */) {
    __shared__ int32_t s_buf[SM_WARPS][SMALL_MAX];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int32_t* buf = s_buf[warp];
    for (int q = blockIdx.x * SM_WARPS + warp; q < n_q; q += gridDim.x * SM_WARPS) {
        const uint64_t r64 = raw_cnt[q];
        if (r64 > SMALL_MAX) continue;  // the block path owns it
        const int r = (int)r64;
        if (r == 0) {
            if (lane == 0) uniq_cnt[q] = 0;
            continue;
        }
        int m = 32;
        while (m < r) m <<= 1;
        // gather the bucket lists: 32 tables at a time, one lane per table, so the dependent loads
        // (bucket id -> list bounds -> ids) of all tables overlap.  A lane copies up to four ids
        // of its own list with independent loads; longer lists are copied by the whole warp.
        int fill = 0;
        for (int t0 = 0; t0 < L; t0 += 32) {
            const int t = t0 + lane;
            int s = 0, e = 0;
            if (bounds) {  // one coalesced read instead of two dependent, scattered ones
                if (t < L) { const int2 be = bounds[(size_t)q * L + t]; s = be.x; e = be.y; }
            } else {
                const int b = t < L ? matched[(size_t)q * L + t] : -1;
                if (b >= 0) { s = bucket_offsets[b]; e = bucket_offsets[b + 1]; }
            }
            const int len = e - s;
            int inc = len;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                if (lane >= o) inc += x;
            }
            const int dst0 = fill + inc - len;
            int32_t v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = i < len ? cand[s + i] : 0;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (i < len) buf[dst0 + i] = v[i];
            uint32_t longer = __ballot_sync(0xFFFFFFFFu, len > 4);
            while (longer) {
                const int src = __ffs(longer) - 1;
                longer &= longer - 1;
                const int ls = __shfl_sync(0xFFFFFFFFu, s, src);
                const int ll = __shfl_sync(0xFFFFFFFFu, len, src);
                const int ld = __shfl_sync(0xFFFFFFFFu, dst0, src);
                for (int i = 4 + lane; i < ll; i += 32) buf[ld + i] = cand[ls + i];
            }
            fill += __shfl_sync(0xFFFFFFFFu, inc, 31);
        }
        __syncwarp();
        int32_t* out = tmp + raw_off[q];
        int written;
        if (m <= 32) written = warp_sort_unique<1>(buf, r, lane, out);
        else if (m <= 64) written = warp_sort_unique<2>(buf, r, lane, out);
        else if (m <= 128) written = warp_sort_unique<4>(buf, r, lane, out);
        else if (m <= 256) written = warp_sort_unique<8>(buf, r, lane, out);
        else if (m <= 512) written = warp_sort_unique<16>(buf, r, lane, out);
        else written = warp_sort_unique<32>(buf, r, lane, out);
        if (lane == 0) uniq_cnt[q] = (uint64_t)written;
        __syncwarp();
    }
}

// ---------------------------------------------------------------------------------------
// Sort path: one CTA per query of mid_list (SMALL_MAX < raw <= MID_MAX), used when the index
// has so many rows that a bitmap would need several windows.  The ids are gathered into
// shared memory, LSD radix sorted there on 8-bit digits (as many passes as the row ids have
// bytes), then adjacent duplicates are dropped while writing out.
// ---------------------------------------------------------------------------------------
constexpr int MS_THREADS = 512;
constexpr int MS_WARPS = MS_THREADS / 32;
constexpr int MS_IPT = 16;
constexpr int MID_MAX = MS_THREADS * MS_IPT;  // 8192

inline size_t sort_path_smem_bytes() {
    return sizeof(uint32_t) * (2 * (size_t)MID_MAX + MS_WARPS * 256 + 256 + 64);
}

__global__ void __launch_bounds__(MS_THREADS)
dedupe_sort_kernel(const uint32_t* __restrict__ mid_list, const int32_t* __restrict__ matched,
                   const int32_t* __restrict__ bucket_offsets, const int32_t* __restrict__ cand,
                   const uint64_t* __restrict__ raw_cnt, const uint64_t* __restrict__ raw_off, int L,
                   int id_bytes, int32_t* __restrict__ tmp, uint64_t* __restrict__ uniq_cnt) {
    extern __shared__ __align__(16) uint32_t s_ms[];
    uint32_t* bufA = s_ms;
    uint32_t* bufB = bufA + MID_MAX;
    uint32_t* s_whist = bufB + MID_MAX;       // [MS_WARPS][256]
    uint32_t* s_binstart = s_whist + MS_WARPS * 256;  // [256]
    uint32_t* s_misc = s_binstart + 256;      // [64]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q = (int)mid_list[blockIdx.x];
    const int r = (int)raw_cnt[q];
    // gather the bucket lists one after another
    int fill = 0;
    for (int t = 0; t < L; ++t) {
        const int b = matched[(size_t)q * L + t];
        if (b < 0) continue;
        const int s = bucket_offsets[b], e = bucket_offsets[b + 1];
        for (int i = s + tid; i < e; i += MS_THREADS) bufA[fill + (i - s)] = (uint32_t)cand[i];
        fill += e - s;
    }
    __syncthreads();
    const int n_iter = (r + MS_THREADS - 1) / MS_THREADS;  // uniform
    uint32_t* src = bufA;
    uint32_t* dst = bufB;
    for (int p = 0; p < id_bytes; ++p) {
        for (int i = tid; i < MS_WARPS * 256; i += MS_THREADS) s_whist[i] = 0;
        __syncthreads();
        uint32_t key[MS_IPT];
        uint16_t rank[MS_IPT];
#pragma unroll
        for (int i = 0; i < MS_IPT; ++i) {
            if (i < n_iter) {
                const int li = warp * (32 * n_iter) + i * 32 + lane;
                const bool valid = li < r;
                key[i] = valid ? src[li] : 0u;
                const uint32_t d = valid ? ((key[i] >> (8 * p)) & 0xFFu) : 0x100u;
                const uint32_t peers = __match_any_sync(0xFFFFFFFFu, d);
                const int leader = __ffs(peers) - 1;
                const uint32_t below = __popc(peers & ((1u << lane) - 1));
                uint32_t old = 0;
                if (valid && lane == leader) old = atomicAdd(&s_whist[warp * 256 + d], (uint32_t)__popc(peers));
                old = __shfl_sync(0xFFFFFFFFu, old, leader);
                rank[i] = (uint16_t)(old + below);
            }
        }
        __syncthreads();
        if (tid < 256) {
            uint32_t cnt = 0;
#pragma unroll
            for (int w = 0; w < MS_WARPS; ++w) {
                uint32_t x = s_whist[w * 256 + tid];
                s_whist[w * 256 + tid] = cnt;
                cnt += x;
            }
            uint32_t inc = cnt;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                if (lane >= o) inc += x;
            }
            if (lane == 31) s_misc[warp] = inc;
            s_binstart[tid] = inc - cnt;  // exclusive inside the warp; warp bases added below
        }
        __syncthreads();
        if (tid < 256) {
            uint32_t wb = 0;
            for (int w = 0; w < warp; ++w) wb += s_misc[w];
            s_binstart[tid] += wb;
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < MS_IPT; ++i) {
            if (i < n_iter) {
                const int li = warp * (32 * n_iter) + i * 32 + lane;
                if (li < r) {
                    const uint32_t d = (key[i] >> (8 * p)) & 0xFFu;
                    dst[s_binstart[d] + s_whist[warp * 256 + d] + rank[i]] = key[i];
                }
            }
        }
        __syncthreads();
        uint32_t* tsw = src; src = dst; dst = tsw;
    }
    // adjacent-unique + block compaction, ascending order kept
    int32_t* out = tmp + raw_off[q];
    uint32_t written = 0;  // uniform
    for (int i0 = 0; i0 < r; i0 += MS_THREADS) {
        const int i = i0 + tid;
        bool keep = false;
        uint32_t v = 0;
        if (i < r) {
            v = src[i];
            keep = i == 0 || src[i - 1] != v;
        }
        const uint32_t mask = __ballot_sync(0xFFFFFFFFu, keep);
        if (lane == 0) s_misc[32 + warp] = __popc(mask);
        __syncthreads();
        uint32_t wb = 0, tot = 0;
        for (int w = 0; w < MS_WARPS; ++w) {
            const uint32_t x = s_misc[32 + w];
            if (w < warp) wb += x;
            tot += x;
        }
        if (keep) out[written + wb + __popc(mask & ((1u << lane) - 1))] = (int32_t)v;
        written += tot;
        __syncthreads();
    }
    if (tid == 0) uniq_cnt[q] = (uint64_t)written;
}

// ---------------------------------------------------------------------------------------
// Block path: one CTA per query of big_list.  Row ids are marked in a shared-memory bitmap
// covering a window of `window_bits` ids; windows are visited in increasing order, and as
// every bucket list is ascending each window's slice of a list is found by binary search.
// A pop-count scan of the bitmap then emits the window's ids sorted and unique.
// ---------------------------------------------------------------------------------------
constexpr int BM_THREADS = 1024;
constexpr int BM_WARPS = BM_THREADS / 32;
constexpr int BM_MAX_L = 1024;   // lists kept in shared memory
constexpr int BM_STAGE = 256;    // ids staged per warp before a coalesced flush

__device__ __forceinline__ int lower_bound_i32(const int32_t* __restrict__ a, int lo, int hi, int32_t v) {
    while (lo < hi) {
        int mid = lo + ((hi - lo) >> 1);
        if (a[mid] < v) lo = mid + 1; else hi = mid;
    }
    return lo;
}

inline size_t bitmap_smem_bytes(int window_bits) {
    return (size_t)window_bits / 8 + 3 * BM_MAX_L * sizeof(int) + (size_t)BM_WARPS * BM_STAGE * sizeof(int32_t);
}


// Marks the ids of Lg ascending lists [s_lo[t], s_we[t]) of `cand` in the bitmap.  The lists are
// laid end to end (s_pre = exclusive prefix of their lengths) and that flat sequence is cut
// into equal stretches, one per warp, so the work is balanced however uneven the lists are.
// Must be called by all BM_THREADS threads; s_lo / s_we must be visible (barrier before).
template <int NT = BM_THREADS>
__device__ __forceinline__ void mark_lists_flat(uint32_t* __restrict__ bitmap, const int32_t* __restrict__ cand,
                                                const int* __restrict__ s_lo, const int* __restrict__ s_we,
                                                int* __restrict__ s_pre, uint32_t* __restrict__ s_wtot, int Lg,
                                                int win_lo) {
    constexpr int NWARP = NT / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int len = tid < Lg ? s_we[tid] - s_lo[tid] : 0;
    int inc = len;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        int x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += x;
    }
    if (lane == 31) s_wtot[warp] = (uint32_t)inc;
    __syncthreads();
    int base = 0, total = 0;
    for (int w = 0; w < NWARP; ++w) {
        const int x = (int)s_wtot[w];
        if (w < warp) base += x;
        total += x;
    }
    if (tid < Lg) s_pre[tid] = base + inc - len;
    __syncthreads();
    // Each warp takes a contiguous stretch of the flat sequence; a lane's list index only moves
    // forward (one binary search per warp, then cheap advances), loads stay coalesced and MK of
    // them are in flight per lane.
    constexpr int MK = 20;
    const int per_warp = (((total + NWARP - 1) / NWARP) + 31) & ~31;
    const int w_begin = warp * per_warp, w_end = min(total, w_begin + per_warp);
    if (w_begin < w_end) {
        int t = 0;
        {
            int a = 0, b = Lg - 1;
            while (a < b) {  // largest t with s_pre[t] <= w_begin
                const int mid = (a + b + 1) >> 1;
                if (s_pre[mid] <= w_begin) a = mid; else b = mid - 1;
            }
            t = a;
        }
        for (int e0 = w_begin + lane; e0 - lane < w_end; e0 += 32 * MK) {
            int32_t v[MK];
#pragma unroll
            for (int j = 0; j < MK; ++j) {
                const int e = e0 + 32 * j;
                v[j] = -1;
                if (e < w_end) {
                    while (t + 1 < Lg && s_pre[t + 1] <= e) ++t;
                    v[j] = cand[s_lo[t] + (e - s_pre[t])];
                }
            }
#pragma unroll
            for (int j = 0; j < MK; ++j) {
                if (v[j] >= 0) {
                    const uint32_t id = (uint32_t)(v[j] - win_lo);
                    atomicOr(&bitmap[id >> 5], 1u << (id & 31));
                }
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(BM_THREADS)
dedupe_bitmap_kernel(const uint32_t* __restrict__ big_list, const int32_t* __restrict__ matched,
                     const int32_t* __restrict__ bucket_offsets, const int32_t* __restrict__ cand,
                     const uint64_t* __restrict__ raw_off, int L, int n_rows, int window_bits,
                     int32_t* __restrict__ tmp, uint64_t* __restrict__ uniq_cnt) {
    extern __shared__ __align__(16) uint32_t s_dyn[];
    uint32_t* bitmap = s_dyn;                                       // [window_bits / 32]
    int* s_lo = reinterpret_cast<int*>(bitmap + window_bits / 32);  // [Lc] slice start (global position)
    int* s_hi = s_lo + BM_MAX_L;                                    // [Lc] end of list
    int* s_we = s_hi + BM_MAX_L;                                    // [Lc] end of the window's slice
    int32_t* s_stage = reinterpret_cast<int32_t*>(s_we + BM_MAX_L); // [BM_WARPS][BM_STAGE]
    __shared__ uint32_t s_wtot[BM_WARPS];
    __shared__ int s_any;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int q = (int)big_list[blockIdx.x];
    const int words = window_bits / 32;
    int32_t* out = tmp + raw_off[q];
    int32_t* stage = s_stage + warp * BM_STAGE;
    uint32_t written = 0;  // uniform across the block

    // L may exceed BM_MAX_L: tables are processed in groups inside the window loop, because
    // every group marks the bitmap of the same window.
    for (int win_lo = 0; win_lo < n_rows; win_lo += window_bits) {
        const int win_hi = min(n_rows, win_lo + window_bits);
        bool cleared = false;
        for (int g0 = 0; g0 < L; g0 += BM_MAX_L) {
            const int Lg = min(BM_MAX_L, L - g0);
            if (tid == 0) s_any = 0;
            __syncthreads();
            for (int t = tid; t < Lg; t += BM_THREADS) {
                int b = matched[(size_t)q * L + g0 + t];
                int lo = 0, hi = 0, we = 0;
                if (b >= 0) {
                    int s = bucket_offsets[b], e = bucket_offsets[b + 1];
                    if (n_rows <= window_bits) { lo = s; we = e; }
                    else {
                        lo = lower_bound_i32(cand, s, e, win_lo);
                        we = lower_bound_i32(cand, lo, e, win_hi);
                    }
                    hi = e;
                    if (we > lo) s_any = 1;
                }
                s_lo[t] = lo; s_hi[t] = hi; s_we[t] = we;
            }
            __syncthreads();
            const int any = s_any;
            __syncthreads();  // s_any is rewritten at the top of the next group
            if (!any) continue;  // uniform
            if (!cleared) {
                uint4* b4 = reinterpret_cast<uint4*>(bitmap);
                for (int w = tid; w < words / 4; w += BM_THREADS) b4[w] = make_uint4(0, 0, 0, 0);
                cleared = true;
                __syncthreads();
            }
            mark_lists_flat(bitmap, cand, s_lo, s_we, s_hi, s_wtot, Lg, win_lo);
        }
        if (!cleared) continue;  // uniform: nothing in this window
        // ---- pop-count scan.  The window is cut into groups of 128 words (one uint4 per lane);
        // warp w owns groups [w*gpw, (w+1)*gpw). ----
        const uint4* b4 = reinterpret_cast<const uint4*>(bitmap);
        const int groups = words / 128;
        const int gpw = (groups + BM_WARPS - 1) / BM_WARPS;
        const int g_begin = warp * gpw, g_end = min(groups, g_begin + gpw);
        uint32_t wsum = 0;
        for (int g = g_begin; g < g_end; ++g) {
            const uint4 v = b4[g * 32 + lane];
            wsum += __popc(v.x) + __popc(v.y) + __popc(v.z) + __popc(v.w);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xFFFFFFFFu, wsum, o);
        if (lane == 0) s_wtot[warp] = wsum;
        __syncthreads();
        uint32_t wbase = 0, wtotal = 0;
        for (int i = 0; i < BM_WARPS; ++i) {
            uint32_t x = s_wtot[i];
            if (i < warp) wbase += x;
            wtotal += x;
        }
        // ---- emit: each lane expands its four words; ids are staged in the warp's slice of
        // shared memory and flushed in coalesced runs; a group denser than the stage is
        // written directly ----
        uint32_t out_pos = written + wbase;  // global position of stage[0]
        uint32_t fill = 0;
        for (int g = g_begin; g < g_end; ++g) {
            const uint4 v = b4[g * 32 + lane];
            const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
            const uint32_t c = __popc(v.x) + __popc(v.y) + __popc(v.z) + __popc(v.w);
            uint32_t inc = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                uint32_t x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                if (lane >= o) inc += x;
            }
            const uint32_t tot = __shfl_sync(0xFFFFFFFFu, inc, 31);
            if (tot == 0) continue;
            const int32_t id0 = win_lo + (g * 128 + lane * 4) * 32;
            if (tot > BM_STAGE || fill + tot > BM_STAGE) {  // flush what is staged
                __syncwarp();
                for (uint32_t i = lane; i < fill; i += 32) out[out_pos + i] = stage[i];
                out_pos += fill;
                fill = 0;
                __syncwarp();
            }
            int32_t* dst = tot > BM_STAGE ? out + out_pos + (inc - c) : stage + fill + (inc - c);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t bits = wv[j];
                while (bits) {
                    const int b = __ffs(bits) - 1;
                    bits &= bits - 1;
                    *dst++ = id0 + j * 32 + b;
                }
            }
            if (tot > BM_STAGE) out_pos += tot; else fill += tot;
        }
        __syncwarp();
        for (uint32_t i = lane; i < fill; i += 32) out[out_pos + i] = stage[i];
        written += wtotal;
        __syncthreads();
    }
    if (tid == 0) uniq_cnt[q] = (uint64_t)written;
}

// ---------------------------------------------------------------------------------------
// Chained single-pass dedupe for query sets dominated by large candidate sets: CTAs take
// (query, window) tickets from an atomic counter IN CSR ORDER, so a CTA only ever waits on CTAs
// that started before it.  After counting its unique ids a CTA publishes the count, obtains the
// sum over all earlier tickets from a chained look-back over `status` (a warp reads 32
// predecessors per round), and writes its sorted ids straight at their final CSR position - no
// scratch copy, no compaction pass.  Queries that took the warp / sort paths have their count
// and ids in `tmp` already; their first ticket joins the chain with that count and copies the
// ids, their other tickets publish zero.
// status word: bits 62-63 flag (0 empty, 1 own count, 2 inclusive prefix), low 62 bits value.
// Every wait is bounded; on expiry DEV_ERR_LOOKBACK_TIMEOUT is recorded and the CTA goes on.
// ---------------------------------------------------------------------------------------
constexpr unsigned long long CH_FLAG_AGG = 1ull << 62;
constexpr unsigned long long CH_FLAG_INC = 2ull << 62;
constexpr unsigned long long CH_VAL_MASK = (1ull << 62) - 1;
constexpr int CH_SPIN_LIMIT = 1 << 22;

__device__ __forceinline__ unsigned long long ld_volatile_u64(const unsigned long long* p) {
    return *reinterpret_cast<const volatile unsigned long long*>(p);
}

// Executed by warp 0 of the CTA that owns ticket q; returns the exclusive prefix.
// `publish` stores this query's own count first (done once); with `blocking` false the walk
// gives up (returns false, nothing published) as soon as a needed predecessor is missing.
__device__ __forceinline__ bool chain_exclusive_prefix(unsigned long long* status, int q,
                                                       unsigned long long own, int lane, int* d_error,
                                                       bool publish, bool blocking, unsigned long long& excl_out) {
    unsigned long long* mine = status + q;
    excl_out = 0ull;
    if (q == 0) {
        if (lane == 0) *reinterpret_cast<volatile unsigned long long*>(mine) = CH_FLAG_INC | own;
        return true;
    }
    if (publish && lane == 0) *reinterpret_cast<volatile unsigned long long*>(mine) = CH_FLAG_AGG | own;
    unsigned long long excl = 0;
    int j = q - 1;
    bool done = false;
    while (!done) {
        const int idx = j - lane;
        unsigned long long s = idx >= 0 ? ld_volatile_u64(status + idx) : CH_FLAG_INC;  // before query 0: prefix 0
        int spins = 0;
        while (__any_sync(0xFFFFFFFFu, (s >> 62) == 0)) {  // someone in the window has not published yet
            if (!blocking) {
                // usable only if a prefix sits nearer than the first missing entry
                const uint32_t miss = __ballot_sync(0xFFFFFFFFu, (s >> 62) == 0);
                const uint32_t inc = __ballot_sync(0xFFFFFFFFu, (s >> 62) == 2);
                if (inc && (__ffs(inc) < __ffs(miss))) break;
                return false;
            }
            if (++spins > CH_SPIN_LIMIT) {
                if (lane == 0) atomicOr(d_error, DEV_ERR_LOOKBACK_TIMEOUT);
                s |= CH_FLAG_INC;  // give up: treat as a prefix so that the walk ends
                break;
            }
            if (spins > 16) __nanosleep(64);
            if ((s >> 62) == 0) s = ld_volatile_u64(status + idx);
        }
        const uint32_t inc_mask = __ballot_sync(0xFFFFFFFFu, (s >> 62) == 2);
        const int stop = inc_mask ? __ffs(inc_mask) - 1 : 32;  // nearest predecessor holding a prefix
        unsigned long long v = lane <= stop ? (s & CH_VAL_MASK) : 0ull;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
        excl += v;
        done = inc_mask != 0;
        j -= 32;
    }
    if (lane == 0) *reinterpret_cast<volatile unsigned long long*>(mine) = CH_FLAG_INC | ((excl + own) & CH_VAL_MASK);
    excl_out = excl;
    return true;
}

// ---------------------------------------------------------------------------------------
// Rank form of the chained kernel.  The row range is cut into n_win windows of window_bits rows
// and one CTA handles one (query, window) pair, tickets in (query, window) order - the order of
// the ids in the CSR.  A CTA
//   1. narrows every bucket list (ascending row ids) to its window with a 32-way warp search,
//   2. marks the ids of those slices in a shared-memory bitmap,
//   3. scans the bitmap once: pop-count prefix per 32-bit word (16 bits, inside blocks of 512
//      rows), a base per block and the number of unique ids, which it publishes to the chain,
//   4. goes over the ids a second time (from registers when a warp's share fits one batch, else
//      from L2): the rank of an id among the unique ids of the window is base[block] +
//      prefix[word] + popc(bits below it), so the id is dropped at stage[rank] in shared memory -
//      duplicates write the same value to the same slot,
//   5. resolves its exclusive prefix from the chain and copies the staged ids, now sorted and
//      unique, to their final CSR position with coalesced stores.
// Work is proportional to the candidates (two walks) plus one pass over the window, there is no
// per-bit emission loop and no scratch copy; windows of 32 KB let several CTAs share an SM so the
// dependent loads of one overlap the work of the others.  A window with more unique ids than the
// stage holds repeats steps 4-5 per stage-sized chunk of ranks.
// ---------------------------------------------------------------------------------------
constexpr int CW_MAX_L = 256;    // lists per query kept in shared memory (<= threads per CTA)

inline size_t chain_window_smem_bytes(int window_bits, int stage_ids) {
    // bitmap (1 bit per row) + 16-bit prefix per 32-bit word + 32-bit base per 512 rows + stage + lists
    return (size_t)window_bits / 8 + (size_t)window_bits / 16 + (size_t)window_bits / 128 +
           (size_t)stage_ids * sizeof(int32_t) + (3 * CW_MAX_L + 1) * sizeof(int);
}

// First position p in [lo, hi) with a[p] >= target (hi if there is none).  Called by a full warp.
__device__ __forceinline__ int warp_lower_bound(const int32_t* __restrict__ a, int lo, int hi, int32_t target,
                                                int lane) {
    while (hi - lo > 32) {
        const int len = hi - lo;
        const int p = lo + (int)(((long long)(lane + 1) * len) / 33);  // 32 distinct probes inside (lo, hi)
        const uint32_t below = __ballot_sync(0xFFFFFFFFu, a[p] < target);  // lanes 0..c-1
        const int c = __popc(below);
        const int p_prev = __shfl_sync(0xFFFFFFFFu, p, max(c - 1, 0));
        const int p_next = __shfl_sync(0xFFFFFFFFu, p, min(c, 31));
        if (c > 0) lo = p_prev + 1;
        if (c < 32) hi = p_next;
    }
    const bool below = lo + lane < hi && a[lo + lane] < target;
    return lo + __popc(__ballot_sync(0xFFFFFFFFu, below));
}

// Walk over the Lg lists [s_lo[t], s_lo[t] + len_t) laid end to end (s_pre[t] = exclusive prefix
// of the lengths, s_pre[Lg] = total).  The flat sequence is cut into equal stretches, one per warp;
// a batch is 32 * MK consecutive elements of the stretch: lanes read consecutive elements
// (coalesced) and every lane has MK independent loads in flight.  The loaded ids are handed back
// untouched (-1 past the end) so that the caller decides when to consume them.
template <int NT, int MK>
struct ListWalk {
    int t, next, base, w_begin, w_end, per_warp;

    __device__ __forceinline__ void init(const int* __restrict__ s_lo, const int* __restrict__ s_pre, int Lg) {
        constexpr int NWARP = NT / 32;
        const int warp = threadIdx.x >> 5;
        const int total = s_pre[Lg];
        per_warp = (((total + NWARP - 1) / NWARP) + 31) & ~31;
        w_begin = warp * per_warp;
        w_end = min(total, w_begin + per_warp);
        t = 0; next = 0; base = 0;
        if (w_begin < w_end) {
            int a = 0, b = Lg - 1;
            while (a < b) {  // largest t with s_pre[t] <= w_begin
                const int mid = (a + b + 1) >> 1;
                if (s_pre[mid] <= w_begin) a = mid; else b = mid - 1;
            }
            t = a;
            next = s_pre[t + 1];        // first flat position past list t
            base = s_lo[t] - s_pre[t];  // flat position -> position in cand
        }
    }
    // batch whose first element (of lane 0) is the flat position e0 - lane
    __device__ __forceinline__ void load(const int32_t* __restrict__ cand, const int* __restrict__ s_lo,
                                         const int* __restrict__ s_pre, int e0, int32_t (&v)[MK]) {
#pragma unroll
        for (int j = 0; j < MK; ++j) {
            const int e = e0 + 32 * j;
            v[j] = -1;
            if (e < w_end) {
                while (e >= next) {  // e < total, so t stays below Lg
                    ++t;
                    next = s_pre[t + 1];
                    base = s_lo[t] - s_pre[t];
                }
                v[j] = cand[base + e];
            }
        }
    }
};

// Slice of every bucket list that falls into every window: slices[(q * n_win + w) * L + t] =
// [a, b) in cand.  One thread per (query, list, window) finds the window's lower boundary with a
// binary search and writes it as the start of its own slice and the end of the previous one;
// with a million independent searches in flight the dependent loads cost nothing, whereas
// inside the chained kernel they would sit on the critical path of every CTA.
__global__ void __launch_bounds__(256)
slice_lists_kernel(const int32_t* __restrict__ matched, const int32_t* __restrict__ bucket_offsets,
                   const int32_t* __restrict__ cand, const uint64_t* __restrict__ raw_cnt, int n_q, int L,
                   int window_bits, int n_win, int mid_max, int2* __restrict__ slices) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_q * L * n_win) return;
    const int w = (int)(idx % n_win);
    const size_t pair = idx / n_win;  // q * L + t
    const int q = (int)(pair / L), t = (int)(pair - (size_t)q * L);
    const uint64_t raw = raw_cnt[q];
    if (!(raw > (uint64_t)SMALL_MAX && raw > (uint64_t)mid_max)) return;  // not a bitmap-path query
    const int b = matched[pair];
    int lo = 0, we = 0;
    if (b >= 0) { lo = bucket_offsets[b]; we = bucket_offsets[b + 1]; }
    int* flat = reinterpret_cast<int*>(slices);
    const size_t mine = (((size_t)q * n_win + w) * L + t) * 2;
    int a = lo;
    if (w > 0) {
        const long long bound = (long long)w * window_bits;
        a = bound > 0x7FFFFFFFll ? we : lower_bound_i32(cand, lo, we, (int32_t)bound);
        flat[mine - (size_t)L * 2 + 1] = a;  // end of the previous window's slice
    }
    flat[mine] = a;
    if (w == n_win - 1) flat[mine + 1] = we;
}

template <int NT, int MK>
__global__ void __launch_bounds__(NT)
dedupe_chained_rank_kernel(const int32_t* __restrict__ matched, const int32_t* __restrict__ bucket_offsets,
                           const int32_t* __restrict__ cand, const uint64_t* __restrict__ raw_cnt,
                           const uint64_t* __restrict__ raw_off, int n_q, int L, int n_rows, int window_bits,
                           int n_win, int stage_ids, int mid_max, const int2* __restrict__ slices /* or null */,
                           const int32_t* __restrict__ tmp,
                           unsigned long long* __restrict__ status, uint32_t* __restrict__ ticket,
                           int32_t* __restrict__ out_indices, uint64_t* __restrict__ counts,
                           uint64_t* __restrict__ offsets, int* __restrict__ d_error) {
    constexpr int NWARP = NT / 32;
    extern __shared__ __align__(16) uint32_t s_dyn[];
    const int n32 = window_bits / 32;      // a multiple of 128
    const int n_blocks = n32 / 16;         // blocks of 512 rows
    uint32_t* bm32 = s_dyn;                                                    // [n32] bitmap
    uint16_t* pre16 = reinterpret_cast<uint16_t*>(bm32 + n32);                // [n32] set bits before the word, inside its block
    uint32_t* base32 = reinterpret_cast<uint32_t*>(pre16 + n32);              // [n_blocks] set bits before the block
    int32_t* stage = reinterpret_cast<int32_t*>(base32 + n_blocks);          // [stage_ids]
    int* s_lo = reinterpret_cast<int*>(stage + stage_ids);                    // [L] slice start in cand
    int* s_we = s_lo + CW_MAX_L;                                               // [L] slice end
    int* s_pre = s_we + CW_MAX_L;                                              // [L + 1] prefix of slice lengths
    __shared__ uint32_t s_wtot[NWARP];
    __shared__ unsigned long long s_excl;
    __shared__ int s_tk;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) s_tk = (int)atomicAdd(ticket, 1u);
    __syncthreads();
    const int tk = s_tk;
    const long long n_tk = (long long)n_q * n_win;
    if (tk >= n_tk) return;
    const int q = tk / n_win, w = tk - q * n_win;
    const bool last_ticket = tk == n_tk - 1;
    const uint64_t raw = raw_cnt[q];
    const bool big = raw > (uint64_t)SMALL_MAX && raw > (uint64_t)mid_max;

    if (!big) {  // count and ids are in tmp already: window 0 joins the chain with them and copies
        if (w > 0 && !last_ticket) {
            if (tid == 0) *reinterpret_cast<volatile unsigned long long*>(status + tk) = CH_FLAG_AGG;
            return;
        }
        const unsigned long long c = w == 0 ? counts[q] : 0ull;
        if (warp == 0) {
            unsigned long long e;
            chain_exclusive_prefix(status, tk, c, lane, d_error, true, true, e);
            if (lane == 0) s_excl = e;
        }
        __syncthreads();
        const unsigned long long excl = s_excl;
        const int32_t* src = tmp + raw_off[q];
        for (unsigned long long i = tid; i < c; i += NT) out_indices[excl + i] = src[i];
        if (tid == 0) {
            if (w == 0) offsets[q] = excl;
            if (last_ticket) offsets[n_q] = excl + c;
        }
        return;
    }

    const int win_lo = w * window_bits;
    const int win_hi = min(n_rows, win_lo + window_bits);
    // ---- 1. clear, list bounds, slices ----
    {
        uint4* b4 = reinterpret_cast<uint4*>(s_dyn);
        for (int i = tid; i < n32 / 4; i += NT) b4[i] = make_uint4(0, 0, 0, 0);
    }
    if (slices) {
        if (tid < L) {
            const int2 sl = slices[(size_t)tk * L + tid];
            s_lo[tid] = sl.x; s_we[tid] = sl.y;
        }
    } else {
        if (tid < L) {
            const int b = matched[(size_t)q * L + tid];
            int lo = 0, we = 0;
            if (b >= 0) { lo = bucket_offsets[b]; we = bucket_offsets[b + 1]; }
            s_lo[tid] = lo; s_we[tid] = we;
        }
        if (n_win > 1) {
            __syncthreads();
            for (int t = warp; t < L; t += NWARP) {
                const int lo = s_lo[t], we = s_we[t];
                if (lo >= we) continue;
                int a = lo, b = we;
                if (w > 0) a = warp_lower_bound(cand, lo, we, win_lo, lane);
                if (w < n_win - 1) b = warp_lower_bound(cand, a, we, win_hi, lane);
                if (lane == 0) { s_lo[t] = a; s_we[t] = b; }
            }
        }
    }
    __syncthreads();
    {   // exclusive prefix of the slice lengths (L <= NT)
        const int len = tid < L ? s_we[tid] - s_lo[tid] : 0;
        int inc = len;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += x;
        }
        if (lane == 31) s_wtot[warp] = (uint32_t)inc;
        __syncthreads();
        int base = 0;
        for (int i = 0; i < warp; ++i) base += (int)s_wtot[i];
        if (tid < L) s_pre[tid] = base + inc - len;
        if (tid == L - 1) s_pre[L] = base + inc;
    }
    __syncthreads();
    // ---- 2. mark.  A stretch that fits one batch keeps its ids in registers for step 4. ----
    ListWalk<NT, MK> wk;
    wk.init(s_lo, s_pre, L);
    const bool single = wk.per_warp <= 32 * MK;  // same for every warp
    int32_t v[MK];
    auto mark = [&](int32_t x) {
        const uint32_t id = (uint32_t)(x - win_lo);
        atomicOr(&bm32[id >> 5], 1u << (id & 31));
    };
    if (single) {
        wk.load(cand, s_lo, s_pre, wk.w_begin + lane, v);
#pragma unroll
        for (int j = 0; j < MK; ++j)
            if (v[j] >= 0) mark(v[j]);
    } else {
        for (int e0 = wk.w_begin + lane; e0 - lane < wk.w_end; e0 += 32 * MK) {
            wk.load(cand, s_lo, s_pre, e0, v);
#pragma unroll
            for (int j = 0; j < MK; ++j)
                if (v[j] >= 0) mark(v[j]);
        }
    }
    __syncthreads();
    // ---- 3. pop-count prefixes.  A warp takes 128 words at a time, a lane four of them; four
    // lanes make a block of 512 rows: 16-bit prefixes inside the block, block totals on the side,
    // then one scan over the block totals. ----
    {
        const uint4* bm4 = reinterpret_cast<const uint4*>(bm32);
        uint2* pre2 = reinterpret_cast<uint2*>(pre16);
        for (int g = warp; g < n32 / 128; g += NWARP) {
            const uint4 x = bm4[g * 32 + lane];
            const uint32_t c0 = __popc(x.x), c1 = __popc(x.y), c2 = __popc(x.z), c3 = __popc(x.w);
            const uint32_t sum = c0 + c1 + c2 + c3;
            uint32_t inc = sum;
            uint32_t up = __shfl_up_sync(0xFFFFFFFFu, inc, 1);
            if ((lane & 3) >= 1) inc += up;
            up = __shfl_up_sync(0xFFFFFFFFu, inc, 2);
            if ((lane & 3) >= 2) inc += up;
            const uint32_t p0 = inc - sum, p1 = p0 + c0, p2 = p1 + c1, p3 = p2 + c2;  // each <= 512
            pre2[g * 32 + lane] = make_uint2(p0 | (p1 << 16), p2 | (p3 << 16));
            if ((lane & 3) == 3) base32[g * 8 + (lane >> 2)] = inc;  // block total, turned into a base below
        }
    }
    __syncthreads();
    const int per_thread = (n_blocks + NT - 1) / NT;
    const int b_begin = min(n_blocks, tid * per_thread), b_end = min(n_blocks, b_begin + per_thread);
    uint32_t mine = 0;
    for (int i = b_begin; i < b_end; ++i) mine += base32[i];
    uint32_t inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
        if (lane >= o) inc += x;
    }
    if (lane == 31) s_wtot[warp] = inc;  // safe: every thread passed a barrier after its last read
    __syncthreads();
    uint32_t run = inc - mine, wtotal = 0;
    for (int i = 0; i < NWARP; ++i) {
        const uint32_t x = s_wtot[i];
        if (i < warp) run += x;
        wtotal += x;
    }
    for (int i = b_begin; i < b_end; ++i) {
        const uint32_t x = base32[i];
        base32[i] = run;
        run += x;
    }
    // publish the count now; the prefix is resolved after the first chunk has been ranked
    if (tid == 0 && tk > 0) *reinterpret_cast<volatile unsigned long long*>(status + tk) = CH_FLAG_AGG | wtotal;
    __syncthreads();
    // ---- 4 + 5. rank, stage, copy out ----
    unsigned long long excl = 0;
    if (stage_ids == 0) {
        // Direct form (no stage): ranks are computed while warp 0 walks the chain, then every id
        // is stored at out[excl + rank]; the ~20 KB target span of a window merges in L2.
        auto rank_of = [&](int32_t x) -> uint32_t {
            const uint32_t id = (uint32_t)(x - win_lo);
            const uint32_t word = id >> 5;
            const uint32_t below = bm32[word] & ((1u << (id & 31)) - 1u);
            return base32[id >> 9] + (uint32_t)pre16[word] + (uint32_t)__popc(below);
        };
        uint32_t rk[MK];
        if (single && warp != 0) {
#pragma unroll
            for (int j = 0; j < MK; ++j) rk[j] = v[j] >= 0 ? rank_of(v[j]) : 0u;
        }
        if (warp == 0) {
            unsigned long long e;
            chain_exclusive_prefix(status, tk, (unsigned long long)wtotal, lane, d_error, false, true, e);
            if (lane == 0) s_excl = e;
            if (single) {
#pragma unroll
                for (int j = 0; j < MK; ++j) rk[j] = v[j] >= 0 ? rank_of(v[j]) : 0u;
            }
        }
        __syncthreads();
        excl = s_excl;
        int32_t* dst = out_indices + excl;
        if (single) {
#pragma unroll
            for (int j = 0; j < MK; ++j)
                if (v[j] >= 0) dst[rk[j]] = v[j];
        } else {
            wk.init(s_lo, s_pre, L);
            for (int e0 = wk.w_begin + lane; e0 - lane < wk.w_end; e0 += 32 * MK) {
                wk.load(cand, s_lo, s_pre, e0, v);
#pragma unroll
                for (int j = 0; j < MK; ++j)
                    if (v[j] >= 0) dst[rank_of(v[j])] = v[j];
            }
        }
    } else
    for (uint32_t chunk_lo = 0; chunk_lo == 0 || chunk_lo < wtotal; chunk_lo += (uint32_t)stage_ids) {
        auto rank = [&](int32_t x) {
            const uint32_t id = (uint32_t)(x - win_lo);
            const uint32_t word = id >> 5;
            const uint32_t below = bm32[word] & ((1u << (id & 31)) - 1u);
            const uint32_t r = base32[id >> 9] + (uint32_t)pre16[word] + (uint32_t)__popc(below) - chunk_lo;
            if (r < (uint32_t)stage_ids) stage[r] = x;
        };
        if (wtotal > 0) {
            if (single) {
#pragma unroll
                for (int j = 0; j < MK; ++j)
                    if (v[j] >= 0) rank(v[j]);
            } else {
                wk.init(s_lo, s_pre, L);
                for (int e0 = wk.w_begin + lane; e0 - lane < wk.w_end; e0 += 32 * MK) {
                    wk.load(cand, s_lo, s_pre, e0, v);
#pragma unroll
                    for (int j = 0; j < MK; ++j)
                        if (v[j] >= 0) rank(v[j]);
                }
            }
        }
        if (chunk_lo == 0) {
            if (warp == 0) {
                unsigned long long e;
                chain_exclusive_prefix(status, tk, (unsigned long long)wtotal, lane, d_error, false, true, e);
                if (lane == 0) s_excl = e;
            }
        }
        __syncthreads();
        excl = s_excl;
        const uint32_t n_chunk = min((uint32_t)stage_ids, wtotal - chunk_lo);
        int32_t* dst = out_indices + excl + chunk_lo;
        for (uint32_t i = tid; i < n_chunk; i += NT) dst[i] = stage[i];
        if (chunk_lo + (uint32_t)stage_ids < wtotal) __syncthreads();  // stage is reused by the next chunk
    }
    if (tid == 0) {
        if (w == 0) offsets[q] = excl;
        if (n_win == 1) counts[q] = wtotal;
        if (last_ticket) offsets[n_q] = excl + wtotal;
    }
}

// counts[q] = offsets[q + 1] - offsets[q]
__global__ void counts_from_offsets_kernel(const uint64_t* __restrict__ offsets, int n_q,
                                           uint64_t* __restrict__ counts) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q < n_q) counts[q] = offsets[q + 1] - offsets[q];
}

// ---------------------------------------------------------------------------------------
// Compaction of the per-query segments from their raw offsets to their final offsets.
// ---------------------------------------------------------------------------------------
// Queries of big_list: a whole block copies the segment.
__global__ void __launch_bounds__(256)
compact_big_kernel(const uint32_t* __restrict__ big_list, const int32_t* __restrict__ tmp,
                   const uint64_t* __restrict__ raw_off, const uint64_t* __restrict__ uniq_cnt,
                   const uint64_t* __restrict__ offsets, int32_t* __restrict__ out) {
    const int q = (int)big_list[blockIdx.x];
    const uint64_t c = uniq_cnt[q];
    const int32_t* src = tmp + raw_off[q];
    int32_t* dst = out + offsets[q];
    for (uint64_t i = threadIdx.x; i < c; i += blockDim.x) dst[i] = src[i];
}

// Small queries only (big ones are copied by compact_big_kernel).
__global__ void __launch_bounds__(256)
compact_small_kernel(const int32_t* __restrict__ tmp, const uint64_t* __restrict__ raw_cnt,
                     const uint64_t* __restrict__ raw_off, const uint64_t* __restrict__ uniq_cnt,
                     const uint64_t* __restrict__ offsets, int n_q, int32_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t n_warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t q = warp; q < (size_t)n_q; q += n_warps) {
        if (raw_cnt[q] > SMALL_MAX) continue;
        const uint64_t c = uniq_cnt[q];
        const int32_t* src = tmp + raw_off[q];
        int32_t* dst = out + offsets[q];
        for (uint64_t i = lane; i < c; i += 32) dst[i] = src[i];
    }
}

// ---------------------------------------------------------------------------------------
// Batch / shard merging helpers.
// ---------------------------------------------------------------------------------------
// offsets_out[q0 + i] = offsets_in[i] + shift, i in [0, n]
__global__ void shift_offsets_kernel(const uint64_t* __restrict__ in, size_t n, uint64_t shift,
                                     uint64_t* __restrict__ out) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = in[i] + shift;
}

// counts[q] = sum over shards of (off_r[q+1] - off_r[q])
__global__ void shard_counts_kernel(const uint64_t* const* __restrict__ shard_offsets, int n_shards,
                                    int n_q, uint64_t* __restrict__ counts) {
    int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= n_q) return;
    uint64_t c = 0;
    for (int r = 0; r < n_shards; ++r) c += shard_offsets[r][q + 1] - shard_offsets[r][q];
    counts[q] = c;
}

// One CTA per query (grid-stride): the shards' lists, shifted to global ids, in shard order.  The
// shard buffers may be peer memory, so the per-shard offsets of a query are fetched by one thread
// each (one round trip instead of one per shard), and the lists are copied as one flat sequence
// with eight independent loads in flight per thread to cover the link latency.
constexpr int SI_GROUP = 64;   // shards handled per sweep
constexpr int SI_UNROLL = 8;
__global__ void __launch_bounds__(256)
shard_interleave_kernel(const int32_t* const* __restrict__ shard_indices,
                        const uint64_t* const* __restrict__ shard_offsets,
                        const int64_t* __restrict__ row_base, int n_shards, int n_q,
                        const uint64_t* __restrict__ offsets, int32_t* __restrict__ out) {
    __shared__ const int32_t* s_src[SI_GROUP];   // shard list of this query, already at its start
    __shared__ uint64_t s_pre[SI_GROUP + 1];     // exclusive prefix of the list lengths
    __shared__ int32_t s_base[SI_GROUP];
    const int tid = threadIdx.x;
    for (size_t q = blockIdx.x; q < (size_t)n_q; q += gridDim.x) {
        uint64_t o = offsets[q];
        for (int g0 = 0; g0 < n_shards; g0 += SI_GROUP) {
            const int G = min(SI_GROUP, n_shards - g0);
            __syncthreads();  // the previous sweep is done with the tables
            if (tid < G) {
                const uint64_t* po = shard_offsets[g0 + tid];
                const uint64_t s = po[q], e = po[q + 1];
                s_src[tid] = shard_indices[g0 + tid] + s;
                s_pre[tid + 1] = e - s;  // length for now
                s_base[tid] = (int32_t)row_base[g0 + tid];
            }
            __syncthreads();
            if (tid == 0) {
                uint64_t run = 0;
                for (int r = 0; r < G; ++r) {
                    const uint64_t len = s_pre[r + 1];
                    s_pre[r] = run;
                    run += len;
                }
                s_pre[G] = run;
            }
            __syncthreads();
            const uint64_t total = s_pre[G];
            int r = 0;
            for (uint64_t i0 = tid; i0 < total; i0 += 256 * SI_UNROLL) {
                // the loaded value is not touched before all loads are issued: an add right after
                // the load would make every load wait for the one before it
                int32_t v[SI_UNROLL], shift[SI_UNROLL];
#pragma unroll
                for (int j = 0; j < SI_UNROLL; ++j) {
                    const uint64_t i = i0 + 256 * j;
                    v[j] = 0;
                    shift[j] = 0;
                    if (i < total) {
                        while (i >= s_pre[r + 1]) ++r;  // i < total keeps r below G
                        shift[j] = s_base[r];
                        v[j] = s_src[r][i - s_pre[r]];
                    }
                }
#pragma unroll
                for (int j = 0; j < SI_UNROLL; ++j) {
                    const uint64_t i = i0 + 256 * j;
                    if (i < total) out[o + i] = v[j] + shift[j];
                }
            }
            o += total;
        }
    }
}

// one warp per query, for results with short lists
__global__ void __launch_bounds__(256)
shard_interleave_small_kernel(const int32_t* const* __restrict__ shard_indices,
                              const uint64_t* const* __restrict__ shard_offsets,
                              const int64_t* __restrict__ row_base, int n_shards, int n_q,
                              const uint64_t* __restrict__ offsets, int32_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t n_warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    for (size_t q = warp; q < (size_t)n_q; q += n_warps) {
        uint64_t o = offsets[q];
        for (int r = 0; r < n_shards; ++r) {
            const uint64_t s = shard_offsets[r][q], e = shard_offsets[r][q + 1];
            const int32_t* src = shard_indices[r] + s;
            const int32_t base = (int32_t)row_base[r];
            for (uint64_t i = lane; i < e - s; i += 32) out[o + i] = src[i] + base;
            o += e - s;
        }
    }
}

// ---------------------------------------------------------------------------------------
// Push form of the shard exchange.  Every rank holds the per-query unique counts of all ranks
// (counts_all[r][q]); rank `rank` needs, for each query, where its own list starts inside the
// merged list held by the query's owner (owner = q / per: the ranks own equal slices of the
// queries), and the owner needs the counts / offsets of its slice.
// ---------------------------------------------------------------------------------------
// merged[q] = sum over ranks of counts_all[r][q]; before_me[q] = the part of it from ranks below `rank`
__global__ void __launch_bounds__(256)
exchange_counts_kernel(const uint64_t* __restrict__ counts_all, int n_ranks, int rank, int n_q,
                       uint64_t* __restrict__ merged, uint64_t* __restrict__ before_me) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= n_q) return;
    uint64_t all = 0, below = 0;
    for (int r = 0; r < n_ranks; ++r) {
        const uint64_t c = counts_all[(size_t)r * n_q + q];
        if (r < rank) below += c;
        all += c;
    }
    merged[q] = all;
    before_me[q] = below;
}

// S = exclusive scan of merged over all queries (n_q + 1 entries).  dstpos[q] = position of this
// rank's list of query q inside the owner's merged id array; the owner's own slice [my_lo, my_hi)
// gets its counts and offsets; slice_totals[j] = ids of slice j.
__global__ void __launch_bounds__(256)
exchange_positions_kernel(const uint64_t* __restrict__ S, const uint64_t* __restrict__ merged,
                          const uint64_t* __restrict__ before_me, int n_q, int per, int n_ranks, int my_lo,
                          int my_hi, uint64_t* __restrict__ dstpos, uint64_t* __restrict__ my_counts,
                          uint64_t* __restrict__ my_offsets, uint64_t* __restrict__ slice_totals) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q < n_ranks) {
        const int lo = min(n_q, q * per), hi = min(n_q, lo + per);
        slice_totals[q] = S[hi] - S[lo];
    }
    if (q > n_q) return;
    if (q < n_q) dstpos[q] = S[q] - S[min(n_q, (q / per) * per)] + before_me[q];
    if (q >= my_lo && q <= my_hi) {
        my_offsets[q - my_lo] = S[q] - S[my_lo];
        if (q < my_hi) my_counts[q - my_lo] = merged[q];
    }
}

// This rank's lists, shifted to global row ids, stored into the owners' id arrays (recv[j] may
// be peer memory: plain coalesced stores, reads are local).  Queries are visited in an order
// that deals the owners round-robin, shifted by the rank: step v goes to owner (v + rank) mod
// n_ranks.  In query order every rank would store to owner 0 first, then to owner 1 ... - all
// ranks into one GPU's NVLink ingress while the other links idle (measured at 8 GPUs: push +
// wait for the slowest rank 3.3 ms for 642 MB per GPU, four times the link time).
__device__ __forceinline__ long long exchange_query_of_step(size_t v, int n_ranks, int rank, int per, int n_q) {
    const int owner = (int)((v + (size_t)rank) % (size_t)n_ranks);
    const long long q = (long long)owner * per + (long long)(v / (size_t)n_ranks);
    return q < (long long)n_q ? q : -1;
}

// CTA per query for long lists.  The stores are 16 bytes per thread on 16-byte boundaries of the
// destination (a warp writes 512 contiguous bytes: whole NVLink packets whatever the phase of the
// list inside the owner's array); the few ids before the first boundary and after the last one
// go out one by one.  The local reads are plain 4-byte loads, sixteen in flight per thread.
constexpr int SP_UNROLL = 4;

__global__ void __launch_bounds__(256)
shard_push_kernel(const int32_t* __restrict__ idx, const uint64_t* __restrict__ off,
                  const uint64_t* __restrict__ dstpos, int32_t* const* __restrict__ recv, int per, int n_q,
                  int n_ranks, int rank, int32_t row_base) {
    const size_t n_steps = (size_t)per * n_ranks;
    for (size_t v = blockIdx.x; v < n_steps; v += gridDim.x) {
        const long long q = exchange_query_of_step(v, n_ranks, rank, per, n_q);
        if (q < 0) continue;
        const uint64_t s = off[q], len = off[q + 1] - s;
        if (len == 0) continue;
        const int32_t* src = idx + s;
        int32_t* dst = recv[q / per] + dstpos[q];
        const uint64_t head = min(len, (uint64_t)(((16u - (uint32_t)(reinterpret_cast<uintptr_t>(dst) & 15u)) & 15u) >> 2));
        if (threadIdx.x < head) dst[threadIdx.x] = src[threadIdx.x] + row_base;
        const uint64_t n4 = (len - head) >> 2;
        const int32_t* s2 = src + head;
        int4* d4 = reinterpret_cast<int4*>(dst + head);
        for (uint64_t i0 = threadIdx.x; i0 < n4; i0 += 256 * SP_UNROLL) {
            int4 w[SP_UNROLL];
#pragma unroll
            for (int j = 0; j < SP_UNROLL; ++j) {
                const uint64_t i = i0 + 256 * j;
                if (i < n4) {
                    const int32_t* p = s2 + 4 * i;
                    w[j] = make_int4(p[0], p[1], p[2], p[3]);
                }
            }
#pragma unroll
            for (int j = 0; j < SP_UNROLL; ++j) {
                const uint64_t i = i0 + 256 * j;
                if (i < n4)
                    d4[i] = make_int4(w[j].x + row_base, w[j].y + row_base, w[j].z + row_base, w[j].w + row_base);
            }
        }
        const uint64_t done = head + 4 * n4;
        if (done + threadIdx.x < len) dst[done + threadIdx.x] = src[done + threadIdx.x] + row_base;
    }
}

// warp per query, for results with short lists
__global__ void __launch_bounds__(256)
shard_push_small_kernel(const int32_t* __restrict__ idx, const uint64_t* __restrict__ off,
                        const uint64_t* __restrict__ dstpos, int32_t* const* __restrict__ recv, int per,
                        int n_q, int n_ranks, int rank, int32_t row_base) {
    const int lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const size_t n_warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t n_steps = (size_t)per * n_ranks;
    for (size_t v = warp; v < n_steps; v += n_warps) {
        const long long q = exchange_query_of_step(v, n_ranks, rank, per, n_q);
        if (q < 0) continue;
        const uint64_t s = off[q], len = off[q + 1] - s;
        int32_t* dst = recv[q / per] + dstpos[q];
        for (uint64_t i = lane; i < len; i += 32) dst[i] = idx[s + i] + row_base;
    }
}

}  // namespace culsh_b200
