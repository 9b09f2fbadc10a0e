// Streamed single-pass gather + dedupe for query sets dominated by large candidate sets.
// Replaces collect_candidates_kernel + the segmented sort / flag / reduce / scan / select chain
// of query_from_matched_buckets (core/query.cuh:290-478) for such sets.
//
// Work is cut into TICKETS in CSR order.  A query with a large candidate set gets as many
// tickets as it takes to keep a ticket at about `ids_per_ticket` raw ids: ticket w of the query
// covers the rows [w * win_bits, (w + 1) * win_bits), a multiple of 4096 rows.  A query handled
// by the warp / sort paths is one ticket that only copies its finished list.  The tickets of
// one call are described by two tables built by small kernels: a 16-byte descriptor per ticket
// and, per (ticket, table), the slice of the bucket list that falls into the ticket's rows.
//
// The kernel is persistent: a CTA takes tickets from an atomic counter, four ahead of the one
// it is working on, so that a ticket's descriptor and slices (cp.async, two tickets ahead) and
// its ids (cp.async into one of two shared-memory buffers, one ticket ahead) are on chip when
// its turn comes; no thread ever waits for a load from global memory in the steady state.  The
// slices are laid end to end in the buffer, each at the 16-byte phase of its source so that
// whole groups of four ids travel as one 16-byte copy; the few pad words hold -1.
// Per ticket the CTA then
//   1. marks the ids in a shared-memory bitmap of the ticket's rows,
//   2. scans the bitmap once (16-bit pop-count prefix per word inside blocks of 512 rows, a
//      32-bit base per block) and publishes the number of unique ids to the chain,
//   3. goes over the ids again: the rank of an id among the unique ids is base[block] +
//      prefix[word] + popc(bits below), so the id is dropped at stage[rank] (duplicates write
//      the same value to the same slot),
//   4. resolves its exclusive prefix from the chain of earlier tickets (decoupled look-back,
//      bounded) and copies the stage, now sorted and unique, to its place in the CSR.
// A ticket whose ids do not fit the buffer (rows with skewed id ranges) reads its lists with
// plain loads and ranks in stage-sized chunks instead.
// Tickets are taken in order and a CTA works through its tickets in order, so a CTA only ever
// waits on tickets that are held by CTAs that are running; every wait is bounded.
#pragma once

#include "query.cuh"

namespace culsh_b200 {

struct TicketDesc {
    int q;         // query
    int win_lo;    // first row of the ticket's window
    int win_bits;  // rows in the window (multiple of 4096); 0 for a copy ticket
    int kind;      // TK_COPY / TK_BITMAP
};
static_assert(sizeof(TicketDesc) == 16, "descriptor travels as one 16-byte copy");
constexpr int TK_COPY = 0;
constexpr int TK_BITMAP = 1;
constexpr int TK_MAX_WINDOWS = 8192;  // per query

// number of tickets of a query with `raw` candidate ids
__host__ __device__ __forceinline__ uint32_t tickets_of_query(uint64_t raw, int mid_max, int ids_per_ticket,
                                                              int min_win, int max_win) {
    const bool big = raw > (uint64_t)SMALL_MAX && raw > (uint64_t)mid_max;
    if (!big) return 1u;
    const uint64_t want = (raw + (uint64_t)ids_per_ticket - 1) / (uint64_t)ids_per_ticket;
    uint64_t w = want < (uint64_t)min_win ? (uint64_t)min_win : want;
    if (w > (uint64_t)max_win) w = (uint64_t)max_win;
    return (uint32_t)w;
}

__global__ void __launch_bounds__(256)
ticket_count_kernel(const uint64_t* __restrict__ raw_cnt, int n_q, int mid_max, int ids_per_ticket, int min_win,
                    int max_win, uint32_t* __restrict__ tk_cnt) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q < n_q) tk_cnt[q] = tickets_of_query(raw_cnt[q], mid_max, ids_per_ticket, min_win, max_win);
}

// descriptors of the tickets of every query (tk_base = exclusive prefix of the ticket counts)
__global__ void __launch_bounds__(256)
ticket_table_kernel(const uint64_t* __restrict__ raw_cnt, const uint32_t* __restrict__ tk_base, int n_q,
                    int n_rows, int mid_max, TicketDesc* __restrict__ descs) {
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= n_q) return;
    const uint32_t base = tk_base[q], n = tk_base[q + 1] - base;
    const uint64_t raw = raw_cnt[q];
    const bool big = raw > (uint64_t)SMALL_MAX && raw > (uint64_t)mid_max;
    if (!big) {
        descs[base] = TicketDesc{q, 0, 0, TK_COPY};
        return;
    }
    const int per = (int)(((size_t)n_rows + n - 1) / n);
    const int wbits = (per + 4095) / 4096 * 4096;
    for (uint32_t w = 0; w < n; ++w) {
        const long long lo = (long long)w * wbits;
        descs[base + w] = TicketDesc{q, (int)(lo < (long long)n_rows ? lo : (long long)n_rows), wbits, TK_BITMAP};
    }
}

// slices[tk * L + t] = [a, b): the part of table t's bucket list (ascending row ids) that falls
// into ticket tk's rows.  One thread per (ticket, table) finds the lower boundary of its window
// and writes it as the start of its own slice and as the end of the slice of the window before.
__global__ void __launch_bounds__(256)
ticket_slices_kernel(const TicketDesc* __restrict__ descs, const uint32_t* __restrict__ n_tickets,
                     const int32_t* __restrict__ matched, const int32_t* __restrict__ bucket_offsets,
                     const int32_t* __restrict__ cand, int L, int n_rows, int2* __restrict__ slices) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t tk = idx / L;
    if (tk >= (size_t)*n_tickets) return;
    const int t = (int)(idx - tk * L);
    const TicketDesc d = descs[tk];
    if (d.kind != TK_BITMAP) return;
    const int b = matched[(size_t)d.q * L + t];
    int lo = 0, we = 0;
    if (b >= 0) { lo = bucket_offsets[b]; we = bucket_offsets[b + 1]; }
    int* flat = reinterpret_cast<int*>(slices);
    const size_t mine = idx * 2;
    int a = lo;
    if (d.win_lo > 0) {
        a = lower_bound_i32(cand, lo, we, d.win_lo);
        flat[mine - (size_t)L * 2 + 1] = a;  // the ticket before is the window before of the same query
    }
    flat[mine] = a;
    if ((long long)d.win_lo + d.win_bits >= (long long)n_rows) flat[mine + 1] = we;
}

// ---- asynchronous copies global -> shared (Ampere-style cp.async: no mbarrier, completion by
// commit groups, so nothing here can wait for ever) ----
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async8(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;\n" ::: "memory"); }

struct StreamArgs {
    const int32_t* cand;                 // bucket lists, 16-byte aligned
    const uint64_t* raw_off;             // start of a copy ticket's finished list in tmp
    const int32_t* tmp;
    const TicketDesc* descs;
    const int2* slices;
    const uint32_t* n_tickets;           // device: number of tickets of this call
    unsigned long long* status;          // chain, one word per ticket, zeroed
    uint32_t* ticket;                    // zeroed
    int32_t* out_indices;
    uint64_t* counts;                    // in: unique counts of the copy tickets' queries
    uint64_t* offsets;                   // out: offsets[q] for every query, offsets[n_q]
    int* d_error;
    int n_q, L, n_rows;
    int window_bits;                     // largest window (multiple of 4096)
    int cap;                             // ids per buffer = stage size (multiple of 4)
};

inline size_t stream_smem_bytes(int window_bits, int cap, int L) {
    const int Lp = (L + 1) & ~1;
    return (size_t)window_bits / 8 + (size_t)window_bits / 16 + (size_t)window_bits / 128 +
           (size_t)cap * 4 * 3 + (size_t)Lp * 8 * 3 + 3 * sizeof(TicketDesc);
}

template <int NT>
__global__ void __launch_bounds__(NT)
dedupe_stream_kernel(const StreamArgs a) {
    constexpr int NWARP = NT / 32;
    extern __shared__ __align__(16) uint32_t s_dyn[];
    const int n32max = a.window_bits / 32;   // a multiple of 128
    const int L = a.L, Lp = (L + 1) & ~1;
    uint32_t* bm32 = s_dyn;                                                   // [n32max] bitmap
    uint16_t* pre16 = reinterpret_cast<uint16_t*>(bm32 + n32max);            // [n32max]
    uint32_t* base32 = reinterpret_cast<uint32_t*>(pre16 + n32max);          // [n32max / 16]
    int32_t* stage = reinterpret_cast<int32_t*>(base32 + n32max / 16);      // [cap]
    int32_t* idbuf = stage + a.cap;                                           // [2][cap]
    int2* meta = reinterpret_cast<int2*>(idbuf + 2 * (size_t)a.cap);         // [3][Lp] slices
    TicketDesc* sdesc = reinterpret_cast<TicketDesc*>(meta + 3 * Lp);        // [3]
    __shared__ uint32_t s_wtot[NWARP];
    __shared__ unsigned long long s_excl;
    __shared__ uint32_t s_tk[8];   // tickets of jobs j (slot j & 7)
    __shared__ int s_tot[4];       // padded id count of job j's buffer (slot j & 3), -1: not staged

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t n_tk = *a.n_tickets;
    uint32_t pending = 0xFFFFFFFFu;  // thread 0: ticket taken, not yet in s_tk

    // ---- issue of the copies for job j's ids into buffer j & 1 (every warp computes the layout
    // of all lists by itself, then copies the lists  warp, warp + NWARP, ...) ----
    auto issue_ids = [&](int j) {
        const TicketDesc d = sdesc[j % 3];
        if (d.kind != TK_BITMAP) {
            if (tid == 0) s_tot[j & 3] = -1;
            return;
        }
        const int2* m = meta + (j % 3) * Lp;
        int32_t* buf = idbuf + (size_t)(j & 1) * a.cap;
        // pass 1: padded total (block of a list = align4((src & 3) + len), empty lists take nothing)
        int total = 0;
        for (int t0 = 0; t0 < L; t0 += 32) {
            const int t = t0 + lane;
            int plen = 0;
            if (t < L) {
                const int2 s = m[t];
                const int len = s.y - s.x;
                if (len > 0) plen = ((s.x & 3) + len + 3) & ~3;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) plen += __shfl_xor_sync(0xFFFFFFFFu, plen, o);
            total += plen;
        }
        if (total > a.cap) {  // same decision in every warp
            if (tid == 0) s_tot[j & 3] = -1;
            return;
        }
        if (tid == 0) s_tot[j & 3] = total;
        // pass 2: copies
        int run = 0;
        for (int t0 = 0; t0 < L; t0 += 32) {
            const int t = t0 + lane;
            int src = 0, len = 0, plen = 0;
            if (t < L) {
                const int2 s = m[t];
                src = s.x;
                len = s.y - s.x;
                if (len > 0) plen = ((src & 3) + len + 3) & ~3; else len = 0;
            }
            int inc = plen;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
                if (lane >= o) inc += x;
            }
            const int block = run + inc - plen;
            run += __shfl_sync(0xFFFFFFFFu, inc, 31);
            const int hi = min(32, L - t0);
            for (int u = warp; u < hi; u += NWARP) {   // list t0 + u is this warp's
                const int l_src = __shfl_sync(0xFFFFFFFFu, src, u);
                const int l_len = __shfl_sync(0xFFFFFFFFu, len, u);
                const int l_block = __shfl_sync(0xFFFFFFFFu, block, u);
                if (l_len == 0) continue;
                const int h = l_src & 3;
                const int groups = (h + l_len + 3) >> 2;
                int32_t* dst = buf + l_block;                       // 16-byte aligned
                const int32_t* s = a.cand + (l_src - h);            // 16-byte aligned
                for (int g = lane; g < groups; g += 32) {
                    const int p0 = 4 * g;
                    if (p0 >= h && p0 + 4 <= h + l_len) {
                        cp_async16(dst + p0, s + p0);
                    } else {
#pragma unroll
                        for (int p = p0; p < p0 + 4; ++p) {
                            if (p >= h && p < h + l_len) cp_async4(dst + p, s + p);
                            else dst[p] = -1;
                        }
                    }
                }
            }
        }
    };

    // ---- end-of-job step: everything issued earlier has landed; hand the freed buffers to the
    // jobs further ahead.  i may be negative (prologue). ----
    auto advance = [&](int i) {
        cp_async_wait_all();
        __syncthreads();
        if (tid == 0) {  // ticket of job i + 4 (taken one step earlier, or right here in the prologue)
            if (pending == 0xFFFFFFFFu) pending = atomicAdd(a.ticket, 1u);
            s_tk[(i + 4) & 7] = pending;
            pending = 0xFFFFFFFFu;
        }
        if (i + 3 >= 0) {  // descriptor + slices of job i + 3
            const uint32_t tk3 = s_tk[(i + 3) & 7];
            if (tk3 < n_tk) {
                const int slot = (i + 3) % 3;
                if (tid == 0) cp_async16(sdesc + slot, a.descs + tk3);
                if (tid < L) cp_async8(meta + slot * Lp + tid, a.slices + (size_t)tk3 * L + tid);
            }
        }
        if (i + 2 >= 0) {  // ids of job i + 2
            const uint32_t tk2 = s_tk[(i + 2) & 7];
            if (tk2 < n_tk) issue_ids(i + 2);
        }
        cp_async_commit();
    };

    advance(-4);
    advance(-3);
    advance(-2);
    advance(-1);

    for (int i = 0;; ++i) {
        const uint32_t tk = s_tk[i & 7];
        if (tk >= n_tk) break;
        if (tid == 0) pending = atomicAdd(a.ticket, 1u);  // for job i + 4, stored by advance(i)
        const TicketDesc d = sdesc[i % 3];
        const int q = d.q;
        const bool last_ticket = tk == n_tk - 1;

        if (d.kind != TK_BITMAP) {  // finished list in tmp: join the chain with its count and copy it
            const unsigned long long c = a.counts[q];
            if (warp == 0) {
                unsigned long long e;
                chain_exclusive_prefix(a.status, (int)tk, c, lane, a.d_error, true, true, e);
                if (lane == 0) s_excl = e;
            }
            __syncthreads();
            const unsigned long long excl = s_excl;
            const int32_t* src = a.tmp + a.raw_off[q];
            for (unsigned long long k = tid; k < c; k += NT) a.out_indices[excl + k] = src[k];
            if (tid == 0) {
                a.offsets[q] = excl;
                if (last_ticket) a.offsets[a.n_q] = excl + c;
            }
            advance(i);
            continue;
        }

        const int win_lo = d.win_lo;
        const int n32 = d.win_bits / 32;     // a multiple of 128, <= n32max
        const int n_blocks = n32 / 16;
        const int tot = s_tot[i & 3];
        const int32_t* ids = idbuf + (size_t)(i & 1) * a.cap;
        const int2* m = meta + (i % 3) * Lp;
        // ---- clear ----
        {
            uint4* b4 = reinterpret_cast<uint4*>(bm32);
            for (int k = tid; k < n32 / 4; k += NT) b4[k] = make_uint4(0, 0, 0, 0);
        }
        __syncthreads();
        // ---- 1. mark ----
        auto mark = [&](int32_t x) {
            const uint32_t id = (uint32_t)(x - win_lo);
            atomicOr(&bm32[id >> 5], 1u << (id & 31));
        };
        if (tot >= 0) {
            const int4* ids4 = reinterpret_cast<const int4*>(ids);
            for (int g = tid; g < tot / 4; g += NT) {
                const int4 v = ids4[g];
                if (v.x >= 0) mark(v.x);
                if (v.y >= 0) mark(v.y);
                if (v.z >= 0) mark(v.z);
                if (v.w >= 0) mark(v.w);
            }
        } else {
            for (int t = 0; t < L; ++t) {
                const int2 s = m[t];
                for (int k = s.x + tid; k < s.y; k += NT) mark(a.cand[k]);
            }
        }
        __syncthreads();
        // ---- 2. pop-count prefixes: a warp takes 128 words at a time, a lane four of them; four
        // lanes make a block of 512 rows ----
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
                if ((lane & 3) == 3) base32[g * 8 + (lane >> 2)] = inc;  // block total, a base below
            }
        }
        __syncthreads();
        const int per_thread = (n_blocks + NT - 1) / NT;
        const int b_begin = min(n_blocks, tid * per_thread), b_end = min(n_blocks, b_begin + per_thread);
        uint32_t mine = 0;
        for (int k = b_begin; k < b_end; ++k) mine += base32[k];
        uint32_t inc = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t x = __shfl_up_sync(0xFFFFFFFFu, inc, o);
            if (lane >= o) inc += x;
        }
        if (lane == 31) s_wtot[warp] = inc;
        __syncthreads();
        uint32_t run = inc - mine, wtotal = 0;
        for (int k = 0; k < NWARP; ++k) {
            const uint32_t x = s_wtot[k];
            if (k < warp) run += x;
            wtotal += x;
        }
        for (int k = b_begin; k < b_end; ++k) {
            const uint32_t x = base32[k];
            base32[k] = run;
            run += x;
        }
        if (tid == 0 && tk > 0)
            *reinterpret_cast<volatile unsigned long long*>(a.status + tk) = CH_FLAG_AGG | wtotal;
        __syncthreads();
        // ---- 3 + 4. rank into the stage, resolve the prefix, copy out ----
        unsigned long long excl = 0;
        for (uint32_t chunk_lo = 0; chunk_lo == 0 || chunk_lo < wtotal; chunk_lo += (uint32_t)a.cap) {
            auto rank = [&](int32_t x) {
                const uint32_t id = (uint32_t)(x - win_lo);
                const uint32_t word = id >> 5;
                const uint32_t below = bm32[word] & ((1u << (id & 31)) - 1u);
                const uint32_t r = base32[id >> 9] + (uint32_t)pre16[word] + (uint32_t)__popc(below) - chunk_lo;
                if (r < (uint32_t)a.cap) stage[r] = x;
            };
            if (wtotal > 0) {
                if (tot >= 0) {  // unique <= staged ids <= cap: a single chunk
                    const int4* ids4 = reinterpret_cast<const int4*>(ids);
                    for (int g = tid; g < tot / 4; g += NT) {
                        const int4 v = ids4[g];
                        if (v.x >= 0) rank(v.x);
                        if (v.y >= 0) rank(v.y);
                        if (v.z >= 0) rank(v.z);
                        if (v.w >= 0) rank(v.w);
                    }
                } else {
                    for (int t = 0; t < L; ++t) {
                        const int2 s = m[t];
                        for (int k = s.x + tid; k < s.y; k += NT) rank(a.cand[k]);
                    }
                }
            }
            if (chunk_lo == 0 && warp == 0) {
                unsigned long long e;
                chain_exclusive_prefix(a.status, (int)tk, (unsigned long long)wtotal, lane, a.d_error, false, true, e);
                if (lane == 0) s_excl = e;
            }
            __syncthreads();
            excl = s_excl;
            const uint32_t n_chunk = min((uint32_t)a.cap, wtotal - chunk_lo);
            int32_t* dst = a.out_indices + excl + chunk_lo;
            for (uint32_t k = tid; k < n_chunk; k += NT) dst[k] = stage[k];
            if (chunk_lo + (uint32_t)a.cap < wtotal) __syncthreads();  // the next chunk reuses the stage
        }
        if (tid == 0) {
            if (win_lo == 0) a.offsets[q] = excl;
            if (last_ticket) a.offsets[a.n_q] = excl + wtotal;
        }
        advance(i);
    }
    cp_async_wait_all();
}

}  // namespace culsh_b200
