// MinHash signatures over CSR rows.  Replaces compute_minhash_kernel
// (minhash/hash.cuh:69-128): sig[t][row][j] = min over the row's column ids c of
// (A[h]*c + B[h]) mod 4294967291, h = t*k + j; an empty row gives 0xFFFFFFFF.
//
// One warp per row.  Lanes own hash functions (lane, lane+32, ...), so every lane is busy
// however short the row is and no cross-lane reduction is needed; the row's column ids
// are loaded 32 at a time (coalesced) and broadcast with shuffles.  The modulus is
// folded with 2^32 = 5 (mod p) instead of a 64-bit division.
#pragma once

#include "common.cuh"

namespace culsh_b200 {

constexpr uint32_t MINHASH_PRIME = 4294967291u;  // minhash/hash.cuh:17
constexpr int MH_THREADS = 256;
constexpr int MH_MAX_PER_LANE = 8;               // hashes per lane per sweep (H <= 256 in one sweep)

__device__ __forceinline__ uint64_t mad_wide_u32(uint32_t a, uint32_t b, uint64_t c) {
    uint64_t d;
    asm("mad.wide.u32 %0, %1, %2, %3;" : "=l"(d) : "r"(a), "r"(b), "l"(c));
    return d;
}

// (a*c + b) mod p with p = 2^32 - 5, i.e. 2^32 == 5 (mod p), for a, b < p and c < 2^31.
// x = a*c + b < 2^63; y = 5*x_hi + x_lo < 3.5 * 2^32 is congruent to x; s = 5*y_hi + y_lo
// < 2^32 + 15 is congruent too and lies below 2p, so the result is s or s - p.  s >= p exactly
// when s + 5 carries out of 32 bits, and then (s + 5) mod 2^32 = s - p: one add with a carry
// test replaces the compare-and-subtract.  b64 is b zero-extended (the caller keeps it in
// registers across the row).
__device__ __forceinline__ uint32_t hash_mod_prime(uint32_t a, uint32_t c, uint64_t b64) {
    const uint64_t x = mad_wide_u32(a, c, b64);
    const uint64_t y = mad_wide_u32((uint32_t)(x >> 32), 5u, (uint64_t)(uint32_t)x);
    const uint32_t u = 5u * (uint32_t)(y >> 32) + 5u;   // <= 20
    const uint32_t t = (uint32_t)y + u;                 // (s + 5) mod 2^32
    return t < u ? t : t - 5u;                          // carried: s - p; else s
}

// The same value shifted by 5, without the final correction: returns t = (s + 5) mod 2^32 (s as
// above) and sets `carried` when the addition wrapped, i.e. when s >= p and the result would have
// been s - p instead of s.  That happens for about 20 of 2^32 inputs, so the row loop keeps the
// minimum of t and a flag, and only a flagged (row, hash function) is evaluated again in full.
__device__ __forceinline__ uint32_t hash_plus5(uint32_t a, uint32_t c, uint64_t b64, bool& carried) {
    const uint64_t x = mad_wide_u32(a, c, b64);
    const uint64_t y = mad_wide_u32((uint32_t)(x >> 32), 5u, (uint64_t)(uint32_t)x);
    const uint32_t u = 5u * (uint32_t)(y >> 32) + 5u;
    const uint32_t t = (uint32_t)y + u;
    carried |= t < u;
    return t;
}

// keys: [L][n_total][NW] with NW = round_key_words(4k); word j (right-aligned) = bswap32(min).
// PL = hash functions per lane per sweep; a sweep covers 32*PL consecutive hash functions and
// H > 256 takes several sweeps.  Slots past H hold a = b = 0, evaluate to 0 and are never stored,
// so the inner loop carries no predicate.
template <int PL>
__global__ void __launch_bounds__(MH_THREADS)
minhash_kernel(const int32_t* __restrict__ indices, const int32_t* __restrict__ indptr,
               const uint32_t* __restrict__ A, const uint32_t* __restrict__ B, int n_rows,
               int L, int k, int NW, uint32_t* __restrict__ keys, int n_total, int row_offset) {
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * (MH_THREADS / 32)) + (threadIdx.x >> 5);
    const int n_warps = gridDim.x * (MH_THREADS / 32);
    const int H = L * k;
    const int pad_words = NW - k;  // leading zero words when 4k is not 4, 8, 16 or 32 bytes

    for (int row = warp; row < n_rows; row += n_warps) {
        const int start = indptr[row], end = indptr[row + 1];
        for (int h0 = 0; h0 < H; h0 += 32 * PL) {
            uint32_t a[PL], m[PL];
            uint64_t b[PL];
#pragma unroll
            for (int i = 0; i < PL; ++i) {
                int h = h0 + i * 32 + lane;
                a[i] = h < H ? A[h] : 0u;
                b[i] = h < H ? (uint64_t)B[h] : 0ull;
                m[i] = 0xFFFFFFFFu;
            }
            bool carried[PL];
#pragma unroll
            for (int i = 0; i < PL; ++i) carried[i] = false;
            for (int base = start; base < end; base += 32) {
                const int mine = base + lane < end ? indices[base + lane] : 0;
                const int cnt = min(32, end - base);
#pragma unroll 8
                for (int s = 0; s < cnt; ++s) {
                    const uint32_t c = (uint32_t)__shfl_sync(0xFFFFFFFFu, mine, s);
#pragma unroll
                    for (int i = 0; i < PL; ++i) m[i] = min(m[i], hash_plus5(a[i], c, b[i], carried[i]));
                }
            }
            // m holds min(hash) + 5 unless one of the evaluations wrapped; those few are redone
#pragma unroll
            for (int i = 0; i < PL; ++i) {
                if (carried[i]) {
                    uint32_t exact = 0xFFFFFFFFu;
                    for (int e = start; e < end; ++e)
                        exact = min(exact, hash_mod_prime(a[i], (uint32_t)indices[e], b[i]));
                    m[i] = exact;
                } else if (end > start) {
                    m[i] -= 5u;
                }
            }
#pragma unroll
            for (int i = 0; i < PL; ++i) {
                int h = h0 + i * 32 + lane;
                if (h < H) {
                    int t = h / k, j = h - t * k;
                    size_t item = (size_t)t * n_total + row_offset + row;
                    keys[item * NW + pad_words + j] = __byte_perm(m[i], 0, 0x0123);
                }
            }
        }
        if (pad_words > 0) {
            for (int idx = lane; idx < L * pad_words; idx += 32) {
                int t = idx / pad_words, j = idx - t * pad_words;
                size_t item = (size_t)t * n_total + row_offset + row;
                keys[item * NW + j] = 0u;
            }
        }
    }
}

inline void launch_minhash(const CtxPtr& c, cudaStream_t stream, const int32_t* indices,
                           const int32_t* indptr, const uint32_t* A, const uint32_t* B, int n_rows,
                           int L, int k, const KeySpec& ks, uint32_t* keys, int n_total,
                           int row_offset) {
    if (n_rows == 0) return;
    int warps_per_block = MH_THREADS / 32;
    size_t blocks = ceil_div((size_t)n_rows, warps_per_block);
    size_t cap = (size_t)c->sm_count * 32;
    if (blocks > cap) blocks = cap;
    const int H = L * k;
    const int sweeps = (int)ceil_div(H, 32 * MH_MAX_PER_LANE);
    const int per_lane = (int)ceil_div(H, 32 * sweeps);  // 1..MH_MAX_PER_LANE
#define CULSH_MH_CASE(PLV)                                                                      \
    case PLV:                                                                                   \
        minhash_kernel<PLV><<<(unsigned)blocks, MH_THREADS, 0, stream>>>(                       \
            indices, indptr, A, B, n_rows, L, k, ks.key_words, keys, n_total, row_offset);      \
        break;
    switch (per_lane) {
        CULSH_MH_CASE(1) CULSH_MH_CASE(2) CULSH_MH_CASE(3) CULSH_MH_CASE(4)
        CULSH_MH_CASE(5) CULSH_MH_CASE(6) CULSH_MH_CASE(7) CULSH_MH_CASE(8)
        default: fail(CULSH_ERR_INTERNAL, "minhash: hashes per lane out of range");
    }
#undef CULSH_MH_CASE
    KERNEL_CHECK();
}

}  // namespace culsh_b200
