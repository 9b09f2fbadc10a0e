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

__device__ __forceinline__ uint32_t mod_prime_u64(uint64_t x) {
    // x = hi*2^32 + lo == hi*5 + lo (mod p); two folds bring it below 2p.
    uint64_t y = (x >> 32) * 5ull + (x & 0xFFFFFFFFull);        // < 6 * 2^32
    uint64_t z = (y >> 32) * 5ull + (y & 0xFFFFFFFFull);        // < 2^32 + 25
    if (z >= MINHASH_PRIME) z -= MINHASH_PRIME;
    return (uint32_t)z;
}

// keys: [L][n_total][NW] with NW = round_key_words(4k); word j (right-aligned) = bswap32(min).
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
        for (int h0 = 0; h0 < H; h0 += 32 * MH_MAX_PER_LANE) {
            uint32_t a[MH_MAX_PER_LANE], b[MH_MAX_PER_LANE], m[MH_MAX_PER_LANE];
#pragma unroll
            for (int i = 0; i < MH_MAX_PER_LANE; ++i) {
                int h = h0 + i * 32 + lane;
                a[i] = h < H ? A[h] : 0u;
                b[i] = h < H ? B[h] : 0u;
                m[i] = 0xFFFFFFFFu;
            }
            const int n_live = min(MH_MAX_PER_LANE, (H - h0 + 31) / 32);
            for (int base = start; base < end; base += 32) {
                int mine = base + lane < end ? indices[base + lane] : 0;
                int cnt = min(32, end - base);
                for (int s = 0; s < cnt; ++s) {
                    uint32_t c = (uint32_t)__shfl_sync(0xFFFFFFFFu, mine, s);
#pragma unroll
                    for (int i = 0; i < MH_MAX_PER_LANE; ++i) {
                        if (i < n_live) {
                            uint32_t hv = mod_prime_u64((uint64_t)a[i] * c + (uint64_t)b[i]);
                            m[i] = min(m[i], hv);
                        }
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < MH_MAX_PER_LANE; ++i) {
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
    minhash_kernel<<<(unsigned)blocks, MH_THREADS, 0, stream>>>(indices, indptr, A, B, n_rows, L, k,
                                                               ks.key_words, keys, n_total,
                                                               row_offset);
    KERNEL_CHECK();
}

}  // namespace culsh_b200
