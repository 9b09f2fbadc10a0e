// Projection hash, CUDA-core path: X . P^T with the quantise-and-pack epilogue fused in,
// so neither the [n][H] projection matrix nor unpacked signatures ever reach HBM.
// Replaces upstream's cublasSgemm/Dgemm + compute_signatures_kernel (rplsh/hash.cuh:24-48,
// 93-129) and + bias_floor_reorder_kernel (pslsh/hash.cuh:26-47, 105-142).
//
// This is the exact-precision path (fp32 FMA for float inputs, fp64 FMA for double
// inputs); the tcgen05 3xTF32 kernel in project_tc.cuh is the fast path for fp32.
#pragma once

#include "common.cuh"

namespace culsh_b200 {

constexpr int PS_BM = 128;      // rows per CTA
constexpr int PS_BN = 64;       // hash columns per inner tile
constexpr int PS_BK = 16;       // features per smem stage
constexpr int PS_THREADS = 256;
constexpr int PS_XS = PS_BM + 2;  // padded smem strides
constexpr int PS_PS = PS_BN + 2;

struct ProjectArgs {
    const void* X;       // [n][d]
    const void* P;       // [H][d]
    const void* bias;    // [H] (p-stable) or null
    uint32_t* keys;      // [L][n][NW]
    uint8_t* ovf_rows;   // [L][n] query mode: 1 where a value does not fit elem_bytes; or null
    int* d_error;        // fit mode: NARROW_OVERFLOW is OR-ed here
    int n, d, L, k;
    int tables_per_group;  // G
    int key_words;         // NW
    int elem_bytes;        // p-stable: 1, 2 or 4
    int row_offset;        // first row of this chunk inside the [L][n_total] key array
    int n_total;           // rows of the whole key array (table stride)
};

// Assemble the packed key of one (row, table) from k int32 hash values in shared memory.
template <int FAMILY>
__device__ __forceinline__ void assemble_key(const int32_t* __restrict__ hv, int k, int NW,
                                             int elem_bytes, uint32_t* __restrict__ out,
                                             bool& overflow) {
    overflow = false;
    if (FAMILY == CULSH_RPLSH) {
        for (int wi = 0; wi < NW; ++wi) {
            int lo = 32 * (NW - 1 - wi);  // lowest bit position held by this word
            uint32_t w = 0;
            for (int b = 0; b < 32; ++b) {
                int pos = lo + b;
                if (pos < k) w |= (uint32_t)(hv[k - 1 - pos] & 1) << b;
            }
            out[wi] = w;
        }
    } else {
        const int KB = k * elem_bytes;
        const int pad = NW * 4 - KB;
        if (elem_bytes < 4) {
            const int lim = elem_bytes == 1 ? 128 : 32768;
            for (int j = 0; j < k; ++j) {
                int v = hv[j];
                if (v < -lim || v >= lim) overflow = true;
            }
        }
        for (int wi = 0; wi < NW; ++wi) {
            uint32_t w = 0;
            for (int bb = 0; bb < 4; ++bb) {
                int i = wi * 4 + bb - pad;
                if (i >= 0) {
                    uint32_t v = (uint32_t)hv[i / elem_bytes];
                    uint32_t byte = (v >> (8 * (i % elem_bytes))) & 0xFFu;
                    w |= byte << (24 - 8 * bb);
                }
            }
            out[wi] = w;
        }
    }
}

template <typename T, int FAMILY>
__global__ void __launch_bounds__(PS_THREADS)
project_simt_kernel(ProjectArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* Xs = reinterpret_cast<T*>(smem_raw);                 // [BK][PS_XS]
    T* Ps = Xs + PS_BK * PS_XS;                              // [BK][PS_PS]
    int32_t* hbuf = reinterpret_cast<int32_t*>(Ps + PS_BK * PS_PS);  // [BM][GC]

    const T* __restrict__ X = static_cast<const T*>(a.X);
    const T* __restrict__ P = static_cast<const T*>(a.P);
    const T* __restrict__ bias = static_cast<const T*>(a.bias);

    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int G = a.tables_per_group;
    const int n_groups = (a.L + G - 1) / G;
    const int group = blockIdx.x % n_groups;  // fastest: the groups of one row block share X in L2
    const int row0 = (blockIdx.x / n_groups) * PS_BM;
    const int GC = G * a.k;
    const int H = a.L * a.k;
    const int col_base = group * GC;
    const int gc_valid = min(GC, H - col_base);

    for (int c0 = 0; c0 < gc_valid; c0 += PS_BN) {
        T acc[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = T(0);

        for (int k0 = 0; k0 < a.d; k0 += PS_BK) {
            {   // X tile: thread -> (row tid/2, 8 consecutive features)
                int r = tid >> 1, kk0 = (tid & 1) * 8;
                int row = row0 + r;
                const T* src = X + (size_t)row * a.d + k0 + kk0;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    T v = T(0);
                    if (row < a.n && k0 + kk0 + j < a.d) v = src[j];
                    Xs[(kk0 + j) * PS_XS + r] = v;
                }
            }
            {   // P tile: thread -> (col tid/4, 4 consecutive features)
                int c = tid >> 2, kk0 = (tid & 3) * 4;
                int lc = c0 + c;
                const T* src = P + (size_t)(col_base + lc) * a.d + k0 + kk0;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    T v = T(0);
                    if (lc < gc_valid && k0 + kk0 + j < a.d) v = src[j];
                    Ps[(kk0 + j) * PS_PS + c] = v;
                }
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < PS_BK; ++kk) {
                T xv[8], pv[4];
#pragma unroll
                for (int i = 0; i < 8; ++i) xv[i] = Xs[kk * PS_XS + ty * 8 + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) pv[j] = Ps[kk * PS_PS + tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 8; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fma(xv[i], pv[j], acc[i][j]);
            }
            __syncthreads();
        }
        // quantise into the per-CTA hash buffer
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int lc = c0 + tx * 4 + j;
            if (lc < gc_valid) {
                T bv = T(0);
                if (FAMILY == CULSH_PSLSH) bv = bias[col_base + lc];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    int32_t q;
                    if (FAMILY == CULSH_RPLSH) {
                        // sign bit of the value narrowed to fp32 (rplsh/hash.cuh:47)
                        q = (int32_t)((__float_as_uint((float)acc[i][j]) >> 31) ^ 1u);
                    } else {
                        q = static_cast<int32_t>(floor(acc[i][j] + bv));  // pslsh/hash.cuh:46
                    }
                    hbuf[(ty * 8 + i) * GC + lc] = q;
                }
            }
        }
    }
    __syncthreads();

    // pack and store: consecutive threads -> consecutive rows of one table
    const int NW = a.key_words;
    const int tables_here = gc_valid / a.k;
    for (int idx = tid; idx < PS_BM * tables_here; idx += PS_THREADS) {
        int r = idx % PS_BM, g = idx / PS_BM;
        int row = row0 + r;
        if (row >= a.n) continue;
        int t = group * G + g;
        uint32_t w[8];
        bool ovf;
        assemble_key<FAMILY>(hbuf + r * GC + g * a.k, a.k, NW, a.elem_bytes, w, ovf);
        size_t item = (size_t)t * a.n_total + a.row_offset + row;
        uint32_t* dst = a.keys + item * NW;
        for (int wi = 0; wi < NW; ++wi) dst[wi] = w[wi];
        if (FAMILY == CULSH_PSLSH) {
            if (a.ovf_rows) a.ovf_rows[item] = ovf ? 1 : 0;
            else if (ovf) atomicOr(a.d_error, DEV_ERR_NARROW_OVERFLOW);
        }
    }
}

inline int simt_tables_per_group(int L, int k) {
    int G = 128 / k;
    if (G < 1) G = 1;
    if (G > L) G = L;
    return G;
}

template <typename T>
inline size_t simt_smem_bytes(int G, int k) {
    return sizeof(T) * (PS_BK * PS_XS + PS_BK * PS_PS) + sizeof(int32_t) * PS_BM * (size_t)G * k;
}

// Host launcher.  X may be a chunk (n rows starting at row_offset of an n_total-row index).
template <typename T>
inline void launch_project_simt(const CtxPtr& c, cudaStream_t stream, int family, const T* X,
                                const T* P, const T* bias, int n, int d, int L, int k,
                                const KeySpec& ks, uint32_t* keys, uint8_t* ovf_rows,
                                int row_offset, int n_total) {
    if (n == 0) return;
    ProjectArgs a{};
    a.X = X; a.P = P; a.bias = bias; a.keys = keys; a.ovf_rows = ovf_rows;
    a.d_error = c->d_error;
    a.n = n; a.d = d; a.L = L; a.k = k;
    a.tables_per_group = simt_tables_per_group(L, k);
    a.key_words = ks.key_words;
    a.elem_bytes = ks.elem_bytes;
    a.row_offset = row_offset;
    a.n_total = n_total;
    size_t smem = simt_smem_bytes<T>(a.tables_per_group, k);
    if (smem > c->smem_optin)
        fail(CULSH_ERR_UNSUPPORTED, "n_hashes=%d needs %zu bytes of shared memory per CTA", k, smem);
    dim3 grid((unsigned)(ceil_div(L, a.tables_per_group) * ceil_div(n, PS_BM)));
    auto kern = family == CULSH_RPLSH ? project_simt_kernel<T, CULSH_RPLSH>
                                      : project_simt_kernel<T, CULSH_PSLSH>;
    CU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, PS_THREADS, smem, stream>>>(a);
    KERNEL_CHECK();
}

}  // namespace culsh_b200
