// Projection hash on the 5th-generation tensor cores: X . P^T as a 3xTF32 split GEMM
// (tcgen05.mma kind::tf32, fp32 accumulators in TMEM, operands staged in shared memory by
// TMA) with the sign-test / floor quantisation and the key packing fused into the epilogue,
// so only packed signatures reach HBM.  Replaces cublasSgemm + compute_signatures_kernel
// (rplsh/hash.cuh:24-48, 93-129) and + bias_floor_reorder_kernel (pslsh/hash.cuh:26-47,
// 105-142) for fp32 inputs.
//
// 3xTF32: x = xh + xl with xh = x & 0xFFFFE000 (the 19 bits a TF32 operand keeps) and
// xl = x - xh (exact in fp32); likewise p = ph + pl.  x.p ~= xh.ph + xh.pl + xl.ph, three
// MMAs into one fp32 accumulator; the dropped xl.pl term is below 2^-22 relative.  P is split
// once per index (prepare_project_tc); X tiles are split in shared memory by a transform
// warpgroup after the TMA load lands (element-wise, so the TMA swizzle is preserved).  When a
// tile's xl is identically zero (e.g. integer-valued data below 2^11) its third MMA is skipped.
//
// One persistent CTA per SM, 14 warps:
//   warp 0      TMA producer (one lane)            full[s]  <- TMA bytes
//   warp 1      MMA issuer (one lane), TMEM owner  ready[s] <- transform, empty[s] <- MMA done
//   warps 2-5   split X tiles into hi / lo         acc_full[b] <- MMA done, acc_empty[b] <- epilogue
//   warps 6-13  epilogue: tcgen05.ld -> quantise -> pack -> store
// A work unit is (128-row tile, chunk of whole tables with <= 256 hash columns); two TMEM
// accumulators of 256 columns alternate so the epilogue of one unit overlaps the MMAs of the
// next.  Every mbarrier wait is bounded: when one runs out the CTA raises an abort flag,
// records DEV_ERR_MBAR_TIMEOUT, and all roles leave their loops; TMEM is released at the end.
// No TMA load uses cluster multicast.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace culsh_b200 {

constexpr int TC_BM = 128;          // rows per tile (MMA M)
constexpr int TC_BN = 256;          // accumulator columns (max MMA N)
constexpr int TC_TRANSFORM_THREADS = 128;
constexpr int TC_EPI_WARPS = 8;     // two warps per TMEM lane quarter, each takes half of the tables
constexpr int TC_EPI_THREADS = TC_EPI_WARPS * 32;
constexpr int TC_THREADS = 64 + TC_TRANSFORM_THREADS + TC_EPI_THREADS;
constexpr long long TC_WAIT_CYCLES = 4000000000ll;  // ~2 s at 2 GHz

template <int KBLK>
struct TcCfg {
    static constexpr int STAGES = KBLK == 32 ? 2 : 4;
    static constexpr int SWIZZLE_BYTES = KBLK * 4;              // 128 or 64
    static constexpr int X_BYTES = TC_BM * KBLK * 4;
    static constexpr int P_BYTES = TC_BN * KBLK * 4;
    static constexpr int STAGE_BYTES = 2 * X_BYTES + 2 * P_BYTES;
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 /*barriers*/ + 1024 /*alignment slack*/;
};

struct TcArgs {
    uint32_t* keys;
    uint8_t* ovf_rows;
    int* d_error;
    unsigned long long* d_mma;  // [0] K-blocks issued, [1] of them with the low-part MMA (or null)
    const float* bias;
    int n, d, L, k;
    int n_tiles, n_chunks, tables_per_chunk, n_mma, n_kblocks;
    int key_words, elem_bytes, family;
    int row_offset, n_total;
};

// ------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking probe of a phase (try_wait may suspend the thread for a while, test_wait never does).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false when the CTA is aborting (the caller leaves its loop).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* d_error) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > TC_WAIT_CYCLES) {
            *abort_flag = 1;
            atomicOr(d_error, DEV_ERR_MBAR_TIMEOUT);
            return false;
        }
    }
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x,
                                            int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile whose rows are one swizzle span wide
// (KBLK fp32 = 128 B or 64 B): 8-row groups follow each other every 8 * span bytes.
template <int KBLK>
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    constexpr uint64_t SBO = (8u * KBLK * 4u) >> 4;
    constexpr uint64_t LAYOUT = KBLK == 32 ? 2ull /*SWIZZLE_128B*/ : 4ull /*SWIZZLE_64B*/;
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (SBO << 32) | (1ull << 46) | (LAYOUT << 61);
}

// kind::tf32, fp32 accumulate, both operands K-major: c_format=F32 (bit 4), a/b format TF32 (=2)
__device__ __forceinline__ uint32_t make_idesc_tf32(int M, int N) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// 256-bit shift register that receives the key bytes / bits of one table, first element most
// significant; after k elements it holds the right-aligned key (w[0] most significant).
struct KeyReg {
    uint64_t w[4];
    __device__ __forceinline__ void clear() { w[0] = w[1] = w[2] = w[3] = 0; }
    __device__ __forceinline__ void push(uint32_t v, int bits) {  // bits in {1, 8, 16, 32}
        w[0] = (w[0] << bits) | (w[1] >> (64 - bits));
        w[1] = (w[1] << bits) | (w[2] >> (64 - bits));
        w[2] = (w[2] << bits) | (w[3] >> (64 - bits));
        w[3] = (w[3] << bits) | (uint64_t)v;
    }
    __device__ __forceinline__ void store(uint32_t* dst, int NW) const {
        if (NW == 1) { dst[0] = (uint32_t)w[3]; }
        else if (NW == 2) { *reinterpret_cast<uint2*>(dst) = make_uint2((uint32_t)(w[3] >> 32), (uint32_t)w[3]); }
        else if (NW == 4) {
            *reinterpret_cast<uint4*>(dst) =
                make_uint4((uint32_t)(w[2] >> 32), (uint32_t)w[2], (uint32_t)(w[3] >> 32), (uint32_t)w[3]);
        } else {
            reinterpret_cast<uint4*>(dst)[0] =
                make_uint4((uint32_t)(w[0] >> 32), (uint32_t)w[0], (uint32_t)(w[1] >> 32), (uint32_t)w[1]);
            reinterpret_cast<uint4*>(dst)[1] =
                make_uint4((uint32_t)(w[2] >> 32), (uint32_t)w[2], (uint32_t)(w[3] >> 32), (uint32_t)w[3]);
        }
    }
};

// Epilogue of one work unit for one warp: stream the accumulator columns [c_begin, c_end) of
// this warp's 32 TMEM lanes (= 32 rows), quantise each value and shift it into the key of its
// table; a finished table is stored as NW words.  KW selects the key register: 1 = 32-bit,
// 2 = 64-bit, 0 = 256-bit.  All control flow is warp-uniform (every lane walks the same
// columns), as tcgen05.ld requires.
template <int FAMILY, int KW>
__device__ __forceinline__ bool epilogue_columns(const TcArgs& a, uint32_t taddr, int c_begin, int c_end,
                                                 int first_table, int bias_base, int row, bool row_ok) {
    const int k = a.k, NW = a.key_words;
    const int bits = FAMILY == CULSH_RPLSH ? 1 : 8 * a.elem_bytes;
    const int lim = a.elem_bytes == 1 ? 128 : (a.elem_bytes == 2 ? 32768 : 0);
    uint32_t acc32 = 0;
    uint64_t acc64 = 0;
    KeyReg wide;
    wide.clear();
    int cnt = 0, tbl = first_table;
    bool ovf = false, any_ovf = false;
    const int g_begin = c_begin & ~15;
    for (int g0 = g_begin; g0 < c_end; g0 += 16) {
        uint32_t r[16];
        tc_ld16(taddr + (uint32_t)g0, r);
        tc_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int col = g0 + j;
            if ((unsigned)(col - c_begin) < (unsigned)(c_end - c_begin)) {
                uint32_t e;
                if (FAMILY == CULSH_RPLSH) {
                    e = r[j] >> 31;  // sign bit; inverted when the key is stored
                } else {
                    const int q = (int)floorf(__uint_as_float(r[j]) + a.bias[bias_base + col]);  // pslsh/hash.cuh:46
                    if (lim && (unsigned)(q + lim) >= (unsigned)(2 * lim)) ovf = true;
                    const uint32_t uq = (uint32_t)q;
                    e = a.elem_bytes == 1 ? (uq & 0xFFu)
                        : a.elem_bytes == 2 ? (((uq & 0xFFu) << 8) | ((uq >> 8) & 0xFFu))
                                            : __byte_perm(uq, 0, 0x0123);
                }
                if (KW == 1) {
                    if (FAMILY == CULSH_RPLSH) acc32 = __funnelshift_l(r[j], acc32, 1);
                    else acc32 = bits == 32 ? e : ((acc32 << bits) | e);
                } else if (KW == 2) {
                    acc64 = (acc64 << bits) | (uint64_t)e;
                } else {
                    wide.push(e, bits);
                }
                if (++cnt == k) {
                    if (row_ok) {
                        const size_t item = (size_t)tbl * a.n_total + a.row_offset + row;
                        uint32_t* dst = a.keys + item * NW;
                        if (KW == 1) {
                            // RPLSH: stored bit = 1 where the sign bit is clear (rplsh/hash.cuh:47)
                            dst[0] = FAMILY == CULSH_RPLSH ? (~acc32 & (k == 32 ? 0xFFFFFFFFu : ((1u << k) - 1u)))
                                                           : acc32;
                        } else if (KW == 2) {
                            uint64_t v = acc64;
                            if (FAMILY == CULSH_RPLSH) v = ~v & (k == 64 ? ~0ull : ((1ull << k) - 1ull));
                            *reinterpret_cast<uint2*>(dst) = make_uint2((uint32_t)(v >> 32), (uint32_t)v);
                        } else {
                            if (FAMILY == CULSH_RPLSH) {  // invert the k low bits of the 256-bit register
#pragma unroll
                                for (int w = 0; w < 4; ++w) {
                                    const int lo_bit = 64 * (3 - w);
                                    uint64_t m = k >= lo_bit + 64 ? ~0ull : (k > lo_bit ? ((1ull << (k - lo_bit)) - 1ull) : 0ull);
                                    wide.w[w] = ~wide.w[w] & m;
                                }
                            }
                            wide.store(dst, NW);
                        }
                        if (FAMILY == CULSH_PSLSH) {
                            if (a.ovf_rows) a.ovf_rows[item] = ovf ? 1 : 0;
                            else any_ovf |= ovf;
                        }
                    }
                    acc32 = 0;
                    acc64 = 0;
                    if (KW == 0) wide.clear();
                    cnt = 0;
                    ovf = false;
                    ++tbl;
                }
            }
        }
    }
    return any_ovf;
}

// Fast form of the p-stable epilogue for one-byte elements and K in {1, 2, 4, 8, 16} hashes per
// table (16 accumulator columns = 16 / K whole tables, c_begin a multiple of 16): the 16 values of
// a group are quantised with independent instructions (one add, one float->int with floor
// rounding, one range test, one byte insert each) and the keys are slices of the resulting 16
// bytes - no per-element bookkeeping or branches as in the general form.
template <int K>
__device__ __forceinline__ bool epilogue_pslsh_bytes(const TcArgs& a, uint32_t taddr, int c_begin, int c_end,
                                                     int first_table, int bias_base, int row, bool row_ok) {
    constexpr int PER_GROUP = 16 / K;
    constexpr int NW = K <= 4 ? 1 : K / 4;
    bool any_ovf = false;
    int tbl = first_table;
    int tables_left = (c_end - c_begin) / K;
    for (int g0 = c_begin; g0 < c_end; g0 += 16, tbl += PER_GROUP, tables_left -= PER_GROUP) {
        uint32_t r[16];
        tc_ld16(taddr + (uint32_t)g0, r);
        tc_ld_wait();
        const float* __restrict__ bias = a.bias + bias_base + g0;
#pragma unroll
        for (int ti = 0; ti < PER_GROUP; ++ti) {
            if (ti < tables_left) {  // warp-uniform
                uint32_t w[NW];
#pragma unroll
                for (int i = 0; i < NW; ++i) w[i] = 0u;
                uint32_t bad = 0u;
#pragma unroll
                for (int e = 0; e < K; ++e) {
                    const int j = ti * K + e;
                    const int q = __float2int_rd(__uint_as_float(r[j]) + __ldg(bias + j));  // pslsh/hash.cuh:46
                    bad |= (uint32_t)(q + 128) >> 8;  // non-zero outside [-128, 127]
                    const int pos = NW * 4 - K + e;    // byte position in the key, 0 = most significant
                    w[pos >> 2] |= ((uint32_t)q & 0xFFu) << (24 - 8 * (pos & 3));
                }
                if (row_ok) {
                    const size_t item = (size_t)(tbl + ti) * a.n_total + a.row_offset + row;
                    uint32_t* dst = a.keys + item * NW;
                    if (NW == 1) dst[0] = w[0];
                    else if (NW == 2) *reinterpret_cast<uint2*>(dst) = make_uint2(w[0], w[1]);
                    else *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2 % NW], w[3 % NW]);
                    if (a.ovf_rows) a.ovf_rows[item] = bad ? 1 : 0;
                    else any_ovf |= bad != 0u;
                }
            }
        }
    }
    return any_ovf;
}

// Fast form of the sign-bit epilogue for keys of one word (k <= 32): sixteen accumulator columns
// become sixteen key bits with straight-line code (no per-element counters or branches as in the
// general form), the bits run through a 64-bit buffer from which every finished table takes its k
// bits, and the tensor-memory load of the next sixteen columns is in flight while the current ones
// are packed.  The general form made the epilogue warps the limit of shapes with few K-blocks per
// unit (1M x 128, 32 x 16: 1,200 of every 1,400 cycles busy).
__device__ __forceinline__ void epilogue_rplsh_bits(const TcArgs& a, uint32_t taddr, int c_begin, int c_end,
                                                    int first_table, int row, bool row_ok) {
    const int k = a.k;
    const uint64_t kmask = k == 32 ? 0xFFFFFFFFull : ((1ull << k) - 1ull);
    int tables_left = (c_end - c_begin) / k;
    int tbl = first_table;
    uint64_t buf = 0;
    int nbits = -(c_begin & 15);  // columns of the first group that lie before c_begin are dropped
    auto consume = [&](const uint32_t (&r)[16]) {
        uint32_t m = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) m |= ((~r[j]) >> 31) << (15 - j);  // 1 where the sign bit is clear (rplsh/hash.cuh:47)
        if (nbits < 0) { m &= 0xFFFFu >> (-nbits); }
        buf = (buf << 16) | (uint64_t)m;
        nbits += 16;
        while (nbits >= k && tables_left > 0) {  // warp-uniform
            const uint32_t key = (uint32_t)((buf >> (nbits - k)) & kmask);
            if (row_ok) a.keys[(size_t)tbl * a.n_total + a.row_offset + row] = key;
            nbits -= k; ++tbl; --tables_left;
        }
    };
    // groups of sixteen columns on sixteen-column boundaries (the last group may reach past c_end,
    // never past the accumulator: its width is a multiple of sixteen); the load of the next group
    // is in flight while the current one is packed
    uint32_t ra[16], rb[16];
    int g = c_begin & ~15;
    tc_ld16(taddr + (uint32_t)g, ra);
    tc_ld_wait();
    while (tables_left > 0) {
        const bool n1 = g + 16 < c_end;
        if (n1) tc_ld16(taddr + (uint32_t)(g + 16), rb);
        consume(ra);
        if (!n1) break;
        tc_ld_wait();
        const bool n2 = g + 32 < c_end;
        if (n2) tc_ld16(taddr + (uint32_t)(g + 32), ra);
        consume(rb);
        if (!n2) break;
        tc_ld_wait();
        g += 32;
    }
}

template <int KBLK, int FAMILY>
__global__ void __launch_bounds__(TC_THREADS, 1)
project_tc_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmP, TcArgs a) {
    using Cfg = TcCfg<KBLK>;
    constexpr int STAGES = Cfg::STAGES;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    auto xh = [&](int s) { return reinterpret_cast<float*>(base + (size_t)s * Cfg::STAGE_BYTES); };
    auto xl = [&](int s) { return reinterpret_cast<float*>(base + (size_t)s * Cfg::STAGE_BYTES + Cfg::X_BYTES); };
    auto ph = [&](int s) { return reinterpret_cast<float*>(base + (size_t)s * Cfg::STAGE_BYTES + 2 * Cfg::X_BYTES); };
    auto pl = [&](int s) {
        return reinterpret_cast<float*>(base + (size_t)s * Cfg::STAGE_BYTES + 2 * Cfg::X_BYTES + Cfg::P_BYTES);
    };
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + (size_t)STAGES * Cfg::STAGE_BYTES);
    uint64_t* full = bars;                   // [STAGES]
    uint64_t* ready = bars + STAGES;         // [STAGES]
    uint64_t* empty = bars + 2 * STAGES;     // [STAGES]
    uint64_t* acc_full = bars + 3 * STAGES;  // [2]
    uint64_t* acc_empty = acc_full + 2;      // [2]
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
    volatile int* s_lo_flag = s_abort + 1;   // [STAGES]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&ready[s], TC_TRANSFORM_THREADS / 32);  // one arrival per split warp
            mbar_init(&empty[s], 1);
            s_lo_flag[s] = 0;
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], TC_EPI_WARPS);  // one arrival per epilogue warp
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // whole warp: allocate all 512 TMEM columns (one CTA per SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    const int n_units_per_tile = a.n_chunks;
    const uint32_t stage_tx = (uint32_t)(Cfg::X_BYTES + 2 * a.n_mma * KBLK * 4);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool live = true;
            for (int tile = blockIdx.x; tile < a.n_tiles && live; tile += gridDim.x) {
                for (int c = 0; c < n_units_per_tile && live; ++c) {
                    for (int kb = 0; kb < a.n_kblocks; ++kb, ++it) {
                        const int s = it % STAGES;
                        const uint32_t phs = (it / STAGES) & 1;
                        if (!mbar_wait(&empty[s], phs ^ 1, s_abort, a.d_error)) { live = false; break; }
                        mbar_expect_tx(&full[s], stage_tx);
                        tma_load_2d(xh(s), &tmX, &full[s], kb * KBLK, tile * TC_BM);
                        tma_load_2d(ph(s), &tmP, &full[s], kb * KBLK, (c * 2 + 0) * a.n_mma);
                        tma_load_2d(pl(s), &tmP, &full[s], kb * KBLK, (c * 2 + 1) * a.n_mma);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc_tf32(TC_BM, a.n_mma);
            uint32_t it = 0, u = 0;
            unsigned long long n_kb = 0, n_lo = 0;
            bool pre_ok = false;
            int pre_flag = 0;
            bool live = true;
            for (int tile = blockIdx.x; tile < a.n_tiles && live; tile += gridDim.x) {
                for (int c = 0; c < n_units_per_tile && live; ++c, ++u) {
                    const int ab = u & 1;
                    const uint32_t aph = (u >> 1) & 1;
                    if (!mbar_wait(&acc_empty[ab], aph ^ 1, s_abort, a.d_error)) { live = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)(ab * TC_BN);
                    for (int kb = 0; kb < a.n_kblocks; ++kb, ++it) {
                        const int s = it % STAGES;
                        const uint32_t phs = (it / STAGES) & 1;
                        // The issuing thread is the serial resource of the kernel (a wait that succeeds
                        // at once still costs ~100 cycles), so the barriers and the flag of the next
                        // stage are probed before this stage's MMAs are issued and the answer is used
                        // one iteration later.
                        if (!pre_ok && (!mbar_wait(&full[s], phs, s_abort, a.d_error) ||
                                        !mbar_wait(&ready[s], phs, s_abort, a.d_error))) { live = false; break; }
                        tc_fence_after();
                        const int use_lo = pre_ok ? pre_flag : s_lo_flag[s];
                        s_lo_flag[s] = 0;
                        {
                            const int s1 = (it + 1) % STAGES;
                            const uint32_t ph1 = ((it + 1) / STAGES) & 1;
                            const bool f = mbar_test_wait(&full[s1], ph1);
                            const bool r = mbar_test_wait(&ready[s1], ph1);
                            pre_flag = s_lo_flag[s1];  // meaningful only when both phases have completed
                            pre_ok = f && r;
                        }
                        ++n_kb;
                        n_lo += use_lo ? 1u : 0u;
                        const uint64_t dxh = make_smem_desc<KBLK>(smem_u32(xh(s)));
                        const uint64_t dxl = make_smem_desc<KBLK>(smem_u32(xl(s)));
                        const uint64_t dph = make_smem_desc<KBLK>(smem_u32(ph(s)));
                        const uint64_t dpl = make_smem_desc<KBLK>(smem_u32(pl(s)));
#pragma unroll
                        for (int ks = 0; ks < KBLK / 8; ++ks) {
                            const uint64_t adv = (uint64_t)(ks * 2);  // 32 bytes per K step, in 16-byte units
                            tc_mma_tf32(d_tmem, dxh + adv, dpl + adv, idesc, (kb | ks) != 0);
                            if (use_lo) tc_mma_tf32(d_tmem, dxl + adv, dph + adv, idesc, 1u);
                            tc_mma_tf32(d_tmem, dxh + adv, dph + adv, idesc, 1u);
                        }
                        tc_commit(&empty[s]);  // stage reusable once these MMAs have read it
                    }
                    if (live) tc_commit(&acc_full[ab]);
                }
            }
            if (a.d_mma) {
                atomicAdd(a.d_mma, n_kb);
                atomicAdd(a.d_mma + 1, n_lo);
            }
        }
    } else if (warp < 6) {
        // ---------------- transform: split X tiles into hi / lo ----------------
        const int tt = threadIdx.x - 64;  // 0..127
        uint32_t it = 0;
        bool live = true;
        for (int tile = blockIdx.x; tile < a.n_tiles && live; tile += gridDim.x) {
            for (int c = 0; c < n_units_per_tile && live; ++c) {
                for (int kb = 0; kb < a.n_kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t phs = (it / STAGES) & 1;
                    if (!mbar_wait(&full[s], phs, s_abort, a.d_error)) { live = false; break; }
                    uint4* h4 = reinterpret_cast<uint4*>(xh(s));
                    uint4* l4 = reinterpret_cast<uint4*>(xl(s));
                    bool any_lo = false;
#pragma unroll
                    for (int j = 0; j < Cfg::X_BYTES / 16 / TC_TRANSFORM_THREADS; ++j) {
                        const int idx = tt + j * TC_TRANSFORM_THREADS;
                        uint4 v = h4[idx];
                        uint4 hi = make_uint4(v.x & 0xFFFFE000u, v.y & 0xFFFFE000u, v.z & 0xFFFFE000u,
                                              v.w & 0xFFFFE000u);
                        float lx = __uint_as_float(v.x) - __uint_as_float(hi.x);
                        float ly = __uint_as_float(v.y) - __uint_as_float(hi.y);
                        float lz = __uint_as_float(v.z) - __uint_as_float(hi.z);
                        float lw = __uint_as_float(v.w) - __uint_as_float(hi.w);
                        any_lo |= (lx != 0.f) | (ly != 0.f) | (lz != 0.f) | (lw != 0.f);
                        h4[idx] = hi;
                        l4[idx] = make_uint4(__float_as_uint(lx), __float_as_uint(ly), __float_as_uint(lz),
                                             __float_as_uint(lw));
                    }
                    if (any_lo) s_lo_flag[s] = 1;
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ready[s]);  // 128 arrivals on one barrier would serialise
                }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;        // TMEM lanes this warp may read: 32*quarter ...
        const int half = (warp - 6) >> 2;    // which half of the unit's tables this warp packs
        const int NW = a.key_words;
        const int k = a.k;
        uint32_t u = 0;
        bool live = true;
        bool any_ovf = false;
        for (int tile = blockIdx.x; tile < a.n_tiles && live; tile += gridDim.x) {
            const int row = tile * TC_BM + quarter * 32 + lane;
            const bool row_ok = row < a.n;
            for (int c = 0; c < n_units_per_tile && live; ++c, ++u) {
                const int ab = u & 1;
                const uint32_t aph = (u >> 1) & 1;
                if (!mbar_wait(&acc_full[ab], aph, s_abort, a.d_error)) { live = false; break; }
                tc_fence_after();
                const int t0 = c * a.tables_per_chunk;
                const int tables_here = min(a.tables_per_chunk, a.L - t0);
                const int split = (tables_here + 1) >> 1;
                const int tb = half == 0 ? 0 : split, te = half == 0 ? split : tables_here;
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ab * TC_BN);
                if (te > tb) {
                    bool o;
                    const bool byte_form = FAMILY == CULSH_PSLSH && a.elem_bytes == 1 && ((tb * k) & 15) == 0;
                    if (FAMILY == CULSH_RPLSH && NW == 1) { epilogue_rplsh_bits(a, taddr, tb * k, te * k, t0 + tb, row, row_ok); o = false; }
                    else if (byte_form && k == 8) o = epilogue_pslsh_bytes<8>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else if (byte_form && k == 4) o = epilogue_pslsh_bytes<4>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else if (byte_form && k == 16) o = epilogue_pslsh_bytes<16>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else if (byte_form && k == 2) o = epilogue_pslsh_bytes<2>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else if (NW == 1) o = epilogue_columns<FAMILY, 1>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else if (NW == 2) o = epilogue_columns<FAMILY, 2>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else o = epilogue_columns<FAMILY, 0>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    any_ovf |= o;
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[ab]);
            }
        }
        if (any_ovf) atomicOr(a.d_error, DEV_ERR_NARROW_OVERFLOW);
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// TS form: the X operand comes from tensor memory.  An MMA that takes both operands from shared
// memory reads 4 KB (A) + 32 B x N (B) per K = 8 step, and with the TMA writes and the hi / lo
// split on top the kernel above is bound by shared-memory bandwidth and by the depth of a
// four-stage ring of 48 KB stages.  Here the split warps write xh / xl straight into tensor
// memory (tcgen05.st, 16 + 16 columns per 16-wide K-block) and the MMAs read only P from shared
// memory: a stage is X as loaded + P hi + P lo for BN hash columns (32-wide K-blocks: 48 KB and
// four stages at BN = 128, 64 KB and three stages at BN = 192).  Tensor memory: two accumulators
// of BN columns + an A ring in the remaining columns (hi + lo of a K-block = 64 columns: four
// stages at BN = 128, two at BN = 192, where a split warp therefore waits for the MMAs of the
// K-block two back before it overwrites their operand).  G groups of four
// split warps can take the K-blocks in turn (one group is enough: the issuing thread is the limit).  Roles, barriers, epilogue and abort protocol are those of the
// kernel above; a work unit is (128-row tile, chunk of whole tables with <= 128 hash columns).
// ------------------------------------------------------------------------------------------
constexpr int TS_BN = 128;      // accumulator columns of the narrow form
constexpr int TS_BN_WIDE = 192; // and of the wide form (shapes of several chunks)
template <int KB, int BN>
struct TsCfg {
    static constexpr int A_STAGES = (512 - 2 * BN) / (2 * KB);  // tensor-memory columns left for xh / xl
    static constexpr int X_BYTES = TC_BM * KB * 4;
    static constexpr int P_BYTES = BN * KB * 4;                 // per part
    static constexpr int STAGE_BYTES = X_BYTES + 2 * P_BYTES;
    static constexpr int STAGES = (192 * 1024) / STAGE_BYTES;   // shared-memory ring
    static constexpr int SMEM = STAGES * STAGE_BYTES + 1024 + 1024;
    static_assert(A_STAGES >= 2 && STAGES >= A_STAGES, "ring sizes");
};

__device__ __forceinline__ void tc_mma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tc_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <int FAMILY, int G, int KB, int BN>
__global__ void __launch_bounds__(64 + G * TC_TRANSFORM_THREADS + TC_EPI_THREADS, 1)
project_ts_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmP, TcArgs a) {
    using Cfg = TsCfg<KB, BN>;
    constexpr int STAGES = Cfg::STAGES, A_STAGES = Cfg::A_STAGES;
    constexpr int TS_A_COL0 = 2 * BN;  // first tensor-memory column of the A ring
    constexpr int TS_KBLK = KB, TS_X_BYTES = Cfg::X_BYTES, TS_STAGE_BYTES = Cfg::STAGE_BYTES;
    extern __shared__ unsigned char tc_smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(
        (reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~(uintptr_t)1023);
    auto xs = [&](int s) { return base + (size_t)s * TS_STAGE_BYTES; };
    auto ph = [&](int s) { return base + (size_t)s * TS_STAGE_BYTES + TS_X_BYTES; };
    auto pl = [&](int s) { return base + (size_t)s * TS_STAGE_BYTES + TS_X_BYTES + Cfg::P_BYTES; };
    uint64_t* bars = reinterpret_cast<uint64_t*>(base + (size_t)STAGES * TS_STAGE_BYTES);
    uint64_t* full = bars;                   // [STAGES] TMA bytes landed
    uint64_t* ready = bars + STAGES;         // [STAGES] xh / xl of the stage are in tensor memory
    uint64_t* empty = bars + 2 * STAGES;     // [STAGES] the stage's MMAs have completed
    uint64_t* acc_full = bars + 3 * STAGES;  // [2]
    uint64_t* acc_empty = acc_full + 2;      // [2]
    uint32_t* s_tmem = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
    volatile int* s_lo_flag = s_abort + 1;   // [STAGES]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&ready[s], TC_TRANSFORM_THREADS / 32);  // one arrival per warp of a split group
            mbar_init(&empty[s], 1);
            s_lo_flag[s] = 0;
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], TC_EPI_WARPS);  // one arrival per epilogue warp
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {  // whole warp: allocate all 512 tensor-memory columns (one CTA per SM)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *s_tmem;

    const int n_units_per_tile = a.n_chunks;
    const uint32_t stage_tx = (uint32_t)(TS_X_BYTES + 2 * a.n_mma * TS_KBLK * 4);

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool live = true;
            for (int tile = blockIdx.x; tile < a.n_tiles && live; tile += gridDim.x) {
                for (int c = 0; c < n_units_per_tile && live; ++c) {
                    for (int kb = 0; kb < a.n_kblocks; ++kb, ++it) {
                        const int s = it % STAGES;
                        const uint32_t phs = (it / STAGES) & 1;
                        if (!mbar_wait(&empty[s], phs ^ 1, s_abort, a.d_error)) { live = false; break; }
                        mbar_expect_tx(&full[s], stage_tx);
                        tma_load_2d(xs(s), &tmX, &full[s], kb * TS_KBLK, tile * TC_BM);
                        tma_load_2d(ph(s), &tmP, &full[s], kb * TS_KBLK, (c * 2 + 0) * a.n_mma);
                        tma_load_2d(pl(s), &tmP, &full[s], kb * TS_KBLK, (c * 2 + 1) * a.n_mma);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc_tf32(TC_BM, a.n_mma);
            uint32_t it = 0, u = 0;
            unsigned long long n_kb = 0, n_lo = 0;
            bool pre_ok = false;
            int pre_flag = 0;
            bool live = true;
            for (int tile = blockIdx.x; tile < a.n_tiles && live; tile += gridDim.x) {
                for (int c = 0; c < n_units_per_tile && live; ++c, ++u) {
                    const int ab = u & 1;
                    const uint32_t aph = (u >> 1) & 1;
                    if (!mbar_wait(&acc_empty[ab], aph ^ 1, s_abort, a.d_error)) { live = false; break; }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + (uint32_t)(ab * BN);
                    for (int kb = 0; kb < a.n_kblocks; ++kb, ++it) {
                        const int s = it % STAGES;
                        const uint32_t phs = (it / STAGES) & 1;
                        // next stage's barriers and flag are probed early, as in project_tc_kernel
                        if (!pre_ok && (!mbar_wait(&full[s], phs, s_abort, a.d_error) ||
                                        !mbar_wait(&ready[s], phs, s_abort, a.d_error))) { live = false; break; }
                        tc_fence_after();
                        const int use_lo = pre_ok ? pre_flag : s_lo_flag[s];
                        s_lo_flag[s] = 0;
                        {
                            const int s1 = (it + 1) % STAGES;
                            const uint32_t ph1 = ((it + 1) / STAGES) & 1;
                            const bool f = mbar_test_wait(&full[s1], ph1);
                            const bool r = mbar_test_wait(&ready[s1], ph1);
                            pre_flag = s_lo_flag[s1];  // meaningful only when both phases have completed
                            pre_ok = f && r;
                        }
                        ++n_kb;
                        n_lo += use_lo ? 1u : 0u;
                        const uint32_t axh = tmem_base + (uint32_t)(TS_A_COL0 + (int)(it % A_STAGES) * 2 * TS_KBLK);
                        const uint32_t axl = axh + (uint32_t)TS_KBLK;
                        const uint64_t dph = make_smem_desc<TS_KBLK>(smem_u32(ph(s)));
                        const uint64_t dpl = make_smem_desc<TS_KBLK>(smem_u32(pl(s)));
#pragma unroll
                        for (int ks = 0; ks < TS_KBLK / 8; ++ks) {
                            const uint64_t adv = (uint64_t)(ks * 2);  // 32 bytes per K step, in 16-byte units
                            const uint32_t acol = (uint32_t)(ks * 8);  // 8 tf32 values = 8 columns per K step
                            tc_mma_tf32_ts(d_tmem, axh + acol, dpl + adv, idesc, (kb | ks) != 0);
                            if (use_lo) tc_mma_tf32_ts(d_tmem, axl + acol, dph + adv, idesc, 1u);
                            tc_mma_tf32_ts(d_tmem, axh + acol, dph + adv, idesc, 1u);
                        }
                        tc_commit(&empty[s]);  // shared-memory stage and A stage reusable once these MMAs are done
                    }
                    if (live) tc_commit(&acc_full[ab]);
                }
            }
            if (a.d_mma) {
                atomicAdd(a.d_mma, n_kb);
                atomicAdd(a.d_mma + 1, n_lo);
            }
        }
    } else if (warp < 2 + 4 * G) {
        // ---------------- split X into hi / lo, straight into tensor memory ----------------
        // G groups of four warps take the K-blocks in turn, so that G of them are in flight.
        const int grp = (warp - 2) >> 2;
        // Warp w may touch tensor-memory lanes 32 * (w % 4) ...: a lane owns one row of the tile.
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;
        // TMA swizzle: 16-byte chunk c of row r sits at chunk c ^ sw (64-byte rows: (r >> 1) & 3, 128-byte rows: r & 7)
        const int sw = KB == 32 ? (r & 7) : ((r >> 1) & 3);
        uint32_t it = 0;
        bool live = true;
        for (int tile = blockIdx.x; tile < a.n_tiles && live; tile += gridDim.x) {
            for (int c = 0; c < n_units_per_tile && live; ++c) {
                for (int kb = 0; kb < a.n_kblocks; ++kb, ++it) {
                    if ((int)(it % G) != grp) continue;
                    const int s = it % STAGES;
                    const uint32_t phs = (it / STAGES) & 1;
                    if (!mbar_wait(&full[s], phs, s_abort, a.d_error)) { live = false; break; }
                    const uint4* row = reinterpret_cast<const uint4*>(xs(s) + (size_t)r * (TS_KBLK * 4));
                    uint32_t hi[KB], lo[KB];
                    bool any_lo = false;
#pragma unroll
                    for (int j = 0; j < KB / 4; ++j) {
                        const uint4 v = row[j ^ sw];
                        const uint32_t x[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t h = x[e] & 0xFFFFE000u;
                            const float l = __uint_as_float(x[e]) - __uint_as_float(h);
                            hi[4 * j + e] = h;
                            lo[4 * j + e] = __float_as_uint(l);
                            any_lo |= l != 0.f;
                        }
                    }
                    // The A stage must be free: the MMAs of K-block it - A_STAGES have completed.  With as
                    // many A stages as shared-memory stages the producer's wait on `empty` before it
                    // refilled this stage says so already.
                    if (A_STAGES < STAGES && it >= (uint32_t)A_STAGES) {
                        const uint32_t prev = it - (uint32_t)A_STAGES;
                        if (!mbar_wait(&empty[prev % STAGES], (prev / STAGES) & 1, s_abort, a.d_error)) { live = false; break; }
                    }
                    tc_fence_after();
                    const uint32_t ta = tmem_base + ((uint32_t)(quarter * 32) << 16) +
                                        (uint32_t)(TS_A_COL0 + (int)(it % A_STAGES) * 2 * TS_KBLK);
#pragma unroll
                    for (int j = 0; j < KB / 16; ++j) {
                        tc_st16(ta + (uint32_t)(16 * j), hi + 16 * j);
                        tc_st16(ta + (uint32_t)(TS_KBLK + 16 * j), lo + 16 * j);
                    }
                    tc_st_wait();
                    if (any_lo) s_lo_flag[s] = 1;
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&ready[s]);  // 128 arrivals on one barrier would serialise
                }
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int quarter = warp & 3;        // TMEM lanes this warp may read: 32*quarter ...
        const int half = (warp - (2 + 4 * G)) >> 2;  // which half of the unit's tables this warp packs
        const int NW = a.key_words;
        const int k = a.k;
        uint32_t u = 0;
        bool live = true;
        bool any_ovf = false;
        for (int tile = blockIdx.x; tile < a.n_tiles && live; tile += gridDim.x) {
            const int row = tile * TC_BM + quarter * 32 + lane;
            const bool row_ok = row < a.n;
            for (int c = 0; c < n_units_per_tile && live; ++c, ++u) {
                const int ab = u & 1;
                const uint32_t aph = (u >> 1) & 1;
                if (!mbar_wait(&acc_full[ab], aph, s_abort, a.d_error)) { live = false; break; }
                tc_fence_after();
                const int t0 = c * a.tables_per_chunk;
                const int tables_here = min(a.tables_per_chunk, a.L - t0);
                const int split = (tables_here + 1) >> 1;
                const int tb = half == 0 ? 0 : split, te = half == 0 ? split : tables_here;
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(ab * BN);
                if (te > tb) {
                    bool o;
                    const bool byte_form = FAMILY == CULSH_PSLSH && a.elem_bytes == 1 && ((tb * k) & 15) == 0;
                    if (FAMILY == CULSH_RPLSH && NW == 1) { epilogue_rplsh_bits(a, taddr, tb * k, te * k, t0 + tb, row, row_ok); o = false; }
                    else if (byte_form && k == 8) o = epilogue_pslsh_bytes<8>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else if (byte_form && k == 4) o = epilogue_pslsh_bytes<4>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else if (byte_form && k == 16) o = epilogue_pslsh_bytes<16>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else if (byte_form && k == 2) o = epilogue_pslsh_bytes<2>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else if (NW == 1) o = epilogue_columns<FAMILY, 1>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else if (NW == 2) o = epilogue_columns<FAMILY, 2>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    else o = epilogue_columns<FAMILY, 0>(a, taddr, tb * k, te * k, t0 + tb, t0 * k, row, row_ok);
                    any_ovf |= o;
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[ab]);
            }
        }
        if (any_ovf) atomicOr(a.d_error, DEV_ERR_NARROW_OVERFLOW);
    }

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512) : "memory");
    }
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
struct TcPlan {
    int kblk, d_pad, n_chunks, tables_per_chunk, n_mma, bn;
    bool ts;
};

inline int tc_kblk_choice() {
    static int v = [] {
        const char* e = getenv("CULSH_TC_KBLK");
        int k = e ? atoi(e) : 16;
        return k == 32 ? 32 : 16;
    }();
    return v;
}

// Which kernel projects a shape.  Three forms: both operands in shared memory with chunks of
// <= 256 hash columns (project_tc_kernel), X in tensor memory with chunks of <= 128 columns, or of
// <= 192 columns (project_ts_kernel).  Measured on B200 (fit, ms):
//                                        shared, 256   tensor, 128   tensor, 192
//   12.5M x 96,  16 x 8  (one chunk)         2.31          1.85           -
//   1M x 128,    32 x 16                     0.62          0.66          0.62
//   10M x 256,   48 x 24                     24.8          29            22.7
// One chunk: the 128-column form.  Several chunks: a unit of n_mma columns costs about
// 40 + 1.3 * n_mma cycles per K step in every form (the tensor-memory form 9 % less), so the form
// with the smaller chunks * (40 + 1.3 * n_mma) is taken, the shared-memory one on a tie.
// CULSH_TC_VARIANT (read once per process) overrides: 0 = shared memory always, 1 = tensor memory /
// 128 columns wherever it applies, 3 = tensor memory / 192 columns for shapes of several chunks
// (the tests run every shape through each).
inline int tc_variant() {
    static int v = [] {
        const char* e = getenv("CULSH_TC_VARIANT");
        return e && *e ? atoi(e) : 2;
    }();
    return v;
}

inline void tc_chunking(int L, int k, int bn, int& tables_per_chunk, int& n_chunks, int& n_mma) {
    tables_per_chunk = std::min(L, bn / k);
    n_chunks = (L + tables_per_chunk - 1) / tables_per_chunk;
    n_mma = (tables_per_chunk * k + 15) / 16 * 16;
}

inline bool tc_plan(int d, int L, int k, TcPlan& p) {
    const int variant = tc_variant();
    bool ts;
    int bn;
    if (variant == 0) { ts = false; bn = TC_BN; }
    else if (variant == 1) { ts = k <= TS_BN; bn = ts ? TS_BN : TC_BN; }
    else if (variant == 3) { ts = k <= TS_BN_WIDE; bn = ts ? (L * k > TS_BN ? TS_BN_WIDE : TS_BN) : TC_BN; }
    else if (L * k <= TS_BN) { ts = true; bn = TS_BN; }
    else {
        ts = false; bn = TC_BN;
        if (k <= TS_BN_WIDE && k <= TC_BN) {
            int t, c, m;
            tc_chunking(L, k, TC_BN, t, c, m);
            const double cost_shared = c * (40.0 + 1.3 * m);
            tc_chunking(L, k, TS_BN_WIDE, t, c, m);
            const double cost_tensor = 0.91 * c * (40.0 + 1.3 * m);
            if (cost_tensor < 0.97 * cost_shared) { ts = true; bn = TS_BN_WIDE; }
        }
    }
    p.bn = bn;
    if (k > bn || d % 4 != 0) return false;
    p.ts = ts;
    p.kblk = ts ? 32 : tc_kblk_choice();
    p.d_pad = (d + p.kblk - 1) / p.kblk * p.kblk;
    tc_chunking(L, k, bn, p.tables_per_chunk, p.n_chunks, p.n_mma);
    return true;
}

// P_split layout: [chunk][hi | lo][n_mma rows][d_pad] fp32, zero where padded.
__global__ void split_projection_kernel(const float* __restrict__ P, int H, int d, int k, int d_pad,
                                        int tables_per_chunk, int n_mma, int n_chunks, float* __restrict__ out) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t per_part = (size_t)n_mma * d_pad;
    size_t total = (size_t)n_chunks * 2 * per_part;
    if (idx >= total) return;
    int c = (int)(idx / (2 * per_part));
    size_t rem = idx - (size_t)c * 2 * per_part;
    int part = (int)(rem / per_part);
    size_t rr = rem - (size_t)part * per_part;
    int r = (int)(rr / d_pad), col = (int)(rr - (size_t)r * d_pad);
    int h = c * tables_per_chunk * k + r;
    float v = 0.f;
    if (r < tables_per_chunk * k && h < H && col < d) {
        float p = P[(size_t)h * d + col];
        float hi = __uint_as_float(__float_as_uint(p) & 0xFFFFE000u);
        v = part == 0 ? hi : p - hi;
    }
    out[idx] = v;
}

inline void prepare_project_tc(const CtxPtr& c, const float* P, int H, int d, int L, int k,
                               DevBuf<uint8_t>& out) {
    TcPlan p;
    if (c->projection_path == 1 || !tc_plan(d, L, k, p)) return;
    size_t total = (size_t)p.n_chunks * 2 * p.n_mma * p.d_pad;
    out.alloc(c, total * sizeof(float));
    split_projection_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, c->stream>>>(
        P, H, d, k, p.d_pad, p.tables_per_chunk, p.n_mma, p.n_chunks, reinterpret_cast<float*>(out.p));
    KERNEL_CHECK();
}

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_tiled() {
    static PFN_encodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        cudaGetLastError();
        return reinterpret_cast<PFN_encodeTiled>(p);
    }();
    return fn;
}

inline bool make_map_2d(CUtensorMap* m, const void* base, uint64_t inner, uint64_t rows, uint64_t pitch_bytes,
                        uint32_t box_inner, uint32_t box_rows, int kblk) {
    PFN_encodeTiled enc = get_encode_tiled();
    if (!enc) return false;
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE,
                     kblk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Returns false when this shape / pointer cannot take the tensor-core path (caller falls back).
inline bool launch_project_tc(const CtxPtr& c, cudaStream_t stream, int family, const float* X, const float* P,
                              const uint8_t* p_split, const float* bias, int n, int d, int L, int k,
                              const KeySpec& ks, uint32_t* keys, uint8_t* ovf_rows, int row_offset,
                              int n_total) {
    (void)P;
    TcPlan p;
    if (!p_split || !tc_plan(d, L, k, p)) return false;
    if (ks.key_words > 8) return false;                       // key wider than the 256-bit packer
    if ((reinterpret_cast<uintptr_t>(X) & 15) != 0) return false;  // TMA base alignment
    if (n <= 0) return true;
    CUtensorMap tmX, tmP;
    if (!make_map_2d(&tmX, X, (uint64_t)d, (uint64_t)n, (uint64_t)d * 4, (uint32_t)p.kblk, TC_BM, p.kblk))
        return false;
    if (!make_map_2d(&tmP, p_split, (uint64_t)p.d_pad, (uint64_t)p.n_chunks * 2 * p.n_mma, (uint64_t)p.d_pad * 4,
                     (uint32_t)p.kblk, (uint32_t)p.n_mma, p.kblk))
        return false;
    TcArgs a{};
    a.keys = keys; a.ovf_rows = ovf_rows; a.d_error = c->d_error; a.bias = bias;
    a.d_mma = c->d_mma;
    a.n = n; a.d = d; a.L = L; a.k = k;
    a.n_tiles = (int)ceil_div(n, TC_BM);
    a.n_chunks = p.n_chunks; a.tables_per_chunk = p.tables_per_chunk; a.n_mma = p.n_mma;
    a.n_kblocks = p.d_pad / p.kblk;
    a.key_words = ks.key_words; a.elem_bytes = ks.elem_bytes; a.family = family;
    a.row_offset = row_offset; a.n_total = n_total;
    int grid = std::min(a.n_tiles, c->sm_count);
    if (p.ts) {
        auto go = [&](auto kern, int smem_bytes) -> bool {
            if ((size_t)smem_bytes > c->smem_optin) return false;
            CU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
            kern<<<grid, 64 + TC_TRANSFORM_THREADS + TC_EPI_THREADS, smem_bytes, stream>>>(tmX, tmP, a);
            KERNEL_CHECK();
            return true;
        };
        const bool rp = family == CULSH_RPLSH;
        if (p.bn == TS_BN_WIDE)
            return rp ? go(project_ts_kernel<CULSH_RPLSH, 1, 32, TS_BN_WIDE>, TsCfg<32, TS_BN_WIDE>::SMEM)
                      : go(project_ts_kernel<CULSH_PSLSH, 1, 32, TS_BN_WIDE>, TsCfg<32, TS_BN_WIDE>::SMEM);
        return rp ? go(project_ts_kernel<CULSH_RPLSH, 1, 32, TS_BN>, TsCfg<32, TS_BN>::SMEM)
                  : go(project_ts_kernel<CULSH_PSLSH, 1, 32, TS_BN>, TsCfg<32, TS_BN>::SMEM);
    }
    auto kern = p.kblk == 32
                    ? (family == CULSH_RPLSH ? project_tc_kernel<32, CULSH_RPLSH> : project_tc_kernel<32, CULSH_PSLSH>)
                    : (family == CULSH_RPLSH ? project_tc_kernel<16, CULSH_RPLSH> : project_tc_kernel<16, CULSH_PSLSH>);
    size_t smem = p.kblk == 32 ? (size_t)TcCfg<32>::SMEM : (size_t)TcCfg<16>::SMEM;
    if (smem > c->smem_optin) return false;
    CU_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, TC_THREADS, smem, stream>>>(tmX, tmP, a);
    KERNEL_CHECK();
    return true;
}

}  // namespace culsh_b200
