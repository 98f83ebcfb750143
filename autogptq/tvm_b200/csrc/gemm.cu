// Prefill dequant-GEMM on the 5th-generation tensor cores (tcgen05 + tensor memory), sm_100a.
//
//   y[M, N] = x[M, K] @ W[K, N] (+ bias),   W[k, n] = scales[g, n] * (q[k, n] - zero[g, n])
//
// One CTA computes a (128*MT) x 128 tile of y.  Roles of its six warps:
//   warp 0      TMA producer: x tiles (128 rows x 64 k, 128-byte swizzle) into the stage ring
//               and the matching packed weight rows (plain 2-D tile) into the same stage
//   warps 1..4  weight producers: each thread owns one of the 128 columns, reads that column's
//               packed words from the stage, dequantises them to the exact fp16
//               value of the reference (auto_gptq/nn_modules/qlinear.py:242: one rounding) and
//               writes 128-byte-swizzled K-major rows of the B operand; afterwards the same
//               warps run the epilogue (tcgen05.ld -> fp16 -> global)
//   warp 5      allocates tensor memory and issues tcgen05.mma (M=128, N=128, K=16, f16 -> f32)
// Stages hand over through mbarriers; tcgen05.commit releases a stage when its MMAs retire.
// Every wait is bounded: on expiry the kernel raises a sticky status word, unwinds, frees its
// tensor memory and returns.
//
// k order inside a 32-row block: 4-bit fields are produced in natural order, so x is read as
// it is; 3-bit fields come out of the 96-bit stream in a fixed permuted order, and layers with
// re-ordered rows need x gathered, so in those cases a small pre-pass writes a permuted copy
// of x into the scratch and the TMA reads that copy.
//
// Replaces the TVM-generated wmma kernels src/kernels/gemm_kernel.cu:25-142 of the reference.
#include <cuda.h>

#include "common.cuh"

namespace b200gptq {

namespace {

constexpr int BN = 128, BK = 64, BM = 128;
constexpr int kGemmThreads = 192;
constexpr int kATileBytes = BM * BK * 2;  // 16 KB
constexpr int kBTileBytes = BN * BK * 2;  // 16 KB
constexpr int kStatusWord = kMaxCounters - 1;  // sticky error word inside the counter region

constexpr int kPackedTileBytes = 4096;     // up to 8 word-rows x 128 columns of packed weights per k-tile

template <int MT> struct GemmCfg {
    static constexpr int kStages = MT == 1 ? 5 : 4;
    static constexpr int kStageBytes = MT * kATileBytes + kBTileBytes + kPackedTileBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
    static constexpr int kTmemCols = MT * BN;  // 128 or 256: powers of two
};

// 3-bit: order in which the 32 fields of a row block leave the 7-window unpack (pairs are
// adjacent entries).  x is permuted the same way by the pre-pass.
__constant__ unsigned char kOrder3[32] = {0, 3, 1, 7, 2, 8, 4, 9, 5, 10, 6, 11, 12, 17, 13, 18,
                                          14, 19, 15, 20, 16, 21, 22, 27, 23, 28, 24, 29, 25, 30, 26, 31};

// ---- small PTX wrappers -----------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2e9 clocks or as soon as another role has raised `abort_flag`.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > 2000000000LL) { *abort_flag = 1; return false; }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

// K-major, 128-byte-swizzled operand tile: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset: next 8-row group
    d |= (uint64_t)1 << 46;                    // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t magic) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(magic));
    return r;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// (field + offset) pair -> scale * (field - zero), exactly as the reference rounds it:
// the subtraction is exact in fp16 and the product is rounded once.
__device__ __forceinline__ uint32_t finish_pair(uint32_t biased, __half2 offset_plus_zero, __half2 scale2) {
    return h2_as_u32(__hmul2(__hsub2(u32_as_h2(biased), offset_plus_zero), scale2));
}

// fp16 exponent pattern that turns a field at bit p of a 16-bit half into 2^(10-p) + field.
__host__ __device__ constexpr uint32_t magic_at(int p) { return (uint32_t)(25 - p) << 10; }
__host__ __device__ constexpr float offset_at(int p) { return (float)(1 << (10 - p)); }

// ---- dequantisation of one 32-row block of one column into 4 chunks of 8 fp16 ---------------
template <int BITS> struct Dequant;

template <> struct Dequant<4> {
    static constexpr int kWords = 4;
    // Byte i of a word holds fields 2i (low nibble) and 2i+1 (high nibble).  PRMT copies the byte
    // into both halves; one LOP3 keeps the low nibble in the low half (offset 1024) and the
    // high nibble in the high half (offset 64): a pair in natural order.
    __device__ static __forceinline__ void run(const uint32_t (&w)[kWords], __half s, int z, uint4 (&out)[4]) {
        const __half2 s2 = __half2half2(s);
        const __half2 oz = __floats2half2_rn(1024.f + (float)z, 64.f + (float)z);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            uint32_t v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t rep = __byte_perm(w[r], 0u, 0x1111u * i);  // byte i in every byte lane
                v[i] = finish_pair(lop3_and_or(rep, 0x00f0000fu, 0x54006400u), oz, s2);
            }
            out[r] = make_uint4(v[0], v[1], v[2], v[3]);
        }
    }
};

template <> struct Dequant<3> {
    static constexpr int kWords = 3;
    template <int PLO, int PHI>
    __device__ static __forceinline__ uint32_t pair(uint32_t window, int z, __half2 s2) {
        constexpr uint32_t mask = (7u << PLO) | (7u << (PHI + 16));
        constexpr uint32_t magic = magic_at(PLO) | (magic_at(PHI) << 16);
        const __half2 oz = __floats2half2_rn(offset_at(PLO) + (float)z, offset_at(PHI) + (float)z);
        return finish_pair(lop3_and_or(window, mask, magic), oz, s2);
    }
    // Seven windows of the 96-bit stream cover the 32 fields exactly once with 16 pairs, in the
    // order of kOrder3: (0,3) (1,7)(2,8) (4,9)(5,10)(6,11) (12,17)(13,18) (14,19)(15,20)(16,21)
    // (22,27)(23,28) (24,29)(25,30)(26,31).
    __device__ static __forceinline__ void run(const uint32_t (&w)[kWords], __half s, int z, uint4 (&out)[4]) {
        const __half2 s2 = __half2half2(s);
        const uint32_t v0 = w[0] << 7;                        // stream offset -7
        const uint32_t v1 = w[0] >> 1;                        // 1
        const uint32_t v2 = __funnelshift_r(w[0], w[1], 11);  // 11
        const uint32_t v3 = w[1];                             // 32
        const uint32_t v4 = __funnelshift_r(w[1], w[2], 9);   // 41
        const uint32_t v5 = w[2] << 2;                        // 62
        const uint32_t v6 = w[2] >> 7;                        // 71
        out[0] = make_uint4(pair<7, 0>(v0, z, s2), pair<2, 4>(v1, z, s2), pair<5, 7>(v1, z, s2), pair<1, 0>(v2, z, s2));
        out[1] = make_uint4(pair<4, 3>(v2, z, s2), pair<7, 6>(v2, z, s2), pair<4, 3>(v3, z, s2), pair<7, 6>(v3, z, s2));
        out[2] = make_uint4(pair<1, 0>(v4, z, s2), pair<4, 3>(v4, z, s2), pair<7, 6>(v4, z, s2), pair<4, 3>(v5, z, s2));
        out[3] = make_uint4(pair<7, 6>(v5, z, s2), pair<1, 0>(v6, z, s2), pair<4, 3>(v6, z, s2), pair<7, 6>(v6, z, s2));
    }
};

// ---- x pre-pass: gather through x_perm and/or permute each 32-block into the 3-bit field order ----
__global__ void __launch_bounds__(256)
prep_x_kernel(const __half* __restrict__ x, const int32_t* __restrict__ x_perm, __half* __restrict__ xp, int M, int K,
              int permute3) {
    const size_t total = (size_t)M * K;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int m = (int)(i / K), k = (int)(i % K);
        int src = permute3 ? (k & ~31) + kOrder3[k & 31] : k;
        if (x_perm) src = __ldg(x_perm + src);
        xp[i] = x[(size_t)m * K + src];
    }
}

template <int BITS, int MT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
            const int32_t* __restrict__ qzeros, const __half* __restrict__ scales,
            const int32_t* __restrict__ g_idx, const __half* __restrict__ bias, __half* __restrict__ y, int M, int K,
            int N, int group_size, unsigned int* __restrict__ status) {
    using Cfg = GemmCfg<MT>;
    constexpr int S = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;            // operand tiles need 1024-byte alignment
    uint8_t* base_ptr = smem_raw + (base - raw);
    const uint32_t bar_base = base + S * Cfg::kStageBytes;   // tma_full[S], b_full[S], empty[S], accum
    __shared__ uint32_t tmem_base_holder;
    __shared__ volatile int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.y * BN, m0 = blockIdx.x * (BM * MT);
    const int KT = (K + BK - 1) / BK;

    auto tma_bar = [&](int s) { return bar_base + 8u * s; };          // x tiles + packed weights have landed
    auto full_bar = [&](int s) { return bar_base + 8u * (S + s); };    // the B operand has been written
    auto empty_bar = [&](int s) { return bar_base + 8u * (2 * S + s); };
    const uint32_t accum_bar = bar_base + 8u * (3 * S);
    auto a_tile = [&](int s, int mt) { return base + s * Cfg::kStageBytes + mt * kATileBytes; };
    auto b_tile = [&](int s) { return base + s * Cfg::kStageBytes + MT * kATileBytes; };
    auto p_tile = [&](int s) { return base + s * Cfg::kStageBytes + MT * kATileBytes + kBTileBytes; };
    constexpr int kWordRowsPerTile = 2 * Dequant<BITS>::kWords;     // word-rows of qweight per 64 rows of K
    constexpr uint32_t kPackedBytes = kWordRowsPerTile * BN * 4;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < S; ++s) {
            mbar_init(tma_bar(s), 1);    // the TMA producer's expect_tx arrive
            mbar_init(full_bar(s), 4);   // one arrive per weight warp
            mbar_init(empty_bar(s), 1);  // tcgen05.commit
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_holder)), "r"((uint32_t)Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_holder;

    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            for (int kt = 0; kt < KT; ++kt) {
                const int s = kt % S, round = kt / S;
                if (round > 0 && !mbar_wait(empty_bar(s), (round - 1) & 1, &abort_flag)) break;
                mbar_arrive_expect_tx(tma_bar(s), MT * kATileBytes + kPackedBytes);
                tma_load_2d(p_tile(s), &tmap_w, n0, kt * kWordRowsPerTile, tma_bar(s));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
                    tma_load_2d(a_tile(s, mt), &tmap_x, kt * BK, m0 + mt * BM, tma_bar(s));
            }
        }
    } else if (warp == 5) {
        // ===== MMA issuer =====
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true;
            for (int kt = 0; kt < KT && ok; ++kt) {
                const int s = kt % S, round = kt / S;
                ok = mbar_wait(tma_bar(s), round & 1, &abort_flag) && mbar_wait(full_bar(s), round & 1, &abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t bdesc = make_smem_desc(b_tile(s));
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint64_t adesc = make_smem_desc(a_tile(s, mt));
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16)
                        umma_f16(tmem_base + mt * BN, adesc + 2u * k16, bdesc + 2u * k16, idesc,
                                 (kt > 0 || k16 > 0) ? 1u : 0u);
                }
                umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
            }
            if (ok) umma_commit(accum_bar);
        }
    } else {
        // ===== weight producers (128 threads, one column each), then epilogue =====
        const int t = threadIdx.x - 32;     // 0..127
        const int n = n0 + t;
        const bool col_ok = n < N;
        const int wt = t >> 5;              // weight warp 0..3
        constexpr int W = Dequant<BITS>::kWords;
        const int zwords = N / 32 * BITS;
        const int RB = K / 32;
        const uint32_t row_off = (uint32_t)(t >> 3) * 1024u + (uint32_t)(t & 7) * 128u;
        int g_cur = -1;
        __half s_cur = __float2half(0.f);
        int z_cur = 0;

        bool ok = true;
        for (int kt = 0; kt < KT; ++kt) {
            const int s = kt % S, round = kt / S;
            // the stage is free (its previous MMAs retired) before the TMA refilled it, so waiting for
            // the refill also orders this thread's B writes after those MMAs
            ok = mbar_wait(tma_bar(s), round & 1, &abort_flag);
            if (!ok) break;
            const uint32_t* pw = reinterpret_cast<const uint32_t*>(base_ptr + (p_tile(s) - base)) + t;
            uint32_t cur[2][W];
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int r = 0; r < W; ++r) cur[h][r] = pw[(h * W + r) * BN];
            uint8_t* brow = base_ptr + (b_tile(s) - base) + row_off;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int rb = 2 * kt + h;
                uint4 out[4];
                if (col_ok && rb < RB) {
                    const int g = g_idx ? __ldg(g_idx + 32 * rb) : (32 * rb) / group_size;
                    if (g != g_cur) {
                        g_cur = g;
                        s_cur = scales[(size_t)g * N + n];
                        z_cur = zero_point<BITS>(qzeros + (size_t)g * zwords, n);
                    }
                    Dequant<BITS>::run(cur[h], s_cur, z_cur, out);
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) out[c] = make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int chunk = 4 * h + c;
                    *reinterpret_cast<uint4*>(brow + (((uint32_t)chunk ^ (uint32_t)(t & 7)) << 4)) = out[c];
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> tensor core reads
            __syncwarp();
            if (lane == 0) mbar_arrive(full_bar(s));
        }

        // ----- epilogue: TMEM -> registers -> fp16 -> global -----
        if (ok) ok = mbar_wait(accum_bar, 0, &abort_flag);
        ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below are warp-collective
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int quarter = warp & 3;  // the TMEM lane quarter this warp may read
#pragma unroll 1
            for (int mt = 0; mt < MT; ++mt) {
                const int m = m0 + mt * BM + quarter * 32 + lane;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(mt * BN + c * 32), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int nc = n0 + c * 32;
                    if (m < M && nc < N) {
                        __half* dst = y + (size_t)m * N + nc;
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t o[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                float f0 = __uint_as_float(r[8 * q + 2 * e]), f1 = __uint_as_float(r[8 * q + 2 * e + 1]);
                                if (bias) {
                                    f0 += __half2float(bias[nc + 8 * q + 2 * e]);
                                    f1 += __half2float(bias[nc + 8 * q + 2 * e + 1]);
                                }
                                o[e] = h2_as_u32(__floats2half2_rn(f0, f1));
                            }
                            *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(o[0], o[1], o[2], o[3]);
                        }
                    }
                }
            }
        }
        (void)wt;
    }

    // ----- teardown: every role arrives here, also after a timed-out wait -----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag) atomicExch(status + kStatusWord, 1u);
    if (warp == 5) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)Cfg::kTmemCols) : "memory");
    }
}

// ---- host side ----------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

template <int BITS, int MT>
int launch_gemm(const __half* x_for_tma, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                const int32_t* g_idx, const __half* bias, __half* y, int M, int K, int N, int group_size,
                unsigned int* status, cudaStream_t stream) {
    using Cfg = GemmCfg<MT>;
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) { set_last_cuda_error((int)cudaErrorNotSupported); return B200GPTQ_ERR_CUDA; }
    CUtensorMap tmap;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(__half)};
    const cuuint32_t box[2] = {BK, BM};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x_for_tma), dims, strides,
                              box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_last_cuda_error((int)cudaErrorInvalidValue); return B200GPTQ_ERR_CUDA; }
    // packed weights: int32 [K/32*bits, N], a box of (word-rows of one k-tile) x 128 columns, no swizzle
    CUtensorMap tmap_w;
    const cuuint64_t wdims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 32 * BITS)};
    const cuuint64_t wstrides[1] = {(cuuint64_t)N * sizeof(int32_t)};
    const cuuint32_t wbox[2] = {BN, 2 * Dequant<BITS>::kWords};
    const CUresult rw = encode(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t*>(qweight), wdims, wstrides,
                               wbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rw != CUDA_SUCCESS) { set_last_cuda_error((int)cudaErrorInvalidValue); return B200GPTQ_ERR_CUDA; }

    static bool attr_set[64][2][2] = {};
    int dev = 0;
    B200GPTQ_CUDA_TRY(cudaGetDevice(&dev));
    auto kernel = gemm_kernel<BITS, MT>;
    if (dev >= 0 && dev < 64 && !attr_set[dev][BITS == 4][MT - 1]) {
        B200GPTQ_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes));
        attr_set[dev][BITS == 4][MT - 1] = true;
    }
    dim3 grid((M + BM * MT - 1) / (BM * MT), (N + BN - 1) / BN);
    kernel<<<grid, kGemmThreads, Cfg::kSmemBytes, stream>>>(tmap, tmap_w, qzeros, scales, g_idx, bias, y, M, K, N,
                                                           group_size, status);
    B200GPTQ_CUDA_TRY(cudaGetLastError());
    return B200GPTQ_OK;
}

}  // namespace

// Scratch: the counter region (its last word is the sticky status word) and, when x has to be
// gathered or permuted, a copy of x.
size_t gemm_workspace_bytes(int M, int K, int N, int bits) {
    (void)N; (void)bits;
    return kCounterBytes + (size_t)M * K * sizeof(__half);
}

int gemm_dispatch(const __half* x, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                  const int32_t* g_idx, const int32_t* x_perm, const __half* bias, __half* y, int M, int K, int N,
                  int bits, int group_size, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    (void)workspace_bytes;
    unsigned int* status = reinterpret_cast<unsigned int*>(workspace);
    const __half* xt = x;
    if (bits == 3 || x_perm) {
        __half* xp = reinterpret_cast<__half*>(reinterpret_cast<char*>(workspace) + kCounterBytes);
        const size_t total = (size_t)M * K;
        int blocks = (int)((total + 256 * 8 - 1) / (256 * 8));
        if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
        if (blocks < 1) blocks = 1;
        prep_x_kernel<<<blocks, 256, 0, stream>>>(x, x_perm, xp, M, K, bits == 3 ? 1 : 0);
        B200GPTQ_CUDA_TRY(cudaGetLastError());
        xt = xp;
    }
    const bool two = M > BM;
    if (bits == 4)
        return two ? launch_gemm<4, 2>(xt, qweight, qzeros, scales, g_idx, bias, y, M, K, N, group_size, status, stream)
                   : launch_gemm<4, 1>(xt, qweight, qzeros, scales, g_idx, bias, y, M, K, N, group_size, status, stream);
    if (bits == 3)
        return two ? launch_gemm<3, 2>(xt, qweight, qzeros, scales, g_idx, bias, y, M, K, N, group_size, status, stream)
                   : launch_gemm<3, 1>(xt, qweight, qzeros, scales, g_idx, bias, y, M, K, N, group_size, status, stream);
    return B200GPTQ_ERR_BITS;
}

}  // namespace b200gptq
