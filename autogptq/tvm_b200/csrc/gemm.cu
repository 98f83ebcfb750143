// Prefill dequant-GEMM on the 5th-generation tensor cores (tcgen05 + tensor memory), sm_100a.
//
//   y[M, N] = x[M, K] @ W[K, N] (+ bias),   W[k, n] = scales[g, n] * (q[k, n] - zero[g, n])
//
// The product is computed transposed, y^T = W^T x^T, so that the dequantised weights are the
// A operand of tcgen05.mma and can live in TENSOR MEMORY: they never touch shared memory, which
// on this part is the resource a mixed-input GEMM runs out of first (an MMA whose operands both
// come from shared memory already consumes its whole read bandwidth at 128 x 128 tiles).
// One CTA computes 128 output columns for a tile of TN <= 256 rows of x:
//   warp 0      TMA producer: per k-tile (64 rows of K) an x tile (TN rows x 64 k, 128-byte
//               swizzle) and the packed weight rows of the CTA's 128 columns, into a stage ring
//   warps 1..16 weight producers in two groups that take k-tiles in turn: each thread owns one of the 128 columns and one 32-row block of
//               the k-tile; it reads its packed words from the stage, dequantises them to the
//               exact fp16 value of the reference (auto_gptq/nn_modules/qlinear.py:242: one
//               rounding) and stores 16 registers into the A buffer of that stage in tensor memory
//               (tcgen05.st); afterwards the same warps run the epilogue (tcgen05.ld -> fp16 -> y)
//   warp 17     allocates tensor memory and issues tcgen05.mma (M = 128 columns, N = TN rows of x,
//               K = 16, f16 x f16 -> f32 accumulators in tensor memory columns 0..TN-1)
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

#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace b200gptq {

namespace {

constexpr int BN = 128;                 // output columns per CTA = rows of the MMA's A operand
constexpr int BK = 64;                  // rows of K per stage
constexpr int kMaxTN = 256;             // rows of x per CTA = N of the MMA
constexpr int kWeightWarps = 8;         // warps that build one k-tile's A operand
// Groups of weight warps, taking k-tiles in turn.
__host__ __device__ constexpr int mma_warp(int groups) { return 1 + kWeightWarps * groups; }
__host__ __device__ constexpr int gemm_threads(int groups) { return 32 * (2 + kWeightWarps * groups); }  // TMA warp, weight warps, MMA warp
constexpr int kPackedTileBytes = 4096;  // up to 8 word-rows x 128 columns of packed weights per k-tile
constexpr int kMaxStages = 16;
constexpr int kTmemCols = 512;          // accumulators in columns [0, TN), A buffers behind them (as many stages as fit)
constexpr int kTmemAColsPerStage = 32;  // 64 k x fp16 = 32 columns of 32 bits
constexpr int kSmemBudget = 222 * 1024;  // ring bytes; the opt-in maximum per CTA is 227 KB
constexpr int kStatusWord = kMaxCounters - 1;  // sticky error word inside the counter region
constexpr int kMaxSplits = 4;            // CTAs that share the k-tiles of one output tile (split K)
constexpr int kGroups = 3;               // weight groups of the launched kernel (one CTA per SM)
// two CTAs on an SM share what bounds a k-tile (its k-tiles count 19/10): the second CTA pays only where it
// fills a half-empty wave or halves the k-tiles of a CTA
constexpr int kTwoPerSmPenaltyNum = 19, kTwoPerSmPenaltyDen = 10;

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
// The same test, but the thread may stay suspended for up to `ns` nanoseconds (it is woken when the phase completes):
// a waiting warp then issues a handful of instructions per microsecond instead of spinning, and the issue slots go to
// the warps that share its scheduler and have work (measured before the change: 60 % of all issued warp
// instructions of this kernel were barrier polls).
__device__ __forceinline__ bool mbar_try_wait_for(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~2e9 clocks or as soon as another role has raised `abort_flag`.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (true) {
        for (int i = 0; i < 8; ++i)
            if (mbar_try_wait_for(bar, parity, 4000u)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > 2000000000LL) { *abort_flag = 1; return false; }
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint4 (&v)[4]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(v[0].x), "r"(v[0].y), "r"(v[0].z), "r"(v[0].w), "r"(v[1].x), "r"(v[1].y), "r"(v[1].z),
          "r"(v[1].w), "r"(v[2].x), "r"(v[2].y), "r"(v[2].z), "r"(v[2].w), "r"(v[3].x), "r"(v[3].y), "r"(v[3].z),
          "r"(v[3].w) : "memory");
}
// A operand in tensor memory, B operand described in shared memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
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

template <int BITS, int kWeightGroups>
__global__ void __launch_bounds__(gemm_threads(kWeightGroups), kWeightGroups == 1 ? 2 : 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
            const int32_t* __restrict__ qzeros, const __half* __restrict__ scales,
            const int32_t* __restrict__ g_idx, const __half* __restrict__ bias, __half* __restrict__ y, int M, int K,
            int N, int group_size, int TN, int S, int tab_groups, int a_off, unsigned int* __restrict__ status,
            int splits, int tmem_cols, float* __restrict__ partial) {
    // splits > 1 (few rows of x, fewer column tiles than SMs): blockIdx.z takes a contiguous run of the k-tiles, two
    // such CTAs fit on an SM (half of the shared and tensor memory each), every CTA leaves its fp32 sums in
    // `partial[z][row][column]`, and the last one of a tile to arrive adds them up in the order of z.
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;            // swizzled tiles need 1024-byte alignment
    uint8_t* base_ptr = smem_raw + (base - raw);
    __shared__ __align__(8) uint64_t bars[3 * kMaxStages + 1];  // tma[S], a_full[S], empty[S], accum
    __shared__ uint32_t tmem_base_holder;
    __shared__ volatile int abort_flag;
    __shared__ volatile int epi_bad;      // split K: an epilogue warp's wait ran out
    __shared__ unsigned int arrived;     // split K: CTAs of this tile that had arrived before this one

    constexpr int kMmaWarp = mma_warp(kWeightGroups);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.y * BN, m0 = blockIdx.x * TN;
    const int KT_all = (K + BK - 1) / BK;
    const int kt_first = (int)(((long long)blockIdx.z * KT_all) / splits);
    const int KT = (int)(((long long)(blockIdx.z + 1) * KT_all) / splits) - kt_first;   // k-tiles of this CTA
    const uint32_t x_tile_bytes = (uint32_t)TN * BK * 2;
    const uint32_t stage_bytes = x_tile_bytes + kPackedTileBytes;

    const uint32_t bar_base = smem_u32(bars);
    auto tma_bar = [&](int s) { return bar_base + 8u * s; };                      // x tile + packed weights landed
    auto full_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };      // A operand stored in tensor memory
    auto empty_bar = [&](int s) { return bar_base + 8u * (2 * kMaxStages + s); }; // the stage's MMAs have retired
    const uint32_t accum_bar = bar_base + 8u * (3 * kMaxStages);
    auto x_tile = [&](int s) { return base + s * stage_bytes; };
    auto p_tile = [&](int s) { return base + s * stage_bytes + x_tile_bytes; };
    constexpr int kWordRowsPerTile = 2 * Dequant<BITS>::kWords;     // word-rows of qweight per 64 rows of K
    constexpr uint32_t kPackedBytes = kWordRowsPerTile * BN * 4;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        epi_bad = 0;
        for (int s = 0; s < S; ++s) {
            mbar_init(tma_bar(s), 1);               // the TMA producer's expect_tx arrive
            mbar_init(full_bar(s), kWeightWarps);   // one arrive per weight warp
            mbar_init(empty_bar(s), 1);             // tcgen05.commit
        }
        mbar_init(accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&tmem_base_holder)), "r"((uint32_t)tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_holder;

    if (warp == 0) {
        // ===== TMA producer =====
        if (lane == 0) {
            int s = 0, round = 0;
            for (int kt = 0; kt < KT; ++kt) {
                if (round > 0 && !mbar_wait(empty_bar(s), (round - 1) & 1, &abort_flag)) break;
                mbar_arrive_expect_tx(tma_bar(s), x_tile_bytes + kPackedBytes);
                tma_load_2d(p_tile(s), &tmap_w, n0, (kt_first + kt) * kWordRowsPerTile, tma_bar(s));
                tma_load_2d(x_tile(s), &tmap_x, (kt_first + kt) * BK, m0, tma_bar(s));
                if (++s == S) { s = 0; ++round; }
            }
        }
    } else if (warp == kMmaWarp) {
        // ===== MMA issuer =====
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(BN >> 4) << 24);
            bool ok = true;
            int s = 0, round = 0;
            for (int kt = 0; kt < KT; ++kt) {
                ok = mbar_wait(tma_bar(s), round & 1, &abort_flag) && mbar_wait(full_bar(s), round & 1, &abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t bdesc = make_smem_desc(x_tile(s));
                const uint32_t a_addr = tmem_base + (uint32_t)a_off + kTmemAColsPerStage * s;
#pragma unroll
                for (int k16 = 0; k16 < BK / 16; ++k16)
                    umma_f16_ts(tmem_base, a_addr + 8u * k16, bdesc + 2u * k16, idesc, (kt > 0 || k16 > 0) ? 1u : 0u);
                umma_commit(empty_bar(s));  // frees the stage once these MMAs have read it
                if (++s == S) { s = 0; ++round; }
            }
            if (ok) umma_commit(accum_bar);
        }
    } else {
        // ===== weight producers (256 threads: one column x one 32-row block each), then epilogue =====
        const int quarter = warp & 3;                 // tensor-memory lanes 32*quarter .. +31 belong to this warp
        const int wgroup = (warp - 1) / kWeightWarps; // this group takes k-tiles wgroup, wgroup + kWeightGroups, ...
        const int kh = ((warp - 1) % kWeightWarps) >> 2;  // which 32-row block of the 64-row k-tile
        const int col = 32 * quarter + lane;          // column inside the tile = tensor-memory lane
        const int n = n0 + col;
        const bool col_ok = n < N;
        constexpr int W = Dequant<BITS>::kWords;
        const int zwords = N / 32 * BITS;
        const int RB = K / 32;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(32 * quarter) << 16);

        // ---- scale / zero-point of (group, column) ----
        // When they fit, the CTA's 128 columns x all groups are staged once in shared memory, packed as
        // (fp16 scale | zero-point << 16), together with the group of every 32-row block; the producers
        // then never wait on global memory inside the k loop.  Larger layers read them from global
        // memory one k-tile ahead.
        uint32_t* tab = reinterpret_cast<uint32_t*>(base_ptr + (size_t)S * stage_bytes);
        uint16_t* gmap = reinterpret_cast<uint16_t*>(tab + (size_t)tab_groups * BN);
        auto group_of = [&](int rb) { return g_idx ? __ldg(g_idx + 32 * rb) : (32 * rb) / group_size; };
        // The table holds the groups this CTA's k-tiles can touch: with the trivial g_idx that is a contiguous run
        // (a split-K CTA needs a fraction of the layer's groups); a stored g_idx may name any group.
        const int rb_first = 2 * kt_first, rb_end = min(RB, 2 * (kt_first + KT));
        const int g_first = (tab_groups && !g_idx) ? (32 * rb_first) / group_size : 0;
        const int g_count = !tab_groups ? 0 : (g_idx ? tab_groups : (32 * rb_end - 1) / group_size - g_first + 1);
        if (tab_groups) {
            constexpr int kFillThreads = kWeightWarps * kWeightGroups * 32;
            const int pt = threadIdx.x - 32;   // 0 .. kFillThreads - 1
            const int total = g_count * BN;
            // four entries per thread and pass, their global loads issued together (one entry at a time the fill
            // was a chain of 16 memory round trips per thread, a third of a 16-row launch)
#pragma unroll 1
            for (int i0 = pt; i0 < total; i0 += 4 * kFillThreads) {
                uint32_t sc[4];
                int z[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + j * kFillThreads;
                    const int g = g_first + i / BN, c = i % BN;
                    sc[j] = 0u; z[j] = 0;
                    if (i < total && n0 + c < N) {
                        sc[j] = __half_as_ushort(__ldg(scales + (size_t)g * N + n0 + c));
                        z[j] = zero_point<BITS>(qzeros + (size_t)g * zwords, n0 + c);
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + j * kFillThreads;
                    if (i < total) tab[i] = sc[j] | ((uint32_t)z[j] << 16);
                }
            }
            for (int rb = rb_first + pt; rb < rb_end; rb += kFillThreads)
                gmap[rb - rb_first] = (uint16_t)(group_of(rb) - g_first);
            asm volatile("bar.sync 1, %0;" ::"n"(kFillThreads) : "memory");
        }
        auto load_group = [&](int rb, int& g, __half& sc, int& z) {
            if (col_ok && rb < rb_end) {
                if (tab_groups) {
                    g = gmap[rb - rb_first];
                    const uint32_t e = tab[g * BN + col];
                    sc = __ushort_as_half((unsigned short)(e & 0xffffu));
                    z = (int)(e >> 16);
                } else {
                    g = group_of(rb);
                    sc = scales[(size_t)g * N + n];
                    z = zero_point<BITS>(qzeros + (size_t)g * zwords, n);
                }
            }
        };
        int g_cur = -1, g_nxt = -1, z_cur = 0, z_nxt = 0;
        __half s_cur = __float2half(0.f), s_nxt = __float2half(0.f);
        load_group(2 * (kt_first + wgroup) + kh, g_cur, s_cur, z_cur);

        bool ok = true;
        int s = wgroup % S, round = wgroup / S;
        for (int kt = wgroup; kt < KT; kt += kWeightGroups) {
            const int rb = 2 * (kt_first + kt) + kh;
            // fetch the scale / zero-point of this thread's next k-tile now, a whole iteration ahead of their use
            const int rb_nxt = rb + 2 * kWeightGroups;
            if (rb_nxt < rb_end && col_ok) {
                if (tab_groups) {
                    load_group(rb_nxt, g_nxt, s_nxt, z_nxt);
                } else {
                    const int gn = group_of(rb_nxt);
                    if (gn != g_cur) load_group(rb_nxt, g_nxt, s_nxt, z_nxt);
                    else { g_nxt = g_cur; s_nxt = s_cur; z_nxt = z_cur; }
                }
            }
            // The TMA refilled this stage only after its previous MMAs retired (empty barrier), so the
            // A buffer of the stage in tensor memory is free as well.
            ok = mbar_wait(tma_bar(s), round & 1, &abort_flag);
            ok = __all_sync(0xffffffffu, ok);   // the tensor-memory store below is warp-collective
            if (!ok) break;
            const uint32_t* pw = reinterpret_cast<const uint32_t*>(base_ptr + (p_tile(s) - base)) + col;
            uint32_t cur[W];
#pragma unroll
            for (int r = 0; r < W; ++r) cur[r] = pw[(kh * W + r) * BN];
            uint4 out[4];
            if (col_ok && rb < RB) {
                Dequant<BITS>::run(cur, s_cur, z_cur, out);
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) out[c] = make_uint4(0, 0, 0, 0);
            }
            tmem_st16(lane_addr + (uint32_t)a_off + kTmemAColsPerStage * s + 16 * kh, out);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(full_bar(s));
            g_cur = g_nxt; s_cur = s_nxt; z_cur = z_nxt;
            s += kWeightGroups;
            while (s >= S) { s -= S; ++round; }
        }

        // ----- epilogue: accumulators (lane = output column, column = row of x) -> fp16 -> y -----
        if (ok) ok = mbar_wait(accum_bar, 0, &abort_flag);
        ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below are warp-collective
        const float b = (bias && col_ok) ? __half2float(bias[n]) : 0.f;
        constexpr int kEpiWarps = kWeightWarps * kWeightGroups;
        if (splits == 1) {
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                // the warps that share a lane quarter take the 16-row chunks in turn
                for (int c = (warp - 1) >> 2; c < TN / 16; c += kEpiWarps / 4) {
                    uint32_t r[16];
                    tmem_ld16(lane_addr + 16u * c, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int m = m0 + 16 * c;
                    if (col_ok) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (m + i < M) y[(size_t)(m + i) * N + n] = __float2half_rn(__uint_as_float(r[i]) + b);
                    }
                }
            }
        } else {
            // ---- split K: fp32 sums of this CTA's k-tiles to the scratch, then the last CTA of the tile adds them.
            //      The hardware barriers below are reached by all epilogue warps whatever happened before: a CTA whose
            //      wait ran out still counts itself in, so that the tile's counter returns to zero (the results are then
            //      undefined and the status word says so). ----
            if (!ok && lane == 0) epi_bad = 1;
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
            const int rows_pad = gridDim.x * TN;
            if (epi_bad == 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float* mine = partial + (size_t)blockIdx.z * rows_pad * N;
#pragma unroll 1
                for (int c = (warp - 1) >> 2; c < TN / 16; c += kEpiWarps / 4) {
                    uint32_t r[16];
                    tmem_ld16(lane_addr + 16u * c, r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    const int m = m0 + 16 * c;
                    if (col_ok) {
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (m + i < M) mine[(size_t)(m + i) * N + n] = __uint_as_float(r[i]);
                    }
                }
            }
            __threadfence();   // this thread's sums are visible before the tile's arrival is counted
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
            unsigned int* counter = status + (blockIdx.y * gridDim.x + blockIdx.x);
            if (threadIdx.x == 32) arrived = atomicAdd(counter, 1u);
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
            if (arrived == (unsigned int)splits - 1u) {
                __threadfence();   // the other CTAs' sums, published before their arrivals
#pragma unroll 1
                for (int c = (warp - 1) >> 2; c < TN / 16; c += kEpiWarps / 4) {
                    const int m = m0 + 16 * c;
                    if (col_ok) {
                        // all loads of the chunk are issued before the first is used: one round trip to L2, not 64
                        float v[kMaxSplits][16];
#pragma unroll
                        for (int z = 0; z < kMaxSplits; ++z)
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                v[z][i] = (z < splits && m + i < M)
                                              ? __ldcg(partial + ((size_t)z * rows_pad + m + i) * N + n) : 0.f;
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            if (m + i < M) {
                                float sum = v[0][i];
#pragma unroll
                                for (int z = 1; z < kMaxSplits; ++z) sum += v[z][i];   // in the order of z
                                y[(size_t)(m + i) * N + n] = __float2half_rn(sum + b);
                            }
                    }
                }
                if (threadIdx.x == 32) *counter = 0u;   // the counter region is left as it was found
            }
        }
    }

    // ----- teardown: every role arrives here, also after a timed-out wait -----
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag) atomicExch(status + kStatusWord, 1u);
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)tmem_cols) : "memory");
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

// Work split of a launch.  With few rows of x a tile's time is the chain of hand-overs per k-tile, not its arithmetic:
// the time of a launch is (waves of CTAs) x (k-tiles per CTA).  Two things shorten it.  Split K: the k-tiles of a
// column tile are spread over up to kMaxSplits CTAs (blockIdx.z), only for one row tile (M <= 128) and when every
// run keeps at least 16 k-tiles (40 above 64 rows: taller partial sums).  Two CTAs per SM (M <= 64): one group of
// weight warps instead of three (320 threads, so that two CTAs fit the register file) and half of the shared and
// tensor memory each.  An SM works through k-tiles at about the same rate either way (0.4-0.5 us per k-tile), so the
// second CTA is taken only where it fills a half-empty second wave or halves the k-tiles of a CTA: 16 rows,
// 4096 x 12288 33.1 -> 29.5 us, 4096 x 22016 64.5 -> 48.5 us, 9216 x 27648 (3-bit) 141 -> 114 us.
struct GemmSplit { int splits, per_sm; };
int splits_for(int M, int tiles, int KT, int slots) {
    if (M > 128 || tiles >= kMaxCounters - 1) return 1;
    int sp = slots / tiles;
    if (sp > kMaxSplits) sp = kMaxSplits;
    // every run keeps enough k-tiles to pay for its own start-up and for the final sum: measured on 4096 x 4096,
    // 16 rows 33.5 -> 21 us with four runs, 128 rows 34.6 -> 37.4 us with two
    const int min_tiles = M <= 64 ? 16 : 40;
    while (sp > 1 && KT / sp < min_tiles) --sp;
    return sp < 1 ? 1 : sp;
}
GemmSplit pick_split(int M, int N, int K) {
    const int tiles = (N + BN - 1) / BN, KT = (K + BK - 1) / BK, sms = sm_count();
    GemmSplit one = {splits_for(M, tiles, KT, sms), 1};
    if (M > 64) return one;
    GemmSplit two = {splits_for(M, tiles, KT, 2 * sms), 2};
    auto cost = [&](const GemmSplit& g) {
        const long long ctas = (long long)tiles * g.splits, slots = (long long)sms * g.per_sm;
        return ((ctas + slots - 1) / slots) * ((KT + g.splits - 1) / g.splits);
    };
    return cost(two) * kTwoPerSmPenaltyNum < cost(one) * kTwoPerSmPenaltyDen ? two : one;
}
int pick_splits(int M, int N, int K) { return pick_split(M, N, K).splits; }
size_t split_partial_bytes(int M, int N, int K) {
    const int sp = pick_splits(M, N, K);
    if (sp == 1) return 0;
    const int TN = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    return (size_t)sp * TN * N * sizeof(float);
}

int pick_tn(int M) {
    if (M <= 16) return 16;
    if (M <= 32) return 32;
    if (M <= 64) return 64;
    if (M <= 128) return 128;
    return kMaxTN;
}

template <int BITS>
int launch_gemm(const __half* x_for_tma, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                const int32_t* g_idx, const __half* bias, __half* y, int M, int K, int N, int group_size,
                unsigned int* status, float* partial, cudaStream_t stream) {
    EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) { set_last_cuda_error((int)cudaErrorNotSupported); return B200GPTQ_ERR_CUDA; }
    const int TN = pick_tn(M);
    const int stage_bytes = TN * BK * 2 + kPackedTileBytes;
    // scale / zero-point table of the CTA's columns for every group, if it leaves room for >= 4 stages
    const int gs_eff = group_size;
    const int G = (K + gs_eff - 1) / gs_eff;
    const GemmSplit split = pick_split(M, N, K);
    const int splits = split.splits;
    const int smem_budget = split.per_sm == 2 ? kSmemBudget / 2 - 2048 : kSmemBudget;
    const int tmem_cols = kTmemCols / split.per_sm;
    int tab_bytes = G * BN * 4 + ((K / 32 * 2 + 15) / 16) * 16;
    int tab_groups = G;
    if (G > 65535 || smem_budget - tab_bytes < 4 * stage_bytes) { tab_bytes = 0; tab_groups = 0; }
    // Stages: a small-M tile moves 4..6 KB per k-tile and its round trip (TMA, dequantisation, MMA, commit) lasts
    // microseconds, so throughput is the number of k-tiles in flight: as many as shared memory and the tensor-memory
    // columns behind the accumulators hold.
    const int a_off = TN < 32 ? 32 : TN;
    int S = (smem_budget - tab_bytes) / stage_bytes;
    if (S > kMaxStages) S = kMaxStages;
    if (S > (tmem_cols - a_off) / kTmemAColsPerStage) S = (tmem_cols - a_off) / kTmemAColsPerStage;
    if (S < 2) return B200GPTQ_ERR_TOO_LARGE;
    const int smem_bytes = S * stage_bytes + tab_bytes + 1024;  // + slack to align the ring to 1024 bytes

    CUtensorMap tmap_x, tmap_w;
    const cuuint32_t estr[2] = {1, 1};
    {   // x: fp16 [M, K]; a box is 64 k x TN rows, 128-byte swizzle, rows beyond M read as zero
        const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
        const cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(__half)};
        const cuuint32_t box[2] = {BK, (cuuint32_t)TN};
        const CUresult r = encode(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(x_for_tma), dims,
                                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)cudaErrorInvalidValue); return B200GPTQ_ERR_CUDA; }
    }
    {   // packed weights: int32 [K/32*bits, N]; a box is the word-rows of one k-tile x 128 columns
        const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 32 * BITS)};
        const cuuint64_t strides[1] = {(cuuint64_t)N * sizeof(int32_t)};
        const cuuint32_t box[2] = {BN, 2 * Dequant<BITS>::kWords};
        const CUresult r = encode(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t*>(qweight), dims,
                                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)cudaErrorInvalidValue); return B200GPTQ_ERR_CUDA; }
    }

    dim3 grid((M + TN - 1) / TN, (N + BN - 1) / BN, splits);
    auto launch = [&](auto groups) -> int {
        constexpr int kG = decltype(groups)::value;
        // the shared-memory opt-in is set once per device and instantiation; afterwards the launch path only reads
        static std::once_flag attr_once[64];
        static int attr_result[64];
        int dev = 0;
        B200GPTQ_CUDA_TRY(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64) return B200GPTQ_ERR_TOO_LARGE;
        std::call_once(attr_once[dev], [dev] {
            attr_result[dev] = (int)cudaFuncSetAttribute(gemm_kernel<BITS, kG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                         226 * 1024);
        });
        if (attr_result[dev] != 0) { set_last_cuda_error(attr_result[dev]); return B200GPTQ_ERR_CUDA; }
        gemm_kernel<BITS, kG><<<grid, gemm_threads(kG), smem_bytes, stream>>>(
            tmap_x, tmap_w, qzeros, scales, g_idx, bias, y, M, K, N, group_size, TN, S, tab_groups, a_off, status, splits,
            tmem_cols, partial);
        return B200GPTQ_OK;
    };
    const int st = split.per_sm == 2 ? launch(std::integral_constant<int, 1>{}) : launch(std::integral_constant<int, kGroups>{});
    if (st != B200GPTQ_OK) return st;
    B200GPTQ_CUDA_TRY(cudaGetLastError());
    return B200GPTQ_OK;
}

}  // namespace

// Scratch: the counter region (its last word is the sticky status word) and, when x has to be
// gathered or permuted, a copy of x.
size_t gemm_workspace_bytes(int M, int K, int N, int bits) {
    (void)bits;
    // counters | copy of x (gathered / permuted) | fp32 partial sums of a split-K launch
    return kCounterBytes + (((size_t)M * K * sizeof(__half) + 255) & ~(size_t)255) + split_partial_bytes(M, N, K);
}

void gemm_split_query(int M, int K, int N, int* splits, int* ctas_per_sm) {
    const GemmSplit g = pick_split(M, N, K);
    *splits = g.splits;
    *ctas_per_sm = g.per_sm;
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
    float* partial = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kCounterBytes +
                                              (((size_t)M * K * sizeof(__half) + 255) & ~(size_t)255));
    if (bits == 4) return launch_gemm<4>(xt, qweight, qzeros, scales, g_idx, bias, y, M, K, N, group_size, status, partial, stream);
    if (bits == 3) return launch_gemm<3>(xt, qweight, qzeros, scales, g_idx, bias, y, M, K, N, group_size, status, partial, stream);
    return B200GPTQ_ERR_BITS;
}

}  // namespace b200gptq
