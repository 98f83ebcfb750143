// Decode GEMV, streaming form (M <= 8, bits in {3,4}, groups = k / group_size).
//
//   y[m, n] = sum_k x[m, xk(k)] * scales[g, n] * (q[k, n] - zero[g, n]),   g = k / group_size
//
// The kernel is bound by HBM bandwidth and, on B200, almost by instruction issue as well
// (about two instructions per weight are available at full bandwidth), and a single layer lasts
// only a few microseconds, so three things shape it:
//
//  * Weight stream: qweight reaches shared memory through a ring of "units" filled by TMA, one
//    cp.async.bulk.tensor box per unit (12 or 16 KB, completion counted on an mbarrier).  Measured on
//    B200: 1 KB bulk copies cap a CTA's stream at ~25 GB/s however many are in flight, one box per unit
//    streams at the full 5.6 TB/s from 148 CTAs.  The box is laid out with the 128-byte swizzle so the
//    quad lanes' 128-bit reads of different word-rows fall into different banks.  The ring is filled at
//    the start of the kernel, before the dependency on the previous kernel is awaited (weights are
//    constants), and every warp counts itself in when it has read a unit: the last one refills the slot.
//  * Unpack without shifts into place or integer->float conversion: a LOP3 masks two fields of a
//    word and ORs in an fp16 exponent, which yields the half2 (c_lo + q_lo, c_hi + q_hi) with known
//    offsets c = 2^(10-p) for a field at bit p of its half.  Integer instructions are the scarce
//    resource (the INT pipe issues at half the FP32 rate), so the count per weight is what is
//    minimised: 5 per 8 weights (4-bit), 23 per 32 weights (3-bit).
//  * The products are done by mma.sync m16n8k16 (f16 x f16 -> f32): the 16 rows of the A tile
//    are 16 output columns, the 8 columns of B are the (up to 8) rows of x, so one instruction
//    retires 256 weights of a warp for every M <= 8.  Offsets and zero-points are removed
//    afterwards: per group, sum_k (c_k + q_k) x_k is scaled by s, and
//    sum_g s * (sum_k c_k x_k + zero * sum_k x_k) -- which needs only x, scales and qzeros -- is
//    computed once per column while the weights are in flight.
//
// Work split: a "unit" is 256 columns x 128 rows of K.  A CTA is 8 warps (128 registers per thread, two
// CTAs per SM).  A thread-block cluster of up to 8 CTAs owns one 256-column group and splits its K range
// evenly; the CTAs' partial sums are combined in the cluster's first CTA in rank order, either pushed
// there with asynchronous shared-memory stores (small M) or read from it through distributed shared memory
// (results do not depend on scheduling; no global scratch, atomics or fences are involved).
// The cluster size is the largest that still lets every CTA of the grid be resident at once.
// Every mbarrier wait is bounded; if one expires the kernel raises a sticky status word and runs
// on without waiting.
//
// Reference semantics: auto_gptq/nn_modules/qlinear.py:197-243; the kernel this replaces is
// the TVM-generated SIMT GEMV src/kernels/gemv_kernel.cu:25-55.
#include <cuda.h>

#include <cstdlib>

#include "common.cuh"

namespace b200gptq {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = 32 * kConsumerWarps;   // 256
constexpr int kThreads = kConsumerThreads;               // warp 0 also issues the weight copies
constexpr int kCgCols = 32 * kConsumerWarps;             // 256 columns per column group
constexpr int kMaxM = 8;
constexpr int kMaxStageRows = 2048;         // rows of x staged in shared memory at a time (fewer when M is large)
constexpr int kStageGroups = 16;            // and at most this many groups
constexpr int kSmemBudget = 107 * 1024;     // dynamic shared memory of a CTA: just under half an SM, so that two CTAs
                                            // are resident on an SM at the same time
constexpr int kRowPitch = kCgCols * 4;      // bytes of one word-row of a unit
constexpr int kMaxRing = 32;
constexpr int kStatusWord = kMaxCounters - 1;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t magic) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(magic));  // (a & mask) | magic
    return r;
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
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
// Bounded wait.  After ~1e9 clocks, or once any thread of the CTA has given up, waiting stops for
// good: the kernel then finishes with undefined results and a raised status word instead of hanging.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* gave_up) {
    if (mbar_try_wait(bar, parity)) return;
    const long long t0 = clock64();
    while (!*gave_up) {
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return;
        if (clock64() - t0 > 1000000000LL) *gave_up = 1;
    }
}
// One TMA copy of a 3-D box into shared memory of this CTA.  qweight is described to the TMA unit as
// [N/32 column chunks][word-rows][32 columns]; a box is 8 chunks x the unit's word-rows x 32 columns and lands as
// [chunk][word-row][128 bytes] with the 128-byte swizzle (16-byte piece p of line L sits at piece p ^ (L & 7)),
// which is what lets the four lanes of a quad read different word-rows of the same columns without bank conflicts.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory"); }

// 3-bit: the 32 fields of a row block leave the seven-window unpack as the 16 pairs (0,3) (1,7) (2,8)
// (4,9) (5,10) (6,11) (12,17) (13,18) (14,19) (15,20) (16,21) (22,27) (23,28) (24,29) (25,30) (26,31);
// the x values are staged in the same order.  kSlot3[f] = half index of field f inside a fragment entry.
__constant__ unsigned char kSlot3[32] = {0, 2, 4, 1, 6, 8, 10, 3, 5, 7, 9, 11, 12, 14, 16, 18,
                                         20, 13, 15, 17, 19, 21, 22, 24, 26, 28, 30, 23, 25, 27, 29, 31};
// bit position (inside its 16-bit half) at which the field of each slot is masked: offset = 2^(10 - p)
__constant__ unsigned char kPos3[32] = {7, 0, 2, 4, 5, 7, 1, 0, 4, 3, 7, 6, 4, 3, 7, 6,
                                        1, 0, 4, 3, 7, 6, 4, 3, 7, 6, 1, 0, 4, 3, 7, 6};

// fp16 exponent pattern that turns a field at bit p of a 16-bit half into 2^(10-p) + field.
__host__ __device__ constexpr uint32_t magic_at(int p) { return (uint32_t)(25 - p) << 10; }

// ---------------------------------------------------------------------------------------
// Per-bit-width traits.  A unit is 256 columns x 128 rows of K for both widths.
//   kWordRows     word-rows of qweight per unit (= rows of the unit's ring buffer)
//   kVecs         128-bit reads per thread per unit
//   kBRegs        32-bit registers of B fragments per (unit, x row, quad lane)
// Lane (g = lane/4, j = lane%4) of warp w holds columns 32w + 4g .. +3 of the column group.
// ---------------------------------------------------------------------------------------
template <int BITS> struct Traits;

// 4-bit: the quad's lane j owns word-rows 2j, 2j+1, 8+2j, 9+2j of the unit's 16 (8 rows of K each): with the
// swizzled ring layout the four lanes of a quad then read from different banks.  Pair i of a word is
// (nibble i, nibble i + 4); even pairs are masked in place (offset 1024), odd pairs sit at bit 4 (offset 64);
// pairs 2, 3 come from the word shifted right by 8.
template <> struct Traits<4> {
    static constexpr int kUnitRows = 128;
    static constexpr int kVecs = 4;
    static constexpr int kBRegs = 16;
    static constexpr int kWordRows = 16;
    // word-row of the unit that holds vec r of quad lane j
    __device__ static __forceinline__ int vec_row(int j, int r) { return 2 * j + (r & 1) + 8 * (r >> 1); }

    // d[cp] + d[2 + cp] accumulate column pair cp (columns 2cp, 2cp+1 of the lane's 4) over this unit;
    // two accumulator sets halve the length of the dependent mma chains.
    __device__ static __forceinline__ void compute(const uint4 (&buf)[kVecs], const uint32_t* __restrict__ bsm,
                                                   bool has_x, float (&d)[4][4]) {
        constexpr uint32_t MASK_E = 0x000f000fu, MAGIC_E = 0x64006400u;   // 1024 + q
        constexpr uint32_t MASK_O = 0x00f000f0u, MAGIC_O = 0x54005400u;   //   64 + q
#pragma unroll
        for (int rb = 0; rb < 4; ++rb) {
            uint4 bf = make_uint4(0, 0, 0, 0);
            if (has_x) bf = *reinterpret_cast<const uint4*>(bsm + 4 * rb);
            const uint32_t wcol[4] = {buf[rb].x, buf[rb].y, buf[rb].z, buf[rb].w};
#pragma unroll
            for (int cp = 0; cp < 2; ++cp) {
                const uint32_t wa = wcol[2 * cp], wb = wcol[2 * cp + 1];
                const uint32_t wa8 = wa >> 8, wb8 = wb >> 8;
                mma16816(d[cp], lop3_and_or(wa, MASK_E, MAGIC_E), lop3_and_or(wb, MASK_E, MAGIC_E),
                         lop3_and_or(wa, MASK_O, MAGIC_O), lop3_and_or(wb, MASK_O, MAGIC_O), bf.x, bf.y);
                mma16816(d[2 + cp], lop3_and_or(wa8, MASK_E, MAGIC_E), lop3_and_or(wb8, MASK_E, MAGIC_E),
                         lop3_and_or(wa8, MASK_O, MAGIC_O), lop3_and_or(wb8, MASK_O, MAGIC_O), bf.z, bf.w);
            }
        }
    }

    // Where row r (0..127) of a unit goes: the quad lane that consumes it and the half index inside that
    // lane's fragment entry.  Pairs are (x0,x4)(x1,x5)(x2,x6)(x3,x7) per row block.
    __device__ static __forceinline__ void locate(int r, int& jl, int& h) {
        const int wr = r >> 3, i8 = r & 7;             // word-row of the unit, row inside the word
        jl = (wr & 7) >> 1;
        const int rb = (wr & 1) + 2 * (wr >> 3);        // which of the lane's four vecs
        h = 8 * rb + 2 * (i8 & 3) + (i8 >> 2);
    }
    __device__ static __forceinline__ float coef(int h) { return (h & 2) ? 64.f : 1024.f; }
};

// 3-bit: the quad's lane j owns row block 4*kb + j (32 rows of K = three word-rows, a 96-bit stream
// per column).  Seven 32-bit windows of the stream expose the 32 fields exactly once as 16 pairs
// (kOrder3); a field at bit p of its half gets the offset 2^(10-p).
template <> struct Traits<3> {
    static constexpr int kUnitRows = 128;
    static constexpr int kVecs = 3;
    static constexpr int kBRegs = 16;
    static constexpr int kWordRows = 12;
    __device__ static __forceinline__ int vec_row(int j, int r) { return 3 * j + r; }

    template <int PLO, int PHI>
    __device__ static __forceinline__ uint32_t pair(uint32_t window) {
        constexpr uint32_t mask = (7u << PLO) | (7u << (PHI + 16));
        constexpr uint32_t magic = magic_at(PLO) | (magic_at(PHI) << 16);
        return lop3_and_or(window, mask, magic);
    }
    // the 16 pairs of one column, in kOrder3 order
    __device__ static __forceinline__ void unpack(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t (&p)[16]) {
        const uint32_t v0 = w0 << 7;                        // stream offset -7
        const uint32_t v1 = w0 >> 1;                        // 1
        const uint32_t v2 = __funnelshift_r(w0, w1, 11);    // 11
        const uint32_t v3 = w1;                             // 32
        const uint32_t v4 = __funnelshift_r(w1, w2, 9);     // 41
        const uint32_t v5 = w2 << 2;                        // 62
        const uint32_t v6 = w2 >> 7;                        // 71
        p[0] = pair<7, 0>(v0); p[1] = pair<2, 4>(v1); p[2] = pair<5, 7>(v1); p[3] = pair<1, 0>(v2);
        p[4] = pair<4, 3>(v2); p[5] = pair<7, 6>(v2); p[6] = pair<4, 3>(v3); p[7] = pair<7, 6>(v3);
        p[8] = pair<1, 0>(v4); p[9] = pair<4, 3>(v4); p[10] = pair<7, 6>(v4); p[11] = pair<4, 3>(v5);
        p[12] = pair<7, 6>(v5); p[13] = pair<1, 0>(v6); p[14] = pair<4, 3>(v6); p[15] = pair<7, 6>(v6);
    }
    __device__ static __forceinline__ void compute(const uint4 (&buf)[kVecs], const uint32_t* __restrict__ bsm,
                                                   bool has_x, float (&d)[4][4]) {
        uint4 bf[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            bf[i] = make_uint4(0, 0, 0, 0);
            if (has_x) bf[i] = *reinterpret_cast<const uint4*>(bsm + 4 * i);
        }
        const uint32_t* b = reinterpret_cast<const uint32_t*>(bf);
#pragma unroll
        for (int cp = 0; cp < 2; ++cp) {
            uint32_t pa[16], pb[16];
            if (cp == 0) { unpack(buf[0].x, buf[1].x, buf[2].x, pa); unpack(buf[0].y, buf[1].y, buf[2].y, pb); }
            else         { unpack(buf[0].z, buf[1].z, buf[2].z, pa); unpack(buf[0].w, buf[1].w, buf[2].w, pb); }
#pragma unroll
            for (int t = 0; t < 8; ++t)
                mma16816(d[2 * (t & 1) + cp], pa[2 * t], pb[2 * t], pa[2 * t + 1], pb[2 * t + 1], b[2 * t], b[2 * t + 1]);
        }
    }
    __device__ static __forceinline__ void locate(int r, int& jl, int& h) {
        jl = r >> 5;
        h = kSlot3[r & 31];
    }
    __device__ static __forceinline__ float coef(int h) { return (float)(1 << (10 - kPos3[h])); }
};

struct Plan {
    int cgs;          // column groups (256 columns each) = clusters
    int kbs;          // units per column group
    int cluster;      // CTAs per cluster: the column group's K range is split evenly among them
    int stage_units;  // units whose x values are staged in shared memory at a time
    int ring_units;   // unit buffers in the shared-memory ring
    int push;         // 1: the K slices are combined by pushing partial sums into the first CTA's shared memory
};

// Rows of x staged at a time: the whole K slice of a CTA for the usual decode shapes.
__host__ __device__ inline int max_stage_rows(int M) { return M <= 2 ? kMaxStageRows : (M <= 4 ? 1024 : 512); }

// Dynamic shared memory, in this order: ring | xs | s_sm | z_sm | corr_sm | ps | red
template <int BITS> __host__ __device__ constexpr int unit_bytes() { return Traits<BITS>::kWordRows * kRowPitch; }
template <int BITS> __host__ __device__ inline int xs_bytes(int M) {
    return (max_stage_rows(M) / Traits<BITS>::kUnitRows) * M * 4 * Traits<BITS>::kBRegs * 4;
}
__host__ __device__ inline int s_sm_bytes() { return kStageGroups * kCgCols * 4; }
__host__ __device__ inline int z_sm_bytes() { return kStageGroups * kCgCols * 4; }
__host__ __device__ inline int corr_bytes(int M) { return M * kCgCols * 4; }
__host__ __device__ inline int ps_bytes(int M) { return M * (max_stage_rows(M) / 128) * 8; }
// landing zone of the other CTAs' partial sums (push combine): red[rank - 1][m][column]
__host__ __device__ inline int red_bytes(int M, int cluster) { return (cluster - 1) * M * kCgCols * 4; }
constexpr int kMaxRedBytes = 16 * 1024;   // larger combines read the partial sums remotely instead

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Asynchronous store of a float into the shared memory of CTA `rank` of this cluster, at the offset of
// `local_ptr`; the 4 bytes are counted on that CTA's mbarrier at the offset of `local_bar`.
__device__ __forceinline__ void st_async_cluster_f32(const float* local_ptr, uint32_t local_bar, uint32_t rank, float v) {
    uint32_t dst, bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(smem_u32(local_ptr)), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(local_bar), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.f32 [%0], %1, [%2];"
                 ::"r"(dst), "f"(v), "r"(bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Read a float from the same shared-memory offset in CTA `rank` of this cluster.
__device__ __forceinline__ float ld_cluster_f32(const float* local_ptr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local_ptr)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

#ifdef B200GPTQ_TRACE
// Timeline recorder for experiments (never compiled into the library that ships): every CTA takes a
// ticket and records a tag (the weight pointer, i.e. the launch) plus the global timer at up to 8 marks.
constexpr int kTraceSlots = 8192;
__device__ unsigned long long g_trace[kTraceSlots * 10];
__device__ unsigned int g_ticket;
__device__ __forceinline__ void trace_mark(int slot, const void* tag = nullptr) {
    __shared__ unsigned int s_ticket;
    if (threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        if (slot == 0) {
            s_ticket = atomicAdd(&g_ticket, 1u);
            if (s_ticket < kTraceSlots) {
                unsigned int smid;
                asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
                g_trace[s_ticket * 10 + 9] = (unsigned long long)(blockIdx.x + 1) | ((unsigned long long)smid << 32);
                g_trace[s_ticket * 10 + 8] = (unsigned long long)tag;
            }
        }
        if (s_ticket < kTraceSlots) g_trace[s_ticket * 10 + slot] = t;
    }
}
__global__ void trace_clear_kernel() {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < kTraceSlots * 10) g_trace[i] = 0;
    if (i == 0) g_ticket = 0;
}
__device__ unsigned long long g_trace_units[8 * 64];
__device__ __forceinline__ void trace_unit(int blk, int i) {
    if ((threadIdx.x & 31) == 0 && (blockIdx.x == blk) && i < 64) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        g_trace_units[(threadIdx.x >> 5) * 64 + i] = t;
    }
}
#define TRACE_UNIT(i)
#define CLK_DECL long long c_wait = 0, c_load = 0, c_comp = 0, c_flush = 0, c_stage = 0, c_t, c_s0 = 0, c_s1 = 0, c_s2 = 0, c_s3 = 0, c_s4 = 0, c_s5 = 0
#define CLK_START c_t = clock64()
#define CLK_ADD(acc) do { const long long c_n = clock64(); acc += c_n - c_t; c_t = c_n; } while (0)
#define CLK_STORE do { if ((threadIdx.x & 31) == 0 && blockIdx.x == 35) { unsigned long long* o = g_trace_units + (threadIdx.x >> 5) * 64; \
    o[0] = c_wait; o[1] = c_load; o[2] = c_comp; o[3] = c_flush; o[4] = c_stage; o[5] = c_s0; o[6] = c_s1; o[7] = c_s2; o[8] = c_s3; o[9] = c_s4; o[10] = c_s5; } } while (0)
#define TRACE(slot) trace_mark(slot)
#define TRACE0(tag) trace_mark(0, tag)
#else
#define TRACE(slot)
#define TRACE0(tag)
#define TRACE_UNIT(i)
#define CLK_DECL
#define CLK_START
#define CLK_ADD(acc)
#define CLK_STORE
#endif

// One cluster per column group; CTA `rank` of the cluster owns units [rank*kbs/C, (rank+1)*kbs/C).
// MULTI = false is the single-row instantiation (M == 1, the decode case that is timed): every loop over the
// rows of x and every multi-row code path folds away, which keeps the code that runs once per launch short.
// PERM = false is the instantiation for layers whose x needs no gather (x_perm == NULL).
template <int BITS, bool MULTI, bool PERM>
__global__ void __launch_bounds__(kThreads, 2)
gemv_stream_kernel(const __grid_constant__ CUtensorMap tmap_w, const __half* __restrict__ x,
                   const int32_t* __restrict__ qweight,
                   const int32_t* __restrict__ qzeros, const __half* __restrict__ scales,
                   const int32_t* __restrict__ x_perm_arg, const __half* __restrict__ bias, __half* __restrict__ y,
                   int M_rows, int K, int N, int group_size, Plan plan, unsigned int* __restrict__ status) {
    const int M = MULTI ? M_rows : 1;
    const int32_t* __restrict__ x_perm = PERM ? x_perm_arg : nullptr;
    using T = Traits<BITS>;
    constexpr int UR = T::kUnitRows;
    constexpr int UB = unit_bytes<BITS>();

    extern __shared__ __align__(128) uint8_t dsm[];
    __shared__ __align__(8) uint64_t bars[2 * kMaxRing + 1];   // full[R] at 0, red at 2 * kMaxRing
    __shared__ float t_x[kStageGroups * kMaxM], t_cx[kStageGroups * kMaxM];
    __shared__ volatile int gave_up;
    __shared__ unsigned int taken[kMaxRing];   // warps that have moved the unit in a ring slot to registers

    TRACE0(qweight);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int R = plan.ring_units, C = plan.cluster, kbs = plan.kbs;
    const int cg = blockIdx.x / C, rank = blockIdx.x - cg * C;
    const int kb_begin = (int)(((long long)rank * kbs) / C), kb_end = (int)(((long long)(rank + 1) * kbs) / C);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };

    // the swizzle pattern is a function of the address: the ring starts on a 1024-byte boundary
    uint8_t* ring = dsm + ((1024u - (smem_u32(dsm) & 1023u)) & 1023u);
    uint8_t* after_xs = ring + (size_t)R * UB + xs_bytes<BITS>(M);
    float (*s_sm)[kCgCols] = reinterpret_cast<float (*)[kCgCols]>(after_xs);
    float (*z_sm)[kCgCols] = reinterpret_cast<float (*)[kCgCols]>(after_xs + s_sm_bytes());
    float (*corr_sm)[kCgCols] = reinterpret_cast<float (*)[kCgCols]>(after_xs + s_sm_bytes() + z_sm_bytes());
    float2* ps = reinterpret_cast<float2*>(after_xs + s_sm_bytes() + z_sm_bytes() + corr_bytes(M));
    // (computed where they are used, to keep them out of registers during the main loop)
    auto red_ptr = [&]() {
        return reinterpret_cast<float*>(ring + (size_t)plan.ring_units * UB + xs_bytes<BITS>(M) + s_sm_bytes() +
                                        z_sm_bytes() + corr_bytes(M) + ps_bytes(M));
    };
    auto red_bar_addr = [&]() { return smem_u32(bars) + 8u * (2 * kMaxRing); };

    if (tid < kMaxRing) taken[tid] = 0u;
    if (tid == 0) {
        gave_up = 0;
        for (int s = 0; s < R; ++s) {
            mbar_init(full_bar(s), 1);                 // the expect_tx arrive of the lane that issues the copies
        }
        mbar_init(red_bar_addr(), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the first CTA of the cluster expects one float per (other CTA, x row, column)
        if (plan.push && rank == 0) mbar_arrive_expect_tx(red_bar_addr(), (uint32_t)red_bytes(M, C));
    }
    __syncthreads();
    if (plan.push) cluster_arrive();   // matched by the wait in front of the first store into another CTA

    // Copy unit `kb` of this CTA's column group into ring slot `slot`: one TMA box of kWordRows x 256 words
    // (columns past N are filled with zeros and count towards the expected bytes like the rest).
    auto issue_unit = [&](int kb, int slot) {
        if (lane == 0) {
            mbar_arrive_expect_tx(full_bar(slot), (uint32_t)UB);
            tma_load_3d(smem_u32(ring) + slot * UB, &tmap_w, 0, kb * T::kWordRows, cg * (kCgCols / 32), full_bar(slot));
        }
    };
    // Weights are constants: the ring is filled before the dependency on the previous kernel is awaited.
    if (warp == 0)
        for (int u = 0; u < R && kb_begin + u < kb_end; ++u) issue_unit(kb_begin + u, u);

    {
        const int g = lane >> 2, j = lane & 3;
        const int zwords = N / 32 * BITS;
        const int lane_col = warp * 32 + 4 * g;  // first of the lane's 4 columns inside the column group
        const int units_per_group = group_size / UR;
        uint32_t* xs = reinterpret_cast<uint32_t*>(ring + (size_t)R * UB);
        const int ps_pitch = max_stage_rows(M) / 128;   // ps[m * ps_pitch + c]: (sum x, sum c*x) of staged rows 128c .. 128c+127
        // byte offsets of the lane's vecs inside a unit: line L = chunk (= warp) * word-rows + word-row, piece g ^ (L & 7)
        uint32_t vec_off[T::kVecs];
#pragma unroll
        for (int r = 0; r < T::kVecs; ++r) {
            const uint32_t L = (uint32_t)(warp * T::kWordRows + T::vec_row(j, r));
            vec_off[r] = L * 128u + (((uint32_t)g ^ (L & 7u)) << 4);
        }

        for (int m = 0; m < M; ++m) corr_sm[m][tid] = 0.f;

        float out[2][4], d[4][4];
#pragma unroll
        for (int cp = 0; cp < 2; ++cp)
#pragma unroll
            for (int r = 0; r < 4; ++r) { out[cp][r] = 0.f; d[cp][r] = 0.f; d[2 + cp][r] = 0.f; }

        bool first_stage = true;
        int stage_g0 = 0;

        // out += scale[group] * d for the lane's 4 columns, then clear d.
        auto flush_group = [&](int grp) {
            const float4 s = *reinterpret_cast<const float4*>(&s_sm[grp - stage_g0][lane_col]);
            out[0][0] = fmaf(s.x, d[0][0] + d[2][0], out[0][0]); out[0][1] = fmaf(s.x, d[0][1] + d[2][1], out[0][1]);
            out[0][2] = fmaf(s.y, d[0][2] + d[2][2], out[0][2]); out[0][3] = fmaf(s.y, d[0][3] + d[2][3], out[0][3]);
            out[1][0] = fmaf(s.z, d[1][0] + d[3][0], out[1][0]); out[1][1] = fmaf(s.z, d[1][1] + d[3][1], out[1][1]);
            out[1][2] = fmaf(s.w, d[1][2] + d[3][2], out[1][2]); out[1][3] = fmaf(s.w, d[1][3] + d[3][3], out[1][3]);
#pragma unroll
            for (int cp = 0; cp < 4; ++cp)
#pragma unroll
                for (int r = 0; r < 4; ++r) d[cp][r] = 0.f;
        };

        CLK_DECL;
        // Stage x for units [kb_a, kb_b): fragments into xs, scales and zero-points into s_sm / z_sm, and
        // the offset / zero-point term  sum_groups s * (sum c x + zero * sum x)  into corr_sm.
        auto stage = [&](int kb_a, int kb_b) {
            const int r0 = kb_a * UR, rows = (kb_b - kb_a) * UR;
            const int g0 = r0 / group_size, ng = (r0 + rows - 1) / group_size - g0 + 1;
            const int n = min(cg * kCgCols + tid, N - 1);
            int zw, zsh;
            bool zstr = false;
            if constexpr (BITS == 3) {
                const int bit = 3 * (n & 31);
                zw = 3 * (n >> 5) + (bit >> 5); zsh = bit & 31; zstr = zsh > 29;
            } else {
                zw = n >> 3; zsh = 4 * (n & 7);
            }
            const __half* sp = scales + (size_t)g0 * N + n;
            const uint32_t* zp = reinterpret_cast<const uint32_t*>(qzeros) + (size_t)g0 * zwords + zw;
            __half* xh = reinterpret_cast<__half*>(xs);
            consumer_sync();  // the previous stage's fragments, scales and zero-points are no longer in use

            // 4 rows of K of up to 4 rows of x per thread and pass
            auto x_issue = [&](int qi, int m0, int4 pidx, __half (&v)[4][4]) {
                const int kq = r0 + 4 * qi;
#pragma unroll
                for (int mm = 0; mm < 4; ++mm) {
                    const int m = m0 + mm;
                    if (qi < rows / 4 && m < M) {
                        const __half* xr = x + (size_t)m * K;
                        if (x_perm) {
                            v[mm][0] = xr[pidx.x]; v[mm][1] = xr[pidx.y]; v[mm][2] = xr[pidx.z]; v[mm][3] = xr[pidx.w];
                        } else {
                            const uint2 raw = *reinterpret_cast<const uint2*>(xr + kq);
                            v[mm][0] = __ushort_as_half((unsigned short)(raw.x & 0xffffu));
                            v[mm][1] = __ushort_as_half((unsigned short)(raw.x >> 16));
                            v[mm][2] = __ushort_as_half((unsigned short)(raw.y & 0xffffu));
                            v[mm][3] = __ushort_as_half((unsigned short)(raw.y >> 16));
                        }
                    }
                }
            };
            auto x_consume = [&](int qi, int m0, const __half (&v)[4][4]) {
                const bool has_q = qi < rows / 4;
                const int kl = 4 * qi;                                // row inside the stage
                const int ul = kl / UR, r_in_unit = kl % UR;
                int jl = 0, hh[4];
                float cf[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    T::locate(r_in_unit + i, jl, hh[i]);   // the four rows share jl
                    cf[i] = T::coef(hh[i]);
                }
                // Sums over the warp's 128 consecutive rows, which lie in one group (group_size is a multiple of
                // 128).  With several rows of x the reductions are written level by level over all rows, so that
                // the shuffles of different rows overlap instead of forming one long dependent chain per row.
                float sx[4], scx[4];
                const int nrows = min(4, M - m0);   // uniform
#pragma unroll
                for (int mm = 0; mm < 4; ++mm) {
                    sx[mm] = 0.f; scx[mm] = 0.f;
                    if (mm < nrows && has_q) {
                        const int m = m0 + mm;
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            xh[(size_t)(((ul * M + m) * 4 + jl) * T::kBRegs) * 2 + hh[i]] = v[mm][i];
                            const float xf = __half2float(v[mm][i]);
                            sx[mm] += xf;
                            scx[mm] = fmaf(cf[i], xf, scx[mm]);
                        }
                    }
                }
                if (nrows == 1) {
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1) {
                        sx[0] += __shfl_xor_sync(0xffffffffu, sx[0], o);
                        scx[0] += __shfl_xor_sync(0xffffffffu, scx[0], o);
                    }
                } else {
#pragma unroll
                    for (int o = 1; o < 32; o <<= 1)
#pragma unroll
                        for (int mm = 0; mm < 4; ++mm) {
                            sx[mm] += __shfl_xor_sync(0xffffffffu, sx[mm], o);
                            scx[mm] += __shfl_xor_sync(0xffffffffu, scx[mm], o);
                        }
                }
                if (has_q && lane == 0) {
#pragma unroll
                    for (int mm = 0; mm < 4; ++mm)
                        if (mm < nrows) ps[(m0 + mm) * ps_pitch + (qi >> 5)] = make_float2(sx[mm], scx[mm]);
                }
            };
            auto perm_of = [&](int qi) {
                const int kq = r0 + 4 * qi;
                int4 pidx = make_int4(kq, kq + 1, kq + 2, kq + 3);
                if (qi < rows / 4 && x_perm) pidx = __ldg(reinterpret_cast<const int4*>(x_perm + kq));
                return pidx;
            };

            // -- constants (scales, zero-points, gather indices): 8 groups of loads in flight at a time; the
            //    first pass of x loads is issued before the first constants are consumed, so that a stage
            //    costs one round trip to memory, not two
            CLK_START;
            __half v0[4][4];
            const int4 pidx0 = perm_of(tid);
#pragma unroll 1
            for (int gb = 0; gb < ng; gb += 8) {
                __half sv[8];
                uint32_t lo[8], hi[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    sv[i] = __float2half(0.f); lo[i] = 0u; hi[i] = 0u;
                    if (gb + i < ng) {
                        sv[i] = __ldg(sp + (size_t)(gb + i) * N);
                        lo[i] = __ldg(zp + (size_t)(gb + i) * zwords);
                        if (BITS == 3 && zstr) hi[i] = __ldg(zp + (size_t)(gb + i) * zwords + 1);
                    }
                }
                // later stages: x can be requested before the first constants are consumed (one round trip, not two)
                if (gb == 0 && !first_stage) x_issue(tid, 0, pidx0, v0);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    if (gb + i < ng) {
                        uint32_t q;
                        if constexpr (BITS == 3) q = __funnelshift_r(lo[i], hi[i], zsh) & 7u;
                        else q = (lo[i] >> zsh) & 15u;
                        s_sm[gb + i][tid] = __half2float(sv[i]);
                        z_sm[gb + i][tid] = __uint_as_float(0x4B000000u | (q + 1u)) - 8388608.f;  // exact small integer
                    }
                }
            }
            CLK_ADD(c_s0);
            if (first_stage) {
                // Everything above used constants only.  x is the one operand a preceding kernel may still be
                // writing: under programmatic dependent launch this is where the kernel waits for it, with its
                // scales and zero-points staged and its ring full.
                TRACE(1);
                // One warp waits for the previous kernel; the others sleep at a hardware barrier meanwhile, so a CTA
                // that is waiting here takes no issue slots from the CTA of the previous kernel on the same SM.
                if (warp == 0) asm volatile("griddepcontrol.wait;" ::: "memory");
                consumer_sync();
                // Only now may the next kernel of the stream take SM space (it initialises, fetches its scales and
                // zero-points and fills its ring with weights before it waits for this kernel's result).  Released
                // any earlier, a third kernel could occupy free halves of SMs ahead of the second one; measured
                // slower for grids that leave half of every SM free.
                asm volatile("griddepcontrol.launch_dependents;");
                TRACE(2);
                first_stage = false;
                x_issue(tid, 0, pidx0, v0);
            }
            CLK_ADD(c_s1);
            x_consume(tid, 0, v0);
            CLK_ADD(c_s2);
#pragma unroll 1
            for (int q0 = 0; q0 < rows / 4; q0 += kConsumerThreads) {
                const int qi = q0 + tid;
                const int4 pidx = q0 == 0 ? pidx0 : perm_of(qi);
#pragma unroll 1
                for (int m0 = (q0 == 0 ? 4 : 0); m0 < M; m0 += 4) {
                    __half v[4][4];
                    x_issue(qi, m0, pidx, v);
                    x_consume(qi, m0, v);
                }
            }
            CLK_ADD(c_s3);
            consumer_sync();
            TRACE(3);
            if (tid < ng * M) {
                const int m = tid % M, gl = tid / M;
                const int ra = max(r0, (g0 + gl) * group_size), rb = min(r0 + rows, (g0 + gl + 1) * group_size);
                float sx = 0.f, scx = 0.f;
                for (int o = (ra - r0) >> 7; o < (rb - r0) >> 7; ++o) {
                    const float2 p = ps[m * ps_pitch + o];
                    sx += p.x;
                    scx += p.y;
                }
                t_x[gl * kMaxM + m] = sx;
                t_cx[gl * kMaxM + m] = scx;
            }
            consumer_sync();
            if (M == 1) {
                float c = 0.f;
#pragma unroll 4
                for (int gl = 0; gl < ng; ++gl)
                    c = fmaf(s_sm[gl][tid], fmaf(z_sm[gl][tid], t_x[gl * kMaxM], t_cx[gl * kMaxM]), c);
                corr_sm[0][tid] += c;
            } else {
                // groups outermost, rows of x innermost: eight independent sums instead of eight chains in a row
                // (every sum still adds its groups in increasing order)
                float c[kMaxM];
#pragma unroll
                for (int m = 0; m < kMaxM; ++m) c[m] = 0.f;
#pragma unroll 2
                for (int gl = 0; gl < ng; ++gl) {
                    const float sg = s_sm[gl][tid], zg = z_sm[gl][tid];
#pragma unroll
                    for (int m = 0; m < kMaxM; ++m)
                        if (m < M) c[m] = fmaf(sg, fmaf(zg, t_x[gl * kMaxM + m], t_cx[gl * kMaxM + m]), c[m]);
                }
#pragma unroll
                for (int m = 0; m < kMaxM; ++m)
                    if (m < M) corr_sm[m][tid] += c[m];
            }
            stage_g0 = g0;
            CLK_ADD(c_s4);
            TRACE(4);
        };

        int kb = kb_begin, slot = 0, round = 0;
        int grp = 0;
        bool pending = false;  // d holds products that have not been scaled into out yet
        while (kb < kb_end) {
            // stage as far as the stage grid and this CTA's range allow
            const int su = plan.stage_units;
            const int kb_stop = min((kb / su + 1) * su, kb_end);
            CLK_START;
            stage(kb, kb_stop);
            CLK_ADD(c_stage);
            grp = (kb * UR) / group_size;
            int grp_left = units_per_group - (kb - grp * units_per_group);
            const uint32_t* bsm = xs + (size_t)(g * 4 + j) * T::kBRegs;
            const int bsm_step = M * 4 * T::kBRegs;
#pragma unroll 1
            for (; kb < kb_stop; ++kb) {
                mbar_wait(full_bar(slot), round & 1, &gave_up);
                CLK_ADD(c_wait);
                uint4 cur[T::kVecs];
                const uint8_t* src = ring + slot * UB;
#pragma unroll
                for (int r = 0; r < T::kVecs; ++r) cur[r] = *reinterpret_cast<const uint4*>(src + vec_off[r]);
                __syncwarp();
                // The unit is on its way to registers.  Each warp counts itself in; the last one refills the slot with
                // the unit R further on (nobody waits for anybody).  The count is looked at after the products, so
                // that its round trip through shared memory is not waited for.
                unsigned int before = 0u;
                if (lane == 0) before = atomicAdd(&taken[slot], 1u);
                const int done_slot = slot;
                if (++slot == R) { slot = 0; ++round; }
                CLK_ADD(c_load);
                T::compute(cur, bsm, g < M, d);
                CLK_ADD(c_comp);
                before = __shfl_sync(0xffffffffu, before, 0);
                if (before == kConsumerWarps - 1) {
                    if (lane == 0) taken[done_slot] = 0u;
                    if (kb + R < kb_end) issue_unit(kb + R, done_slot);
                }
                bsm += bsm_step;
                pending = true;
                if (--grp_left == 0) {
                    flush_group(grp);
                    ++grp;
                    grp_left = units_per_group;
                    pending = false;
                }
                CLK_ADD(c_flush);
            }
            TRACE(5);
        }
        if (pending) flush_group(grp);
        CLK_STORE;

        // ---- this CTA's partial result: combine the lanes, remove the offset / zero-point term ----
        consumer_sync();  // corr_sm is complete
        const bool push = plan.push != 0;
        if (push) cluster_wait();   // every CTA of the cluster is running and has initialised its barriers
        float* red = red_ptr();
        const uint32_t red_bar = red_bar_addr();
#pragma unroll
        for (int cp = 0; cp < 2; ++cp)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int m = 2 * j + (r & 1);
                const int c = lane_col + 2 * cp + (r >> 1);
                if (m < M) {
                    const float v = out[cp][r] - corr_sm[m][c];
                    if (push && rank > 0) st_async_cluster_f32(red + ((rank - 1) * M + m) * kCgCols + c, red_bar, 0u, v);
                    else corr_sm[m][c] = v;
                }
            }
        consumer_sync();
    }

    if (plan.push) {
        float* red = red_ptr();
        const uint32_t red_bar = red_bar_addr();
        // ---- push combine: the other CTAs are done once their stores are issued (nothing reads their shared
        //      memory); the first CTA waits for all of them on its barrier and adds them up in rank order ----
        TRACE(6);
        if (rank == 0 && warp < kConsumerWarps) {
            mbar_wait(red_bar, 0, &gave_up);
            const int n = cg * kCgCols + tid;
            if (n < N) {
#pragma unroll 1
                for (int m = 0; m < M; ++m) {
                    float v = corr_sm[m][tid];
                    for (int r = 1; r < C; ++r) v += red[((r - 1) * M + m) * kCgCols + tid];
                    if (bias) v += __half2float(bias[n]);
                    y[(size_t)m * N + n] = __float2half_rn(v);
                }
            }
        }
        if (tid == 0 && gave_up) atomicExch(status + kStatusWord, 1u);
        TRACE(7);
        return;
    }

    // ---- combine the K slices of the cluster through distributed shared memory, in rank order ----
    // (a single row of x is always pushed when the cluster has several CTAs: the single-row kernels get here with
    // one CTA per cluster only, and the remote part below is compiled out of them)
    if (MULTI && C > 1) cluster_sync_all();   // every CTA's partial result is in its corr_sm
    TRACE(6);
    if (rank == 0 && warp < kConsumerWarps) {
        const int n = cg * kCgCols + tid;
        if (n < N) {
#pragma unroll 1
            for (int m = 0; m < M; ++m) {
                // all remote reads are issued before the first is used; the sum stays in rank order
                float part[8];
#pragma unroll
                for (int r = 1; r < 8; ++r)
                    part[r] = (MULTI && r < C) ? ld_cluster_f32(&corr_sm[m][tid], (uint32_t)r) : 0.f;
                float v = corr_sm[m][tid];
#pragma unroll
                for (int r = 1; r < 8; ++r) v += part[r];
                if (bias) v += __half2float(bias[n]);
                y[(size_t)m * N + n] = __float2half_rn(v);
            }
        }
    }
    if (MULTI && C > 1) cluster_sync_all();   // the other CTAs keep their shared memory alive until it has been read
    if (tid == 0 && gave_up) atomicExch(status + kStatusWord, 1u);
    TRACE(7);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
}

int ctas_per_sm() {
    static const int v = [] {
        const char* e = std::getenv("B200GPTQ_GEMV_CTAS_PER_SM");
        const int n = e ? std::atoi(e) : 0;
        return (n == 1 || n == 2) ? n : 2;
    }();
    return v;
}

template <int BITS>
Plan make_plan(int M, int K, int N, int group_size, int* smem_bytes) {
    Plan p;
    constexpr int unit_rows = Traits<BITS>::kUnitRows;
    p.cgs = (N + kCgCols - 1) / kCgCols;
    p.kbs = K / unit_rows;
    // cluster size: as many K slices as keep every CTA of the grid resident at once (two per SM: a CTA takes just
    // under half an SM's registers and shared memory), at most 8.  Measured against one CTA per SM with the next
    // launch of the stream resident beside it: two CTAs of the same launch keep the SM's issue slots busier
    // (16 warps instead of 8 in the unpack loop), which is worth more than hiding the next launch's start-up.
    const int per_sm = ctas_per_sm();
    const int slots = per_sm * sm_count();
    int c = slots / p.cgs;
    if (c > 8) c = 8;
    if (c > p.kbs) c = p.kbs;
    if (c < 1) c = 1;
    p.cluster = c;
    // a stage spans at most max_stage_rows(M) rows and at most kStageGroups groups, and starts on a multiple of itself
    const int cap = max_stage_rows(M);
    long long stage_rows = (long long)kStageGroups * group_size;
    if (stage_rows > cap) stage_rows = group_size <= cap ? (cap / group_size) * group_size : cap;
    p.stage_units = (int)(stage_rows / unit_rows);
    if (p.stage_units < 1) p.stage_units = 1;
    // ring: what is left of the shared-memory budget, no more than the slice needs
    const int other = xs_bytes<BITS>(M) + s_sm_bytes() + z_sm_bytes() + corr_bytes(M) + ps_bytes(M);
    static const bool push_env = [] {
        const char* e = std::getenv("B200GPTQ_GEMV_PUSH");
        return !(e && e[0] == '0');
    }();
    p.push = (c > 1 && (M == 1 || push_env) && red_bytes(M, c) <= kMaxRedBytes) ? 1 : 0;
    const int fixed = other + (p.push ? red_bytes(M, c) : 0);
    static const int inflight_env = [] {
        const char* e = std::getenv("B200GPTQ_GEMV_INFLIGHT_KB");
        const int kb = e ? std::atoi(e) : 0;
        return kb > 0 ? kb * 1024 : 0;
    }();
    const int inflight = inflight_env ? inflight_env : kSmemBudget - fixed;
    int ring = inflight / unit_bytes<BITS>();
    const int longest = (p.kbs + c - 1) / c;
    if (ring > longest) ring = longest;
    if (ring > kMaxRing) ring = kMaxRing;
    if (ring < 2) ring = 2;
    p.ring_units = ring;
    *smem_bytes = ring * unit_bytes<BITS>() + fixed + 1024;   // + slack to start the ring on a 1024-byte boundary
    return p;
}

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("B200GPTQ_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

template <int BITS>
int launch_stream(const __half* x, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                  const int32_t* x_perm, const __half* bias, __half* y, int M, int K, int N, int group_size,
                  void* workspace, cudaStream_t stream) {
    int smem_bytes = 0;
    const Plan plan = make_plan<BITS>(M, K, N, group_size, &smem_bytes);
    unsigned int* status = reinterpret_cast<unsigned int*>(workspace);

    static bool attr_set[64] = {};
    int dev = 0;
    B200GPTQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        B200GPTQ_CUDA_TRY(cudaFuncSetAttribute(gemv_stream_kernel<BITS, false, false>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200GPTQ_CUDA_TRY(cudaFuncSetAttribute(gemv_stream_kernel<BITS, false, true>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200GPTQ_CUDA_TRY(cudaFuncSetAttribute(gemv_stream_kernel<BITS, true, false>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        B200GPTQ_CUDA_TRY(cudaFuncSetAttribute(gemv_stream_kernel<BITS, true, true>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[dev] = true;
    }
    // qweight [K/32*bits, N] as a 3-D tensor {32 columns, word-rows, N/32 column chunks}; a box is one unit
    static const EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) { set_last_cuda_error((int)cudaErrorNotSupported); return B200GPTQ_ERR_CUDA; }
    CUtensorMap tmap_w;
    {
        const cuuint64_t dims[3] = {32, (cuuint64_t)(K / 32 * BITS), (cuuint64_t)(N / 32)};
        const cuuint64_t strides[2] = {(cuuint64_t)N * sizeof(int32_t), 32 * sizeof(int32_t)};
        const cuuint32_t box[3] = {32, (cuuint32_t)Traits<BITS>::kWordRows, (cuuint32_t)(kCgCols / 32)};
        const cuuint32_t estr[3] = {1, 1, 1};
        const CUresult r = encode(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<int32_t*>(qweight), dims,
                                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)cudaErrorInvalidValue); return B200GPTQ_ERR_CUDA; }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.cgs * plan.cluster);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    attr[na].id = cudaLaunchAttributeClusterDimension;
    attr[na].val.clusterDim.x = plan.cluster;
    attr[na].val.clusterDim.y = 1;
    attr[na].val.clusterDim.z = 1;
    ++na;
    if (pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    auto kernel = M == 1 ? (x_perm ? gemv_stream_kernel<BITS, false, true> : gemv_stream_kernel<BITS, false, false>)
                         : (x_perm ? gemv_stream_kernel<BITS, true, true> : gemv_stream_kernel<BITS, true, false>);
    B200GPTQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tmap_w, x, qweight, qzeros, scales, x_perm, bias, y, M, K, N,
                                         group_size, plan, status));
    return B200GPTQ_OK;
}

}  // namespace

#ifdef B200GPTQ_TRACE
extern "C" __attribute__((visibility("default"))) int b200gptq_trace_read(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, g_trace, sizeof(unsigned long long) * n);
}
extern "C" __attribute__((visibility("default"))) int b200gptq_trace_units(unsigned long long* host) {
    return (int)cudaMemcpyFromSymbol(host, g_trace_units, sizeof(unsigned long long) * 8 * 64);
}
extern "C" __attribute__((visibility("default"))) int b200gptq_trace_clear(void) {
    trace_clear_kernel<<<80, 1024>>>();
    return (int)cudaDeviceSynchronize();
}
#endif

// The streaming kernel handles groups k / group_size only (no g_idx), whole units per group, and
// x rows that can be read 8 bytes at a time.
bool gemv_stream_supported(int M, int K, int N, int bits, int group_size) {
    (void)N;
    if (M < 1 || M > kMaxM) return false;
    if (bits == 3 || bits == 4) return group_size % 128 == 0 && K % 128 == 0;
    return false;
}

size_t gemv_stream_workspace_bytes(int M, int K, int N, int bits) {
    (void)M;
    if (bits != 3 && bits != 4) return 0;
    if (bits == 3 && K % 128 != 0) return 0;
    (void)K; (void)N;
    return kCounterBytes;  // only the status word: partial sums travel through distributed shared memory
}

int gemv_stream_dispatch(const __half* x, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                         const int32_t* g_idx, const int32_t* x_perm, const __half* bias, __half* y, int M, int K,
                         int N, int bits, int group_size, void* workspace, cudaStream_t stream) {
    if (g_idx) return B200GPTQ_ERR_GROUPS;
    if (bits == 4)
        return launch_stream<4>(x, qweight, qzeros, scales, x_perm, bias, y, M, K, N, group_size, workspace, stream);
    if (bits == 3)
        return launch_stream<3>(x, qweight, qzeros, scales, x_perm, bias, y, M, K, N, group_size, workspace, stream);
    return B200GPTQ_ERR_BITS;
}

}  // namespace b200gptq
