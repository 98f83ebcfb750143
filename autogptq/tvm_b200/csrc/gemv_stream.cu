// Decode GEMV, streaming form (M <= 8, bits in {3,4}, groups = k / group_size).
//
//   y[m, n] = sum_k x[m, xk(k)] * scales[g, n] * (q[k, n] - zero[g, n]),   g = k / group_size
//
// A single layer moves 8..17 MB and lasts a few microseconds, so the kernel is shaped by the fixed costs
// of one launch as much as by bandwidth.  Measured on B200 while designing it: with all weight loads
// removed a launch takes as long as with them, and with loads and arithmetic removed the rest (start-up,
// x, combine) still costs 4..6 us: instruction issue and latency on the SMs bound a launch of this size,
// not HBM (a bare TMA loop over the same boxes streams at 6.6 TB/s).  The alternatives to the split below
// were built and timed too: one CTA per 32-column strip over all of K (no combine, but every CTA prepares
// the whole of x) and K slices combined through global scratch by the last CTA to arrive (the fence /
// counter / re-read chain costs 2 us at the end of every launch); both were slower.
//
//  * Everything that does not depend on the previous kernel is requested in the first instructions:
//    the CTA's scales (one TMA box), its zero-points and gather indices (plain loads) and its weights
//    (a ring of "units" of 256 columns x 128 rows of K, one cp.async.bulk.tensor box of 12 or 16 KB per
//    unit, 128-byte swizzle, completion on an mbarrier).  Under programmatic dependent launch this happens
//    while the previous kernel is still running.  Only x is read after `griddepcontrol.wait`.
//  * x is laid out in shared memory in the order in which the tensor-core fragments consume it: a
//    thread gathers the eight values of one 16-byte piece and stores it with one instruction; the sums
//    of x that the offset removal needs are reduced over 16 lanes on the way.  Layers with a gather
//    first copy the whole of x into shared memory with one linear bulk copy and gather from there
//    (2-byte gathers from global memory by every CTA at the same moment queue up at the few L2 lines
//    that hold x: 34 us instead of 10 for the 3-bit benchmark layer when every CTA gathers all of x).
//    The unpack + MMA loop starts right after that one barrier; scales are first needed at the end of
//    the first unit (their TMA box has its own mbarrier), zero-points only after the loop.
//  * Unpack without shifts into place or integer->float conversion: a LOP3 masks two fields of a
//    word and ORs in an fp16 exponent, which yields the half2 (c_lo + q_lo, c_hi + q_hi) with known
//    offsets c = 2^(10-p) for a field at bit p of its half: 5 integer instructions per 8 weights
//    (4-bit), 23 per 32 weights (3-bit).
//  * The products are done by mma.sync m16n8k16 (f16 x f16 -> f32): the 16 rows of the A tile
//    are 16 output columns, the 8 columns of B are the (up to 8) rows of x, so one instruction
//    retires 256 weights of a warp for every M <= 8.  After each unit the sums are scaled by the
//    unit's group scale.  Offsets and zero-points are removed at the end: per column
//    sum_units s * (sum_k c_k x_k + zero * sum_k x_k), which needs only x, scales and qzeros.
//
// Work split: a CTA is 8 warps; warp w owns columns 32w..32w+31 of its column group, the four lanes of a
// quad own different rows of a unit.  A thread-block cluster of up to 8 CTAs owns one 256-column group and
// splits its K range evenly, so a CTA prepares only its own slice of x; the CTAs' partial sums are combined
// in the cluster's first CTA in rank order, either pushed there with asynchronous shared-memory stores
// (small M) or read from it through distributed shared memory (results do not depend on scheduling; no
// global scratch, atomics or fences).  Every mbarrier wait is bounded; if one expires the kernel raises a
// sticky status word and runs on without waiting.
//
// Reference semantics: auto_gptq/nn_modules/qlinear.py:197-243; the kernel this replaces is
// the TVM-generated SIMT GEMV src/kernels/gemv_kernel.cu:25-55.
#include <cuda.h>

#include <mutex>
#include <new>

#include "common.cuh"
#include "tp_exchange.cuh"

namespace b200gptq {

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = 32 * kWarps;       // 256
constexpr int kCgCols = 32 * kWarps;        // 256 columns per column group
constexpr int kMaxM = 8;
constexpr int kUnitRows = 128;
constexpr int kRowPitch = kCgCols * 4;      // bytes of one word-row of a unit
constexpr int kMaxRing = 32;
constexpr int kXsBytes = 16 * 1024;         // x fragments staged at a time
constexpr int kXFullMax = 32 * 1024;        // largest x (all rows) that is copied whole before a gather
constexpr int kStatusWord = kMaxCounters - 1;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t magic) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(magic));  // (a & mask) | magic
    return r;
}

// d += a * b, or d = a * b when FIRST (the accumulators of a unit start at zero without being cleared)
template <bool FIRST>
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    if (FIRST) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
            : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
    } else {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    }
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
// The same test with a suspend-time hint: the thread may stay suspended for up to `ns` nanoseconds and is woken when
// the phase completes, so a waiting warp leaves its scheduler's issue slots to the warps that have work.
__device__ __forceinline__ bool mbar_try_wait_for(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Bounded wait.  After ~1e9 clocks, or once any thread of the CTA has given up, waiting stops for
// good: the kernel then finishes with undefined results and a raised status word instead of hanging.
__device__ __noinline__ void mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* gave_up) {
    const long long t0 = clock64();
    while (!*gave_up) {
        for (int i = 0; i < 8; ++i)
            if (mbar_try_wait_for(bar, parity, 2000u)) return;
        if (clock64() - t0 > 1000000000LL) *gave_up = 1;
    }
}
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* gave_up) {
    if (mbar_try_wait(bar, parity)) return;
    if (mbar_try_wait(bar, parity)) return;
    mbar_wait_slow(bar, parity, gave_up);
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
// scales [G, N] fp16: a box is 256 columns x the groups of a stage, rows past G and columns past N read as zero
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}

// 3-bit: the 32 fields of a row block leave the seven-window unpack as the 16 pairs (0,3) (1,7) (2,8)
// (4,9) (5,10) (6,11) (12,17) (13,18) (14,19) (15,20) (16,21) (22,27) (23,28) (24,29) (25,30) (26,31);
// x is staged in the same order.  kField3[h] = field (row of the block) that sits at half h of a fragment entry,
// kPos3[h] = bit position (inside its 16-bit half) at which that field is masked: its offset is 2^(10 - p).
struct Table32 { unsigned char v[32]; };
constexpr Table32 kField3 = {{0, 3, 1, 7, 2, 8, 4, 9, 5, 10, 6, 11, 12, 17, 13, 18,
                              14, 19, 15, 20, 16, 21, 22, 27, 23, 28, 24, 29, 25, 30, 26, 31}};
constexpr Table32 kPos3 = {{7, 0, 2, 4, 5, 7, 1, 0, 4, 3, 7, 6, 4, 3, 7, 6,
                            1, 0, 4, 3, 7, 6, 4, 3, 7, 6, 1, 0, 4, 3, 7, 6}};
// eight consecutive table entries as the bytes of one 64-bit word
constexpr unsigned long long pack8(const Table32& t, int first) {
    unsigned long long r = 0;
    for (int i = 0; i < 8; ++i) r |= (unsigned long long)t.v[first + i] << (8 * i);
    return r;
}

// fp16 exponent pattern that turns a field at bit p of a 16-bit half into 2^(10-p) + field.
__host__ __device__ constexpr uint32_t magic_at(int p) { return (uint32_t)(25 - p) << 10; }

// ---------------------------------------------------------------------------------------
// Per-bit-width traits.  A unit is 256 columns x 128 rows of K for both widths.
//   kWordRows     word-rows of qweight per unit (= rows of the unit's ring buffer)
//   kVecs         128-bit reads per thread per unit
// Lane (g = lane/4, j = lane%4) of warp w holds columns 32w + 4g .. +3 of the column group; a fragment entry
// is the 32 halves (16 registers) of x that quad lane j multiplies with its share of a unit.
//   piece_rows(j, t8, r, pos)   rows of the unit (0..127) whose x values form halves 8*t8 .. 8*t8+7 of quad lane
//                               j's fragment entry, and the bit positions of the fields they multiply
// ---------------------------------------------------------------------------------------
template <int BITS> struct Traits;

// 4-bit: the quad's lane j owns word-rows 2j, 2j+1, 8+2j, 9+2j of the unit's 16 (8 rows of K each): with the
// swizzled ring layout the four lanes of a quad then read from different banks.  Pair i of a word is
// (nibble i, nibble i + 4); even pairs are masked in place (offset 1024), odd pairs sit at bit 4 (offset 64);
// pairs 2, 3 come from the word shifted right by 8.
template <> struct Traits<4> {
    static constexpr int kVecs = 4;
    static constexpr int kWordRows = 16;
    // word-row of the unit that holds vec r of quad lane j
    __device__ static __forceinline__ int vec_row(int j, int r) { return 2 * j + (r & 1) + 8 * (r >> 1); }

    // d[cp], d[2 + cp]: column pair cp (columns 2cp, 2cp+1 of the lane's 4) over this unit;
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
                if (rb == 0) {
                    mma16816<true>(d[cp], lop3_and_or(wa, MASK_E, MAGIC_E), lop3_and_or(wb, MASK_E, MAGIC_E),
                                   lop3_and_or(wa, MASK_O, MAGIC_O), lop3_and_or(wb, MASK_O, MAGIC_O), bf.x, bf.y);
                    mma16816<true>(d[2 + cp], lop3_and_or(wa8, MASK_E, MAGIC_E), lop3_and_or(wb8, MASK_E, MAGIC_E),
                                   lop3_and_or(wa8, MASK_O, MAGIC_O), lop3_and_or(wb8, MASK_O, MAGIC_O), bf.z, bf.w);
                } else {
                    mma16816<false>(d[cp], lop3_and_or(wa, MASK_E, MAGIC_E), lop3_and_or(wb, MASK_E, MAGIC_E),
                                    lop3_and_or(wa, MASK_O, MAGIC_O), lop3_and_or(wb, MASK_O, MAGIC_O), bf.x, bf.y);
                    mma16816<false>(d[2 + cp], lop3_and_or(wa8, MASK_E, MAGIC_E), lop3_and_or(wb8, MASK_E, MAGIC_E),
                                    lop3_and_or(wa8, MASK_O, MAGIC_O), lop3_and_or(wb8, MASK_O, MAGIC_O), bf.z, bf.w);
                }
            }
        }
    }

    // Piece t8 of lane j is one word-row (8 consecutive rows of K) in the order 0 4 1 5 2 6 3 7.
    __device__ static __forceinline__ void piece_rows(int j, int t8, int (&r)[8], int (&pos)[8]) {
        const int wr = (t8 & 1) + 2 * j + 8 * (t8 >> 1);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            r[i] = 8 * wr + (i >> 1) + 4 * (i & 1);
            pos[i] = (i & 2) ? 4 : 0;
        }
    }
};

// 3-bit: the quad's lane j owns row block j of the unit (32 rows of K = three word-rows, a 96-bit stream
// per column).  Seven 32-bit windows of the stream expose the 32 fields exactly once as 16 pairs.
template <> struct Traits<3> {
    static constexpr int kVecs = 3;
    static constexpr int kWordRows = 12;
    __device__ static __forceinline__ int vec_row(int j, int r) { return 3 * j + r; }

    template <int PLO, int PHI>
    __device__ static __forceinline__ uint32_t pair(uint32_t window) {
        constexpr uint32_t mask = (7u << PLO) | (7u << (PHI + 16));
        constexpr uint32_t magic = magic_at(PLO) | (magic_at(PHI) << 16);
        return lop3_and_or(window, mask, magic);
    }
    // the 16 pairs of one column, in fragment order
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
            for (int t = 0; t < 8; ++t) {
                if (t < 2)
                    mma16816<true>(d[2 * (t & 1) + cp], pa[2 * t], pb[2 * t], pa[2 * t + 1], pb[2 * t + 1], b[2 * t], b[2 * t + 1]);
                else
                    mma16816<false>(d[2 * (t & 1) + cp], pa[2 * t], pb[2 * t], pa[2 * t + 1], pb[2 * t + 1], b[2 * t], b[2 * t + 1]);
            }
        }
    }
    __device__ static __forceinline__ void piece_rows(int j, int t8, int (&r)[8], int (&pos)[8]) {
        constexpr unsigned long long F0 = pack8(kField3, 0), F1 = pack8(kField3, 8), F2 = pack8(kField3, 16),
                                     F3 = pack8(kField3, 24);
        constexpr unsigned long long P0 = pack8(kPos3, 0), P1 = pack8(kPos3, 8), P2 = pack8(kPos3, 16),
                                     P3 = pack8(kPos3, 24);
        const unsigned long long f = t8 == 0 ? F0 : (t8 == 1 ? F1 : (t8 == 2 ? F2 : F3));
        const unsigned long long p = t8 == 0 ? P0 : (t8 == 1 ? P1 : (t8 == 2 ? P2 : P3));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            r[i] = 32 * j + (int)((f >> (8 * i)) & 0xffu);
            pos[i] = (int)((p >> (8 * i)) & 0xffu);
        }
    }
};

// ---------------------------------------------------------------------------------------
// Integer tensor path of the single-row 3-bit instantiation.  Measured on B200: mma.sync retires one m16n8k32 u8 x s8
// product in the same 8 cycles per SM sub-partition as one m16n8k16 f16 product (twice the weights), integer and
// logic instructions issue at half rate, and bytes need far fewer of them than halves: a 96-bit run of 3-bit fields
// becomes nine operand registers with twelve instructions (bytes q << p, p <= 5) against 23 for halves; the factor
// 2^p is taken out on the x side.  x is turned into fixed point per
// unit (X = x * 2^e, |X| < 2^22: exact for every element within 2^-12 of the unit's largest), pre-shifted by what
// its weight byte lacks, and split into four signed byte planes, which are the columns 0..3 of the B operand: one
// instruction multiplies 512 weights by all four planes.  The four sums are recombined in fp32 once per unit
// together with the group's scale; the zero-point term is  zero * sum X.
//   kSteps      tensor instructions per unit and pair of columns
//   kPre        log2 of the common factor of (weight byte) * (pre-shifted X) over q * X
//   item_rows   x preparation: the 8 rows (relative to the unit) that item 4 j + t of a unit handles (quad lane t,
//               part j) and the left shift each X gets
// ---------------------------------------------------------------------------------------
// d += a (u8, 16 x 32) * b (s8, 32 x 8)
__device__ __forceinline__ void imma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                     uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// exact int -> float for |d| < 2^22 without a conversion instruction (those issue at a fraction of the arithmetic rate)
__device__ __forceinline__ float small_int_to_float(int d) { return __int_as_float(d + 0x4B400000) - 12582912.f; }
// 4 x 4 byte transpose: plane p of the result holds byte p of a, b, c, d
__device__ __forceinline__ void planes_of(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&pl)[4]) {
    const uint32_t ab01 = __byte_perm(a, b, 0x5140), cd01 = __byte_perm(c, d, 0x5140);
    const uint32_t ab23 = __byte_perm(a, b, 0x7362), cd23 = __byte_perm(c, d, 0x7362);
    pl[0] = __byte_perm(ab01, cd01, 0x5410); pl[1] = __byte_perm(ab01, cd01, 0x7632);
    pl[2] = __byte_perm(ab23, cd23, 0x5410); pl[3] = __byte_perm(ab23, cd23, 0x7632);
}
// one step's B operands of a quad lane: [plane][b0, b1]
__device__ __forceinline__ void store_step(uint8_t* dst, const uint32_t (&lo)[4], const uint32_t (&hi)[4]) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(lo[0], hi[0], lo[1], hi[1]);
    *reinterpret_cast<uint4*>(dst + 16) = make_uint4(lo[2], hi[2], lo[3], hi[3]);
}
struct Table8 { unsigned char v[8]; };
constexpr unsigned long long pack8b(const Table8& t) {
    unsigned long long r = 0;
    for (int i = 0; i < 8; ++i) r |= (unsigned long long)t.v[i] << (8 * i);
    return r;
}

// 3-bit: quad lane t owns row block t of the unit (a 96-bit run per column, field f at bit 3 f).  Every byte of the
// three words holds two whole fields, which two ANDs per word expose as q << p; the eight fields that straddle
// bytes (2 5 10 13 18 21 26 29) sit at the start of a byte after a shift of the run by 6 bits.  Nine registers hold
// the 32 fields (and four empty bytes):
//   R0 = w0 & A: f0 p0, f3 p1, f6 p2, f8 p0      R1 = w0 & B: f1 p3, f4 p4, f7 p5, f9 p3
//   R2 = w1 & A': f11 p1, f14 p2, f16 p0, f19 p1  R3 = w1 & B': f12 p4, f15 p5, f17 p3, f20 p4
//   R4 = w2 & A": f22 p2, f24 p0, f27 p1, f30 p2  R5 = w2 & B": f23 p5, f25 p3, f28 p4, f31 p5
//   R6 = (run >> 6)  : f2 p0, f5 p1, -, f10 p0    R7 = (run >> 38): f13 p1, -, f18 p0, f21 p1
//   R8 = (run >> 70) : -, f26 p0, f29 p1, -
// Step s multiplies (R[2s], R[2s+1]); the fifth step has only R8.
struct IT3 {
    static constexpr int kSteps = 5, kPre = 5;
    static constexpr uint32_t m(int p0, int p1, int p2, int p3) {
        return (p0 < 0 ? 0u : 7u << p0) | (p1 < 0 ? 0u : 7u << (8 + p1)) | (p2 < 0 ? 0u : 7u << (16 + p2)) |
               (p3 < 0 ? 0u : 7u << (24 + p3));
    }
    __device__ static __forceinline__ void unpack(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t (&r)[9]) {
        r[0] = w0 & m(0, 1, 2, 0); r[1] = w0 & m(3, 4, 5, 3);
        r[2] = w1 & m(1, 2, 0, 1); r[3] = w1 & m(4, 5, 3, 4);
        r[4] = w2 & m(2, 0, 1, 2); r[5] = w2 & m(5, 3, 4, 5);
        r[6] = __funnelshift_r(w0, w1, 6) & m(0, 1, -1, 0);
        r[7] = __funnelshift_r(w1, w2, 6) & m(1, -1, 0, 1);
        r[8] = (w2 >> 6) & m(-1, 0, 1, -1);
    }
    // items j = 0..2 fill step j; item 3 holds the eight straddling fields, which fill steps 3 and 4
    __device__ static __forceinline__ void item_rows(int j, int t, int (&row)[8], int (&pre)[8]) {
        constexpr unsigned long long F0 = pack8b({{0, 3, 6, 8, 1, 4, 7, 9}}), P0 = pack8b({{0, 1, 2, 0, 3, 4, 5, 3}});
        constexpr unsigned long long F1 = pack8b({{11, 14, 16, 19, 12, 15, 17, 20}}), P1 = pack8b({{1, 2, 0, 1, 4, 5, 3, 4}});
        constexpr unsigned long long F2 = pack8b({{22, 24, 27, 30, 23, 25, 28, 31}}), P2 = pack8b({{2, 0, 1, 2, 5, 3, 4, 5}});
        constexpr unsigned long long F3 = pack8b({{2, 5, 10, 13, 18, 21, 26, 29}}), P3 = pack8b({{0, 1, 0, 1, 0, 1, 0, 1}});
        const unsigned long long f = j == 0 ? F0 : (j == 1 ? F1 : (j == 2 ? F2 : F3));
        const unsigned long long p = j == 0 ? P0 : (j == 1 ? P1 : (j == 2 ? P2 : P3));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            row[i] = 32 * t + (int)((f >> (8 * i)) & 0xffu);
            pre[i] = 5 - (int)((p >> (8 * i)) & 0xffu);
        }
    }
    // cur[i] = columns 4g..4g+3 of word-row 3t + i
    __device__ static __forceinline__ void compute(const uint4 (&cur)[3], const uint8_t* __restrict__ xb, bool has_x,
                                                   int (&da)[4], int (&db)[4]) {
        uint2 bx[5];
#pragma unroll
        for (int s = 0; s < 5; ++s) {
            bx[s] = make_uint2(0u, 0u);
            if (has_x) bx[s] = *reinterpret_cast<const uint2*>(xb + s * 128);
        }
#pragma unroll
        for (int cp = 0; cp < 2; ++cp) {
            uint32_t ra[9], rb[9];
            if (cp == 0) { unpack(cur[0].x, cur[1].x, cur[2].x, ra); unpack(cur[0].y, cur[1].y, cur[2].y, rb); }
            else         { unpack(cur[0].z, cur[1].z, cur[2].z, ra); unpack(cur[0].w, cur[1].w, cur[2].w, rb); }
            int (&d)[4] = cp == 0 ? da : db;
            int e[4] = {0, 0, 0, 0};
            imma(d, ra[0], rb[0], ra[1], rb[1], bx[0].x, bx[0].y);
            imma(e, ra[2], rb[2], ra[3], rb[3], bx[1].x, bx[1].y);
            imma(d, ra[4], rb[4], ra[5], rb[5], bx[2].x, bx[2].y);
            imma(e, ra[6], rb[6], ra[7], rb[7], bx[3].x, bx[3].y);
            imma(d, ra[8], rb[8], 0u, 0u, bx[4].x, 0u);
#pragma unroll
            for (int r = 0; r < 4; ++r) d[r] += e[r];
        }
    }
};
// bytes of one unit's B operands in shared memory: [step][quad lane][plane][b0, b1]
constexpr int kIntUnitBytes = IT3::kSteps * 4 * 32;

struct Plan {
    int cgs;          // column groups (256 columns each) = clusters
    int kbs;          // units per column group
    int cluster;      // CTAs per cluster: the column group's K range is split evenly among them
    int stage_units;  // units whose x values are staged in shared memory at a time
    int ring_units;   // unit buffers in the shared-memory ring
    int group_box;    // groups of scales / zero-points held per stage (rows of the scales TMA box)
    int push;         // 1: the K slices are combined by pushing partial sums into the first CTA's shared memory
    int xfull;        // x is bulk-copied to shared memory before it is re-ordered (the whole of x for layers with x_perm,
                      // the CTA's rows otherwise): 2 into bytes of its own, 1 into the bytes of the partial sums, 0 not
    int early;        // when dependents may be launched: 0 once this CTA has passed its own wait, 1 as soon as it runs,
                      // 2 once all its weights are requested
    int xact;         // activation applied to x as it is read: 0 none, 1 SwiGLU (x holds [gate | up], 2 K values per
                      // row), 2 ReLU -- the element-wise kernel between two linears of a decode step folded into the second
};

// The two activations, rounded exactly like the stand-alone kernel (b200gptq_act): SiLU to fp16, then the product.
__device__ __forceinline__ unsigned short act_relu(unsigned short h) {
    return __half_as_ushort(__float2half_rn(fmaxf(__half2float(__ushort_as_half(h)), 0.f)));
}
__device__ __forceinline__ unsigned short act_swiglu(unsigned short g, unsigned short u) {
    const float gf = __half2float(__ushort_as_half(g));
    const float s = __half2float(__float2half_rn(gf / (1.f + __expf(-gf))));
    return __half_as_ushort(__float2half_rn(s * __half2float(__ushort_as_half(u))));
}

template <int BITS> __host__ __device__ constexpr int unit_bytes() { return Traits<BITS>::kWordRows * kRowPitch; }
// Dynamic shared memory, in this order: ring | xs | s_sm | z_sm | ps | part | red
// x as staged for the tensor instructions: fp16 fragments (several rows of x) or byte planes (one row)
__host__ __device__ inline int xs_bytes(int S, int M) { return S * M * 256; }
// The integer path pays for a longer preparation of x with a shorter loop: measured on B200 it wins for 3-bit layers
// (8.2 against 8.6 us on the 4096 x 11008 benchmark layer) and loses for 4-bit ones, whose fp16 unpacking is cheap
// (5.5 against 5.0 us on 4096 x 4096).
template <int BITS> __host__ __device__ constexpr bool int_path(int M) { return M == 1 && BITS == 3; }
template <int BITS> __host__ __device__ constexpr int xs_total(int S, int M) {
    return int_path<BITS>(M) ? S * kIntUnitBytes : xs_bytes(S, M);
}
__host__ __device__ inline int s_sm_bytes(int gbox) { return gbox * kCgCols * 2; }
__host__ __device__ inline int z_sm_bytes(int gbox) { return gbox * kCgCols; }
__host__ __device__ inline int ps_bytes(int S, int M) { return (S * M * 8 + 15) & ~15; }
__host__ __device__ inline int part_bytes(int M) { return M * kCgCols * 4; }
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

// One cluster per column group; CTA `rank` of the cluster owns units [rank*kbs/C, (rank+1)*kbs/C).
// MULTI = false is the single-row instantiation (M == 1, the decode case that is timed): every loop over the
// rows of x folds away and the CTA is small enough for three per SM.
// PERM = false is the instantiation for layers whose x needs no gather (x_perm == NULL).
// XACT: the activation applied to x as it is read (Plan::xact), a template parameter because a run-time test per
// element of x on the path between the dependency wait and the first product costs 3 % of a decode step.
template <int BITS, bool MULTI, bool PERM, int XACT>
__global__ void __launch_bounds__(kThreads, MULTI ? 2 : 3)
gemv_stream_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_s,
                   const __half* x, const int32_t* __restrict__ qzeros, const int32_t* __restrict__ x_perm,
                   const __half* __restrict__ bias, __half* __restrict__ y, int M_rows, int K, int N,
                   int group_size, Plan plan, unsigned int* __restrict__ status, const __grid_constant__ TpArgs tp) {
    const int M = MULTI ? M_rows : 1;
    constexpr bool INT = int_path<BITS>(MULTI ? 2 : 1);   // products on the integer tensor path
    constexpr int MM = MULTI ? kMaxM : 1;
    using T = Traits<BITS>;
    constexpr int UB = unit_bytes<BITS>();

    extern __shared__ __align__(128) uint8_t dsm[];
    __shared__ __align__(8) uint64_t bars[kMaxRing + 3];   // full[R] at 0, scales, combine, whole-x copy
    __shared__ unsigned int taken[kMaxRing];               // warps that have moved the unit in a ring slot to registers
    __shared__ volatile int gave_up;
    __shared__ unsigned int tp_epoch;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int R = plan.ring_units, C = plan.cluster, S = plan.stage_units, GB = plan.group_box;
    const int cg = blockIdx.x / C, rank = blockIdx.x - cg * C;
    const int kb_begin = (int)(((long long)rank * plan.kbs) / C), kb_end = (int)(((long long)(rank + 1) * plan.kbs) / C);
    const bool refill = kb_end - kb_begin > R;   // the slice does not fit the ring: slots are re-used
    const bool push = plan.push != 0;
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    const uint32_t s_bar = bar_base + 8u * kMaxRing, red_bar = bar_base + 8u * (kMaxRing + 1);
    const uint32_t x_bar = bar_base + 8u * (kMaxRing + 2);

    // the swizzle pattern is a function of the address: the ring starts on a 1024-byte boundary
    uint8_t* ring = dsm + ((1024u - (smem_u32(dsm) & 1023u)) & 1023u);
    uint32_t* xs = reinterpret_cast<uint32_t*>(ring + (size_t)R * UB);
    const __half* s_sm = reinterpret_cast<const __half*>(reinterpret_cast<uint8_t*>(xs) + xs_total<BITS>(S, M));
    uint8_t* z_sm = reinterpret_cast<uint8_t*>(xs) + xs_total<BITS>(S, M) + s_sm_bytes(GB);
    float2* ps = reinterpret_cast<float2*>(z_sm + z_sm_bytes(GB));       // (sum x, sum c*x) per (unit, x row)
    // `part` / `red` hold partial sums at the end of the kernel; before that the same bytes hold the whole of x
    // while it is gathered (PERM with plan.xfull): the other CTAs of the cluster store into `red` only after this
    // CTA has arrived at the cluster barrier, which it does once its last fragment of x is staged.
    float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(ps) + ps_bytes(S, M));
    float* red = part + M * kCgCols;
    // x as copied from global memory: the whole of x for layers with a gather, the CTA's own rows otherwise; either
    // in bytes of its own behind `red` (plan.xfull == 2) or, when it is larger, in the bytes of `part` / `red`
    const bool use_xfull = plan.xfull != 0;
    const bool xfull_aliased = plan.xfull == 1;
    const unsigned short* xfull = reinterpret_cast<const unsigned short*>(
        xfull_aliased ? part : red + (plan.push ? (plan.cluster - 1) * M * kCgCols : 0));
    const int xrow_halves = PERM ? K : (kb_end - kb_begin) * kUnitRows;    // halves per row of x in the copy
    const int xrow_first = PERM ? 0 : kb_begin * kUnitRows;                // first row of K held by the copy

    const int units_per_group = group_size / kUnitRows;

    // Copy unit `kb` of this CTA's column group into ring slot `slot`: one TMA box of kWordRows x 256 words
    // (columns past N are filled with zeros and count towards the expected bytes like the rest).
    auto issue_unit = [&](int kb, int slot) {
        mbar_arrive_expect_tx(full_bar(slot), (uint32_t)UB);
        tma_load_3d(smem_u32(ring) + slot * UB, &tmap_w, 0, kb * T::kWordRows, cg * (kCgCols / 32), full_bar(slot));
    };
    auto issue_scales = [&](int g0) {
        mbar_arrive_expect_tx(s_bar, (uint32_t)s_sm_bytes(GB));
        tma_load_2d(smem_u32(s_sm), &tmap_s, cg * kCgCols, g0, s_bar);
    };

    if (tid == 0) {
        gave_up = 0;
        for (int s = 0; s < R; ++s) mbar_init(full_bar(s), 1);   // the expect_tx arrive of the thread that issues the copy
        mbar_init(s_bar, 1);
        mbar_init(red_bar, 1);
        mbar_init(x_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        // Weights and scales are constants: they are requested before the dependency on the previous kernel is awaited.
        issue_scales((kb_begin * kUnitRows) / group_size);
        for (int u = 0; u < R && kb_begin + u < kb_end; ++u) issue_unit(kb_begin + u, u);
        // the first CTA of the cluster expects one float per (other CTA, x row, column)
        if (push && rank == 0) mbar_arrive_expect_tx(red_bar, (uint32_t)red_bytes(M, C));
    }
    if (tid < kMaxRing) taken[tid] = 0u;
    __syncthreads();
    // matched by the wait in front of the first store into another CTA; a CTA that gathers x through `part` / `red`
    // arrives only when it has finished with those bytes
    if (push && !xfull_aliased) cluster_arrive();
    if (plan.early == 1) asm volatile("griddepcontrol.launch_dependents;");

    const int g = lane >> 2, j = lane & 3;
    const int lane_col = warp * 32 + 4 * g;  // first of the lane's 4 columns inside the column group
    // byte offsets of the lane's vecs inside a unit: line L = chunk (= warp) * word-rows + word-row, piece g ^ (L & 7)
    uint32_t vec_off[T::kVecs];
#pragma unroll
    for (int r = 0; r < T::kVecs; ++r) {
        const uint32_t L = (uint32_t)(warp * T::kWordRows + T::vec_row(j, r));
        vec_off[r] = L * 128u + (((uint32_t)g ^ (L & 7u)) << 4);
    }

    // several rows of x: this lane's columns (2cp, 2cp+1) x rows of x (2j, 2j+1), scaled; one row: out[0][c] is this
    // lane's pair of planes of column 4g + c
    float out[2][4];
#pragma unroll
    for (int cp = 0; cp < 2; ++cp)
#pragma unroll
        for (int r = 0; r < 4; ++r) out[cp][r] = 0.f;
    const float plane_weight = j == 0 ? 1.f : (j == 1 ? 65536.f : 0.f);   // one row: quad lane j holds planes 2j, 2j+1
    float corr[MM];    // column `tid`: offset / zero-point term of every row of x
#pragma unroll
    for (int m = 0; m < MM; ++m) corr[m] = 0.f;

    // zero-point field of column `tid`
    const int zn = min(cg * kCgCols + tid, N - 1);
    const int zwords = N / 32 * BITS;
    int zw, zsh;
    if constexpr (BITS == 3) {
        const int bit = 3 * (zn & 31);
        zw = 3 * (zn >> 5) + (bit >> 5); zsh = bit & 31;
    } else {
        zw = zn >> 3; zsh = 4 * (zn & 7);
    }
    const bool zstr = BITS == 3 && zsh > 29;   // the field straddles two words

    const unsigned short* xu = reinterpret_cast<const unsigned short*>(x);
    // x[m, k] as the products see it (k: row of K after the gather)
    auto load_x = [&](int m, int k) -> unsigned short {
        if constexpr (XACT == 1) {
            const unsigned short* row = xu + (size_t)m * 2 * K;
            return act_swiglu(__ldcg(row + k), __ldcg(row + K + k));
        } else {
            const unsigned short h = use_xfull ? xfull[m * xrow_halves + k - xrow_first] : __ldcg(xu + (size_t)m * K + k);
            return XACT == 2 ? act_relu(h) : h;
        }
    };

    int slot = 0, round = 0;
    bool first = true, triggered = false;
    for (int kb_a = kb_begin, st = 0; kb_a < kb_end; kb_a += S, ++st) {
        const int kb_b = min(kb_a + S, kb_end);
        const int nu = kb_b - kb_a;
        const int g0 = (kb_a * kUnitRows) / group_size;
        const int ng = (kb_b * kUnitRows - 1) / group_size - g0 + 1;
        if (!first) {
            __syncthreads();   // the previous stage's fragments, scales and sums are no longer in use
            if (tid == 0) issue_scales(g0);
        }
        // ---- zero-points of this stage's groups (column tid), eight loads in flight at a time ----
        {
            const uint32_t* zp = reinterpret_cast<const uint32_t*>(qzeros) + (size_t)g0 * zwords + zw;
#pragma unroll 1
            for (int gb = 0; gb < ng; gb += 8) {
                uint32_t lo[8], hi[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    lo[i] = 0u; hi[i] = 0u;
                    if (gb + i < ng) {
                        lo[i] = __ldg(zp + (size_t)(gb + i) * zwords);
                        if (zstr) hi[i] = __ldg(zp + (size_t)(gb + i) * zwords + 1);
                    }
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (gb + i < ng) {
                        uint32_t q;
                        if constexpr (BITS == 3) q = __funnelshift_r(lo[i], hi[i], zsh) & 7u;
                        else q = (lo[i] >> zsh) & 15u;
                        z_sm[(gb + i) * kCgCols + tid] = (uint8_t)(q + 1u);   // the reference's unmasked "+1"
                    }
            }
        }
        // Everything before this point uses constants only.  x is the one operand a preceding kernel may still be
        // writing: under programmatic dependent launch `await_x` is where the kernel waits for it, with its ring,
        // scales, zero-points and gather indices requested.
        auto await_x = [&]() {
            asm volatile("griddepcontrol.wait;" ::: "memory");
            if (plan.early == 0) asm volatile("griddepcontrol.launch_dependents;");
            if (use_xfull) {
                // A gather straight from global memory would send every CTA's 2-byte requests to the same few
                // L2 lines at the same moment; one linear bulk copy of x per CTA and a gather from shared memory
                // costs the L2 a twelfth of the requests.
                if (tid == 0) {
                    const uint32_t row_bytes = (uint32_t)(xrow_halves * 2);
                    mbar_arrive_expect_tx(x_bar, row_bytes * (uint32_t)M);
                    for (int mm = 0; mm < M; ++mm)
                        asm volatile(
                            "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                            ::"r"(smem_u32(xfull) + mm * row_bytes), "l"(x + (size_t)mm * K + xrow_first),
                              "r"(row_bytes), "r"(x_bar) : "memory");
                }
                mbar_wait(x_bar, 0, &gave_up);
            }
        };
        if constexpr (!INT) {
            // ---- x: fragment pieces of 8 halves, one per thread and pass ----
            const int items = nu * M * 16;
    #pragma unroll 1
            for (int q0 = 0; q0 < items; q0 += kThreads) {
                const int q = q0 + tid;
                const bool active = q < items;
                const int um = q >> 4;
                const int u = MULTI ? um / M : um, m = MULTI ? um - u * M : 0;
                int rr[8], pos[8];
                T::piece_rows((q >> 2) & 3, q & 3, rr, pos);
                const int row0 = (kb_a + u) * kUnitRows;
                int kx[8];
    #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    kx[i] = row0 + rr[i];
                    if (PERM && active) kx[i] = __ldg(x_perm + kx[i]);
                }
                if (first && q0 == 0) {
                    await_x();
                }
                unsigned short xv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) xv[i] = active ? load_x(m, kx[i]) : (unsigned short)0;
                float sx = 0.f, scx = 0.f;
    #pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float xf = __half2float(__ushort_as_half(xv[i]));
                    sx += xf;
                    scx = fmaf(__int_as_float((137 - pos[i]) << 23), xf, scx);   // 2^(10 - pos)
                }
                if (active) {
                    uint4 piece;
                    piece.x = (uint32_t)xv[0] | ((uint32_t)xv[1] << 16);
                    piece.y = (uint32_t)xv[2] | ((uint32_t)xv[3] << 16);
                    piece.z = (uint32_t)xv[4] | ((uint32_t)xv[5] << 16);
                    piece.w = (uint32_t)xv[6] | ((uint32_t)xv[7] << 16);
                    *reinterpret_cast<uint4*>(xs + 4 * q) = piece;
                }
                // the 16 pieces of one (unit, x row) sit in 16 adjacent lanes
    #pragma unroll
                for (int o = 1; o < 16; o <<= 1) {
                    sx += __shfl_xor_sync(0xffffffffu, sx, o);
                    scx += __shfl_xor_sync(0xffffffffu, scx, o);
                }
                if (active && (lane & 15) == 0) ps[um] = make_float2(sx, scx);
            }
        } else {
            // ---- x, one row: fixed point per unit, four signed byte planes in the order of the B operand.  Item
            //      q = 16 u + 4 j + t of the stage: unit u, quad lane t, part j (8 rows); the 16 items of a unit sit
            //      in 16 adjacent lanes ----
            using I = IT3;
            const int items = nu * 16;
#pragma unroll 1
            for (int q0 = 0; q0 < items; q0 += kThreads) {
                const int q = q0 + tid;
                const bool active = q < items;
                const int u = q >> 4, jq = (q >> 2) & 3, tq = q & 3;
                int rr[8], pre[8];
                I::item_rows(jq, tq, rr, pre);
                const int row0 = (kb_a + u) * kUnitRows;
                int kx[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    kx[i] = row0 + rr[i];
                    if (PERM && active) kx[i] = __ldg(x_perm + kx[i]);
                }
                if (first && q0 == 0) await_x();
                float xf[8];
                unsigned int mx = 0u;   // bits of the largest |x|: the order of non-negative floats, NaN above infinity
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    unsigned short h = 0;
                    if (active) h = load_x(0, kx[i]);
                    xf[i] = __half2float(__ushort_as_half(h));
                    mx = max(mx, __float_as_uint(fabsf(xf[i])));
                }
#pragma unroll
                for (int o = 1; o < 16; o <<= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                // 2^ex > max |x| of the unit; X = x * 2^(148 - ex) has |X| < 2^22.  A unit of zeros takes any scale; a
                // unit with an infinity or a NaN gets a NaN factor, so that its columns come out as NaN.
                int ex = (int)(mx >> 23);
                const bool bad = ex == 255;
                if (ex == 0 || bad) ex = 127;
                const float scale = __uint_as_float((uint32_t)(275 - ex) << 23);
                int sum = 0;
                int dg[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // round to nearest through the fp32 adder: |x * scale| <= 2^22
                    const int X = __float_as_int(fmaf(xf[i], scale, 12582912.f)) - 0x4B400000;
                    sum += X;
                    dg[i] = ((X << pre[i]) + 0x00808080) ^ 0x00808080;   // four signed base-256 digits
                }
#pragma unroll
                for (int o = 1; o < 16; o <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                if (active) {
                    if ((lane & 15) == 0) {
                        const float delta = __uint_as_float((uint32_t)(ex - 21) << 23);   // 2^(ex - 148)
                        float cq = __uint_as_float((uint32_t)(ex - 21 - I::kPre) << 23);
                        if (bad) cq = __uint_as_float(0x7fc00000u);
                        ps[u] = make_float2(cq, delta * (float)sum);   // (factor of the plane sums, sum of x)
                    }
                    uint8_t* dst = reinterpret_cast<uint8_t*>(xs) + (size_t)u * kIntUnitBytes;
                    uint32_t lo[4], hi[4];
                    if (jq < 3) {
                        planes_of(dg[0], dg[1], dg[2], dg[3], lo);
                        planes_of(dg[4], dg[5], dg[6], dg[7], hi);
                        store_step(dst + (jq * 4 + tq) * 32, lo, hi);
                    } else {
                        planes_of(dg[0], dg[1], 0, dg[2], lo);
                        planes_of(dg[3], 0, dg[4], dg[5], hi);
                        store_step(dst + (3 * 4 + tq) * 32, lo, hi);
                        planes_of(0, dg[6], dg[7], 0, lo);
                        hi[0] = hi[1] = hi[2] = hi[3] = 0u;
                        store_step(dst + (4 * 4 + tq) * 32, lo, hi);
                    }
                }
            }
        }
        __syncthreads();   // fragments and sums are in shared memory
        first = false;
        if (push && xfull_aliased && kb_b == kb_end) cluster_arrive();

        // ---- the units of this stage ----
        int gl = 0;                                                            // group of the current unit, relative to g0
        int left = units_per_group - (kb_a - (kb_a / units_per_group) * units_per_group);
        const uint32_t* bsm = xs + (size_t)(g * 4 + j) * 16;
        const int bsm_step = M * 64;
        bool scales_ready = false;
#pragma unroll 1
        for (int kb = kb_a; kb < kb_b; ++kb) {
            if (plan.early == 2 && !triggered && kb + R >= kb_end) {
                // every unit of this CTA has been requested: CTAs of the next launch may come in and queue their
                // weights behind it without delaying it
                asm volatile("griddepcontrol.launch_dependents;");
                triggered = true;
            }
            mbar_wait(full_bar(slot), round & 1, &gave_up);
            uint4 cur[T::kVecs];
            const uint8_t* src = ring + slot * UB;
#pragma unroll
            for (int r = 0; r < T::kVecs; ++r) cur[r] = *reinterpret_cast<const uint4*>(src + vec_off[r]);
            // The unit is on its way to registers.  When slots are re-used each warp counts itself in; the last one
            // refills the slot with the unit R further on (nobody waits for anybody).  The count is looked at after
            // the products, so that its round trip through shared memory is not waited for.
            unsigned int before = 0u;
            if (refill) {
                __syncwarp();
                if (lane == 0) before = atomicAdd(&taken[slot], 1u);
            }
            const int done_slot = slot;
            if (++slot == R) { slot = 0; ++round; }
            float d[4][4];
            int da[4] = {0, 0, 0, 0}, db[4] = {0, 0, 0, 0};
            if constexpr (!INT) T::compute(cur, bsm, g < M, d);
            else IT3::compute(cur, reinterpret_cast<const uint8_t*>(xs) + (size_t)(kb - kb_a) * kIntUnitBytes + j * 32 + g * 8,
                                   g < 4, da, db);
            if (refill) {
                before = __shfl_sync(0xffffffffu, before, 0);
                if (before == kWarps - 1 && lane == 0) {
                    taken[done_slot] = 0u;
                    if (kb + R < kb_end) issue_unit(kb + R, done_slot);
                }
            }
            bsm += bsm_step;
            if (!scales_ready) { mbar_wait(s_bar, st & 1, &gave_up); scales_ready = true; }
            // out += scale[group] * d for the lane's 4 columns
            const uint2 sv = *reinterpret_cast<const uint2*>(s_sm + gl * kCgCols + lane_col);
            const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sv.x));
            const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sv.y));
            if constexpr (!INT) {
                out[0][0] = fmaf(s01.x, d[0][0] + d[2][0], out[0][0]); out[0][1] = fmaf(s01.x, d[0][1] + d[2][1], out[0][1]);
                out[0][2] = fmaf(s01.y, d[0][2] + d[2][2], out[0][2]); out[0][3] = fmaf(s01.y, d[0][3] + d[2][3], out[0][3]);
                out[1][0] = fmaf(s23.x, d[1][0] + d[3][0], out[1][0]); out[1][1] = fmaf(s23.x, d[1][1] + d[3][1], out[1][1]);
                out[1][2] = fmaf(s23.y, d[1][2] + d[3][2], out[1][2]); out[1][3] = fmaf(s23.y, d[1][3] + d[3][3], out[1][3]);
            } else {
                // recombine this lane's two planes (sums S_p of plane p: 256^p S_p), scale by the unit's factor and the group's scale
                const float c = ps[kb - kb_a].x * plane_weight;
                out[0][0] = fmaf(s01.x * c, fmaf(256.f, small_int_to_float(da[1]), small_int_to_float(da[0])), out[0][0]);
                out[0][1] = fmaf(s01.y * c, fmaf(256.f, small_int_to_float(da[3]), small_int_to_float(da[2])), out[0][1]);
                out[0][2] = fmaf(s23.x * c, fmaf(256.f, small_int_to_float(db[1]), small_int_to_float(db[0])), out[0][2]);
                out[0][3] = fmaf(s23.y * c, fmaf(256.f, small_int_to_float(db[3]), small_int_to_float(db[2])), out[0][3]);
            }
            if (--left == 0) { ++gl; left = units_per_group; }
        }

        // ---- offset / zero-point term of this stage for column tid: sum_units s * (sum c x + zero * sum x) ----
        {
            int gc = 0;
            int lc = units_per_group - (kb_a - (kb_a / units_per_group) * units_per_group);
#pragma unroll 1
            for (int u = 0; u < nu; ++u) {
                const float sg = __half2float(s_sm[gc * kCgCols + tid]);
                const float zg = (float)z_sm[gc * kCgCols + tid];
#pragma unroll
                for (int m = 0; m < MM; ++m)
                    if (m < M) {
                        const float2 p = ps[u * M + m];
                        if constexpr (!INT) corr[m] = fmaf(sg, fmaf(zg, p.x, p.y), corr[m]);
                        else corr[m] = fmaf(sg * zg, p.y, corr[m]);   // one row: zero * sum x
                    }
                if (--lc == 0) { ++gc; lc = units_per_group; }
            }
        }
    }

    // ---- this CTA's partial result: lane layout -> one column per thread, minus the offset term ----
    if constexpr (!INT) {
#pragma unroll
        for (int cp = 0; cp < 2; ++cp)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int m = 2 * j + (r & 1);
                if (m < M) part[m * kCgCols + lane_col + 2 * cp + (r >> 1)] = out[cp][r];
            }
    } else {
        // one row: the quad's lanes hold different planes of the same four columns
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            float v = out[0][c];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            out[0][c] = v;
        }
        if (j == 0) *reinterpret_cast<float4*>(part + lane_col) = make_float4(out[0][0], out[0][1], out[0][2], out[0][3]);
    }
    __syncthreads();
    const int n = cg * kCgCols + tid;
    // The column group's sums over all of K end up in v[] of ONE CTA (the only one of a group, or the cluster's
    // first); `finish` adds the other ranks' sums (tensor-parallel row shards) and the bias and writes y.
    auto finish = [&](float (&v)[MM]) {
        if (tp.world > 1) tp_exchange_group<MM>(tp, cg, tid, M, v, &tp_epoch);
        if (n < N) {
#pragma unroll
            for (int m = 0; m < MM; ++m)
                if (m < M) {
                    float o = v[m];
                    if (bias) o += __half2float(bias[n]);
                    y[(size_t)m * N + n] = __float2half_rn(o);
                }
        }
    };
    float v[MM];
    if (C == 1) {
#pragma unroll
        for (int m = 0; m < MM; ++m) v[m] = m < M ? part[m * kCgCols + tid] - corr[m] : 0.f;
        finish(v);
        if (tid == 0 && gave_up) atomicExch(status + kStatusWord, 1u);
        return;
    }
    if (push) {
        // ---- push combine: the other CTAs are done once their stores are issued (nothing reads their shared
        //      memory); the first CTA waits for all of them on its barrier and adds them up in rank order ----
        cluster_wait();   // every CTA of the cluster is running and has initialised its barriers
        if (rank > 0) {
#pragma unroll
            for (int m = 0; m < MM; ++m)
                if (m < M)
                    st_async_cluster_f32(red + ((rank - 1) * M + m) * kCgCols + tid, red_bar, 0u,
                                         part[m * kCgCols + tid] - corr[m]);
        } else {
            mbar_wait(red_bar, 0, &gave_up);
#pragma unroll
            for (int m = 0; m < MM; ++m) {
                v[m] = 0.f;
                if (m < M) {
                    v[m] = part[m * kCgCols + tid] - corr[m];
                    for (int r = 1; r < C; ++r) v[m] += red[((r - 1) * M + m) * kCgCols + tid];
                }
            }
            finish(v);
        }
        if (tid == 0 && gave_up) atomicExch(status + kStatusWord, 1u);
        return;
    }
    // ---- combine the K slices of the cluster through distributed shared memory, in rank order ----
    if (MULTI) {
#pragma unroll
        for (int m = 0; m < MM; ++m)
            if (m < M) part[m * kCgCols + tid] -= corr[m];   // column tid is this thread's own
        cluster_sync_all();   // every CTA's partial result is in its `part`
        if (rank == 0) {
#pragma unroll
            for (int m = 0; m < MM; ++m) {
                v[m] = 0.f;
                if (m < M) {
                    // all remote reads are issued before the first is used; the sum stays in rank order
                    float rem[8];
#pragma unroll
                    for (int r = 1; r < 8; ++r) rem[r] = r < C ? ld_cluster_f32(&part[m * kCgCols + tid], (uint32_t)r) : 0.f;
                    v[m] = part[m * kCgCols + tid];
#pragma unroll
                    for (int r = 1; r < 8; ++r) v[m] += rem[r];
                }
            }
            finish(v);
        }
        cluster_sync_all();   // the other CTAs keep their shared memory alive until it has been read
    }
    if (tid == 0 && gave_up) atomicExch(status + kStatusWord, 1u);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static const EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

constexpr int kSmemPerSm = 227 * 1024;   // shared memory an SM can give to its CTAs
constexpr int kSmemCtaReserve = 1024;    // and what the system takes per resident CTA

// Largest group count any stage of any CTA touches.
int max_groups_per_stage(const Plan& p, int group_size) {
    int best = 1;
    for (int r = 0; r < p.cluster; ++r) {
        const int a = (int)(((long long)r * p.kbs) / p.cluster), b = (int)(((long long)(r + 1) * p.kbs) / p.cluster);
        for (int s = a; s < b; s += p.stage_units) {
            const int e = s + p.stage_units < b ? s + p.stage_units : b;
            const int ng = (e * kUnitRows - 1) / group_size - (s * kUnitRows) / group_size + 1;
            if (ng > best) best = ng;
        }
    }
    return best;
}

// knobs (all optional, 0 = the default): [0] CTAs of one grid per SM that the cluster size is chosen for,
// [1] CTAs per SM that the shared-memory footprint is sized for, [2] cap on ring units, [3] trigger of dependents
// (1 after the own wait, 2 at entry, 3 once all weights are requested), [4] 1 = gather x from global memory,
// [5] activation applied to x as it is read (Plan::xact)
// Clusters of `cluster` CTAs with `smem_bytes` of dynamic shared memory that the device holds at once (0: unknown).
// Answers are kept per thread: a plan is made once per layer, a direct call asks on every launch.
int resident_clusters(const void* kernel, int cluster, int smem_bytes) {
    struct Entry { const void* kernel; int dev, cluster, smem, answer; };
    thread_local Entry cache[16];
    thread_local int used = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    for (int i = 0; i < used; ++i)
        if (cache[i].kernel == kernel && cache[i].dev == dev && cache[i].cluster == cluster && cache[i].smem == smem_bytes)
            return cache[i].answer;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cluster * 1024);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { (void)cudaGetLastError(); n = 0; }
    if (used < 16) cache[used++] = Entry{kernel, dev, cluster, smem_bytes, n};
    return n;
}

template <int BITS> const void* kernel_for(bool multi, bool perm, int xact);
template <int BITS> int set_smem_attr_once();

template <int BITS>
Plan make_plan(int M, int K, int N, int group_size, bool has_perm, const int* knobs, int* smem_bytes) {
    Plan p;
    p.cgs = (N + kCgCols - 1) / kCgCols;
    p.kbs = K / kUnitRows;
    // Cluster size: as many K slices as give the grid about three CTAs per SM (two with several rows of x), at
    // most 8: measured on B200, more and shorter slices beat fewer and longer ones.
    const int grid_per_sm = (knobs && knobs[0] > 0) ? knobs[0] : (M == 1 ? 3 : 2);
    int c = (grid_per_sm * sm_count()) / p.cgs;
    if (c > 8) c = 8;
    if (c > p.kbs) c = p.kbs;
    if (c < 1) c = 1;
    p.cluster = c;
    const int longest = (p.kbs + c - 1) / c;
    p.stage_units = int_path<BITS>(M) ? kXsBytes / kIntUnitBytes : kXsBytes / (M * 256);
    if (p.stage_units > longest) p.stage_units = longest;
    p.group_box = max_groups_per_stage(p, group_size);
    p.push = (c > 1 && red_bytes(M, c) <= kMaxRedBytes) ? 1 : 0;
    p.early = (knobs && knobs[3] > 0) ? knobs[3] - 1 : 0;
    p.xact = knobs ? knobs[5] : 0;
    // layers with a gather, and several rows of x, take x through linear bulk copies when it is small enough
    // (knobs[4] == 1 switches it off): small copies get bytes of their own, larger ones share the bytes of the partial
    // sums (the CTA then joins its cluster's barrier only when it has finished with x).  One row without a gather: a
    // CTA reads only its own rows of x, and plain loads measured faster than the copy; with M rows the 2-byte loads
    // of all CTAs queue up at the same L2 lines (8 rows of a 4096 x 12288 layer: 27 us with loads).
    const int xcopy_bytes = M * (has_perm ? K : longest * kUnitRows) * 2;
    p.xfull = ((!has_perm && M == 1) || (knobs && knobs[4] == 1)) ? 0 : (xcopy_bytes <= 4096 ? 2 : (xcopy_bytes <= kXFullMax ? 1 : 0));
    if (p.xact == 1) p.xfull = 0;   // gate and up are two runs of the row: no single copy (callers fuse SwiGLU only without a gather)
    int tail = part_bytes(M) + (p.push ? red_bytes(M, c) : 0);
    if (p.xfull == 2) tail += xcopy_bytes;
    if (p.xfull == 1 && tail < xcopy_bytes) tail = xcopy_bytes;
    const int fixed = xs_total<BITS>(p.stage_units, M) + s_sm_bytes(p.group_box) + z_sm_bytes(p.group_box) +
                      ps_bytes(p.stage_units, M) + tail + 1024;
    // Footprint (CTAs per SM that the shared memory is sized for).  A launch should be resident at once: clusters are
    // placed inside one GPC, so whether `cgs` clusters of `c` CTAs fit is asked of the occupancy calculator, not
    // computed from the SM count (36 clusters of 8 do not fit at two CTAs per SM, 36864 x 9216: 73 -> 55 us at
    // three).  Among footprints with the same number of waves the one with the longer ring wins, then the
    // smaller one (CTAs of the next launch of the stream find room beside the running ones and fetch their weights
    // early).
    int fit_per_sm = 0;
    if (knobs && knobs[1] > 0) fit_per_sm = knobs[1];
    else {
        // (the calculator needs the kernels' shared-memory limit raised first)
        const void* kernel = set_smem_attr_once<BITS>() == B200GPTQ_OK ? kernel_for<BITS>(M > 1, has_perm, p.xact) : nullptr;
        int best_waves = 0, best_ring = 0;
        for (int f = (M == 1 ? 4 : 3); f >= 2; --f) {
            int r = (kSmemPerSm / f - kSmemCtaReserve - fixed) / unit_bytes<BITS>();
            if (r > longest) r = longest;
            if (r > kMaxRing) r = kMaxRing;
            if (r < 2) continue;
            const int resident = kernel ? resident_clusters(kernel, c, r * unit_bytes<BITS>() + fixed) : 0;
            if (resident <= 0) { fit_per_sm = 0; break; }
            const int waves = (p.cgs + resident - 1) / resident;
            if (!fit_per_sm || waves < best_waves || (waves == best_waves && r > best_ring)) {
                fit_per_sm = f; best_waves = waves; best_ring = r;
            }
        }
        if (!fit_per_sm)   // no answer from the calculator: the largest footprint count that holds the whole slice
            for (int f = (M == 1 ? 3 : 2); f >= 2 && !fit_per_sm; --f)
                if (fixed + longest * unit_bytes<BITS>() <= kSmemPerSm / f - kSmemCtaReserve) fit_per_sm = f;
    }
    if (!fit_per_sm) fit_per_sm = 2;
    const int budget = kSmemPerSm / fit_per_sm - kSmemCtaReserve;
    int ring = (budget - fixed) / unit_bytes<BITS>();
    if (knobs && knobs[2] > 0 && ring > knobs[2]) ring = knobs[2];
    if (ring > longest) ring = longest;
    if (ring > kMaxRing) ring = kMaxRing;
    if (ring < 2) ring = 2;
    p.ring_units = ring;
    *smem_bytes = ring * unit_bytes<BITS>() + fixed;   // `fixed` includes the slack to start the ring on a 1024-byte boundary
    return p;
}

// The instantiation for (several rows of x, gather, activation); SwiGLU is not built together with a gather.
template <int BITS>
const void* kernel_for(bool multi, bool perm, int xact) {
#define B200GPTQ_K(MU, PE, XA) reinterpret_cast<const void*>(gemv_stream_kernel<BITS, MU, PE, XA>)
    if (xact == 0) return multi ? (perm ? B200GPTQ_K(true, true, 0) : B200GPTQ_K(true, false, 0))
                                : (perm ? B200GPTQ_K(false, true, 0) : B200GPTQ_K(false, false, 0));
    if (xact == 2) return multi ? (perm ? B200GPTQ_K(true, true, 2) : B200GPTQ_K(true, false, 2))
                                : (perm ? B200GPTQ_K(false, true, 2) : B200GPTQ_K(false, false, 2));
    if (xact == 1 && !perm) return multi ? B200GPTQ_K(true, false, 1) : B200GPTQ_K(false, false, 1);
    return nullptr;
#undef B200GPTQ_K
}

template <int BITS>
int set_smem_attr_once() {
    static std::once_flag once[64];
    static int result[64];
    int dev = 0;
    B200GPTQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B200GPTQ_ERR_TOO_LARGE;
    std::call_once(once[dev], [dev] {
        cudaError_t e = cudaSuccess;
        auto set = [&](const void* f) {
            if (e == cudaSuccess) e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        };
        for (int multi = 0; multi < 2; ++multi)
            for (int perm = 0; perm < 2; ++perm)
                for (int xact = 0; xact < 3; ++xact)
                    if (const void* f = kernel_for<BITS>(multi != 0, perm != 0, xact)) set(f);
        result[dev] = (int)e;
    });
    if (result[dev] != 0) { set_last_cuda_error(result[dev]); return B200GPTQ_ERR_CUDA; }
    return B200GPTQ_OK;
}

// Everything about a launch that does not change from call to call: the plan, the two tensor maps (which name
// the layer's qweight and scales) and the kernel instantiation.
struct PreparedStream {
    Plan plan;
    int smem_bytes;
    int M, K, N, group_size;
    CUtensorMap tmap_w, tmap_s;
    const void* kernel;
};

template <int BITS>
int prepare_stream(PreparedStream* ps, const int32_t* qweight, const __half* scales, bool has_perm, int M, int K, int N,
                   int group_size, const int* knobs) {
    ps->plan = make_plan<BITS>(M, K, N, group_size, has_perm, knobs, &ps->smem_bytes);
    ps->M = M; ps->K = K; ps->N = N; ps->group_size = group_size;
    const EncodeTiledFn encode = encode_tiled_fn();
    if (!encode) { set_last_cuda_error((int)cudaErrorNotSupported); return B200GPTQ_ERR_CUDA; }
    {
        // qweight [K/32*bits, N] as a 3-D tensor {32 columns, word-rows, N/32 column chunks}; a box is one unit
        const cuuint64_t dims[3] = {32, (cuuint64_t)(K / 32 * BITS), (cuuint64_t)(N / 32)};
        const cuuint64_t strides[2] = {(cuuint64_t)N * sizeof(int32_t), 32 * sizeof(int32_t)};
        const cuuint32_t box[3] = {32, (cuuint32_t)Traits<BITS>::kWordRows, (cuuint32_t)(kCgCols / 32)};
        const cuuint32_t estr[3] = {1, 1, 1};
        const CUresult r = encode(&ps->tmap_w, CU_TENSOR_MAP_DATA_TYPE_INT32, 3, const_cast<int32_t*>(qweight), dims,
                                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)cudaErrorInvalidValue); return B200GPTQ_ERR_CUDA; }
    }
    {
        // scales [G, N] fp16; a box is the groups of one stage x 256 columns
        const int G = (K + group_size - 1) / group_size;
        const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)G};
        const cuuint64_t strides[1] = {(cuuint64_t)N * sizeof(__half)};
        const cuuint32_t box[2] = {(cuuint32_t)kCgCols, (cuuint32_t)ps->plan.group_box};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r = encode(&ps->tmap_s, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(scales), dims,
                                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)cudaErrorInvalidValue); return B200GPTQ_ERR_CUDA; }
    }
    ps->kernel = kernel_for<BITS>(M != 1, has_perm, ps->plan.xact);
    if (!ps->kernel) return B200GPTQ_ERR_SHAPE;   // SwiGLU together with a gather: not instantiated
    return B200GPTQ_OK;
}

template <int BITS>
int launch_prepared(const PreparedStream& ps, const __half* x, const int32_t* qzeros, const int32_t* x_perm,
                    const __half* bias, __half* y, void* workspace, cudaStream_t stream, const TpArgs* tp_args) {
    unsigned int* status = reinterpret_cast<unsigned int*>(workspace);
    if (int st = set_smem_attr_once<BITS>()) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ps.plan.cgs * ps.plan.cluster);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = ps.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ps.plan.cluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    TpArgs tp = {};
    if (tp_args) {
        if (ps.plan.cgs > kTpMaxGroups) return B200GPTQ_ERR_TOO_LARGE;
        tp = *tp_args;
    }
    int M = ps.M, K = ps.K, N = ps.N, group_size = ps.group_size;
    Plan plan = ps.plan;
    void* args[] = {const_cast<CUtensorMap*>(&ps.tmap_w), const_cast<CUtensorMap*>(&ps.tmap_s), &x, &qzeros, &x_perm,
                    &bias, &y, &M, &K, &N, &group_size, &plan, &status, &tp};
    B200GPTQ_CUDA_TRY(cudaLaunchKernelExC(&cfg, ps.kernel, args));
    return B200GPTQ_OK;
}

template <int BITS>
int launch_stream(const __half* x, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                  const int32_t* x_perm, const __half* bias, __half* y, int M, int K, int N, int group_size,
                  void* workspace, cudaStream_t stream, const int* knobs, const TpArgs* tp_args) {
    PreparedStream ps;
    if (int st = prepare_stream<BITS>(&ps, qweight, scales, x_perm != nullptr, M, K, N, group_size, knobs)) return st;
    return launch_prepared<BITS>(ps, x, qzeros, x_perm, bias, y, workspace, stream, tp_args);
}

}  // namespace

// The streaming kernel handles groups k / group_size only (no g_idx), whole units per group,
// at most 64 groups per stage of a CTA and scales rows that TMA can address (N % 8 == 0 always holds).
bool gemv_stream_supported(int M, int K, int N, int bits, int group_size) {
    (void)N;
    if (M < 1 || M > kMaxM) return false;
    if (bits == 3 || bits == 4) return group_size % kUnitRows == 0 && K % kUnitRows == 0;
    return false;
}

size_t gemv_stream_workspace_bytes(int M, int K, int N, int bits) {
    (void)M; (void)K; (void)N;
    if (bits != 3 && bits != 4) return 0;
    return kCounterBytes;  // only the status word: partial sums travel through distributed shared memory
}

// `knobs` (NULL = the defaults) overrides plan heuristics: b200gptq_gemv_tuned passes the first two, parameter sweeps
// that link this translation unit directly use all of them.
int gemv_stream_dispatch_tp(const __half* x, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                            const int32_t* x_perm, const __half* bias, __half* y, int M, int K, int N, int bits,
                            int group_size, void* workspace, cudaStream_t stream, const int* knobs, const TpArgs* tp) {
    if (bits == 4)
        return launch_stream<4>(x, qweight, qzeros, scales, x_perm, bias, y, M, K, N, group_size, workspace, stream, knobs, tp);
    if (bits == 3)
        return launch_stream<3>(x, qweight, qzeros, scales, x_perm, bias, y, M, K, N, group_size, workspace, stream, knobs, tp);
    return B200GPTQ_ERR_BITS;
}

int gemv_stream_dispatch_knobs(const __half* x, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                               const int32_t* x_perm, const __half* bias, __half* y, int M, int K, int N, int bits,
                               int group_size, void* workspace, cudaStream_t stream, const int* knobs) {
    return gemv_stream_dispatch_tp(x, qweight, qzeros, scales, x_perm, bias, y, M, K, N, bits, group_size, workspace,
                                   stream, knobs, nullptr);
}

// A prepared launch as an opaque object (b200gptq_gemv_plan_*): built once per (layer, row count), run many times.
struct GemvStreamPlan {
    int bits;
    PreparedStream ps;
};

GemvStreamPlan* gemv_stream_plan_create(const int32_t* qweight, const __half* scales, bool has_perm, int M, int K, int N,
                                        int bits, int group_size, const int* knobs, int* status_out) {
    GemvStreamPlan* p = new (std::nothrow) GemvStreamPlan;
    if (!p) { *status_out = B200GPTQ_ERR_CUDA; return nullptr; }
    p->bits = bits;
    *status_out = bits == 4 ? prepare_stream<4>(&p->ps, qweight, scales, has_perm, M, K, N, group_size, knobs)
                            : prepare_stream<3>(&p->ps, qweight, scales, has_perm, M, K, N, group_size, knobs);
    if (*status_out != B200GPTQ_OK) { delete p; return nullptr; }
    return p;
}

int gemv_stream_plan_run(const GemvStreamPlan* p, const __half* x, const int32_t* qzeros, const int32_t* x_perm,
                         const __half* bias, __half* y, void* workspace, cudaStream_t stream) {
    return p->bits == 4 ? launch_prepared<4>(p->ps, x, qzeros, x_perm, bias, y, workspace, stream, nullptr)
                        : launch_prepared<3>(p->ps, x, qzeros, x_perm, bias, y, workspace, stream, nullptr);
}

void gemv_stream_plan_destroy(GemvStreamPlan* p) { delete p; }

int gemv_stream_dispatch(const __half* x, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                         const int32_t* g_idx, const int32_t* x_perm, const __half* bias, __half* y, int M, int K,
                         int N, int bits, int group_size, void* workspace, cudaStream_t stream) {
    if (g_idx) return B200GPTQ_ERR_GROUPS;
    return gemv_stream_dispatch_knobs(x, qweight, qzeros, scales, x_perm, bias, y, M, K, N, bits, group_size,
                                      workspace, stream, nullptr);
}

}  // namespace b200gptq
