// Decode GEMV, strip form (M == 1, bits in {3,4}, groups = k / group_size): one persistent CTA per SM owns
// whole 32-column strips of the layer over ALL of K, so nothing is combined between CTAs, and the products run
// on the integer tensor path.
//
//   y[n] = sum_k x[xk(k)] * scales[g, n] * (q[k, n] - zero[g, n]),   g = k / group_size
//
// What the measurements on B200 that shaped it say:
//  * the legacy tensor instruction mma.sync retires one m16n8k16 f16 product per 8 cycles and SM sub-partition,
//    and one m16n8k32 u8 x s8 product in the same 8 cycles: twice the weights.  Integer and logic instructions
//    issue at half rate (two cycles per warp instruction), so the cost of a weight is the number of such
//    instructions that make it an operand.  Bytes need far fewer than halves: a 4-bit word becomes two operand
//    registers with two ANDs (q and 16 q), a 96-bit run of 3-bit fields nine registers with twelve
//    instructions (q << p, p <= 5).  The factor 2^p is taken out on the x side.
//  * x is turned into fixed point per 128 rows of K (X = x * 2^e, |X| < 2^22, exact for every element within
//    2^-12 of the largest), pre-shifted by what its weight byte lacks, and split into four signed byte planes,
//    which are the columns of the B operand: one instruction multiplies 512 weights by all four planes.
//    The four partial sums are recombined in fp32 once per 128 rows, together with the group's scale and the
//    zero-point term  zero * sum X.
//  * a chain of dependent launches costs each launch the time from its release by the previous kernel to its
//    own last store.  With one CTA per SM that takes less than half of the SM's shared memory and registers,
//    the next launch's CTA sits beside the running one and has its weights in shared memory when it is
//    released (`griddepcontrol.launch_dependents` is the first instruction).
//
// Work split: CTA b owns strips [b*S/G, (b+1)*S/G) of 32 columns.  A producer warp streams their weights
// through a ring of TMA boxes (32 columns x 1024 rows of K, 128-byte swizzle); 16 consumer warps split K
// (warp w takes the 128-row units u = w mod 16), each runs the two 16-column tiles of a strip over its units,
// and the warps' sums are added up in shared memory in warp order at the end (results do not depend on
// scheduling).  Every mbarrier wait is
// bounded; if one expires the kernel raises the sticky status word and runs on without waiting.
//
// Reference semantics: auto_gptq/nn_modules/qlinear.py:197-243; the kernel this replaces is the TVM-generated
// SIMT GEMV src/kernels/gemv_kernel.cu:25-55.
#include <cuda.h>

#include <mutex>
#include <new>

#include "common.cuh"

namespace b200gptq {

namespace {

constexpr int kCWarps = 16;                 // consumer warps: K slices
constexpr int kCThreads = 32 * kCWarps;     // 512
constexpr int kSThreads = kCThreads + 32;   // + the producer warp
constexpr int kUnitRows = 128;              // rows of K between two recombinations in fp32
constexpr int kBoxUnits = 8;                // units per TMA box
constexpr int kStripCols = 32;
constexpr int kMaxRing = 12;
constexpr int kMaxStrips = 6;               // strips per CTA
constexpr int kMaxK = 8192;                 // two passes of the x preparation
constexpr int kStatusWord = kMaxCounters - 1;
constexpr int kDynBudget = 112 * 1024;      // two CTAs per SM

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// Bounded wait: after ~1e9 clocks, or once any thread of the CTA has given up, waiting stops for good.
__device__ __noinline__ void mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* gave_up) {
    const long long t0 = clock64();
    while (!*gave_up) {
        for (int i = 0; i < 32; ++i)
            if (mbar_try_wait(bar, parity)) return;
        if (clock64() - t0 > 1000000000LL) *gave_up = 1;
    }
}
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, volatile int* gave_up) {
    if (mbar_try_wait(bar, parity)) return;
    mbar_wait_slow(bar, parity, gave_up);
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCThreads) : "memory"); }

// d += a (u8, 16 x 32) * b (s8, 32 x 8)
__device__ __forceinline__ void imma(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                     uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct Table8 { unsigned char v[8]; };
constexpr unsigned long long pack8(const Table8& t) {
    unsigned long long r = 0;
    for (int i = 0; i < 8; ++i) r |= (unsigned long long)t.v[i] << (8 * i);
    return r;
}

// ---------------------------------------------------------------------------------------------------------
// Per-bit-width traits.  A unit is 128 rows of K; lane (g = lane / 4, t = lane % 4) of a warp feeds rows
// g and g + 8 of the A operand (columns 2g and 2g + 1 of a 16-column tile) and k-bytes of quarter t.
//   kWordRows   word-rows of qweight per unit
//   kSteps      tensor instructions per unit and tile
//   kPre        log2 of the common factor of (weight byte) * (pre-shifted X) over q * X
//   item_rows   x preparation: the 8 rows (relative to the unit) that item q = 4 j + t of a unit handles, and
//               the left shift each X gets
// ---------------------------------------------------------------------------------------------------------
template <int BITS> struct ST;

// 4-bit: step s of quarter t is word-row (s & 1) + 2 t + 8 (s >> 1) of the unit's 16 (with the 128-byte swizzle
// the sixteen lanes of a half warp then read sixteen different 8-byte bank pairs).  w & 0x0f0f0f0f holds rows
// 0 2 4 6 of the word-row as bytes q, w & 0xf0f0f0f0 rows 1 3 5 7 as bytes 16 q.
template <> struct ST<4> {
    static constexpr int kWordRows = 16, kSteps = 4, kPre = 4;
    __device__ static __forceinline__ int step_row(int s, int t) { return (s & 1) + 2 * t + 8 * (s >> 1); }
    static constexpr int kReads = 4;            // 8-byte weight reads per unit and tile: one per step
    __device__ static __forceinline__ int read_row(int i, int t) { return step_row(i, t); }
    __device__ static __forceinline__ void item_rows(int j, int t, int (&row)[8], int (&pre)[8]) {
        const int wr = step_row(j, t);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            row[i] = 8 * wr + 2 * (i & 3) + (i >> 2);   // slots 0..3: rows 0 2 4 6, slots 4..7: rows 1 3 5 7
            pre[i] = (i < 4) ? 4 : 0;
        }
    }
};

// 3-bit: quarter t owns row block t of the unit (32 rows = three word-rows = a 96-bit run per column, field f
// at bit 3 f).  Every byte of the three words holds two whole fields, which two ANDs per word expose as
// q << p; the eight fields that straddle bytes (2 5 10 13 18 21 26 29) sit at the start of a byte after a
// shift of the run by 6 bits.  Nine registers hold the 32 fields (and four empty bytes):
//   R0 = w0 & A: f0 p0, f3 p1, f6 p2, f8 p0      R1 = w0 & B: f1 p3, f4 p4, f7 p5, f9 p3
//   R2 = w1 & A': f11 p1, f14 p2, f16 p0, f19 p1  R3 = w1 & B': f12 p4, f15 p5, f17 p3, f20 p4
//   R4 = w2 & A": f22 p2, f24 p0, f27 p1, f30 p2  R5 = w2 & B": f23 p5, f25 p3, f28 p4, f31 p5
//   R6 = (run >> 6)  : f2 p0, f5 p1, -, f10 p0    R7 = (run >> 38): f13 p1, -, f18 p0, f21 p1
//   R8 = (run >> 70) : -, f26 p0, f29 p1, -
// Step s multiplies (R[2s], R[2s+1]); the fifth step has only R8.
template <> struct ST<3> {
    static constexpr int kWordRows = 12, kSteps = 5, kPre = 5;
    static constexpr int kReads = 3;            // the three word-rows of the quarter's row block
    __device__ static __forceinline__ int read_row(int i, int t) { return 3 * t + i; }
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
        constexpr unsigned long long F0 = pack8({{0, 3, 6, 8, 1, 4, 7, 9}}), P0 = pack8({{0, 1, 2, 0, 3, 4, 5, 3}});
        constexpr unsigned long long F1 = pack8({{11, 14, 16, 19, 12, 15, 17, 20}}), P1 = pack8({{1, 2, 0, 1, 4, 5, 3, 4}});
        constexpr unsigned long long F2 = pack8({{22, 24, 27, 30, 23, 25, 28, 31}}), P2 = pack8({{2, 0, 1, 2, 5, 3, 4, 5}});
        constexpr unsigned long long F3 = pack8({{2, 5, 10, 13, 18, 21, 26, 29}}), P3 = pack8({{0, 1, 0, 1, 0, 1, 0, 1}});
        const unsigned long long f = j == 0 ? F0 : (j == 1 ? F1 : (j == 2 ? F2 : F3));
        const unsigned long long p = j == 0 ? P0 : (j == 1 ? P1 : (j == 2 ? P2 : P3));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            row[i] = 32 * t + (int)((f >> (8 * i)) & 0xffu);
            pre[i] = 5 - (int)((p >> (8 * i)) & 0xffu);
        }
    }
};

struct StripPlan {
    int strips;        // 32-column strips of the layer
    int grid;          // CTAs
    int units;         // K / 128
    int boxes;         // TMA boxes per strip
    int ring;          // boxes in the shared-memory ring
    int tw;            // columns of the scales / zero-point tables of a CTA (strips per CTA * 32)
    int groups;        // K / group_size
    int upg;           // units per group
    int upg_shift;     // log2(upg) when it is a power of two, else -1
    int passes;        // passes of the x preparation (512 items of 8 rows each)
};

template <int BITS> __host__ __device__ constexpr int box_bytes() { return kBoxUnits * ST<BITS>::kWordRows * 128; }
template <int BITS> __host__ __device__ constexpr int unit_plane_bytes() { return ST<BITS>::kSteps * 4 * 32; }

// 4 x 4 byte transpose: plane p of the result holds byte p of a, b, c, d
__device__ __forceinline__ void planes_of(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&pl)[4]) {
    const uint32_t ab01 = __byte_perm(a, b, 0x5140), cd01 = __byte_perm(c, d, 0x5140);
    const uint32_t ab23 = __byte_perm(a, b, 0x7362), cd23 = __byte_perm(c, d, 0x7362);
    pl[0] = __byte_perm(ab01, cd01, 0x5410); pl[1] = __byte_perm(ab01, cd01, 0x7632);
    pl[2] = __byte_perm(ab23, cd23, 0x5410); pl[3] = __byte_perm(ab23, cd23, 0x7632);
}
// one step's B operands of a quarter: [plane][b0, b1]
__device__ __forceinline__ void store_step(uint8_t* dst, const uint32_t (&lo)[4], const uint32_t (&hi)[4]) {
    *reinterpret_cast<uint4*>(dst) = make_uint4(lo[0], hi[0], lo[1], hi[1]);
    *reinterpret_cast<uint4*>(dst + 16) = make_uint4(lo[2], hi[2], lo[3], hi[3]);
}

template <int BITS, bool PERM>
__global__ void __launch_bounds__(kSThreads, 2)
gemv_strip_kernel(const __grid_constant__ CUtensorMap tmap_w, const __half* __restrict__ scales,
                  const __half* x, const int32_t* __restrict__ qzeros, const int32_t* __restrict__ x_perm,
                  const __half* __restrict__ bias, __half* __restrict__ y, int K, int N, StripPlan plan,
                  unsigned int* __restrict__ status) {
    using T = ST<BITS>;
    constexpr int BOX = box_bytes<BITS>();
    constexpr int UPB = unit_plane_bytes<BITS>();
    constexpr int UW = T::kWordRows * 128;     // bytes of a unit inside a box

    // dependents may start at once: they fetch their own weights beside this CTA and wait for its results
    asm volatile("griddepcontrol.launch_dependents;");

    extern __shared__ __align__(128) uint8_t dsm[];
    __shared__ __align__(8) uint64_t bars[2 * kMaxRing + 1];   // full[R], empty[R], x
    __shared__ volatile int gave_up;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int R = plan.ring;
    const int s0 = (int)(((long long)blockIdx.x * plan.strips) / plan.grid);
    const int s1 = (int)(((long long)(blockIdx.x + 1) * plan.strips) / plan.grid);
    const int nstrips = s1 - s0;
    if (nstrips == 0) return;   // narrow layers leave some CTAs without a strip (the grid always fills the device)
    const int nbox = nstrips * plan.boxes;
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxRing + s); };
    const uint32_t x_bar = bar_base + 8u * (2 * kMaxRing);

    // dynamic shared memory: ring | planes | copy of x | scales as fp32 | zero-points | per-unit factors | partial sums
    uint8_t* ring = dsm + ((1024u - (smem_u32(dsm) & 1023u)) & 1023u);
    uint8_t* planes = ring + (size_t)R * BOX;
    const unsigned short* raw = reinterpret_cast<const unsigned short*>(planes + (size_t)plan.units * UPB);
    float* s_sm = reinterpret_cast<float*>(planes + (size_t)plan.units * UPB + (size_t)K * 2);
    uint8_t* z_sm = reinterpret_cast<uint8_t*>(s_sm + (size_t)plan.groups * plan.tw);
    float2* ps = reinterpret_cast<float2*>(z_sm + (((size_t)plan.groups * plan.tw + 15) & ~(size_t)15));
    float* partial = reinterpret_cast<float*>(ps + plan.units);

    if (tid == 0) {
        gave_up = 0;
        for (int s = 0; s < R; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), kBoxUnits); }
        mbar_init(x_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    if (warp == kCWarps) {
        // ---- producer: the CTA's boxes in the order in which they are consumed ----
        if (lane == 0) {
            // (no division or remainder by run-time values anywhere in the loops: their latency is hundreds of cycles)
            int slot = 0, round = 0, strip = s0, b = 0;
            for (int i = 0; i < nbox; ++i) {
                if (round > 0) {
                    // slots free up only after the consumers have been released by the previous kernel: wait for
                    // that first, so that the bounded wait below times the consumers and not the predecessor
                    if (i == R) asm volatile("griddepcontrol.wait;" ::: "memory");
                    mbar_wait(empty_bar(slot), (round - 1) & 1, &gave_up);
                }
                mbar_arrive_expect_tx(full_bar(slot), (uint32_t)BOX);
                tma_load_2d(smem_u32(ring) + slot * BOX, &tmap_w, strip * kStripCols, b * (kBoxUnits * T::kWordRows),
                            full_bar(slot));
                if (++slot == R) { slot = 0; ++round; }
                if (++b == plan.boxes) { b = 0; ++strip; }
            }
        }
        return;
    }

    // ---- consumers ----
    const int g = lane >> 2, t = lane & 3;
    const int U = plan.units;
    // Warp w runs the units u = w (mod 16): a box holds 8 consecutive units, so a strip's boxes are used by the two
    // halves of the CTA in turn and go back to the producer one after the other, not all at the end of the strip.

    // scales (as fp32: type conversions issue at a fraction of the arithmetic rate on this GPU, so none is left for
    // the loop) and zero-points (field + 1) of the CTA's columns: constants
    {
        const int zwords = N / 32 * BITS;
        for (int grp = warp; grp < plan.groups; grp += kCWarps)
            for (int sp = 0; sp < nstrips; ++sp) {
                const int c = sp * kStripCols + lane, n = s0 * kStripCols + c;
                z_sm[grp * plan.tw + c] = (uint8_t)zero_point<BITS>(qzeros + (size_t)grp * zwords, n);
                s_sm[grp * plan.tw + c] = __half2float(scales[(size_t)grp * N + n]);
            }
    }
    consumer_sync();   // the tables are complete (still before the dependency wait: nothing of this is on the timed path)
    // x preparation: a warp prepares the units it multiplies (u = warp + 16 i), two per pass: lanes 0..15 one unit,
    // lanes 16..31 the next; item = (unit, quarter t, part j), 16 items of 8 rows per unit
    int kx[2][8], pre[8];
    {
        int row[8];
        T::item_rows((lane >> 2) & 3, lane & 3, row, pre);
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const int u = warp + kCWarps * (2 * p + (lane >> 4));
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                kx[p][i] = u * kUnitRows + row[i];
                if (PERM && u < U) kx[p][i] = min(max(__ldg(x_perm + kx[p][i]), 0), K - 1);
            }
        }
    }
    // byte offsets of this lane's weight reads inside a unit: [row of the step or block][tile]
    constexpr int NR = T::kReads;
    uint32_t woff[NR][2];
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int row = T::read_row(i, t);
#pragma unroll
        for (int h = 0; h < 2; ++h)
            woff[i][h] = (uint32_t)row * 128u + ((((uint32_t)(4 * h + (g >> 1))) ^ ((uint32_t)row & 7u)) << 4) + (uint32_t)(g & 1) * 8u;
    }

    // Everything above used constants only.  x is the one operand a preceding kernel may still be writing.
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // ---- x: copy, fixed point per unit, byte planes in the order of the B operand (each warp its own units) ----
    {
        if (tid == 0) {
            mbar_arrive_expect_tx(x_bar, (uint32_t)(K * 2));
            asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(raw)), "l"(x), "r"(K * 2), "r"(x_bar) : "memory");
        }
        mbar_wait(x_bar, 0, &gave_up);
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const int u = warp + kCWarps * (2 * p + (lane >> 4));
            const bool active = u < U;
            float xf[8];
            unsigned int mx = 0u;   // bits of the largest |x|: the order of non-negative floats, with NaN above infinity
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                xf[i] = active ? __half2float(__ushort_as_half(raw[kx[p][i]])) : 0.f;
                mx = max(mx, __float_as_uint(fabsf(xf[i])));
            }
#pragma unroll
            for (int o = 1; o < 16; o <<= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            // 2^ex > max |x| of the unit; X = x * 2^(148 - ex) has |X| < 2^22.  A unit of zeros takes any scale; a unit
            // with an infinity or a NaN gets a NaN factor, so that its columns come out as NaN.
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
                    const float delta = __uint_as_float((uint32_t)(ex - 21) << 23);              // 2^(ex - 148)
                    float cq = __uint_as_float((uint32_t)(ex - 21 - T::kPre) << 23);
                    if (bad) cq = __uint_as_float(0x7fc00000u);
                    ps[u] = make_float2(cq, delta * (float)sum);
                }
                const int j = (lane >> 2) & 3, tq = lane & 3;
                uint32_t lo[4], hi[4];
                if (BITS == 4 || j < 3) {
                    planes_of(dg[0], dg[1], dg[2], dg[3], lo);
                    planes_of(dg[4], dg[5], dg[6], dg[7], hi);
                    store_step(planes + (size_t)u * UPB + (j * 4 + tq) * 32, lo, hi);
                } else {
                    constexpr int Z = 0x00000000;   // the digits of zero are zero
                    planes_of(dg[0], dg[1], Z, dg[2], lo);
                    planes_of(dg[3], Z, dg[4], dg[5], hi);
                    store_step(planes + (size_t)u * UPB + (3 * 4 + tq) * 32, lo, hi);
                    planes_of(Z, dg[6], dg[7], Z, lo);
                    hi[0] = hi[1] = hi[2] = hi[3] = 0u;
                    store_step(planes + (size_t)u * UPB + (4 * 4 + tq) * 32, lo, hi);
                }
            }
        }
        __syncwarp();   // the warp's planes and factors are in shared memory; nobody else reads them
    }

    // ---- the strips ----
    const float pw = t == 0 ? 1.f : (t == 1 ? 65536.f : 0.f);   // weight of this lane's pair of planes
    const uint8_t* xb_base = planes + t * 32 + g * 8;
    // exact int -> float for |d| < 2^22 without a conversion instruction
    auto tofloat = [](int d) { return __int_as_float(d + 0x4B400000) - 12582912.f; };
    int slot = 0, phase = 0;
#pragma unroll 1
    for (int sp = 0; sp < nstrips; ++sp) {
        float acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};   // [tile][column 2g, 2g + 1]
        float zc = 0.f;                                // zero-point term of column `lane` of the strip over this warp's units
#pragma unroll 1
        for (int b = 0; b < plan.boxes; ++b) {
            // a box holds 8 units, which belong to 8 warps: only they wait for it and hand it back (a warp touches a
            // slot's empty barrier only after it has seen the same box full, so phases cannot run into one another)
            const int ul = (warp - b * kBoxUnits) & (kCWarps - 1);   // this warp's unit of the box, if below 8
            const int u = b * kBoxUnits + ul;
            if (ul < kBoxUnits) mbar_wait(full_bar(slot), phase, &gave_up);
            if (ul < kBoxUnits && u < U) {
                const uint8_t* ubase = ring + (size_t)slot * BOX + ul * UW;
                const uint8_t* xb = xb_base + (size_t)u * UPB;
                int d[2][4];
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int r = 0; r < 4; ++r) d[h][r] = 0;
                if constexpr (BITS == 4) {
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        uint2 bx = make_uint2(0u, 0u);
                        if (g < 4) bx = *reinterpret_cast<const uint2*>(xb + s * 128);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint2 w = *reinterpret_cast<const uint2*>(ubase + woff[s][h]);
                            imma(d[h], w.x & 0x0f0f0f0fu, w.y & 0x0f0f0f0fu, w.x & 0xf0f0f0f0u, w.y & 0xf0f0f0f0u, bx.x, bx.y);
                        }
                    }
                } else {
                    // a unit is 1536 bytes: odd units start half-way into the swizzle pattern
                    const uint32_t par = (uint32_t)(ul & 1) << 6;
                    uint2 bx[5];
#pragma unroll
                    for (int s = 0; s < 5; ++s) {
                        bx[s] = make_uint2(0u, 0u);
                        if (g < 4) bx[s] = *reinterpret_cast<const uint2*>(xb + s * 128);
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint2 w[3];
#pragma unroll
                        for (int i = 0; i < 3; ++i) w[i] = *reinterpret_cast<const uint2*>(ubase + (woff[i][h] ^ par));
                        uint32_t ra[9], rb[9];
                        T::unpack(w[0].x, w[1].x, w[2].x, ra);
                        T::unpack(w[0].y, w[1].y, w[2].y, rb);
                        int e[4] = {0, 0, 0, 0};
                        imma(d[h], ra[0], rb[0], ra[1], rb[1], bx[0].x, bx[0].y);
                        imma(e, ra[2], rb[2], ra[3], rb[3], bx[1].x, bx[1].y);
                        imma(d[h], ra[4], rb[4], ra[5], rb[5], bx[2].x, bx[2].y);
                        imma(e, ra[6], rb[6], ra[7], rb[7], bx[3].x, bx[3].y);
                        imma(d[h], ra[8], rb[8], 0u, 0u, bx[4].x, 0u);
#pragma unroll
                        for (int r = 0; r < 4; ++r) d[h][r] += e[r];
                    }
                }
                // recombine the planes and scale:  s * 2^-e' * sum_p 256^p S_p
                const int grow = (plan.upg_shift >= 0 ? u >> plan.upg_shift : u / plan.upg) * plan.tw + sp * kStripCols;
                const float2 f = ps[u];
                const float c = f.x * pw;
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const float2 sc = *reinterpret_cast<const float2*>(s_sm + grow + 16 * h + 2 * g);
                    const float v0 = fmaf(256.f, tofloat(d[h][1]), tofloat(d[h][0]));
                    const float v1 = fmaf(256.f, tofloat(d[h][3]), tofloat(d[h][2]));
                    acc[h][0] = fmaf(sc.x * c, v0, acc[h][0]);
                    acc[h][1] = fmaf(sc.y * c, v1, acc[h][1]);
                }
                // the zero-point term of the unit, one column per lane:  s * zero * sum x
                zc = fmaf(s_sm[grow + lane] * (float)z_sm[grow + lane], f.y, zc);
            }
            __syncwarp();
            if (ul < kBoxUnits && lane == 0) mbar_arrive(empty_bar(slot));
            if (++slot == R) { slot = 0; phase ^= 1; }
        }
        // this warp's units of the strip: add the four quarters, take off the zero-point term, keep per warp
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float v = acc[h][c];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                acc[h][c] = v;
            }
        float* dst = partial + ((size_t)sp * kCWarps + warp) * kStripCols;
        if (t == 0) {
            *reinterpret_cast<float2*>(dst + 2 * g) = make_float2(acc[0][0], acc[0][1]);
            *reinterpret_cast<float2*>(dst + 16 + 2 * g) = make_float2(acc[1][0], acc[1][1]);
        }
        __syncwarp();
        dst[lane] -= zc;
    }
    consumer_sync();
    // ---- add the K slices in warp order, bias, store ----
    for (int c = tid; c < nstrips * kStripCols; c += kCThreads) {
        const int sp = c >> 5, cc = c & 31;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kCWarps; ++w) v += partial[((size_t)sp * kCWarps + w) * kStripCols + cc];
        const int n = s0 * kStripCols + c;
        if (bias) v += __half2float(bias[n]);
        y[n] = __float2half_rn(v);
    }
    if (tid == 0 && gave_up) atomicExch(status + kStatusWord, 1u);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn strip_encode_fn() {
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

// Shared memory of a plan besides the ring.
template <int BITS>
int fixed_bytes(const StripPlan& p) {
    const int per_cta = (p.strips + p.grid - 1) / p.grid;
    return p.units * unit_plane_bytes<BITS>() + p.units * kUnitRows * 2 + p.groups * p.tw * 4 + ((p.groups * p.tw + 15) & ~15) + p.units * 8 +
           per_cta * kCWarps * kStripCols * 4 + 1024;
}

template <int BITS>
bool make_strip_plan(int K, int N, int group_size, StripPlan* out, int* smem_bytes) {
    if (K % kUnitRows || K > kMaxK || group_size % kUnitRows || N % kStripCols) return false;
    StripPlan p;
    p.strips = N / kStripCols;
    p.grid = sm_count();   // always the whole device: the next launch's CTAs then find one free place per SM
    const int per_cta = (p.strips + p.grid - 1) / p.grid;
    if (per_cta > kMaxStrips) return false;
    p.units = K / kUnitRows;
    p.boxes = (p.units + kBoxUnits - 1) / kBoxUnits;
    p.tw = per_cta * kStripCols;
    p.groups = K / group_size;
    p.upg = group_size / kUnitRows;
    p.upg_shift = -1;
    for (int b = 0; b < 16; ++b)
        if (p.upg == (1 << b)) p.upg_shift = b;
    p.passes = (p.units + 2 * kCWarps - 1) / (2 * kCWarps);   // a warp prepares two units per pass
    if (p.tw > 256 || p.groups > 256 || p.passes > 2) return false;
    const int fixed = fixed_bytes<BITS>(p);
    int ring = (kDynBudget - fixed) / box_bytes<BITS>();
    if (ring > per_cta * p.boxes) ring = per_cta * p.boxes;
    if (ring > kMaxRing) ring = kMaxRing;
    if (ring < 2) return false;
    p.ring = ring;
    *out = p;
    *smem_bytes = ring * box_bytes<BITS>() + fixed;
    return true;
}

struct PreparedStrip {
    StripPlan plan;
    int smem_bytes, K, N;
    CUtensorMap tmap_w;
    const __half* scales;
    const void* kernel;
};

template <int BITS>
int set_strip_attr_once() {
    static std::once_flag once[64];
    static int result[64];
    int dev = 0;
    B200GPTQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return B200GPTQ_ERR_TOO_LARGE;
    std::call_once(once[dev], [dev] {
        cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(gemv_strip_kernel<BITS, false>),
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, kDynBudget);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(reinterpret_cast<const void*>(gemv_strip_kernel<BITS, true>),
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, kDynBudget);
        result[dev] = (int)e;
    });
    if (result[dev] != 0) { set_last_cuda_error(result[dev]); return B200GPTQ_ERR_CUDA; }
    return B200GPTQ_OK;
}

template <int BITS>
int prepare_strip(PreparedStrip* ps, const int32_t* qweight, const __half* scales, bool has_perm, int K, int N,
                  int group_size) {
    if (!make_strip_plan<BITS>(K, N, group_size, &ps->plan, &ps->smem_bytes)) return B200GPTQ_ERR_SHAPE;
    ps->K = K; ps->N = N;
    const EncodeTiledFn encode = strip_encode_fn();
    if (!encode) { set_last_cuda_error((int)cudaErrorNotSupported); return B200GPTQ_ERR_CUDA; }
    {
        // qweight [K/32*bits, N] int32; a box is 32 columns x the word-rows of 8 units, rows past the end read as zero
        const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K / 32 * BITS)};
        const cuuint64_t strides[1] = {(cuuint64_t)N * sizeof(int32_t)};
        const cuuint32_t box[2] = {(cuuint32_t)kStripCols, (cuuint32_t)(kBoxUnits * ST<BITS>::kWordRows)};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r = encode(&ps->tmap_w, CU_TENSOR_MAP_DATA_TYPE_INT32, 2, const_cast<int32_t*>(qweight), dims,
                                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { set_last_cuda_error((int)cudaErrorInvalidValue); return B200GPTQ_ERR_CUDA; }
    }
    ps->scales = scales;
    ps->kernel = has_perm ? (const void*)gemv_strip_kernel<BITS, true> : (const void*)gemv_strip_kernel<BITS, false>;
    return B200GPTQ_OK;
}

template <int BITS>
int launch_strip(const PreparedStrip& ps, const __half* x, const int32_t* qzeros, const int32_t* x_perm,
                 const __half* bias, __half* y, void* workspace, cudaStream_t stream) {
    unsigned int* status = reinterpret_cast<unsigned int*>(workspace);
    if (int st = set_strip_attr_once<BITS>()) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ps.plan.grid);
    cfg.blockDim = dim3(kSThreads);
    cfg.dynamicSmemBytes = ps.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int K = ps.K, N = ps.N;
    StripPlan plan = ps.plan;
    const __half* scales = ps.scales;
    void* args[] = {const_cast<CUtensorMap*>(&ps.tmap_w), &scales, &x, &qzeros, &x_perm,
                    &bias, &y, &K, &N, &plan, &status};
    B200GPTQ_CUDA_TRY(cudaLaunchKernelExC(&cfg, ps.kernel, args));
    return B200GPTQ_OK;
}

}  // namespace

// The strip kernel serves single-row calls whose layer has a strip for at least three quarters of the SMs and whose
// per-CTA tables fit beside a ring of at least two boxes.
bool gemv_strip_supported(int M, int K, int N, int bits, int group_size) {
    if (M != 1 || (bits != 3 && bits != 4) || group_size <= 0) return false;
    if (4 * (N / kStripCols) < 3 * sm_count()) return false;
    StripPlan p;
    int smem = 0;
    return bits == 4 ? make_strip_plan<4>(K, N, group_size, &p, &smem) : make_strip_plan<3>(K, N, group_size, &p, &smem);
}

struct GemvStripPlan {
    int bits;
    PreparedStrip ps;
};

GemvStripPlan* gemv_strip_plan_create(const int32_t* qweight, const __half* scales, bool has_perm, int K, int N, int bits,
                                      int group_size, int* status_out) {
    GemvStripPlan* p = new (std::nothrow) GemvStripPlan;
    if (!p) { *status_out = B200GPTQ_ERR_CUDA; return nullptr; }
    p->bits = bits;
    *status_out = bits == 4 ? prepare_strip<4>(&p->ps, qweight, scales, has_perm, K, N, group_size)
                            : prepare_strip<3>(&p->ps, qweight, scales, has_perm, K, N, group_size);
    if (*status_out != B200GPTQ_OK) { delete p; return nullptr; }
    return p;
}

int gemv_strip_plan_run(const GemvStripPlan* p, const __half* x, const int32_t* qzeros, const int32_t* x_perm,
                        const __half* bias, __half* y, void* workspace, cudaStream_t stream) {
    return p->bits == 4 ? launch_strip<4>(p->ps, x, qzeros, x_perm, bias, y, workspace, stream)
                        : launch_strip<3>(p->ps, x, qzeros, x_perm, bias, y, workspace, stream);
}

void gemv_strip_plan_destroy(GemvStripPlan* p) { delete p; }

int gemv_strip_dispatch(const __half* x, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                        const int32_t* x_perm, const __half* bias, __half* y, int K, int N, int bits, int group_size,
                        void* workspace, cudaStream_t stream) {
    GemvStripPlan p;
    p.bits = bits;
    const int st = bits == 4 ? prepare_strip<4>(&p.ps, qweight, scales, x_perm != nullptr, K, N, group_size)
                             : prepare_strip<3>(&p.ps, qweight, scales, x_perm != nullptr, K, N, group_size);
    if (st != B200GPTQ_OK) return st;
    return gemv_strip_plan_run(&p, x, qzeros, x_perm, bias, y, workspace, stream);
}

}  // namespace b200gptq
