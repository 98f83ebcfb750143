// Decode GEMV, streaming form (M <= 8, bits in {3,4}, groups = k / group_size).
//
//   y[m, n] = sum_k x[m, xk(k)] * scales[g, n] * (q[k, n] - zero[g, n]),   g = k / group_size
//
// The kernel is bound by HBM bandwidth and, on B200, almost by instruction issue as well
// (about two instructions per weight are available at full bandwidth), so the inner loop
// is built to spend roughly one instruction per weight:
//
//  * weights go from global memory straight to registers with 128-bit loads, several
//    units ahead of their use (no shared-memory staging, no barriers on the weight path);
//  * fields are never shifted into place or converted: a LOP3 masks two fields of a word
//    and ORs in an fp16 exponent, which yields the half2 (c_lo + q_lo, c_hi + q_hi) with
//    small known offsets c (8..128);
//  * the products are done by mma.sync m16n8k16 (f16 x f16 -> f32): the 16 rows of the A
//    tile are 16 output columns, the 8 columns of B are the (up to 8) rows of x, so one
//    instruction retires 256 weights of a warp for every M <= 8;
//  * the offsets and zero-points are removed afterwards: per group, sum_k (c_k + q_k) x_k is
//    scaled by s, and  sum_g s * (sum_k c_k x_k + zero * sum_k x_k)  -- which needs only x,
//    scales and qzeros -- is computed per column while the first weight loads are in flight.
//
// Work split: a "unit" is 256 columns x 32 rows (4-bit) or x 128 rows (3-bit).  Units are
// numbered column-group-major and dealt out in equal contiguous ranges to 2 CTAs per SM,
// so every shape is balanced; a range that ends inside a column group leaves a partial
// sum in the fp32 scratch and the last CTA of that column group adds the partials in a
// fixed order (results do not depend on scheduling).
//
// Reference semantics: auto_gptq/nn_modules/qlinear.py:197-243; the kernel this replaces is
// the TVM-generated SIMT GEMV src/kernels/gemv_kernel.cu:25-55.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"

namespace b200gptq {

namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerCta = kThreads / 32;
constexpr int kCgCols = 32 * kWarpsPerCta;  // 256 columns per column group
constexpr int kMaxM = 8;
constexpr int kStageRows = 1024;            // rows of x staged in shared memory at a time

__device__ __forceinline__ uint4 ldg_stream(const int32_t* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

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

// 3-bit: half index, inside a fragment entry, of the x value that meets field f of a row block.
__constant__ unsigned char kSlot3[32] = {0, 2, 4, 6, 8, 1, 3, 5, 7, 9, 11, 12, 14, 16, 18, 20,
                                         13, 15, 17, 19, 21, 23, 24, 26, 28, 30, 32, 25, 27, 29, 31, 33};

// ---------------------------------------------------------------------------------------
// Per-bit-width traits.
//   kUnitRows     rows of K covered by one unit
//   kVecs         128-bit loads per thread per unit
//   kBRegs        32-bit registers of B fragments per (unit, x row, quad lane), padded to x4
// Lane (g = lane/4, j = lane%4) of warp w holds columns 32w + 4g .. +3 of the column group.
// ---------------------------------------------------------------------------------------
template <int BITS> struct Traits;

// 4-bit: the quad's lane j owns word-row 4*rb + j (8 rows of K).  Fields are brought to bit 4
// of each 16-bit half, where OR-ing 0x5400 gives 64 + q.  Pair i = (nibble i, nibble i + 4).
template <> struct Traits<4> {
    static constexpr int kUnitRows = 32;
    static constexpr int kVecs = 1;
    static constexpr int kBRegs = 4;
    static constexpr int kDepth = 8;   // units in flight per thread

    static constexpr int kWordRows = 4;  // word-rows of qweight per unit

    // p points at word-row 4*kb + j of the lane's first column.
    __device__ static __forceinline__ void load(uint4 (&buf)[kVecs], const int32_t* __restrict__ p, int N,
                                                bool active) {
        (void)N;
        if (active) buf[0] = ldg_stream(p);
        else buf[0] = make_uint4(0, 0, 0, 0);
    }
    __device__ static __forceinline__ int first_word_row(int kb, int j) { return 4 * kb + j; }

    // d[cp] accumulates column pair cp (columns 2cp, 2cp+1 of the lane's 4) over this unit.
    __device__ static void compute(const uint4 (&buf)[kVecs], const uint32_t* __restrict__ bsm, bool has_x,
                                   float (&d)[2][4]) {
        uint4 bf = make_uint4(0, 0, 0, 0);
        if (has_x) bf = *reinterpret_cast<const uint4*>(bsm);
        const uint32_t wcol[4] = {buf[0].x, buf[0].y, buf[0].z, buf[0].w};
        constexpr uint32_t MASK = 0x00f000f0u, MAGIC = 0x54005400u;
#pragma unroll
        for (int cp = 0; cp < 2; ++cp) {
            const uint32_t wa = wcol[2 * cp], wb = wcol[2 * cp + 1];
            const uint32_t a_p0 = lop3_and_or(wa << 4, MASK, MAGIC), b_p0 = lop3_and_or(wb << 4, MASK, MAGIC);
            const uint32_t a_p1 = lop3_and_or(wa, MASK, MAGIC), b_p1 = lop3_and_or(wb, MASK, MAGIC);
            const uint32_t a_p2 = lop3_and_or(wa >> 4, MASK, MAGIC), b_p2 = lop3_and_or(wb >> 4, MASK, MAGIC);
            const uint32_t a_p3 = lop3_and_or(wa >> 8, MASK, MAGIC), b_p3 = lop3_and_or(wb >> 8, MASK, MAGIC);
            mma16816(d[cp], a_p0, b_p0, a_p1, b_p1, bf.x, bf.y);
            mma16816(d[cp], a_p2, b_p2, a_p3, b_p3, bf.z, bf.w);
        }
    }

    // Position (in halfs) inside a (unit, x row, quad lane) fragment entry of the x value that meets
    // field i8 (0..7) of the lane's word: pairs are (x0,x4)(x1,x5)(x2,x6)(x3,x7).  Offset constant: 64.
    __device__ static __forceinline__ int slot(int i8) { return 2 * (i8 & 3) + (i8 >> 2); }
    __device__ static __forceinline__ float coef(int) { return 64.f; }
    static constexpr int kRowsPerLane = 8;   // rows of K per quad lane and unit
};

// 3-bit: the quad's lane j owns row block 4*kb + j (32 rows of K = three word-rows, a 96-bit
// stream per column).  Nine 32-bit windows of the stream each expose two clean pairs:
// window base b (stream offset 3b - 1, so -4 for b = -1) has fields b+1 (bit 4) and b+2 (bit 7) in its low half
// and b+6 (bit 3), b+7 (bit 6) in its high half, with exponents giving offsets 64, 8, 128, 16.
// Fields 5, 16, 27 appear twice and field "32" does not exist: their second slot gets x = 0.
template <> struct Traits<3> {
    static constexpr int kUnitRows = 128;
    static constexpr int kVecs = 3;
    static constexpr int kBRegs = 20;  // 18 used
    static constexpr int kDepth = 3;

    static constexpr int kWordRows = 12;

    // p points at word-row 3*(4*kb + j) of the lane's first column.
    __device__ static __forceinline__ void load(uint4 (&buf)[kVecs], const int32_t* __restrict__ p, int N,
                                                bool active) {
#pragma unroll
        for (int r = 0; r < 3; ++r) {
            if (active) buf[r] = ldg_stream(p + (size_t)r * N);
            else buf[r] = make_uint4(0, 0, 0, 0);
        }
    }
    __device__ static __forceinline__ int first_word_row(int kb, int j) { return 3 * (4 * kb + j); }

    // Window t (0..8) of one column's stream (w0, w1, w2); stream offsets -4, 2, 8, 29, 35, 41, 62, 68, 74.
    template <int T_>
    __device__ static __forceinline__ uint32_t window(uint32_t w0, uint32_t w1, uint32_t w2) {
        if constexpr (T_ == 0) return w0 << 4;
        else if constexpr (T_ == 1) return w0 >> 2;
        else if constexpr (T_ == 2) return __funnelshift_r(w0, w1, 8);
        else if constexpr (T_ == 3) return w1 << 3;
        else if constexpr (T_ == 4) return w1 >> 3;
        else if constexpr (T_ == 5) return __funnelshift_r(w1, w2, 9);
        else if constexpr (T_ == 6) return w2 << 2;
        else if constexpr (T_ == 7) return w2 >> 4;
        else return w2 >> 10;
    }

    template <int T_>
    __device__ static __forceinline__ void step(const uint4 (&buf)[kVecs], const uint32_t* __restrict__ bsm,
                                                bool has_x, float (&d)[2][4]) {
        constexpr uint32_t MASK_A = 0x00380070u, MAGIC_A = 0x58005400u;  // (64 + f[b+1], 128 + f[b+6])
        constexpr uint32_t MASK_B = 0x01C00380u, MAGIC_B = 0x4C004800u;  // ( 8 + f[b+2],  16 + f[b+7])
        uint2 bf = make_uint2(0, 0);
        if (has_x) bf = *reinterpret_cast<const uint2*>(bsm + 2 * T_);
        {
            const uint32_t va = window<T_>(buf[0].x, buf[1].x, buf[2].x);
            const uint32_t vb = window<T_>(buf[0].y, buf[1].y, buf[2].y);
            mma16816(d[0], lop3_and_or(va, MASK_A, MAGIC_A), lop3_and_or(vb, MASK_A, MAGIC_A),
                     lop3_and_or(va, MASK_B, MAGIC_B), lop3_and_or(vb, MASK_B, MAGIC_B), bf.x, bf.y);
        }
        {
            const uint32_t va = window<T_>(buf[0].z, buf[1].z, buf[2].z);
            const uint32_t vb = window<T_>(buf[0].w, buf[1].w, buf[2].w);
            mma16816(d[1], lop3_and_or(va, MASK_A, MAGIC_A), lop3_and_or(vb, MASK_A, MAGIC_A),
                     lop3_and_or(va, MASK_B, MAGIC_B), lop3_and_or(vb, MASK_B, MAGIC_B), bf.x, bf.y);
        }
    }

    __device__ static void compute(const uint4 (&buf)[kVecs], const uint32_t* __restrict__ bsm, bool has_x,
                                   float (&d)[2][4]) {
        step<0>(buf, bsm, has_x, d); step<1>(buf, bsm, has_x, d); step<2>(buf, bsm, has_x, d);
        step<3>(buf, bsm, has_x, d); step<4>(buf, bsm, has_x, d); step<5>(buf, bsm, has_x, d);
        step<6>(buf, bsm, has_x, d); step<7>(buf, bsm, has_x, d); step<8>(buf, bsm, has_x, d);
    }

    // Half index inside a fragment entry for field f (0..31) of the lane's row block: window t,
    // position 0..3 = (A low, A high, B low, B high) -> 4t + position.  Offsets by position: 64, 128, 8, 16.
    __device__ static __forceinline__ int slot(int f) { return kSlot3[f]; }
    __device__ static __forceinline__ float coef(int h) {
        const int pos = h & 3;
        return pos == 0 ? 64.f : pos == 1 ? 128.f : pos == 2 ? 8.f : 16.f;
    }
    static constexpr int kRowsPerLane = 32;
};

struct Plan {
    int cgs;          // column groups (256 columns each)
    int kbs;          // units per column group
    int units;        // cgs * kbs
    int ctas;
    int stage_units;  // units whose x values are staged in shared memory at a time (<= 1024 rows, <= 8 groups)
};

__host__ __device__ inline int cta_first_unit(int i, int units, int ctas) {
    return (int)(((long long)i * units) / ctas);
}
// CTA that owns unit u (largest i with cta_first_unit(i) <= u).
__host__ __device__ inline int unit_owner(int u, int units, int ctas) {
    return (int)((((long long)u + 1) * ctas - 1) / units);
}

constexpr int kStageGroups = 8;

#ifdef B200GPTQ_TRACE
__device__ unsigned long long g_trace[1024 * 8];
__device__ __forceinline__ void trace_mark(int slot) {
    if (threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        g_trace[blockIdx.x * 8 + slot] = t;
    }
}
#define TRACE(slot) trace_mark(slot)
#else
#define TRACE(slot)
#endif

template <int BITS>
__global__ void __launch_bounds__(kThreads, 2)
gemv_stream_kernel(const __half* __restrict__ x, const int32_t* __restrict__ qweight,
                   const int32_t* __restrict__ qzeros, const __half* __restrict__ scales,
                   const int32_t* __restrict__ x_perm, const __half* __restrict__ bias, __half* __restrict__ y,
                   int M, int K, int N, int group_size, Plan plan, float* __restrict__ partials,
                   unsigned int* __restrict__ counters) {
    using T = Traits<BITS>;
    constexpr int UR = T::kUnitRows;
    constexpr int D = T::kDepth;
    constexpr int MAX_STAGE_UNITS = kStageRows / UR;

    __shared__ __align__(16) uint32_t xs[MAX_STAGE_UNITS * kMaxM * 4 * T::kBRegs];  // x in fragment order
    __shared__ float2 ps[kMaxM][kStageRows / 8];            // (sum x, sum c*x) of each 8 staged rows
    __shared__ __align__(16) float s_sm[kStageGroups][kCgCols];  // scales of the staged groups
    __shared__ float corr_sm[kMaxM][kCgCols];               // offset / zero-point term, then the segment result
    __shared__ float t_x[kStageGroups * kMaxM], t_cx[kStageGroups * kMaxM];
    __shared__ bool is_last;

    TRACE(0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, j = lane & 3;
    const int u_begin = cta_first_unit(blockIdx.x, plan.units, plan.ctas);
    const int u_end = cta_first_unit(blockIdx.x + 1, plan.units, plan.ctas);
    const int kbs = plan.kbs;
    const int zwords = N / 32 * BITS;
    const int lane_col = warp * 32 + 4 * g;  // first of the lane's 4 columns inside the column group
    const size_t unit_stride = (size_t)T::kWordRows * N;
    const int units_per_group = group_size / UR;

    // ---- the weight stream: a register ring of D units, refilled as it is consumed ----
    int pf_cg = u_begin / kbs;
    int pf_left_cg = kbs - (u_begin - pf_cg * kbs);   // units left in the prefetch column group
    int pf_left = u_end - u_begin;                    // units left in this CTA's range
    bool pf_col_ok = pf_cg * kCgCols + lane_col < N;
    const int32_t* pf_ptr =
        qweight + (size_t)T::first_word_row(kbs - pf_left_cg, j) * N + (size_t)pf_cg * kCgCols + lane_col;
    auto prefetch = [&](uint4 (&dst)[T::kVecs]) {
        T::load(dst, pf_ptr, N, pf_left > 0 && pf_col_ok);
        pf_ptr += unit_stride;
        --pf_left;
        if (--pf_left_cg == 0) {
            ++pf_cg;
            pf_left_cg = kbs;
            pf_col_ok = pf_cg * kCgCols + lane_col < N;
            pf_ptr = qweight + (size_t)T::first_word_row(0, j) * N + (size_t)pf_cg * kCgCols + lane_col;
        }
    };
    uint4 buf[D][T::kVecs];

#pragma unroll
    for (int m = 0; m < kMaxM; ++m) corr_sm[m][tid] = 0.f;

    float out[2][4], d[2][4];
#pragma unroll
    for (int cp = 0; cp < 2; ++cp)
#pragma unroll
        for (int r = 0; r < 4; ++r) { out[cp][r] = 0.f; d[cp][r] = 0.f; }

    bool waited = false;
    int stage_g0 = 0;

    // out += scale[group] * d for the lane's 4 columns, then clear d.
    auto flush_group = [&](int grp) {
        const float4 s = *reinterpret_cast<const float4*>(&s_sm[grp - stage_g0][lane_col]);
        out[0][0] = fmaf(s.x, d[0][0], out[0][0]); out[0][1] = fmaf(s.x, d[0][1], out[0][1]);
        out[0][2] = fmaf(s.y, d[0][2], out[0][2]); out[0][3] = fmaf(s.y, d[0][3], out[0][3]);
        out[1][0] = fmaf(s.z, d[1][0], out[1][0]); out[1][1] = fmaf(s.z, d[1][1], out[1][1]);
        out[1][2] = fmaf(s.w, d[1][2], out[1][2]); out[1][3] = fmaf(s.w, d[1][3], out[1][3]);
#pragma unroll
        for (int cp = 0; cp < 2; ++cp)
#pragma unroll
            for (int r = 0; r < 4; ++r) d[cp][r] = 0.f;
    };

    // Stage x for units [kb_a, kb_b) of column group cg: fragments into xs, scales into s_sm, and
    // the offset / zero-point term  sum_groups s * (sum c x + zero * sum x)  into corr_sm.
    auto stage = [&](int cg, int kb_a, int kb_b) {
        const int r0 = kb_a * UR, rows = (kb_b - kb_a) * UR;
        const int g0 = r0 / group_size, ng = (r0 + rows - 1) / group_size - g0 + 1;
        const int n = min(cg * kCgCols + tid, N - 1);
        // -- static data first: scales and zero-points of this thread's column, gather indices
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
        float s_reg[kStageGroups], z_reg[kStageGroups];
#pragma unroll
        for (int gl = 0; gl < kStageGroups; ++gl) {
            s_reg[gl] = 0.f; z_reg[gl] = 0.f;
            if (gl < ng) {
                s_reg[gl] = __half2float(__ldg(sp + (size_t)gl * N));
                const uint32_t lo = __ldg(zp + (size_t)gl * zwords);
                uint32_t q;
                if constexpr (BITS == 3) {
                    const uint32_t hi = zstr ? __ldg(zp + (size_t)gl * zwords + 1) : 0u;
                    q = __funnelshift_r(lo, hi, zsh) & 7u;
                } else {
                    q = (lo >> zsh) & 15u;
                }
                z_reg[gl] = __uint_as_float(0x4B000000u | (q + 1u)) - 8388608.f;  // exact small integer
            }
        }
        const bool has_q = tid < rows / 4;
        const int kq = r0 + 4 * tid;  // this thread stages rows kq .. kq+3 of every x row
        int4 pidx = make_int4(kq, kq + 1, kq + 2, kq + 3);
        if (has_q && x_perm) pidx = __ldg(reinterpret_cast<const int4*>(x_perm + kq));
        if (!waited) {
            // The small loads above are already queued; now start the weight stream behind them.
#pragma unroll
            for (int i = 0; i < D; ++i) prefetch(buf[i]);
            // x is the only operand a preceding kernel may still be writing
            asm volatile("griddepcontrol.launch_dependents;");
            asm volatile("griddepcontrol.wait;" ::: "memory");
            waited = true;
            TRACE(1);
        }
        __syncthreads();  // the previous stage's fragments and scales are no longer in use
#pragma unroll
        for (int gl = 0; gl < kStageGroups; ++gl) s_sm[gl][tid] = s_reg[gl];
        {
            const int kl = 4 * tid;                               // row inside the stage
            const int ul = kl / UR, jl = (kl % UR) / T::kRowsPerLane, f0 = kl % T::kRowsPerLane;
            __half* xh = reinterpret_cast<__half*>(xs);
#pragma unroll 1
            for (int m = 0; m < M; ++m) {
                float sx = 0.f, scx = 0.f;
                if (has_q) {
                    const __half* xr = x + (size_t)m * K;
                    __half v[4];
                    if (x_perm) {
                        v[0] = xr[pidx.x]; v[1] = xr[pidx.y]; v[2] = xr[pidx.z]; v[3] = xr[pidx.w];
                    } else {
                        const uint2 raw = *reinterpret_cast<const uint2*>(xr + kq);
                        v[0] = __ushort_as_half((unsigned short)(raw.x & 0xffffu));
                        v[1] = __ushort_as_half((unsigned short)(raw.x >> 16));
                        v[2] = __ushort_as_half((unsigned short)(raw.y & 0xffffu));
                        v[3] = __ushort_as_half((unsigned short)(raw.y >> 16));
                    }
                    __half* e = xh + (size_t)(((ul * M + m) * 4 + jl) * T::kBRegs) * 2;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int h = T::slot(f0 + i);
                        e[h] = v[i];
                        const float xf = __half2float(v[i]);
                        sx += xf;
                        scx = fmaf(T::coef(h), xf, scx);
                    }
                    if (BITS == 3 && f0 == 0) {  // slots that no field feeds must multiply by zero
                        const __half zero = __float2half(0.f);
                        e[10] = zero; e[22] = zero; e[34] = zero; e[35] = zero;
                    }
                }
                sx += __shfl_xor_sync(0xffffffffu, sx, 1);
                scx += __shfl_xor_sync(0xffffffffu, scx, 1);
                if (has_q && (tid & 1) == 0) ps[m][tid >> 1] = make_float2(sx, scx);
            }
        }
        __syncthreads();
        if (tid < ng * M) {
            const int m = tid % M, gl = tid / M;
            const int ra = max(r0, (g0 + gl) * group_size), rb = min(r0 + rows, (g0 + gl + 1) * group_size);
            float sx = 0.f, scx = 0.f;
#pragma unroll 4
            for (int o = (ra - r0) >> 3; o < (rb - r0) >> 3; ++o) {
                const float2 p = ps[m][o];
                sx += p.x;
                scx += p.y;
            }
            t_x[gl * kMaxM + m] = sx;
            t_cx[gl * kMaxM + m] = scx;
        }
        __syncthreads();
#pragma unroll 1
        for (int m = 0; m < M; ++m) {
            float c = 0.f;
#pragma unroll
            for (int gl = 0; gl < kStageGroups; ++gl)
                if (gl < ng) c = fmaf(s_reg[gl], fmaf(z_reg[gl], t_x[gl * kMaxM + m], t_cx[gl * kMaxM + m]), c);
            corr_sm[m][tid] += c;
        }
        stage_g0 = g0;
        TRACE(2);
    };

    // Close the segment of column group cg: combine lanes, remove the offset / zero-point term,
    // then write y or leave the partial sums in the scratch for the last CTA of the column group.
    auto finish_segment = [&](int cg) {
        __syncthreads();  // corr_sm is complete
#pragma unroll
        for (int cp = 0; cp < 2; ++cp)
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int m = 2 * j + (r & 1);
                const int c = lane_col + 2 * cp + (r >> 1);
                if (m < M) corr_sm[m][c] = out[cp][r] - corr_sm[m][c];
                out[cp][r] = 0.f;
            }
        __syncthreads();
        const int n = cg * kCgCols + tid;
        const int owner_first = unit_owner(cg * kbs, plan.units, plan.ctas);
        const int owner_last = unit_owner(cg * kbs + kbs - 1, plan.units, plan.ctas);
        const bool whole = (owner_first == owner_last);
#pragma unroll 1
        for (int m = 0; m < M; ++m) {
            float v = corr_sm[m][tid];
            corr_sm[m][tid] = 0.f;
            if (n < N) {
                if (whole) {
                    if (bias) v += __half2float(bias[n]);
                    y[(size_t)m * N + n] = __float2half_rn(v);
                } else {
                    partials[((size_t)(blockIdx.x + cg) * kMaxM + m) * kCgCols + tid] = v;
                }
            }
        }
        if (!whole) {
            __threadfence();
            __syncthreads();
            if (tid == 0) {
                const unsigned int expected = (unsigned int)(owner_last - owner_first + 1);
                const unsigned int prev = atomicAdd(counters + cg, 1u);
                is_last = (prev == expected - 1);
                if (is_last) counters[cg] = 0u;  // the scratch is left ready for the next call
            }
            __syncthreads();
            if (is_last) {
                __threadfence();
                if (n < N) {
#pragma unroll 1
                    for (int m = 0; m < M; ++m) {
                        float v = 0.f;
#pragma unroll 4
                        for (int i = owner_first; i <= owner_last; ++i)
                            v += __ldcg(partials + ((size_t)(i + cg) * kMaxM + m) * kCgCols + tid);
                        if (bias) v += __half2float(bias[n]);
                        y[(size_t)m * N + n] = __float2half_rn(v);
                    }
                }
            }
        }
    };

    // One unit: take slot I of the register ring, refill it with the unit D ahead, multiply.
    // The ring slot is a compile-time constant, so the switch below enters an unrolled sequence of D
    // units at the current slot; the heavy, rarely executed stage / finish code exists once.
    int u = u_begin, slot = 0;
    int grp = 0, grp_left = 1;       // group of the next unit, units of it still to come
    const uint32_t* bsm = xs;        // fragments of the next unit for this lane
    const int bsm_step = M * 4 * T::kBRegs;
    bool pending = false;            // d holds products that have not been scaled into out yet
    auto unit = [&](auto slot_c) {
        constexpr int I = decltype(slot_c)::value;
        uint4 cur[T::kVecs];
#pragma unroll
        for (int r = 0; r < T::kVecs; ++r) cur[r] = buf[I][r];
        prefetch(buf[I]);
        T::compute(cur, bsm, g < M, d);
        bsm += bsm_step;
        ++u;
        pending = true;
        if (--grp_left == 0) {
            flush_group(grp);
            ++grp;
            grp_left = units_per_group;
            pending = false;
        }
    };

    while (u < u_end) {
        const int cg = u / kbs;
        const int kb = u - cg * kbs;
        // stage as far as the stage grid, the column group and this CTA's range allow
        const int su = plan.stage_units;
        const int kb_stop = min(min(kbs, (kb / su + 1) * su), kb + (u_end - u));
        stage(cg, kb, kb_stop);
        grp = (kb * UR) / group_size;
        grp_left = units_per_group - (kb - grp * units_per_group);
        bsm = xs + (size_t)(g * 4 + j) * T::kBRegs;
        const int run_end = u + (kb_stop - kb);
        while (u < run_end) {
            switch (slot) {
#define B200GPTQ_UNIT(I)                                             \
    case I:                                                          \
        if constexpr (I < D) {                                       \
            unit(std::integral_constant<int, I>{});                  \
            if (u == run_end) { slot = (I + 1) % D; break; }         \
        }
                B200GPTQ_UNIT(0) B200GPTQ_UNIT(1) B200GPTQ_UNIT(2) B200GPTQ_UNIT(3)
                B200GPTQ_UNIT(4) B200GPTQ_UNIT(5) B200GPTQ_UNIT(6) B200GPTQ_UNIT(7)
#undef B200GPTQ_UNIT
                default: slot = 0;
            }
        }
        TRACE(3);
        // the segment ends here if the next unit belongs to another column group or to another CTA
        if (u == u_end || kb_stop == kbs) {
            if (pending) { flush_group(grp); pending = false; }
            finish_segment(cg);
        }
    }
    TRACE(4);
}

int ctas_per_sm() {
    static const int v = [] {
        const char* e = std::getenv("B200GPTQ_GEMV_CTAS_PER_SM");
        const int n = e ? std::atoi(e) : 0;
        return (n == 1 || n == 2) ? n : 2;
    }();
    return v;
}

Plan make_plan(int K, int N, int bits, int group_size) {
    Plan p;
    const int unit_rows = bits == 4 ? Traits<4>::kUnitRows : Traits<3>::kUnitRows;
    p.cgs = (N + kCgCols - 1) / kCgCols;
    p.kbs = K / unit_rows;
    p.units = p.cgs * p.kbs;
    const int want = ctas_per_sm() * sm_count();
    p.ctas = p.units < want ? p.units : want;
    if (p.ctas < 1) p.ctas = 1;
    // a stage spans at most kStageRows rows and at most kStageGroups groups, and starts on a multiple of itself
    long long stage_rows = (long long)kStageGroups * group_size;
    if (stage_rows > kStageRows) stage_rows = group_size <= kStageRows ? (kStageRows / group_size) * group_size : kStageRows;
    p.stage_units = (int)(stage_rows / unit_rows);
    if (p.stage_units < 1) p.stage_units = 1;
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
    const Plan plan = make_plan(K, N, BITS, group_size);
    if (plan.cgs >= kMaxCounters - 1) return B200GPTQ_ERR_TOO_LARGE;  // the last counter word is reserved
    unsigned int* counters = reinterpret_cast<unsigned int*>(workspace);
    float* partials = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kCounterBytes);

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.ctas);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    B200GPTQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemv_stream_kernel<BITS>, x, qweight, qzeros, scales, x_perm, bias, y,
                                         M, K, N, group_size, plan, partials, counters));
    return B200GPTQ_OK;
}

}  // namespace

#ifdef B200GPTQ_TRACE
extern "C" __attribute__((visibility("default"))) int b200gptq_trace_read(unsigned long long* host, int n) {
    return (int)cudaMemcpyFromSymbol(host, g_trace, sizeof(unsigned long long) * n);
}
#endif

// The streaming kernel handles groups k / group_size only (no g_idx), whole units per group, and
// x rows that can be read 8 bytes at a time.
bool gemv_stream_supported(int M, int K, int N, int bits, int group_size) {
    (void)N;
    if (M < 1 || M > kMaxM) return false;
    if (bits == 4) return group_size % 32 == 0 && K % 32 == 0;
    if (bits == 3) return group_size % 128 == 0 && K % 128 == 0;
    return false;
}

size_t gemv_stream_workspace_bytes(int M, int K, int N, int bits) {
    (void)M;
    if (bits != 3 && bits != 4) return 0;
    if (bits == 3 && K % 128 != 0) return 0;
    const Plan plan = make_plan(K, N, bits, 128);
    return kCounterBytes + (size_t)(plan.ctas + plan.cgs) * kMaxM * kCgCols * sizeof(float);
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
