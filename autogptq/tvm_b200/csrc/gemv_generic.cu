// Decode GEMV, general form: any g_idx, any supported bit width, 1 <= M <= 8.
//
// y[m, n] = sum_k x[m, xk(k)] * scales[g(k), n] * (q[k, n] - zero[g(k), n])      (+ bias[n])
//
// This kernel accepts everything the packed format can express (qlinear.py:197-243 of the
// reference defines the arithmetic) and is the path taken when the streaming kernel's
// layout conditions do not hold.  Work split: a CTA owns a strip of 128 columns and one
// slice of K; its 8 warps walk the slice one 32-row block at a time, each lane holding 4
// adjacent columns (128-bit loads of the packed words).  x values of a row block live one
// per lane and are broadcast with warp shuffles.  Partial sums are combined across warps
// in shared memory and, when K is split across CTAs, across CTAs through an fp32 scratch
// area in a fixed order (the last CTA to arrive adds the slices 0..S-1 in sequence), so
// results do not depend on scheduling.
#include "common.cuh"

namespace b200gptq {

namespace {

constexpr int kStripCols = 128;
constexpr int kWarps = 8;

template <int BITS, int M>
__global__ void __launch_bounds__(kWarps * 32)
gemv_generic_kernel(const __half* __restrict__ x, const int32_t* __restrict__ qweight,
                    const int32_t* __restrict__ qzeros, const __half* __restrict__ scales,
                    const int32_t* __restrict__ g_idx, const int32_t* __restrict__ x_perm,
                    const __half* __restrict__ bias, __half* __restrict__ y, int K, int N,
                    int group_size, int rb_per_slice, float* __restrict__ partials,
                    unsigned int* __restrict__ counters) {
    constexpr int MP = (M + 1) / 2;  // x rows are carried as half2 pairs
    __shared__ float red[kWarps][M][kStripCols];
    __shared__ bool is_last;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int strip = blockIdx.x, slice = blockIdx.y, S = gridDim.y;
    int n0 = strip * kStripCols + lane * 4;
    if (n0 > N - 4) n0 = N - 4;  // clamp: edge lanes repeat the last column quad and are not written
    const int RB = K / kRowsPerBlock;
    const int rb_begin = slice * rb_per_slice;
    const int rb_end = min(RB, rb_begin + rb_per_slice);
    const int zwords = N / 32 * BITS;

    float acc[M][4];
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[m][c] = 0.f;

    for (int rb = rb_begin + warp; rb < rb_end; rb += kWarps) {
        uint32_t w[4][BITS];
#pragma unroll
        for (int r = 0; r < BITS; ++r) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(qweight + (size_t)(rb * BITS + r) * N + n0));
            w[0][r] = v.x; w[1][r] = v.y; w[2][r] = v.z; w[3][r] = v.w;
        }
        const int k_lane = rb * kRowsPerBlock + lane;
        const int g_lane = group_of_row(g_idx, k_lane, group_size);
        const int src = x_perm ? __ldg(x_perm + k_lane) : k_lane;
        uint32_t xv[MP];
#pragma unroll
        for (int p = 0; p < MP; ++p) {
            const __half a = x[(size_t)(2 * p) * K + src];
            const __half b = (2 * p + 1 < M) ? x[(size_t)(2 * p + 1) * K + src] : __float2half(0.f);
            xv[p] = (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16);
        }
        const bool uniform = __all_sync(0xffffffffu, g_lane == __shfl_sync(0xffffffffu, g_lane, 0));

        float s[4], fz[4];
        int g_cur = -1;
        // j is fully unrolled so that every field position is a compile-time constant
#pragma unroll
        for (int j = 0; j < kRowsPerBlock; ++j) {
            if (j == 0 || !uniform) {
                const int g = __shfl_sync(0xffffffffu, g_lane, uniform ? 0 : j);
                if (g != g_cur) {  // warp-uniform: g comes from a shuffle
                    g_cur = g;
                    const uint2 sv = __ldg(reinterpret_cast<const uint2*>(scales + (size_t)g * N + n0));
                    const float2 s01 = __half22float2(*reinterpret_cast<const __half2*>(&sv.x));
                    const float2 s23 = __half22float2(*reinterpret_cast<const __half2*>(&sv.y));
                    s[0] = s01.x; s[1] = s01.y; s[2] = s23.x; s[3] = s23.y;
                    const int32_t* zrow = qzeros + (size_t)g * zwords;
#pragma unroll
                    for (int c = 0; c < 4; ++c) fz[c] = 8388608.f + (float)zero_point<BITS>(zrow, n0 + c);
                }
            }
            float xf[M];
#pragma unroll
            for (int p = 0; p < MP; ++p) {
                const uint32_t v = __shfl_sync(0xffffffffu, xv[p], j);
                const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&v));
                xf[2 * p] = f.x;
                if (2 * p + 1 < M) xf[2 * p + 1] = f.y;
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                // 2^23 + q is exact in fp32, so (2^23 + q) - (2^23 + zero) is the exact integer q - zero
                const float d = __uint_as_float(0x4B000000u | block_field<BITS>(w[c], j)) - fz[c];
                const float wv = d * s[c];
#pragma unroll
                for (int m = 0; m < M; ++m) acc[m][c] = fmaf(wv, xf[m], acc[m][c]);
            }
        }
    }

    // ---- combine the 8 warps of this CTA ----
#pragma unroll
    for (int m = 0; m < M; ++m)
#pragma unroll
        for (int c = 0; c < 4; ++c) red[warp][m][lane * 4 + c] = acc[m][c];
    __syncthreads();

    const int strip_n0 = strip * kStripCols;
    for (int i = threadIdx.x; i < M * kStripCols; i += kWarps * 32) {
        const int m = i / kStripCols, c = i % kStripCols;
        const int n = strip_n0 + c;
        float v = 0.f;
#pragma unroll
        for (int wv = 0; wv < kWarps; ++wv) v += red[wv][m][c];
        if (n < N) {
            if (S == 1) {
                if (bias) v += __half2float(bias[n]);
                y[(size_t)m * N + n] = __float2half_rn(v);
            } else {
                partials[((size_t)slice * M + m) * N + n] = v;
            }
        }
    }
    if (S == 1) return;

    // ---- combine the K slices: the last CTA of this strip to arrive sums them in order ----
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(counters + strip, 1u);
        is_last = (prev == (unsigned int)(S - 1));
        if (is_last) counters[strip] = 0u;  // leave the scratch ready for the next call
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int i = threadIdx.x; i < M * kStripCols; i += kWarps * 32) {
        const int m = i / kStripCols, c = i % kStripCols;
        const int n = strip_n0 + c;
        if (n >= N) continue;
        float v = 0.f;
        for (int sl = 0; sl < S; ++sl) v += __ldcg(partials + ((size_t)sl * M + m) * N + n);
        if (bias) v += __half2float(bias[n]);
        y[(size_t)m * N + n] = __float2half_rn(v);
    }
}

}  // namespace

// Number of K slices for the general kernel: enough CTAs to fill the device a few times over,
// but never fewer than one row block per warp.
int gemv_generic_slices(int K, int N) {
    const int strips = (N + kStripCols - 1) / kStripCols;
    const int RB = K / kRowsPerBlock;
    int S = (4 * sm_count() + strips - 1) / strips;
    const int max_s = (RB + kWarps - 1) / kWarps;
    if (S > max_s) S = max_s;
    if (S < 1) S = 1;
    if (S > 64) S = 64;
    return S;
}

size_t gemv_generic_workspace_bytes(int M, int K, int N) {
    return kCounterBytes + (size_t)gemv_generic_slices(K, N) * M * N * sizeof(float);
}

template <int BITS, int M>
static int launch(const __half* x, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                  const int32_t* g_idx, const int32_t* x_perm, const __half* bias, __half* y, int K, int N,
                  int group_size, void* workspace, cudaStream_t stream) {
    const int strips = (N + kStripCols - 1) / kStripCols;
    const int S = gemv_generic_slices(K, N);
    const int RB = K / kRowsPerBlock;
    const int rbps = (RB + S - 1) / S;
    if (strips >= kMaxCounters - 1) return B200GPTQ_ERR_TOO_LARGE;  // the last counter word is reserved
    unsigned int* cnt = reinterpret_cast<unsigned int*>(workspace);
    float* partials = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kCounterBytes);
    dim3 grid(strips, S);
    gemv_generic_kernel<BITS, M><<<grid, kWarps * 32, 0, stream>>>(
        x, qweight, qzeros, scales, g_idx, x_perm, bias, y, K, N, group_size, rbps, partials, cnt);
    B200GPTQ_CUDA_TRY(cudaGetLastError());
    return B200GPTQ_OK;
}

template <int BITS>
static int dispatch_m(int M, const __half* x, const int32_t* qweight, const int32_t* qzeros,
                      const __half* scales, const int32_t* g_idx, const int32_t* x_perm, const __half* bias,
                      __half* y, int K, int N, int group_size, void* workspace, cudaStream_t stream) {
#define B200GPTQ_CASE(m)                                                                                  \
    case m:                                                                                               \
        return launch<BITS, m>(x, qweight, qzeros, scales, g_idx, x_perm, bias, y, K, N, group_size,      \
                               workspace, stream);
    switch (M) {
        B200GPTQ_CASE(1) B200GPTQ_CASE(2) B200GPTQ_CASE(3) B200GPTQ_CASE(4)
        B200GPTQ_CASE(5) B200GPTQ_CASE(6) B200GPTQ_CASE(7) B200GPTQ_CASE(8)
    }
#undef B200GPTQ_CASE
    return B200GPTQ_ERR_SHAPE;
}

int gemv_generic_dispatch(const __half* x, const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                          const int32_t* g_idx, const int32_t* x_perm, const __half* bias, __half* y, int M,
                          int K, int N, int bits, int group_size, void* workspace, cudaStream_t stream) {
    switch (bits) {
        case 2: return dispatch_m<2>(M, x, qweight, qzeros, scales, g_idx, x_perm, bias, y, K, N, group_size, workspace, stream);
        case 3: return dispatch_m<3>(M, x, qweight, qzeros, scales, g_idx, x_perm, bias, y, K, N, group_size, workspace, stream);
        case 4: return dispatch_m<4>(M, x, qweight, qzeros, scales, g_idx, x_perm, bias, y, K, N, group_size, workspace, stream);
        case 8: return dispatch_m<8>(M, x, qweight, qzeros, scales, g_idx, x_perm, bias, y, K, N, group_size, workspace, stream);
    }
    return B200GPTQ_ERR_BITS;
}

}  // namespace b200gptq
