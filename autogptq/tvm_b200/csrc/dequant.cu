// Whole-layer unpack + dequantise:  packed GPTQ buffers -> q[K,N] int8 and W[K,N] fp16.
//
// Bit-exact counterpart of the unpack/dequantise half of the reference's torch path
// (auto_gptq/nn_modules/qlinear.py:201-242): W = scale * fp16(q - (zero_field + 1)) with a
// single fp16 rounding.  Streaming kernel: each thread owns 4 adjacent columns of one
// 32-row block, reads its `bits` words per column with 128-bit loads and writes 32 rows.
#include "common.cuh"

namespace b200gptq {

template <int BITS>
__global__ void __launch_bounds__(256)
dequant_kernel(const int32_t* __restrict__ qweight, const int32_t* __restrict__ qzeros,
               const __half* __restrict__ scales, const int32_t* __restrict__ g_idx,
               int K, int N, int group_size, int8_t* __restrict__ q_out, __half* __restrict__ w_out) {
    const int n0 = (blockIdx.x * 32 + threadIdx.x) * 4;
    const int rb = blockIdx.y * blockDim.y + threadIdx.y;
    if (n0 >= N || rb * kRowsPerBlock >= K) return;

    uint32_t w[4][BITS];
#pragma unroll
    for (int r = 0; r < BITS; ++r) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(qweight + (size_t)(rb * BITS + r) * N + n0));
        w[0][r] = v.x; w[1][r] = v.y; w[2][r] = v.z; w[3][r] = v.w;
    }

    int g_prev = -1;
    __half s[4];
    int z[4];
#pragma unroll
    for (int j = 0; j < kRowsPerBlock; ++j) {  // fully unrolled: field positions become constants
        const int k = rb * kRowsPerBlock + j;
        const int g = group_of_row(g_idx, k, group_size);
        if (g != g_prev) {
            g_prev = g;
            const uint2 sv = __ldg(reinterpret_cast<const uint2*>(scales + (size_t)g * N + n0));
            const __half2 s01 = *reinterpret_cast<const __half2*>(&sv.x);
            const __half2 s23 = *reinterpret_cast<const __half2*>(&sv.y);
            s[0] = __low2half(s01); s[1] = __high2half(s01);
            s[2] = __low2half(s23); s[3] = __high2half(s23);
            const int32_t* zrow = qzeros + (size_t)g * (N / 32 * BITS);
#pragma unroll
            for (int c = 0; c < 4; ++c) z[c] = zero_point<BITS>(zrow, n0 + c);
        }
        int q[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) q[c] = (int)block_field<BITS>(w[c], j);
        if (q_out) {
            char4 qv = make_char4((signed char)q[0], (signed char)q[1], (signed char)q[2], (signed char)q[3]);
            *reinterpret_cast<char4*>(q_out + (size_t)k * N + n0) = qv;
        }
        if (w_out) {
            __half h[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) h[c] = __hmul(s[c], __int2half_rn(q[c] - z[c]));
            uint2 ov;
            ov.x = (uint32_t)__half_as_ushort(h[0]) | ((uint32_t)__half_as_ushort(h[1]) << 16);
            ov.y = (uint32_t)__half_as_ushort(h[2]) | ((uint32_t)__half_as_ushort(h[3]) << 16);
            *reinterpret_cast<uint2*>(w_out + (size_t)k * N + n0) = ov;
        }
    }
}

template <int BITS>
static int launch_dequant(const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                          const int32_t* g_idx, int K, int N, int group_size, int8_t* q_out,
                          __half* w_out, cudaStream_t stream) {
    dim3 block(32, 8);
    dim3 grid((N + 127) / 128, (K / kRowsPerBlock + 7) / 8);
    dequant_kernel<BITS><<<grid, block, 0, stream>>>(qweight, qzeros, scales, g_idx, K, N, group_size,
                                                     q_out, w_out);
    B200GPTQ_CUDA_TRY(cudaGetLastError());
    return B200GPTQ_OK;
}

int dequant_dispatch(const int32_t* qweight, const int32_t* qzeros, const __half* scales,
                     const int32_t* g_idx, int K, int N, int bits, int group_size, int8_t* q_out,
                     __half* w_out, cudaStream_t stream) {
    switch (bits) {
        case 2: return launch_dequant<2>(qweight, qzeros, scales, g_idx, K, N, group_size, q_out, w_out, stream);
        case 3: return launch_dequant<3>(qweight, qzeros, scales, g_idx, K, N, group_size, q_out, w_out, stream);
        case 4: return launch_dequant<4>(qweight, qzeros, scales, g_idx, K, N, group_size, q_out, w_out, stream);
        case 8: return launch_dequant<8>(qweight, qzeros, scales, g_idx, K, N, group_size, q_out, w_out, stream);
    }
    return B200GPTQ_ERR_BITS;
}

// ---- row re-ordering (act-order layers) --------------------------------------------------
// Output row block rb of column quad n0 gathers, for each of its 32 rows r, the field of
// original row perm[r]; fields are re-packed with the same layout.
template <int BITS>
__global__ void __launch_bounds__(256)
sort_rows_kernel(const int32_t* __restrict__ qweight, const int32_t* __restrict__ g_idx,
                 const int32_t* __restrict__ perm, int K, int N,
                 int32_t* __restrict__ qweight_sorted, int32_t* __restrict__ g_idx_sorted) {
    const int n0 = (blockIdx.x * 32 + threadIdx.x) * 4;
    const int rb = blockIdx.y * blockDim.y + threadIdx.y;
    if (rb * kRowsPerBlock >= K) return;
    if (blockIdx.x == 0 && g_idx_sorted) {
        const int r = rb * kRowsPerBlock + threadIdx.x;
        g_idx_sorted[r] = g_idx ? g_idx[perm[r]] : 0;
    }
    if (n0 >= N) return;
    uint32_t out[4][BITS];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int r = 0; r < BITS; ++r) out[c][r] = 0u;

#pragma unroll 1
    for (int j = 0; j < kRowsPerBlock; ++j) {
        const int src = __ldg(perm + rb * kRowsPerBlock + j);
        const int sb = src / kRowsPerBlock, sj = src % kRowsPerBlock;
        uint32_t q[4];
        if constexpr (BITS == 3) {
            const int bit = 3 * sj, wi = bit >> 5, sh = bit & 31;
            const uint4 lo = __ldg(reinterpret_cast<const uint4*>(qweight + (size_t)(sb * 3 + wi) * N + n0));
            uint4 hi = make_uint4(0, 0, 0, 0);
            if (sh > 29) hi = __ldg(reinterpret_cast<const uint4*>(qweight + (size_t)(sb * 3 + wi + 1) * N + n0));
            q[0] = __funnelshift_r(lo.x, hi.x, sh) & 7u; q[1] = __funnelshift_r(lo.y, hi.y, sh) & 7u;
            q[2] = __funnelshift_r(lo.z, hi.z, sh) & 7u; q[3] = __funnelshift_r(lo.w, hi.w, sh) & 7u;
        } else {
            constexpr int PF = 32 / BITS;
            constexpr uint32_t MASK = (1u << BITS) - 1u;
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(qweight + (size_t)(sb * BITS + sj / PF) * N + n0));
            const int sh = BITS * (sj % PF);
            q[0] = (v.x >> sh) & MASK; q[1] = (v.y >> sh) & MASK;
            q[2] = (v.z >> sh) & MASK; q[3] = (v.w >> sh) & MASK;
        }
        // insert field j of the output block (j is loop-uniform, so indices resolve statically per case)
        if constexpr (BITS == 3) {
            const int bit = 3 * j, wi = bit >> 5, sh = bit & 31;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
                for (int r = 0; r < 3; ++r) {
                    if (r == wi) out[c][r] |= q[c] << sh;
                    if (r == wi + 1 && sh > 29) out[c][r] |= q[c] >> (32 - sh);
                }
            }
        } else {
            constexpr int PF = 32 / BITS;
            const int wi = j / PF, sh = BITS * (j % PF);
#pragma unroll
            for (int c = 0; c < 4; ++c)
#pragma unroll
                for (int r = 0; r < BITS; ++r)
                    if (r == wi) out[c][r] |= q[c] << sh;
        }
    }
#pragma unroll
    for (int r = 0; r < BITS; ++r) {
        uint4 v = make_uint4(out[0][r], out[1][r], out[2][r], out[3][r]);
        *reinterpret_cast<uint4*>(qweight_sorted + (size_t)(rb * BITS + r) * N + n0) = v;
    }
}

template <int BITS>
static int launch_sort_rows(const int32_t* qweight, const int32_t* g_idx, const int32_t* perm, int K, int N,
                            int32_t* qweight_sorted, int32_t* g_idx_sorted, cudaStream_t stream) {
    dim3 block(32, 8);
    dim3 grid((N + 127) / 128, (K / kRowsPerBlock + 7) / 8);
    sort_rows_kernel<BITS><<<grid, block, 0, stream>>>(qweight, g_idx, perm, K, N, qweight_sorted, g_idx_sorted);
    B200GPTQ_CUDA_TRY(cudaGetLastError());
    return B200GPTQ_OK;
}

int sort_rows_dispatch(const int32_t* qweight, const int32_t* g_idx, const int32_t* perm, int K, int N,
                       int bits, int32_t* qweight_sorted, int32_t* g_idx_sorted, cudaStream_t stream) {
    switch (bits) {
        case 2: return launch_sort_rows<2>(qweight, g_idx, perm, K, N, qweight_sorted, g_idx_sorted, stream);
        case 3: return launch_sort_rows<3>(qweight, g_idx, perm, K, N, qweight_sorted, g_idx_sorted, stream);
        case 4: return launch_sort_rows<4>(qweight, g_idx, perm, K, N, qweight_sorted, g_idx_sorted, stream);
        case 8: return launch_sort_rows<8>(qweight, g_idx, perm, K, N, qweight_sorted, g_idx_sorted, stream);
    }
    return B200GPTQ_ERR_BITS;
}

}  // namespace b200gptq
