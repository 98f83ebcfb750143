// Shared device helpers: GPTQ field extraction and launch-side utilities.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/b200gptq.h"

namespace b200gptq {

constexpr int kRowsPerBlock = 32;  // one "row block": 32 rows of K = bits words of qweight per column

// Scratch layout shared by every kernel: the first kCounterBytes hold arrival counters that
// are zero between calls (each kernel resets the ones it used); partial sums follow.  Keeping
// the counter region at a fixed size means no kernel's partial sums ever land on another
// kernel's counters when the same scratch buffer serves different shapes.
constexpr size_t kCounterBytes = 16384;
constexpr int kMaxCounters = (int)(kCounterBytes / sizeof(unsigned int));

__host__ __device__ constexpr int words_per_block(int bits) { return bits; }  // 32 rows * bits / 32

// Thread-local record of the last CUDA runtime error seen by an entry point.
void set_last_cuda_error(int err);

#define B200GPTQ_CUDA_TRY(expr)                                 \
    do {                                                        \
        cudaError_t _e = (expr);                                \
        if (_e != cudaSuccess) {                                \
            ::b200gptq::set_last_cuda_error((int)_e);           \
            return B200GPTQ_ERR_CUDA;                           \
        }                                                       \
    } while (0)

int sm_count();  // multiprocessors of the current device (cached per device)

// ---- field extraction ------------------------------------------------------------------
// Field j (0..31) of one row block whose `BITS` words are w[0..BITS-1].  For 2/4/8 bits
// a word holds 32/BITS fields at bit BITS*i; for 3 bits the three words form one
// 96-bit little-endian stream with field j at bits [3j, 3j+3).
template <int BITS>
__device__ __forceinline__ uint32_t block_field(const uint32_t (&w)[BITS], int j) {
    if constexpr (BITS == 3) {
        const int bit = 3 * j;
        const int wi = bit >> 5, sh = bit & 31;
        uint32_t lo = w[wi];
        uint32_t hi = (wi < 2) ? w[wi + 1] : 0u;
        return __funnelshift_r(lo, hi, sh) & 7u;
    } else {
        constexpr int PF = 32 / BITS;
        return (w[j / PF] >> (BITS * (j % PF))) & ((1u << BITS) - 1u);
    }
}

// Zero-point field of column n from one row of qzeros (packed along N), plus the
// reference's unmasked "+1".
template <int BITS>
__device__ __forceinline__ int zero_point(const int32_t* __restrict__ qzeros_row, int n) {
    const uint32_t* row = reinterpret_cast<const uint32_t*>(qzeros_row);
    if constexpr (BITS == 3) {
        const int t = n >> 5, bit = 3 * (n & 31);
        const int wi = bit >> 5, sh = bit & 31;
        uint32_t lo = __ldg(row + 3 * t + wi);
        uint32_t hi = (wi < 2 && sh > 29) ? __ldg(row + 3 * t + wi + 1) : 0u;
        return (int)(__funnelshift_r(lo, hi, sh) & 7u) + 1;
    } else {
        constexpr int PF = 32 / BITS;
        return (int)((__ldg(row + n / PF) >> (BITS * (n % PF))) & ((1u << BITS) - 1u)) + 1;
    }
}

__device__ __forceinline__ int group_of_row(const int32_t* __restrict__ g_idx, int k, int group_size) {
    return g_idx ? __ldg(g_idx + k) : k / group_size;
}

}  // namespace b200gptq
