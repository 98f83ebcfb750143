// Packing of integer fields into GPTQ int32 words on the GPU (load-time path, HBM-bound).
//
//   vals  int32 [R, C]  (R a multiple of 32): one field per element, packed along R
//   out   int32 [R / 32 * bits, C]
//
// 2/4/8 bits: field j of a word sits at bit bits*j.  3 bits: the 32 fields of a row block form one
// 96-bit little-endian stream over three words.  Values wider than `bits` are NOT masked: they spill
// into the neighbouring fields exactly as the reference's un-masked `|=` does
// (auto_gptq/nn_modules/qlinear.py:111-134 for qweight, :140-170 for qzeros), with the arithmetic done
// on the value as an unsigned 32-bit number, as numpy does there.
//
// One thread packs one row block of one column: its 32 reads are strided by C, so the threads of a warp
// (consecutive columns) read and write consecutive addresses.
#include "common.cuh"

namespace b200gptq {

namespace {

template <int BITS>
__global__ void __launch_bounds__(256)
pack_fields_kernel(const int32_t* __restrict__ vals, int R, int C, int32_t* __restrict__ out) {
    const int c = blockIdx.x * 32 + threadIdx.x;
    const int rb = blockIdx.y * blockDim.y + threadIdx.y;
    if (c >= C || rb * kRowsPerBlock >= R) return;
    const int32_t* src = vals + (size_t)rb * kRowsPerBlock * C + c;
    uint32_t w[BITS];
#pragma unroll
    for (int i = 0; i < BITS; ++i) w[i] = 0u;
#pragma unroll
    for (int j = 0; j < kRowsPerBlock; ++j) {
        const uint32_t v = (uint32_t)src[(size_t)j * C];
        if constexpr (BITS == 3) {
            const int bit = 3 * j, wi = bit >> 5, sh = bit & 31;
            w[wi] |= v << sh;
            if (sh > 29) w[wi + 1] |= (v >> (32 - sh)) & ((1u << (sh + 3 - 32)) - 1u);
        } else {
            constexpr int PF = 32 / BITS;
            w[j / PF] |= v << (BITS * (j % PF));
        }
    }
    int32_t* dst = out + (size_t)rb * BITS * C + c;
#pragma unroll
    for (int i = 0; i < BITS; ++i) dst[(size_t)i * C] = (int32_t)w[i];
}

template <int BITS>
int launch_pack(const int32_t* vals, int R, int C, int32_t* out, cudaStream_t stream) {
    dim3 block(32, 8);
    dim3 grid((C + 31) / 32, (R / kRowsPerBlock + 7) / 8);
    pack_fields_kernel<BITS><<<grid, block, 0, stream>>>(vals, R, C, out);
    B200GPTQ_CUDA_TRY(cudaGetLastError());
    return B200GPTQ_OK;
}

}  // namespace

int pack_fields_dispatch(const int32_t* vals, int R, int C, int bits, int32_t* out, cudaStream_t stream) {
    switch (bits) {
        case 2: return launch_pack<2>(vals, R, C, out, stream);
        case 3: return launch_pack<3>(vals, R, C, out, stream);
        case 4: return launch_pack<4>(vals, R, C, out, stream);
        case 8: return launch_pack<8>(vals, R, C, out, stream);
    }
    return B200GPTQ_ERR_BITS;
}

}  // namespace b200gptq
