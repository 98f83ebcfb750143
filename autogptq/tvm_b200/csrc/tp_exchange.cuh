// One-shot all-reduce over peer memory for the row-parallel decode GEMV (M <= 8 rows of a few thousand
// columns: 8..18 KB per rank, where only latency counts).
//
// Every rank owns an exchange buffer that all ranks of the node have mapped (CUDA IPC or symmetric
// memory; the caller allocates, zero-fills and maps it).  Layout of a buffer, the same on every rank:
//
//   [0, 256)          status word (sticky, raised when a wait ran out) and padding
//   [256, 4096)       flags[src rank][column group]  uint32: how many exchanges that source has completed for
//                     that column group
//   [4096, ...)       data[parity][src rank][row][column]  fp32 partial sums, kTpMaxCols columns per row
//
// An exchange of one 256-column group, done by the ONE thread block that holds the rank's sums of that group
// (no other block touches the group's flags): read the own counter, add one (= epoch), PUSH the rank's
// partial sums into slot `rank` of every rank's buffer (plain stores over NVLink, no reads from peers), fence,
// store the epoch into flags[rank][group] of every buffer, then wait -- on LOCAL memory only -- until all
// sources show that epoch, and add the slots up in rank order, so every rank gets the same bits.
// Two data slots (parity of the epoch) suffice: a rank cannot start exchange e+2 of a group before it has
// finished e+1, which needs every peer's push of e+1, which a peer issues only after it has finished reading
// exchange e.  Counters only grow, so a captured CUDA graph can replay the call.
//
// Every wait is bounded by `timeout` clock cycles; when it runs out the block raises the status word of its own
// buffer and goes on (the result is then undefined, the context stays usable).
//
// No multicast loads, no reads of peer memory at all: peers are only ever written.
#pragma once

#include "common.cuh"

namespace b200gptq {

constexpr int kTpMaxWorld = 8;
constexpr int kTpMaxGroups = 64;                       // 256-column groups per exchange: N <= 16384
constexpr int kTpMaxCols = kTpMaxGroups * 256;
constexpr int kTpMaxRows = 8;
constexpr size_t kTpFlagsOffset = 256;
constexpr size_t kTpDataOffset = 4096;
constexpr size_t kTpBufferBytes = kTpDataOffset + (size_t)2 * kTpMaxWorld * kTpMaxRows * kTpMaxCols * sizeof(float);

struct TpArgs {
    int rank, world;                     // world <= 1: no exchange
    long long timeout;                   // clock cycles a wait may last
    unsigned char* peer[kTpMaxWorld];    // exchange buffers of all ranks as mapped in this process (peer[rank]: own)
};

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Called by all `nthreads` (>= world, a multiple of 32) threads of the block that owns column group `cg`; thread
// `tid` holds the rank's partial sums v[m] of column cg * 256 + tid (tid < 256; other threads only help waiting).
// On return v[m] holds the sum over ranks.  `epoch_sm` is one word of shared memory.
template <int MM>
__device__ __forceinline__ void tp_exchange_group(const TpArgs& tp, int cg, int tid, int M, float (&v)[MM],
                                                  unsigned int* epoch_sm) {
    unsigned char* own = tp.peer[tp.rank];
    unsigned int* own_flags = reinterpret_cast<unsigned int*>(own + kTpFlagsOffset);
    if (tid == 0) *epoch_sm = own_flags[tp.rank * kTpMaxGroups + cg] + 1u;   // only this block writes that word
    __syncthreads();
    const unsigned int epoch = *epoch_sm;
    const size_t slot = (size_t)(epoch & 1u) * kTpMaxWorld;
    const int col = cg * 256 + tid;
    if (tid < 256) {
        for (int p = 0; p < tp.world; ++p) {
            float* dst = reinterpret_cast<float*>(tp.peer[p] + kTpDataOffset) + ((slot + tp.rank) * kTpMaxRows) * kTpMaxCols + col;
#pragma unroll
            for (int m = 0; m < MM; ++m)
                if (m < M) dst[(size_t)m * kTpMaxCols] = v[m];
        }
    }
    __threadfence_system();   // this thread's stores are performed at every GPU before the flags go out
    __syncthreads();
    if (tid < tp.world)
        st_release_sys(reinterpret_cast<unsigned int*>(tp.peer[tid] + kTpFlagsOffset) + tp.rank * kTpMaxGroups + cg, epoch);
    if (tid < tp.world) {
        const unsigned int* f = own_flags + tid * kTpMaxGroups + cg;
        const long long t0 = clock64();
        while ((int)(ld_acquire_sys(f) - epoch) < 0) {
            if (clock64() - t0 > tp.timeout) {
                atomicExch(reinterpret_cast<unsigned int*>(own), 2u);   // sticky: a peer did not show up in time
                break;
            }
        }
    }
    __syncthreads();
    if (tid < 256) {
        const float* src = reinterpret_cast<const float*>(own + kTpDataOffset) + (slot * kTpMaxRows) * kTpMaxCols + col;
#pragma unroll
        for (int m = 0; m < MM; ++m)
            if (m < M) {
                float s = 0.f;
                for (int p = 0; p < tp.world; ++p) s += __ldcv(src + ((size_t)p * kTpMaxRows + m) * kTpMaxCols);
                v[m] = s;
            }
    }
}

}  // namespace b200gptq
