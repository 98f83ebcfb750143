// One-shot all-reduce over peer memory for the row-parallel decode GEMV (M <= 8 rows of a few thousand
// columns: 8..18 KB per rank, where only latency counts).
//
// Every rank owns an exchange buffer that all ranks of the node have mapped (CUDA IPC or symmetric
// memory; the caller allocates, zero-fills and maps it).  Layout of a buffer, the same on every rank:
//
//   [0, 256)          status word (sticky, raised when a wait ran out) and padding
//   [256, 4096)       counters[src rank][column group]  uint32: exchanges this rank has done for that column group
//                     (only row `rank` is used, by its owner)
//   [4096, ...)       data[parity][src rank][row][column]  8-byte words {fp32 partial sum, epoch}
//
// An exchange of one 256-column group, done by the ONE thread block that holds the rank's sums of that group
// (no other block touches the group's counter): read the own counter, add one (= epoch), PUSH the rank's partial
// sums into slot `rank` of every other rank's buffer -- each value travels with the epoch in ONE 8-byte store,
// which arrives whole, so there is no fence and no separate flag: one NVLink write latency instead of a write,
// a fence round trip and a flag.  Then every thread waits -- on LOCAL memory only -- until the words of its
// column carry that epoch from all sources, and adds them up in rank order, so every rank gets the same bits.
// Two data slots (parity of the epoch) suffice: a rank cannot start exchange e+2 of a group before it has
// finished e+1, which needs every peer's push of e+1, which a peer issues only after it has finished reading
// exchange e.  Epochs only grow, so a captured CUDA graph can replay the call.
//
// Every wait is bounded by `timeout` clock cycles; when it runs out the thread raises the status word of its own
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
constexpr size_t kTpBufferBytes = kTpDataOffset + (size_t)2 * kTpMaxWorld * kTpMaxRows * kTpMaxCols * sizeof(uint2);

struct TpArgs {
    int rank, world;                     // world <= 1: no exchange
    long long timeout;                   // clock cycles a wait may last
    unsigned char* peer[kTpMaxWorld];    // exchange buffers of all ranks as mapped in this process (peer[rank]: own)
};

__device__ __forceinline__ void st_word_sys(uint2* p, float v, unsigned int epoch) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(epoch) : "memory");
}
__device__ __forceinline__ uint2 ld_word_sys(const uint2* p) {
    uint2 w;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];" : "=r"(w.x), "=r"(w.y) : "l"(p) : "memory");
    return w;
}

// Called by all threads (>= 256) of the block that owns column group `cg`; thread `tid` < 256 holds the rank's
// partial sums v[m] of column cg * 256 + tid.  On return v[m] holds the sum over ranks.  `epoch_sm` is one word of
// shared memory.
template <int MM>
__device__ __forceinline__ void tp_exchange_group(const TpArgs& tp, int cg, int tid, int M, float (&v)[MM],
                                                  unsigned int* epoch_sm) {
    unsigned char* own = tp.peer[tp.rank];
    unsigned int* counter = reinterpret_cast<unsigned int*>(own + kTpFlagsOffset) + tp.rank * kTpMaxGroups + cg;
    if (tid == 0) {
        const unsigned int e = *counter + 1u;   // only this block touches that word
        *counter = e;
        *epoch_sm = e;
    }
    __syncthreads();
    const unsigned int epoch = *epoch_sm;
    if (tid >= 256) return;
    const size_t slot = (size_t)(epoch & 1u) * kTpMaxWorld;
    const int col = cg * 256 + tid;
    for (int p = 0; p < tp.world; ++p) {
        if (p == tp.rank) continue;
        uint2* dst = reinterpret_cast<uint2*>(tp.peer[p] + kTpDataOffset) + ((slot + tp.rank) * kTpMaxRows) * kTpMaxCols + col;
#pragma unroll
        for (int m = 0; m < MM; ++m)
            if (m < M) st_word_sys(dst + (size_t)m * kTpMaxCols, v[m], epoch);
    }
    const uint2* src = reinterpret_cast<const uint2*>(own + kTpDataOffset) + (slot * kTpMaxRows) * kTpMaxCols + col;
    float sum[MM];
#pragma unroll
    for (int m = 0; m < MM; ++m) sum[m] = 0.f;
    const long long t0 = clock64();
    bool late = false;
    for (int p = 0; p < tp.world; ++p) {
#pragma unroll
        for (int m = 0; m < MM; ++m)
            if (m < M) {
                float val = v[m];
                if (p != tp.rank) {
                    const uint2* w = src + ((size_t)p * kTpMaxRows + m) * kTpMaxCols;
                    uint2 got = ld_word_sys(w);
                    while (got.y != epoch && !late) {
                        if (clock64() - t0 > tp.timeout) late = true;
                        got = ld_word_sys(w);
                    }
                    val = __uint_as_float(got.x);
                }
                sum[m] += val;
            }
    }
    if (late) atomicExch(reinterpret_cast<unsigned int*>(own), 2u);   // sticky: a peer did not show up in time
#pragma unroll
    for (int m = 0; m < MM; ++m) v[m] = sum[m];
}

}  // namespace b200gptq
