// b200gptq_gemv_static: the decode GEMV for callers that cannot hand over scratch memory.
//
// Some hosts of this library have no way to allocate device memory at the point where they call a
// kernel: a plugin that runs inside another runtime's launch callback, an engine that froze its
// memory plan at build time, a real-time loop in which cudaMalloc (a synchronising call of unbounded
// duration) is forbidden.  For them the fp32 partial sums and arrival counters that the GEMV
// kernels need live in a fixed array inside this library's device image instead of a caller buffer.
//
// Consequences, all visible in the interface contract:
//  * every GPU whose context loads the library holds kStaticScratchBytes of device memory until the
//    context dies;
//  * problems whose scratch need exceeds that size are refused (B200GPTQ_ERR_TOO_LARGE);
//  * all calls on a device share the one array, so two calls that may overlap on the GPU (different
//    streams without an ordering between them) race; calls ordered on one stream are safe.  The
//    array keeps whatever the previous call left: the kernels return their arrival counters to
//    zero before they finish and write every partial-sum slot before reading it, so nothing else
//    needs clearing between calls;
//  * the first call on each device resolves the array's device address with a runtime call
//    (cudaGetSymbolAddress).  Make that first call outside any stream capture.
#include <mutex>

#include "common.cuh"

namespace b200gptq {

int gemv_generic_dispatch(const __half*, const int32_t*, const int32_t*, const __half*, const int32_t*,
                          const int32_t*, const __half*, __half*, int, int, int, int, int, void*, cudaStream_t);
bool gemv_stream_supported(int M, int K, int N, int bits, int group_size);
int gemv_stream_dispatch(const __half*, const int32_t*, const int32_t*, const __half*, const int32_t*,
                         const int32_t*, const __half*, __half*, int, int, int, int, int, void*, cudaStream_t);

namespace {

constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB per device

// In host code this name is only a handle for the runtime's symbol table, not a device address;
// the address the kernels receive comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void* g_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device; resolved once per device.
int static_scratch(void** out) {
    int dev = 0;
    B200GPTQ_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return B200GPTQ_ERR_TOO_LARGE;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_ptr[dev]) {
        void* ptr = nullptr;
        // The array is zero-initialised static storage and the kernels leave their counters at zero, so nothing has
        // to be cleared here (a memset on the default stream would not be ordered with the caller's stream anyway).
        B200GPTQ_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return B200GPTQ_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace b200gptq

using namespace b200gptq;

extern "C" {

size_t b200gptq_gemv_static_capacity(void) { return kStaticScratchBytes; }

int b200gptq_gemv_static(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                         const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y, int M, int K, int N,
                         int bits, int group_size, void* stream) {
    if (!x || !qweight || !qzeros || !scales || !y) return B200GPTQ_ERR_NULL_POINTER;
    if (bits != 2 && bits != 3 && bits != 4 && bits != 8) return B200GPTQ_ERR_BITS;
    if (K <= 0 || N <= 0 || K % 32 != 0 || N % 32 != 0 || M < 1 || M > 8) return B200GPTQ_ERR_SHAPE;
    if (group_size == -1) group_size = K;
    if (group_size <= 0) return B200GPTQ_ERR_SHAPE;
    if (!aligned16(qweight) || !aligned16(x) || !aligned16(y) || !aligned16(scales) || !aligned16(qzeros))
        return B200GPTQ_ERR_ALIGNMENT;
    if (b200gptq_workspace_bytes(B200GPTQ_OP_GEMV, M, K, N, bits) > kStaticScratchBytes)
        return B200GPTQ_ERR_TOO_LARGE;
    void* scratch = nullptr;
    if (int st = static_scratch(&scratch)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (!g_idx && gemv_stream_supported(M, K, N, bits, group_size))
        return gemv_stream_dispatch(static_cast<const __half*>(x), qweight, qzeros, static_cast<const __half*>(scales),
                                    g_idx, x_perm, static_cast<const __half*>(bias), static_cast<__half*>(y), M, K, N,
                                    bits, group_size, scratch, s);
    return gemv_generic_dispatch(static_cast<const __half*>(x), qweight, qzeros, static_cast<const __half*>(scales),
                                 g_idx, x_perm, static_cast<const __half*>(bias), static_cast<__half*>(y), M, K, N, bits,
                                 group_size, scratch, s);
}

// The sticky status word of the built-in scratch on the current device (see b200gptq_workspace_status).
int b200gptq_gemv_static_status(void* stream, unsigned int* host_out) {
    if (!host_out) return B200GPTQ_ERR_NULL_POINTER;
    void* scratch = nullptr;
    if (int st = static_scratch(&scratch)) return st;
    return b200gptq_workspace_status(scratch, stream, host_out);
}

}  // extern "C"
