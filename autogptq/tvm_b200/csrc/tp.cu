// Tensor-parallel entry points of the C ABI: the row-parallel decode GEMV with its all-reduce fused into
// the combine step, and the same exchange as a kernel of its own for results that other kernels produced.
// See tp_exchange.cuh for the protocol and include/b200gptq.h for the contract.
#include <cuda.h>

#include <cstring>

#include "common.cuh"
#include "tp_exchange.cuh"

namespace b200gptq {

bool gemv_stream_supported(int M, int K, int N, int bits, int group_size);
int gemv_stream_dispatch_tp(const __half*, const int32_t*, const int32_t*, const __half*, const int32_t*, const __half*,
                            __half*, int, int, int, int, int, void*, cudaStream_t, const int*, const TpArgs*);
int gemv_generic_dispatch(const __half*, const int32_t*, const int32_t*, const __half*, const int32_t*,
                          const int32_t*, const __half*, __half*, int, int, int, int, int, void*, cudaStream_t);

namespace {

// y[M, N] (fp16, this rank's partial sums) -> the sum over ranks (+ bias), in place.  One CTA per 256 columns.
__global__ void __launch_bounds__(256)
allreduce_kernel(__half* __restrict__ y, const __half* __restrict__ bias, int M, int N, const __grid_constant__ TpArgs tp) {
    __shared__ unsigned int epoch;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const int cg = blockIdx.x, tid = threadIdx.x, n = cg * 256 + tid;
    float v[kTpMaxRows];
#pragma unroll
    for (int m = 0; m < kTpMaxRows; ++m) v[m] = (m < M && n < N) ? __half2float(y[(size_t)m * N + n]) : 0.f;
    tp_exchange_group<kTpMaxRows>(tp, cg, tid, M, v, &epoch);
    if (n < N) {
#pragma unroll
        for (int m = 0; m < kTpMaxRows; ++m)
            if (m < M) {
                float o = v[m];
                if (bias) o += __half2float(bias[n]);
                y[(size_t)m * N + n] = __float2half_rn(o);
            }
    }
}

int fill_tp(TpArgs* tp, int rank, int world, void* const* peers, long long timeout_cycles) {
    if (world < 1 || world > kTpMaxWorld || rank < 0 || rank >= world) return B200GPTQ_ERR_SHAPE;
    if (!peers) return B200GPTQ_ERR_NULL_POINTER;
    tp->rank = rank;
    tp->world = world;
    tp->timeout = timeout_cycles > 0 ? timeout_cycles : 20000000000LL;   // ~10 s: ranks may be seconds apart at start-up
    for (int p = 0; p < kTpMaxWorld; ++p) tp->peer[p] = nullptr;
    for (int p = 0; p < world; ++p) {
        if (!peers[p]) return B200GPTQ_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(peers[p]) & 255u) return B200GPTQ_ERR_ALIGNMENT;
        tp->peer[p] = static_cast<unsigned char*>(peers[p]);
    }
    return B200GPTQ_OK;
}

int launch_allreduce(__half* y, const __half* bias, int M, int N, const TpArgs& tp, cudaStream_t stream) {
    const int cgs = (N + 255) / 256;
    if (cgs > kTpMaxGroups) return B200GPTQ_ERR_TOO_LARGE;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(cgs);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200GPTQ_CUDA_TRY(cudaLaunchKernelEx(&cfg, allreduce_kernel, y, bias, M, N, tp));
    return B200GPTQ_OK;
}

}  // namespace
}  // namespace b200gptq

using namespace b200gptq;

extern "C" {

size_t b200gptq_tp_buffer_bytes(void) { return kTpBufferBytes; }

int b200gptq_tp_allreduce(void* y, const void* bias, int M, int N, int rank, int world, void* const* peer_buffers,
                          long long timeout_cycles, void* stream) {
    if (!y) return B200GPTQ_ERR_NULL_POINTER;
    if (M < 1 || M > kTpMaxRows || N < 1) return B200GPTQ_ERR_SHAPE;
    TpArgs tp;
    if (int st = fill_tp(&tp, rank, world, peer_buffers, timeout_cycles)) return st;
    return launch_allreduce(static_cast<__half*>(y), static_cast<const __half*>(bias), M, N, tp,
                            static_cast<cudaStream_t>(stream));
}

int b200gptq_gemv_tp(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                     const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y, int M, int K, int N,
                     int bits, int group_size, void* workspace, size_t workspace_bytes, int rank, int world,
                     void* const* peer_buffers, long long timeout_cycles, int slices_per_sm, int ctas_per_sm,
                     void* stream) {
    return b200gptq_gemv_tp_ex(x, qweight, qzeros, scales, g_idx, x_perm, bias, y, M, K, N, bits, group_size, workspace,
                               workspace_bytes, rank, world, peer_buffers, timeout_cycles, slices_per_sm, ctas_per_sm,
                               B200GPTQ_ACT_NONE, stream);
}

int b200gptq_gemv_tp_ex(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                        const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y, int M, int K, int N,
                        int bits, int group_size, void* workspace, size_t workspace_bytes, int rank, int world,
                        void* const* peer_buffers, long long timeout_cycles, int slices_per_sm, int ctas_per_sm,
                        int input_act, void* stream) {
    if (slices_per_sm < 0 || slices_per_sm > 8 || ctas_per_sm < 0 || ctas_per_sm > 4) return B200GPTQ_ERR_SHAPE;
    if (input_act != B200GPTQ_ACT_NONE && input_act != B200GPTQ_ACT_SWIGLU && input_act != B200GPTQ_ACT_RELU)
        return B200GPTQ_ERR_SHAPE;
    const int knobs[6] = {slices_per_sm, ctas_per_sm, 0, 0, 0, input_act};
    if (!x || !qweight || !qzeros || !scales || !y) return B200GPTQ_ERR_NULL_POINTER;
    if (bits != 2 && bits != 3 && bits != 4 && bits != 8) return B200GPTQ_ERR_BITS;
    if (K <= 0 || N <= 0 || K % 32 != 0 || N % 32 != 0 || M < 1 || M > 8) return B200GPTQ_ERR_SHAPE;
    if (group_size == -1) group_size = K;
    if (group_size <= 0) return B200GPTQ_ERR_SHAPE;
    auto mis = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) != 0; };
    if (mis(qweight) || mis(x) || mis(y) || mis(scales) || mis(qzeros) || mis(workspace)) return B200GPTQ_ERR_ALIGNMENT;
    if (!workspace || workspace_bytes < b200gptq_workspace_bytes(B200GPTQ_OP_GEMV, M, K, N, bits))
        return B200GPTQ_ERR_WORKSPACE;
    TpArgs tp;
    if (int st = fill_tp(&tp, rank, world, peer_buffers, timeout_cycles)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool streams = !g_idx && gemv_stream_supported(M, K, N, bits, group_size);
    // the activation is part of the streaming kernel's read of x only (and SwiGLU not together with a gather)
    if (input_act != B200GPTQ_ACT_NONE && (!streams || (input_act == B200GPTQ_ACT_SWIGLU && x_perm))) return B200GPTQ_ERR_SHAPE;
    if (streams)
        return gemv_stream_dispatch_tp(static_cast<const __half*>(x), qweight, qzeros, static_cast<const __half*>(scales),
                                       x_perm, static_cast<const __half*>(bias), static_cast<__half*>(y), M, K, N, bits,
                                       group_size, workspace, s, (slices_per_sm || ctas_per_sm || input_act) ? knobs : nullptr,
                                       world > 1 ? &tp : nullptr);
    // general kernel: this rank's sums first (without the bias), then the exchange as a kernel of its own
    if (int st = gemv_generic_dispatch(static_cast<const __half*>(x), qweight, qzeros, static_cast<const __half*>(scales),
                                       g_idx, x_perm, world > 1 ? nullptr : static_cast<const __half*>(bias),
                                       static_cast<__half*>(y), M, K, N, bits, group_size, workspace, s))
        return st;
    if (world == 1) return B200GPTQ_OK;
    return launch_allreduce(static_cast<__half*>(y), static_cast<const __half*>(bias), M, N, tp, s);
}

int b200gptq_tp_enable_peer(int peer_device) {
    int dev = 0;
    B200GPTQ_CUDA_TRY(cudaGetDevice(&dev));
    if (peer_device == dev) return B200GPTQ_OK;
    int can = 0;
    B200GPTQ_CUDA_TRY(cudaDeviceCanAccessPeer(&can, dev, peer_device));
    if (!can) { set_last_cuda_error((int)cudaErrorPeerAccessUnsupported); return B200GPTQ_ERR_CUDA; }
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) { (void)cudaGetLastError(); return B200GPTQ_OK; }
    B200GPTQ_CUDA_TRY(e);
    return B200GPTQ_OK;
}

int b200gptq_tp_export(const void* device_ptr, void* ipc_handle_out, size_t* offset_out) {
    if (!device_ptr || !ipc_handle_out || !offset_out) return B200GPTQ_ERR_NULL_POINTER;
    // the handle names the whole allocation that contains the pointer; the offset locates the pointer inside it
    typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    static const RangeFn range = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<RangeFn>(p);
    }();
    if (!range) { set_last_cuda_error((int)cudaErrorNotSupported); return B200GPTQ_ERR_CUDA; }
    CUdeviceptr base = 0;
    size_t size = 0;
    if (range(&base, &size, (CUdeviceptr)device_ptr) != CUDA_SUCCESS) {
        set_last_cuda_error((int)cudaErrorInvalidValue);
        return B200GPTQ_ERR_CUDA;
    }
    cudaIpcMemHandle_t h;
    B200GPTQ_CUDA_TRY(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
    memcpy(ipc_handle_out, &h, sizeof(h));
    *offset_out = (size_t)((CUdeviceptr)device_ptr - base);
    return B200GPTQ_OK;
}

int b200gptq_tp_open_peer(const void* ipc_handle, void** mapped) {
    if (!ipc_handle || !mapped) return B200GPTQ_ERR_NULL_POINTER;
    cudaIpcMemHandle_t h;
    memcpy(&h, ipc_handle, sizeof(h));
    void* p = nullptr;
    // mapped into the CURRENT device's address space; peer access to the owning device is enabled on the way
    B200GPTQ_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *mapped = p;
    return B200GPTQ_OK;
}

int b200gptq_tp_close_peer(void* mapped) {
    if (!mapped) return B200GPTQ_OK;
    B200GPTQ_CUDA_TRY(cudaIpcCloseMemHandle(mapped));
    return B200GPTQ_OK;
}

int b200gptq_tp_probe(const void* device_ptr, unsigned int* host_out) {
    if (!device_ptr || !host_out) return B200GPTQ_ERR_NULL_POINTER;
    B200GPTQ_CUDA_TRY(cudaMemcpy(host_out, device_ptr, sizeof(unsigned int), cudaMemcpyDeviceToHost));
    return B200GPTQ_OK;
}

int b200gptq_tp_status(const void* own_buffer, void* stream, unsigned int* host_out) {
    if (!own_buffer || !host_out) return B200GPTQ_ERR_NULL_POINTER;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    B200GPTQ_CUDA_TRY(cudaMemcpyAsync(host_out, own_buffer, sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
    B200GPTQ_CUDA_TRY(cudaStreamSynchronize(s));
    return B200GPTQ_OK;
}

}  // extern "C"
