// extern "C" boundary: argument validation and dispatch.  See include/b200gptq.h.
#include <mutex>
#include <new>

#include "common.cuh"

namespace b200gptq {

static thread_local int tls_last_cuda_error = 0;
void set_last_cuda_error(int err) { tls_last_cuda_error = err; }

int sm_count() {
    // looked up once per device; afterwards the launch path only reads (no lock)
    static std::once_flag once[64];
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::call_once(once[dev], [dev] {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    });
    return cached[dev];
}

// implemented in the kernel translation units
int dequant_dispatch(const int32_t*, const int32_t*, const __half*, const int32_t*, int, int, int, int, int8_t*,
                     __half*, cudaStream_t);
int pack_fields_dispatch(const int32_t*, int, int, int, int32_t*, cudaStream_t);
int sort_rows_dispatch(const int32_t*, const int32_t*, const int32_t*, int, int, int, int32_t*, int32_t*,
                       cudaStream_t);
int gemv_generic_dispatch(const __half*, const int32_t*, const int32_t*, const __half*, const int32_t*,
                          const int32_t*, const __half*, __half*, int, int, int, int, int, void*, cudaStream_t);
size_t gemv_generic_workspace_bytes(int M, int K, int N);
bool gemv_stream_supported(int M, int K, int N, int bits, int group_size);
size_t gemv_stream_workspace_bytes(int M, int K, int N, int bits);
int gemv_stream_dispatch(const __half*, const int32_t*, const int32_t*, const __half*, const int32_t*,
                         const int32_t*, const __half*, __half*, int, int, int, int, int, void*, cudaStream_t);
int gemv_stream_dispatch_knobs(const __half*, const int32_t*, const int32_t*, const __half*, const int32_t*,
                               const __half*, __half*, int, int, int, int, int, void*, cudaStream_t, const int*);
size_t gemm_workspace_bytes(int M, int K, int N, int bits);
void gemm_split_query(int M, int K, int N, int* splits, int* ctas_per_sm);
int gemm_dispatch(const __half*, const int32_t*, const int32_t*, const __half*, const int32_t*, const int32_t*,
                  const __half*, __half*, int, int, int, int, int, void*, size_t, cudaStream_t);

struct GemvStreamPlan;
GemvStreamPlan* gemv_stream_plan_create(const int32_t*, const __half*, bool, int, int, int, int, int, const int*, int*);
int gemv_stream_plan_run(const GemvStreamPlan*, const __half*, const int32_t*, const int32_t*, const __half*, __half*,
                         void*, cudaStream_t);
void gemv_stream_plan_destroy(GemvStreamPlan*);

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Packing rules shared by every entry point.
static int check_layer(int K, int N, int bits, int* group_size) {
    if (bits != 2 && bits != 3 && bits != 4 && bits != 8) return B200GPTQ_ERR_BITS;
    if (K <= 0 || N <= 0 || K % 32 != 0) return B200GPTQ_ERR_SHAPE;
    if (N % 32 != 0) return B200GPTQ_ERR_SHAPE;  // qzeros holds N/32*bits words per group
    if (*group_size == -1) *group_size = K;
    if (*group_size <= 0) return B200GPTQ_ERR_SHAPE;
    return B200GPTQ_OK;
}

}  // namespace b200gptq

using namespace b200gptq;

extern "C" {

const char* b200gptq_strerror(int status) {
    switch (status) {
        case B200GPTQ_OK: return "ok";
        case B200GPTQ_ERR_NULL_POINTER: return "a required pointer is NULL";
        case B200GPTQ_ERR_BITS: return "unsupported bit width for this entry point";
        case B200GPTQ_ERR_SHAPE: return "K, N, M or group_size violate the packing rules (K % 32 == 0, N % 32 == 0)";
        case B200GPTQ_ERR_ALIGNMENT: return "a device pointer is not 16-byte aligned";
        case B200GPTQ_ERR_WORKSPACE: return "workspace missing or smaller than b200gptq_workspace_bytes()";
        case B200GPTQ_ERR_CUDA: return "CUDA runtime error; see b200gptq_last_cuda_error()";
        case B200GPTQ_ERR_GROUPS: return "g_idx must be constant over aligned 32-row blocks for this entry point";
        case B200GPTQ_ERR_TOO_LARGE: return "problem exceeds a fixed capacity of this entry point";
    }
    return "unknown status";
}

int b200gptq_last_cuda_error(void) { return tls_last_cuda_error; }

int b200gptq_abi_version(void) { return 1; }

int b200gptq_dequant(const int32_t* qweight, const int32_t* qzeros, const void* scales, const int32_t* g_idx,
                     int K, int N, int bits, int group_size, int8_t* q_out, void* w_out, void* stream) {
    if (!qweight || !qzeros || !scales) return B200GPTQ_ERR_NULL_POINTER;
    if (int st = check_layer(K, N, bits, &group_size)) return st;
    if (bits == 8 && q_out) return B200GPTQ_ERR_BITS;
    if (!aligned16(qweight) || (w_out && !aligned16(w_out)) || (q_out && !aligned16(q_out)) ||
        (reinterpret_cast<uintptr_t>(scales) & 7u))
        return B200GPTQ_ERR_ALIGNMENT;
    if (!q_out && !w_out) return B200GPTQ_OK;
    return dequant_dispatch(qweight, qzeros, static_cast<const __half*>(scales), g_idx, K, N, bits, group_size,
                            q_out, static_cast<__half*>(w_out), static_cast<cudaStream_t>(stream));
}

int b200gptq_pack_fields(const int32_t* vals, int R, int C, int bits, int32_t* out, void* stream) {
    if (!vals || !out) return B200GPTQ_ERR_NULL_POINTER;
    if (bits != 2 && bits != 3 && bits != 4 && bits != 8) return B200GPTQ_ERR_BITS;
    if (R <= 0 || C <= 0 || R % 32 != 0) return B200GPTQ_ERR_SHAPE;
    return pack_fields_dispatch(vals, R, C, bits, out, static_cast<cudaStream_t>(stream));
}

int b200gptq_sort_rows(const int32_t* qweight, const int32_t* g_idx, const int32_t* perm, int K, int N, int bits,
                       int32_t* qweight_sorted, int32_t* g_idx_sorted, void* stream) {
    if (!qweight || !perm || !qweight_sorted || !g_idx) return B200GPTQ_ERR_NULL_POINTER;
    int gs = K;
    if (int st = check_layer(K, N, bits, &gs)) return st;
    if (!aligned16(qweight) || !aligned16(qweight_sorted)) return B200GPTQ_ERR_ALIGNMENT;
    return sort_rows_dispatch(qweight, g_idx, perm, K, N, bits, qweight_sorted, g_idx_sorted,
                              static_cast<cudaStream_t>(stream));
}

size_t b200gptq_workspace_bytes(int op, int M, int K, int N, int bits) {
    if (M <= 0 || K <= 0 || N <= 0) return 0;
    if (op == B200GPTQ_OP_GEMV) {
        size_t a = gemv_generic_workspace_bytes(M, K, N);
        size_t b = gemv_stream_workspace_bytes(M, K, N, bits);
        return a > b ? a : b;
    }
    if (op == B200GPTQ_OP_GEMM) return gemm_workspace_bytes(M, K, N, bits);
    return 0;
}

int b200gptq_workspace_status(const void* workspace, void* stream, unsigned int* host_out) {
    if (!workspace || !host_out) return B200GPTQ_ERR_NULL_POINTER;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned int* word = static_cast<const unsigned int*>(workspace) + (kMaxCounters - 1);
    B200GPTQ_CUDA_TRY(cudaMemcpyAsync(host_out, word, sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
    B200GPTQ_CUDA_TRY(cudaStreamSynchronize(s));
    return B200GPTQ_OK;
}

int b200gptq_gemv_path(int M, int K, int N, int bits, int group_size, int has_g_idx) {
    if (int st = check_layer(K, N, bits, &group_size)) return st;
    if (M < 1 || M > 8) return B200GPTQ_ERR_SHAPE;
    return (!has_g_idx && gemv_stream_supported(M, K, N, bits, group_size)) ? B200GPTQ_PATH_STREAM
                                                                           : B200GPTQ_PATH_GENERIC;
}

int b200gptq_gemm_split(int M, int K, int N, int bits, int* splits, int* ctas_per_sm) {
    if (!splits || !ctas_per_sm) return B200GPTQ_ERR_NULL_POINTER;
    int group_size = -1;
    if (int st = check_layer(K, N, bits, &group_size)) return st;
    if (bits != 3 && bits != 4) return B200GPTQ_ERR_BITS;
    if (M < 1) return B200GPTQ_ERR_SHAPE;
    gemm_split_query(M, K, N, splits, ctas_per_sm);
    return B200GPTQ_OK;
}

int b200gptq_gemv(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                  const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y, int M, int K, int N,
                  int bits, int group_size, void* workspace, size_t workspace_bytes, void* stream) {
    return b200gptq_gemv_tuned(x, qweight, qzeros, scales, g_idx, x_perm, bias, y, M, K, N, bits, group_size,
                               workspace, workspace_bytes, 0, 0, stream);
}

int b200gptq_gemv_tuned(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                        const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y, int M, int K, int N,
                        int bits, int group_size, void* workspace, size_t workspace_bytes, int slices_per_sm,
                        int ctas_per_sm, void* stream) {
    return b200gptq_gemv_ex(x, qweight, qzeros, scales, g_idx, x_perm, bias, y, M, K, N, bits, group_size, workspace,
                            workspace_bytes, slices_per_sm, ctas_per_sm, B200GPTQ_ACT_NONE, stream);
}

// An input activation is folded into the streaming kernel's read of x only: the general kernel does not have it,
// and SwiGLU reads two runs of the row, which the gather path's single copy of x does not hold.
static bool act_supported(int input_act, bool streams, const int32_t* x_perm) {
    if (input_act == B200GPTQ_ACT_NONE) return true;
    if (input_act != B200GPTQ_ACT_SWIGLU && input_act != B200GPTQ_ACT_RELU) return false;
    return streams && !(input_act == B200GPTQ_ACT_SWIGLU && x_perm);
}

int b200gptq_gemv_ex(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                     const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y, int M, int K, int N,
                     int bits, int group_size, void* workspace, size_t workspace_bytes, int slices_per_sm,
                     int ctas_per_sm, int input_act, void* stream) {
    if (slices_per_sm < 0 || slices_per_sm > 8 || ctas_per_sm < 0 || ctas_per_sm > 4) return B200GPTQ_ERR_SHAPE;
    if (!x || !qweight || !qzeros || !scales || !y) return B200GPTQ_ERR_NULL_POINTER;
    if (int st = check_layer(K, N, bits, &group_size)) return st;
    if (M < 1 || M > 8) return B200GPTQ_ERR_SHAPE;
    if (!aligned16(qweight) || !aligned16(x) || !aligned16(y) || !aligned16(scales) || !aligned16(qzeros))
        return B200GPTQ_ERR_ALIGNMENT;
    if (!workspace || workspace_bytes < b200gptq_workspace_bytes(B200GPTQ_OP_GEMV, M, K, N, bits))
        return B200GPTQ_ERR_WORKSPACE;
    if (!aligned16(workspace)) return B200GPTQ_ERR_ALIGNMENT;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool streams = !g_idx && gemv_stream_supported(M, K, N, bits, group_size);
    if (!act_supported(input_act, streams, x_perm)) return B200GPTQ_ERR_SHAPE;
    if (streams) {
        const int knobs[6] = {slices_per_sm, ctas_per_sm, 0, 0, 0, input_act};
        return gemv_stream_dispatch_knobs(static_cast<const __half*>(x), qweight, qzeros,
                                          static_cast<const __half*>(scales), x_perm, static_cast<const __half*>(bias),
                                          static_cast<__half*>(y), M, K, N, bits, group_size, workspace, st,
                                          (slices_per_sm || ctas_per_sm || input_act) ? knobs : nullptr);
    }
    return gemv_generic_dispatch(static_cast<const __half*>(x), qweight, qzeros, static_cast<const __half*>(scales),
                                 g_idx, x_perm, static_cast<const __half*>(bias), static_cast<__half*>(y), M, K, N,
                                 bits, group_size, workspace, st);
}

// A plan remembers the layer and everything that can be decided before x is known.
struct b200gptq_gemv_plan {
    const int32_t *qweight, *qzeros, *g_idx, *x_perm;
    const __half *scales, *bias;
    int M, K, N, bits, group_size, slices_per_sm, ctas_per_sm;
    size_t workspace_need;
    b200gptq::GemvStreamPlan* stream;   // NULL: the general kernel serves this problem
};

int b200gptq_gemv_plan_create(b200gptq_gemv_plan** out, const int32_t* qweight, const int32_t* qzeros,
                              const void* scales, const int32_t* g_idx, const int32_t* x_perm, const void* bias,
                              int M, int K, int N, int bits, int group_size, int slices_per_sm, int ctas_per_sm) {
    return b200gptq_gemv_plan_create_ex(out, qweight, qzeros, scales, g_idx, x_perm, bias, M, K, N, bits, group_size,
                                        slices_per_sm, ctas_per_sm, B200GPTQ_ACT_NONE);
}

int b200gptq_gemv_plan_create_ex(b200gptq_gemv_plan** out, const int32_t* qweight, const int32_t* qzeros,
                                 const void* scales, const int32_t* g_idx, const int32_t* x_perm, const void* bias,
                                 int M, int K, int N, int bits, int group_size, int slices_per_sm, int ctas_per_sm,
                                 int input_act) {
    if (!out || !qweight || !qzeros || !scales) return B200GPTQ_ERR_NULL_POINTER;
    *out = nullptr;
    if (int st = check_layer(K, N, bits, &group_size)) return st;
    if (M < 1 || M > 8) return B200GPTQ_ERR_SHAPE;
    if (slices_per_sm < 0 || slices_per_sm > 8 || ctas_per_sm < 0 || ctas_per_sm > 4) return B200GPTQ_ERR_SHAPE;
    if (!aligned16(qweight) || !aligned16(scales) || !aligned16(qzeros)) return B200GPTQ_ERR_ALIGNMENT;
    b200gptq_gemv_plan* p = new (std::nothrow) b200gptq_gemv_plan;
    if (!p) return B200GPTQ_ERR_CUDA;
    *p = {qweight, qzeros, g_idx, x_perm, static_cast<const __half*>(scales), static_cast<const __half*>(bias),
          M, K, N, bits, group_size, slices_per_sm, ctas_per_sm,
          b200gptq_workspace_bytes(B200GPTQ_OP_GEMV, M, K, N, bits), nullptr};
    const bool streams = !g_idx && gemv_stream_supported(M, K, N, bits, group_size);
    if (!act_supported(input_act, streams, x_perm)) { delete p; return B200GPTQ_ERR_SHAPE; }
    if (streams) {
        const int knobs[6] = {slices_per_sm, ctas_per_sm, 0, 0, 0, input_act};
        int st = B200GPTQ_OK;
        p->stream = gemv_stream_plan_create(qweight, p->scales, x_perm != nullptr, M, K, N, bits, group_size,
                                            (slices_per_sm || ctas_per_sm || input_act) ? knobs : nullptr, &st);
        if (!p->stream) { delete p; return st; }
    }
    *out = p;
    return B200GPTQ_OK;
}

int b200gptq_gemv_plan_run(const b200gptq_gemv_plan* p, const void* x, void* y, void* workspace,
                           size_t workspace_bytes, void* stream) {
    if (!p || !x || !y) return B200GPTQ_ERR_NULL_POINTER;
    if (!aligned16(x) || !aligned16(y) || (workspace && !aligned16(workspace))) return B200GPTQ_ERR_ALIGNMENT;
    if (!workspace || workspace_bytes < p->workspace_need) return B200GPTQ_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (p->stream)
        return gemv_stream_plan_run(p->stream, static_cast<const __half*>(x), p->qzeros, p->x_perm, p->bias,
                                    static_cast<__half*>(y), workspace, st);
    return gemv_generic_dispatch(static_cast<const __half*>(x), p->qweight, p->qzeros, p->scales, p->g_idx, p->x_perm,
                                 p->bias, static_cast<__half*>(y), p->M, p->K, p->N, p->bits, p->group_size, workspace,
                                 st);
}

void b200gptq_gemv_plan_destroy(b200gptq_gemv_plan* p) {
    if (!p) return;
    if (p->stream) gemv_stream_plan_destroy(p->stream);
    delete p;
}

int b200gptq_gemm(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                  const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y, int M, int K, int N,
                  int bits, int group_size, void* workspace, size_t workspace_bytes, void* stream) {
    if (!x || !qweight || !qzeros || !scales || !y) return B200GPTQ_ERR_NULL_POINTER;
    if (int st = check_layer(K, N, bits, &group_size)) return st;
    if (bits != 3 && bits != 4) return B200GPTQ_ERR_BITS;
    if (M < 1) return B200GPTQ_ERR_SHAPE;
    // the kernel takes one group per aligned 32-row block: without a g_idx that holds only for such group sizes
    if (!g_idx && group_size % 32 != 0) return B200GPTQ_ERR_GROUPS;
    if (!aligned16(qweight) || !aligned16(x) || !aligned16(y) || !aligned16(scales) || !aligned16(qzeros))
        return B200GPTQ_ERR_ALIGNMENT;
    const size_t need = b200gptq_workspace_bytes(B200GPTQ_OP_GEMM, M, K, N, bits);
    if (need && (!workspace || workspace_bytes < need)) return B200GPTQ_ERR_WORKSPACE;
    if (workspace && !aligned16(workspace)) return B200GPTQ_ERR_ALIGNMENT;
    return gemm_dispatch(static_cast<const __half*>(x), qweight, qzeros, static_cast<const __half*>(scales), g_idx,
                         x_perm, static_cast<const __half*>(bias), static_cast<__half*>(y), M, K, N, bits,
                         group_size, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
