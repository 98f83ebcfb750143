// placeholder until the streaming kernel lands
#include "common.cuh"
namespace b200gptq {
bool gemv_stream_supported(int, int, int, int, int) { return false; }
size_t gemv_stream_workspace_bytes(int, int, int, int) { return 0; }
int gemv_stream_dispatch(const __half*, const int32_t*, const int32_t*, const __half*, const int32_t*,
                         const int32_t*, const __half*, __half*, int, int, int, int, int, void*, cudaStream_t) {
    return B200GPTQ_ERR_SHAPE;
}
}  // namespace b200gptq
