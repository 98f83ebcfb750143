/*
 * b200gptq -- C ABI of the B200 (sm_100a) GPTQ QuantLinear forward kernels.
 *
 * Every entry point takes plain device pointers and sizes, launches on the
 * caller's stream, never synchronises, never allocates device memory, and
 * returns 0 on success or a negative B200GPTQ_ERR_* code.  Nothing throws,
 * aborts or prints.  All buffers are owned by the caller.
 *
 * Buffer formats are the standard AutoGPTQ ones
 * (auto_gptq/nn_modules/qlinear.py:40-59 of the reference):
 *   qweight int32 [K/32*bits, N]   row-major, fields packed along K
 *   qzeros  int32 [G, N/32*bits]   fields packed along N, stored value = zero - 1
 *   scales  fp16  [G, N]
 *   g_idx   int32 [K]              group of row k; NULL means k / group_size
 *   bias    fp16  [N] or NULL
 *   x       fp16  [M, K], y fp16 [M, N], both row-major and dense
 * with G = ceil(K / group_size) (group_size == -1 means one group, G = 1).
 *
 * These functions replace, for the reference, the per-shape kernel handler
 * `handler(x, qweight, y, scales, zeros)` that
 * auto_gptq/nn_modules/tvm_untils/pycuda_warpper.py:138-189 builds with TVM and
 * launches through pycuda, and the dequantise-then-matmul arithmetic of
 * auto_gptq/nn_modules/qlinear.py:197-243 that defines its results.
 */
#ifndef B200GPTQ_H_
#define B200GPTQ_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define B200GPTQ_API __attribute__((visibility("default")))
#else
#define B200GPTQ_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

#define B200GPTQ_OK 0
#define B200GPTQ_ERR_NULL_POINTER (-1)   /* a required pointer is NULL */
#define B200GPTQ_ERR_BITS (-2)           /* bits not supported by this entry point */
#define B200GPTQ_ERR_SHAPE (-3)          /* K, N, M or group_size violate the packing rules */
#define B200GPTQ_ERR_ALIGNMENT (-4)      /* a pointer is not 16-byte aligned */
#define B200GPTQ_ERR_WORKSPACE (-5)      /* workspace missing or smaller than b200gptq_workspace_bytes() */
#define B200GPTQ_ERR_CUDA (-6)           /* the CUDA runtime refused the launch; see b200gptq_last_cuda_error() */
#define B200GPTQ_ERR_GROUPS (-7)         /* this entry point needs g_idx constant over aligned 32-row blocks */
#define B200GPTQ_ERR_TOO_LARGE (-8)      /* the problem exceeds a fixed capacity of this entry point */

/* op selectors of b200gptq_workspace_bytes() */
#define B200GPTQ_OP_GEMV 1
#define B200GPTQ_OP_GEMM 2

/* Text for a status code.  Never NULL. */
B200GPTQ_API const char* b200gptq_strerror(int status);

/* cudaError_t of the most recent B200GPTQ_ERR_CUDA on the calling thread (0 if none). */
B200GPTQ_API int b200gptq_last_cuda_error(void);

/* ABI version; bumped when a signature changes. */
B200GPTQ_API int b200gptq_abi_version(void);

/*
 * Unpack and dequantise a whole layer.
 *   q_out  int8 [K, N]  (nullable)  q[k,n], the integer field
 *   w_out  fp16 [K, N]  (nullable)  W[k,n] = scales[g,n] * fp16(q[k,n] - (qzeros_field[g,n] + 1)),
 *                                   g = g_idx[k]; one fp16 rounding, no flush-to-zero
 * bits in {2,3,4,8} (q_out must be NULL for 8 bits).  Bit-exact restatement of the
 * unpack / dequantise half of qlinear.py:201-242.
 */
B200GPTQ_API int b200gptq_dequant(const int32_t* qweight, const int32_t* qzeros, const void* scales,
                     const int32_t* g_idx, int K, int N, int bits, int group_size,
                     int8_t* q_out, void* w_out, void* stream);

/*
 * Bytes of scratch that b200gptq_gemv / b200gptq_gemm may use for this problem.
 * The scratch must be zero-filled once before its first use; the kernels leave
 * it zero-filled where that matters, so one buffer can serve every later call
 * on the same stream.  Calls that may overlap on the GPU need separate buffers.
 */
B200GPTQ_API size_t b200gptq_workspace_bytes(int op, int M, int K, int N, int bits);

/*
 * Sticky status word of a scratch buffer.  Every wait inside the kernels is bounded (about 1e9 GPU clock
 * cycles); a kernel whose wait runs out raises this word to a non-zero value, finishes with undefined results
 * and returns, so the context stays usable.  The call copies the word to `*host_out` and SYNCHRONISES the
 * stream.  0 = no wait ever ran out since the buffer was zero-filled.  (The word is the last 32-bit word of
 * the first 16 KiB of the buffer; b200gptq_gemv_static_status is the same query for the scratch built into the library.)
 */
B200GPTQ_API int b200gptq_workspace_status(const void* workspace, void* stream, unsigned int* host_out);

/*
 * Decode GEMV, 1 <= M <= 8:  y[m,:] = x[m,:] @ W (+ bias), fp32 accumulation,
 * fp16 result.  bits in {2,3,4,8}.  Replaces the TVM `m1` kernel launch of
 * pycuda_warpper.py:144-149 (kernel: src/kernels/gemv_kernel.cu:25-55).
 *
 *   x_perm  int32 [K] or NULL.  When given, row r of qweight multiplies
 *           x[m, x_perm[r]] instead of x[m, r]: this is how a layer whose rows
 *           were re-ordered by b200gptq_sort_rows() is evaluated.
 *
 * Any g_idx is accepted, but g_idx == NULL is the fast-path contract: only then
 * (and with bits in {3,4}, K and group_size multiples of 128) does the call run
 * the streaming tensor-map kernel; every non-NULL g_idx, even one equal to
 * k / group_size, runs the general kernel, which looks groups up per row block.
 * Callers that hold a checkpoint's g_idx should compare it with k / group_size
 * once at load time and pass NULL when it matches (act-order layers: re-order
 * with b200gptq_sort_rows() first, which usually yields k / group_size again).
 * b200gptq_gemv_path() tells which kernel a call will run.
 */
B200GPTQ_API int b200gptq_gemv(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                  const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y,
                  int M, int K, int N, int bits, int group_size,
                  void* workspace, size_t workspace_bytes, void* stream);

/*
 * b200gptq_gemv with the two tuning parameters of the streaming kernel made explicit (0 = the library's
 * default for that parameter; other kernels ignore them).  The reference tunes its kernels per shape and
 * per row bucket (tile tables of pycuda_warpper.py:77-127, NNI search results in .cache/handler_database.json);
 * here the kernel is one and what remains to tune is how it shares the GPU with its neighbours in the stream:
 *   slices_per_sm  the K range of a 256-column group is cut into as many slices (CTAs) as give the grid about
 *                  this many CTAs per SM (at most 8 slices).  Default 3 for one row of x, 2 otherwise.
 *   ctas_per_sm    shared-memory footprint: a CTA takes at most 1/ctas_per_sm of an SM, so that many CTAs -- of
 *                  this launch and of its neighbours -- can be resident together; a slice that does not fit is
 *                  streamed through a ring.  Default: 3 if the whole slice still fits, else 2.
 * Measured on B200: a chain of nothing but GEMVs (the benchmark's pool of layers) is fastest with the defaults;
 * a decode step, where small kernels sit between the GEMVs, is fastest with (2, 3).
 */
B200GPTQ_API int b200gptq_gemv_tuned(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                        const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y,
                        int M, int K, int N, int bits, int group_size,
                        void* workspace, size_t workspace_bytes,
                        int slices_per_sm, int ctas_per_sm, void* stream);

/*
 * The GEMV with an activation folded into its read of x, so that the element-wise kernel between two linears of
 * a decode step (SiLU(gate) * up before `down_proj`, ReLU before `fc2`: auto_gptq/modeling/llama.py:8-12,
 * opt.py:11-16 name the layer pairs) is not a launch of its own:
 *   B200GPTQ_ACT_SWIGLU   x is [M, 2 K] = [gate | up]; the products see fp16(fp16(silu(gate)) * up), rounded exactly like
 *                         b200gptq_act.  Not together with x_perm.
 *   B200GPTQ_ACT_RELU     x is [M, K]; the products see max(x, 0).
 * Only the streaming kernel has it: a call that the general kernel would serve (non-NULL g_idx, 2/8 bits, ...)
 * returns B200GPTQ_ERR_SHAPE and the caller runs b200gptq_act first.  Otherwise as b200gptq_gemv_tuned
 * (B200GPTQ_ACT_NONE gives exactly that); b200gptq_gemv_plan_create_ex and b200gptq_gemv_tp_ex are the plan and
 * the tensor-parallel form.
 */
#define B200GPTQ_ACT_NONE 0
#define B200GPTQ_ACT_SWIGLU 1
#define B200GPTQ_ACT_RELU 2
B200GPTQ_API int b200gptq_gemv_ex(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                     const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y,
                     int M, int K, int N, int bits, int group_size,
                     void* workspace, size_t workspace_bytes,
                     int slices_per_sm, int ctas_per_sm, int input_act, void* stream);

/*
 * The same GEMV as a plan: what can be decided before x is known (kernel choice, work split, the TMA
 * descriptors of the layer's qweight and scales) is built once per (layer, M) and kept in an opaque HOST
 * object, so that a call costs one kernel launch.  This is the counterpart of the reference's per-shape
 * handler objects (tvm_untils/cache.py:10-60 keeps them in a module-level dict; here the caller owns the plan
 * and the library keeps no table).  The plan holds the layer's device pointers, not copies: the buffers must
 * outlive it and stay where they are.  A plan may be run from several threads and streams at once with
 * different workspaces.  plan_run has the semantics of b200gptq_gemv_tuned with the arguments given at creation.
 */
typedef struct b200gptq_gemv_plan b200gptq_gemv_plan;
B200GPTQ_API int b200gptq_gemv_plan_create(b200gptq_gemv_plan** out, const int32_t* qweight, const int32_t* qzeros,
                              const void* scales, const int32_t* g_idx, const int32_t* x_perm, const void* bias,
                              int M, int K, int N, int bits, int group_size, int slices_per_sm, int ctas_per_sm);
B200GPTQ_API int b200gptq_gemv_plan_create_ex(b200gptq_gemv_plan** out, const int32_t* qweight, const int32_t* qzeros,
                              const void* scales, const int32_t* g_idx, const int32_t* x_perm, const void* bias,
                              int M, int K, int N, int bits, int group_size, int slices_per_sm, int ctas_per_sm,
                              int input_act);
B200GPTQ_API int b200gptq_gemv_plan_run(const b200gptq_gemv_plan* plan, const void* x, void* y,
                           void* workspace, size_t workspace_bytes, void* stream);
B200GPTQ_API void b200gptq_gemv_plan_destroy(b200gptq_gemv_plan* plan);

/*
 * Which kernel b200gptq_gemv runs for this problem: B200GPTQ_PATH_STREAM or
 * B200GPTQ_PATH_GENERIC (a negative B200GPTQ_ERR_* code for an invalid problem).
 * Host-only; launches nothing.  has_g_idx != 0 means a non-NULL g_idx is passed.
 * The reference picks its kernel per (bits, N, K, M bucket) in
 * pycuda_warpper.py:138-189; this is the query for the same decision here.
 */
#define B200GPTQ_PATH_STREAM 1
#define B200GPTQ_PATH_GENERIC 2
B200GPTQ_API int b200gptq_gemv_path(int M, int K, int N, int bits, int group_size, int has_g_idx);

/*
 * Prefill GEMM, any M >= 1 (meant for M >= 16):  y = x @ W (+ bias) on the
 * tcgen05 tensor cores with fp32 accumulators in tensor memory.  bits in {3,4}.
 * Replaces the TVM `m16 .. m256` kernel launches of pycuda_warpper.py:150-189
 * (kernels: src/kernels/gemm_kernel.cu:25-142); no M padding is needed.
 *
 * x_perm as for b200gptq_gemv, except that a non-NULL x_perm needs
 * workspace room for the gathered copy of x (counted by b200gptq_workspace_bytes).
 * With M <= 128 and fewer column tiles than SMs, K is split over up to four
 * thread blocks per tile; their fp32 partial sums live in the workspace (also
 * counted by b200gptq_workspace_bytes) and are added in a fixed order, so the
 * result does not depend on which block finishes last.
 * g_idx must be constant over aligned 32-row blocks: the kernel takes the
 * group of a block from the block's first row and does not check the others
 * (that is the caller's contract); layers with an arbitrary act-order g_idx
 * are first re-ordered with b200gptq_sort_rows().
 */
B200GPTQ_API int b200gptq_gemm(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                  const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y,
                  int M, int K, int N, int bits, int group_size,
                  void* workspace, size_t workspace_bytes, void* stream);

/*
 * How b200gptq_gemm divides this problem on the current device: *splits = thread blocks that share one tile's K
 * (1 = none; their fp32 partial sums are added in a fixed order), *ctas_per_sm = 1 (three groups of weight warps per
 * block) or 2 (one group, half of the shared and tensor memory).  Host-only; launches nothing.  The reference picks
 * a tile per (bits, N, K, M bucket) from its tuned table (pycuda_warpper.py:77-127); this is the query for the
 * corresponding decision here, so that a test can tell which form it exercised.
 */
B200GPTQ_API int b200gptq_gemm_split(int M, int K, int N, int bits, int* splits, int* ctas_per_sm);

/*
 * Pack integer fields into GPTQ words: vals int32 [R, C] (R % 32 == 0, one field per element, packed
 * along R) -> out int32 [R/32*bits, C], bits in {2,3,4,8}.  This is the word-building half of
 * QuantLinear.pack of the reference (auto_gptq/nn_modules/qlinear.py:111-134 for qweight, called on
 * [K, N]; :140-170 for qzeros, called on the transposed [N, G] zero-points), a Python loop over the
 * rows there.  Like that loop it does not mask: a value wider than `bits` spills into the
 * neighbouring fields.
 */
B200GPTQ_API int b200gptq_pack_fields(const int32_t* vals, int R, int C, int bits, int32_t* out, void* stream);

/*
 * Re-order the rows of a packed layer so that rows of one group are adjacent
 * (stable sort of k by g_idx[k]).  Outputs:
 *   qweight_sorted int32 [K/32*bits, N]   row r holds original row perm[r]
 *   perm           int32 [K]              the x_perm to pass to gemv / gemm
 *   g_idx_sorted   int32 [K]              g_idx[perm[r]], non-decreasing
 * `perm` is computed by the caller (it is a host-side argsort of g_idx) and
 * read here from device memory; this entry point does the unpack / gather /
 * repack of the weight fields, bits in {2,3,4,8}.
 */
B200GPTQ_API int b200gptq_sort_rows(const int32_t* qweight, const int32_t* g_idx, const int32_t* perm,
                       int K, int N, int bits,
                       int32_t* qweight_sorted, int32_t* g_idx_sorted, void* stream);

/*
 * Decode GEMV without caller scratch (no counterpart in the reference; the reference's kernels
 * need no scratch because they never split K across thread blocks).
 *
 * Same arithmetic, arguments and results as b200gptq_gemv, for hosts that cannot allocate
 * device memory where they launch: plugins called from inside another runtime, engines whose
 * memory plan is frozen, loops in which cudaMalloc is forbidden.  The partial sums and arrival
 * counters live in a fixed array of b200gptq_gemv_static_capacity() bytes (4 MiB) inside the
 * library's device image; each GPU that loads the library holds that memory until its context
 * ends.  The call never allocates or frees memory.
 *
 *  - Problems with b200gptq_workspace_bytes(B200GPTQ_OP_GEMV, ...) above the capacity return
 *    B200GPTQ_ERR_TOO_LARGE.
 *  - All calls on one device share the array: calls that may overlap on the GPU race with each
 *    other; order them on one stream (or with events).
 *  - The first call on a device looks the array's address up with a runtime call; make that call
 *    before any stream capture begins.  (The array is zero-initialised storage and the kernels
 *    leave their counters at zero, so nothing is cleared.)
 */
B200GPTQ_API int b200gptq_gemv_static(const void* x, const int32_t* qweight, const int32_t* qzeros,
                         const void* scales, const int32_t* g_idx, const int32_t* x_perm, const void* bias,
                         void* y, int M, int K, int N, int bits, int group_size, void* stream);

/* Bytes of the built-in scratch array used by b200gptq_gemv_static (per device). */
B200GPTQ_API size_t b200gptq_gemv_static_capacity(void);
/* b200gptq_workspace_status for the built-in scratch of the current device (synchronises the stream). */
B200GPTQ_API int b200gptq_gemv_static_status(void* stream, unsigned int* host_out);

/*
 * Tensor-parallel row shards (one process per GPU of one node): the decode GEMV of a K shard with the sum
 * over ranks fused into its last step, and that sum as a call of its own.
 *
 * The reference has no tensor parallelism (its only multi-GPU code places whole decoder layers on
 * different devices, quantization/opt.py:270-304); these entry points serve the linears that a
 * tensor-parallel split makes row-parallel -- o_proj / down_proj (auto_gptq/modeling/llama.py:8-12),
 * out_proj / fc2 (auto_gptq/modeling/opt.py:11-16) -- whose per-rank results
 *     y_r = x[:, rows of rank r] @ W[rows of rank r, :]          (arithmetic of qlinear.py:197-243)
 * must be added up.  At decode sizes (8..18 KB per rank) that sum is pure latency, so instead of a
 * collective library call every rank PUSHES its fp32 partial sums into every rank's exchange buffer
 * with plain stores over NVLink, raises a counter there, waits on its own memory until all ranks'
 * counters arrived and adds the slots in rank order (every rank gets the same bits; peers are never
 * read; no multicast).
 *
 * Exchange buffers: every rank allocates b200gptq_tp_buffer_bytes() bytes of device memory (256-byte
 * aligned), zero-fills them ONCE, and makes them addressable by all ranks of the node (CUDA IPC,
 * cuMem fabric / POSIX handles, or torch symmetric memory) with peer access enabled; `peer_buffers`
 * is a HOST array of `world` device pointers, entry r = rank r's buffer as mapped in the calling
 * process (entry `rank` = the own buffer).  All ranks must issue the same sequence of calls with the
 * same M and N.  Limits: world <= 8, M <= 8, N <= 16384.
 *
 * Waits are bounded: a rank that does not see a peer's counter within `timeout_cycles` GPU clock
 * cycles (<= 0: 2e10, about ten seconds) raises the sticky status word at byte 0 of its own buffer to 2, finishes with
 * undefined results and returns control; b200gptq_tp_status() reads the word (it synchronises the
 * stream).  Counters only grow, so the calls can be captured in a CUDA graph and replayed.
 *
 *   b200gptq_gemv_tp       y = sum over ranks of (x_r @ W_r) + bias; same arguments as b200gptq_gemv_tuned
 *                          for this rank's shard.  `bias` (full, the same on every rank) is added
 *                          after the sum.  With g_idx == NULL the exchange runs inside the GEMV
 *                          kernel's combine step; shards that need the general kernel (act-order
 *                          row shards keep global group ids) run it as a second kernel.
 *   b200gptq_tp_allreduce  y[M, N] (fp16, in place) = sum over ranks of y + bias: the same exchange
 *                          for partial results produced elsewhere.
 */
B200GPTQ_API size_t b200gptq_tp_buffer_bytes(void);
B200GPTQ_API int b200gptq_gemv_tp(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                     const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y,
                     int M, int K, int N, int bits, int group_size,
                     void* workspace, size_t workspace_bytes,
                     int rank, int world, void* const* peer_buffers, long long timeout_cycles,
                     int slices_per_sm, int ctas_per_sm, void* stream);
/* b200gptq_gemv_tp with the input activation of b200gptq_gemv_ex (x is this rank's slice: [M, 2 K_local] for SwiGLU). */
B200GPTQ_API int b200gptq_gemv_tp_ex(const void* x, const int32_t* qweight, const int32_t* qzeros, const void* scales,
                     const int32_t* g_idx, const int32_t* x_perm, const void* bias, void* y,
                     int M, int K, int N, int bits, int group_size,
                     void* workspace, size_t workspace_bytes,
                     int rank, int world, void* const* peer_buffers, long long timeout_cycles,
                     int slices_per_sm, int ctas_per_sm, int input_act, void* stream);
B200GPTQ_API int b200gptq_tp_allreduce(void* y, const void* bias, int M, int N, int rank, int world,
                          void* const* peer_buffers, long long timeout_cycles, void* stream);
B200GPTQ_API int b200gptq_tp_status(const void* own_buffer, void* stream, unsigned int* host_out);
/* Let kernels of the current device store into memory of `peer_device` (cudaDeviceEnablePeerAccess; fine if it
 * is enabled already).  A host-side set-up call: once per peer before the first exchange. */
B200GPTQ_API int b200gptq_tp_enable_peer(int peer_device);
/* Set-up helpers for exchange buffers shared through CUDA IPC: export the 64-byte cudaIpcMemHandle_t of the
 * allocation that contains `device_ptr` together with the pointer's offset inside it; map the allocation behind
 * such a handle into the CURRENT device's address
 * space (`*mapped` = base of that allocation; peer access to the owning device is enabled on the way), unmap it,
 * and read one word through the runtime to check a mapping before kernels use it. */
B200GPTQ_API int b200gptq_tp_export(const void* device_ptr, void* ipc_handle_out /* 64 bytes */, size_t* offset_out);
B200GPTQ_API int b200gptq_tp_open_peer(const void* ipc_handle, void** mapped);
B200GPTQ_API int b200gptq_tp_close_peer(void* mapped);
B200GPTQ_API int b200gptq_tp_probe(const void* device_ptr, unsigned int* host_out);

/*
 * Decode-step helpers around the linears (fp16 storage, fp32 arithmetic, one launch each).  The
 * reference has no counterpart: it leaves everything between its QuantLinear calls to the
 * transformers modules (end2end/autogptq-generation-inference-benchmark.py:26-49).  They exist so
 * that a batch-1 decode step is a handful of launches instead of dozens of element-wise kernels.
 *
 *   b200gptq_add_norm     x[rows,H] += add (nullable); h = RMSNorm(x)*w (rms != 0) or LayerNorm(x)*w + beta
 *   b200gptq_rope_cache   one new token per sequence: qkv[b,3,heads,hd] -> rotated q_out[b,heads,hd]; rotated k
 *                         and v written at position pos[0] of the caches [b,heads,max_seq,hd]; rope == 0: no rotation
 *   b200gptq_attn_decode  out[b,heads*hd] = softmax(q k^T * scale) v over cache positions 0..pos[0]; hd in {64,128}
 *   b200gptq_attn_step    b200gptq_rope_cache followed by b200gptq_attn_decode as ONE launch (same caches bit for bit,
 *                         same output up to the order of the softmax accumulation): rotates
 *                         q and the new k inside the attention kernel, attends to the new position from shared
 *                         memory and writes k, v into the caches for the steps to come
 *   b200gptq_act          act[rows,I] = silu(u[:, :I]) * u[:, I:] (gated != 0) or relu(u) (gated == 0)
 * `pos` is a device pointer to one int64, so that a captured graph can advance it.
 */
B200GPTQ_API int b200gptq_add_norm(void* x, const void* add, const void* w, const void* beta, void* h, int rows,
                                   int H, float eps, int rms, void* stream);
B200GPTQ_API int b200gptq_rope_cache(const void* qkv, const void* cos_t, const void* sin_t, const void* pos,
                                     void* q_out, void* k_cache, void* v_cache, int batch, int heads, int hd,
                                     int max_seq, int rope, void* stream);
B200GPTQ_API int b200gptq_attn_decode(const void* q, const void* k_cache, const void* v_cache, const void* pos,
                                      void* out, int batch, int heads, int hd, int max_seq, float scale,
                                      void* stream);
B200GPTQ_API int b200gptq_attn_step(const void* qkv, const void* cos_t, const void* sin_t, const void* pos,
                                    void* k_cache, void* v_cache, void* out, int batch, int heads, int hd,
                                    int max_seq, int rope, float scale, void* stream);
B200GPTQ_API int b200gptq_act(const void* u, void* act, int rows, int I, int gated, void* stream);

/*
 * Dense fp16 projection of up to 8 rows:  y[rows, N] = x[rows, K] @ w[N, K]^T  (fp32 sums of 8-product fp16 partial
 * sums, one fp16 rounding).  This is the vocabulary projection of a decode step, which AutoGPTQ leaves unquantised
 * (auto_gptq/modeling/_base.py:534 keeps `lm_head` out of the quantised modules): one pass over w at stream rate,
 * launched like the other decode-step helpers.  K % 8 == 0, rows * K * 2 <= 96 KiB, x and w 16-byte aligned.
 */
B200GPTQ_API int b200gptq_dense_gemv(const void* x, const void* w, void* y, int rows, int K, int N, void* stream);

/*
 * Greedy token pick of a decode step (the reference leaves it to transformers' generate(),
 * end2end/autogptq-generation-inference-benchmark.py:26-49; here it is one launch on one GPU and two around the
 * exchange on several, instead of a dozen element-wise kernels).
 *
 *   b200gptq_pick_local  per row of fp16 logits[rows, ld]: the largest of columns [0, valid) (lowest column on a tie).
 *                        world == 1: tokens[row] = min(base_index + column, max_token).
 *                        world > 1 : slots[row, 4*world] (fp16) gets {logit, 0, token / 256, token % 256} in this rank's
 *                        four entries and zeros elsewhere; the caller sums `slots` over the ranks
 *                        (b200gptq_tp_allreduce) and calls b200gptq_pick_final.
 *   b200gptq_pick_final  tokens[row] = the token of the rank with the largest logit (lowest rank on a tie), clamped.
 * pos_inc (nullable): a device int64 that the launch increments by one (the step's position), so that a captured
 * graph advances it.  ld % 8 == 0, logits 16-byte aligned.
 */
B200GPTQ_API int b200gptq_pick_local(const void* logits, int rows, int ld, int valid, long long base_index, int world,
                                     int rank, void* slots, long long* tokens, long long max_token, long long* pos_inc,
                                     void* stream);
B200GPTQ_API int b200gptq_pick_final(const void* slots, int rows, int world, long long* tokens, long long max_token,
                                     long long* pos_inc, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200GPTQ_H_ */
