// Small fused kernels for the decode step around the quantised linears: residual-add + RMSNorm /
// LayerNorm, rotary embedding + KV-cache write, single-query attention over the cache, SwiGLU / ReLU.
// They replace the chain of framework element-wise kernels that otherwise dominates a batch-1 decode
// step once the linears are fast (the reference leaves these to transformers' eager modules:
// end2end/autogptq-generation-inference-benchmark.py:26-49).  All are memory-trivial; the point is
// launch count.  fp16 storage, fp32 arithmetic.
#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace b200gptq {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// x[b,:] += add[b,:] (optional); h[b,:] = norm(x[b,:]) * w (+ beta).  rms != 0: RMSNorm, else LayerNorm.
// One CTA of 256 threads per row; H is a multiple of 8.
// Programmatic dependent launch: every kernel of the decode step is launched with the attribute that lets it
// become resident while its predecessor in the stream is still running.  It reads and writes nothing of the
// step's data before the predecessor has completed (griddepcontrol.wait), and only then lets its own successor
// in (so at most two kernels of the chain are resident at a time).  Without the launch attribute both
// instructions do nothing.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
}

bool pdl_enabled() {
    static const bool on = [] {
        const char* e = std::getenv("B200GPTQ_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, void* stream, int cluster_x,
                       Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (cluster_x > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = cluster_x;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    if (pdl_enabled()) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__global__ void __launch_bounds__(256)
add_norm_kernel(__half* __restrict__ x, const __half* __restrict__ add, const __half* __restrict__ w,
                const __half* __restrict__ beta, __half* __restrict__ h, int H, float eps, int rms) {
    extern __shared__ float row[];  // H floats
    __shared__ float red[2][8];
    pdl_enter();
    const int b = blockIdx.x, tid = threadIdx.x;
    __half* xr = x + (size_t)b * H;
    float s = 0.f, s2 = 0.f;
    for (int i = tid * 8; i < H; i += 256 * 8) {
        uint4 v = *reinterpret_cast<const uint4*>(xr + i);
        __half2* p = reinterpret_cast<__half2*>(&v);
        if (add) {
            const uint4 a = *reinterpret_cast<const uint4*>(add + (size_t)b * H + i);
            const __half2* q = reinterpret_cast<const __half2*>(&a);
#pragma unroll
            for (int k = 0; k < 4; ++k) p[k] = __hadd2(p[k], q[k]);
            *reinterpret_cast<uint4*>(xr + i) = v;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(p[k]);
            row[i + 2 * k] = f.x; row[i + 2 * k + 1] = f.y;
            s += f.x + f.y; s2 += f.x * f.x + f.y * f.y;
        }
    }
    s = warp_sum(s); s2 = warp_sum(s2);
    if ((tid & 31) == 0) { red[0][tid >> 5] = s; red[1][tid >> 5] = s2; }
    __syncthreads();
    float ts = 0.f, ts2 = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { ts += red[0][k]; ts2 += red[1][k]; }
    const float mean = rms ? 0.f : ts / H;
    const float var = rms ? ts2 / H : fmaxf(ts2 / H - mean * mean, 0.f);
    const float inv = rsqrtf(var + eps);
    for (int i = tid * 8; i < H; i += 256 * 8) {
        uint4 o;
        __half2* po = reinterpret_cast<__half2*>(&o);
        const uint4 wv = *reinterpret_cast<const uint4*>(w + i);
        const __half2* pw = reinterpret_cast<const __half2*>(&wv);
        uint4 bv = make_uint4(0, 0, 0, 0);
        if (beta) bv = *reinterpret_cast<const uint4*>(beta + i);
        const __half2* pb = reinterpret_cast<const __half2*>(&bv);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 fw = __half22float2(pw[k]), fb = __half22float2(pb[k]);
            // RMSNorm rounds the normalised value to fp16 before the weight, as the usual fp16 modules do
            float a0 = (row[i + 2 * k] - mean) * inv, a1 = (row[i + 2 * k + 1] - mean) * inv;
            if (rms) { a0 = __half2float(__float2half_rn(a0)); a1 = __half2float(__float2half_rn(a1)); }
            po[k] = __floats2half2_rn(a0 * fw.x + fb.x, a1 * fw.y + fb.y);
        }
        *reinterpret_cast<uint4*>(h + (size_t)b * H + i) = o;
    }
}

// qkv[b, 3, heads, hd] (one new token per sequence): rotate q and k by the angle of position `pos[0]`
// (interleaved pairs), write q to q_out[b, heads, hd] and k, v into the caches at that position.
// cache layout [b, heads, max_seq, hd].  rope == 0: no rotation (OPT).  One CTA per (head, b), hd/2 threads.
__global__ void rope_cache_kernel(const __half* __restrict__ qkv, const __half* __restrict__ cos_t,
                                  const __half* __restrict__ sin_t, const long long* __restrict__ pos,
                                  __half* __restrict__ q_out, __half* __restrict__ k_cache,
                                  __half* __restrict__ v_cache, int heads, int hd, int max_seq, int rope) {
    pdl_enter();
    const int head = blockIdx.x, b = blockIdx.y, i = threadIdx.x;  // pair index
    const long long p64 = pos[0];
    // The position lives in device memory (a captured graph advances it), so the host cannot check it per launch:
    // a position outside the caches is refused here, with no access issued.
    if (p64 < 0 || p64 >= max_seq) return;
    const int p = (int)p64;
    const size_t tok = (size_t)b * 3 * heads * hd;
    const __half2 q2 = *reinterpret_cast<const __half2*>(qkv + tok + (size_t)head * hd + 2 * i);
    const __half2 k2 = *reinterpret_cast<const __half2*>(qkv + tok + (size_t)(heads + head) * hd + 2 * i);
    const __half2 v2 = *reinterpret_cast<const __half2*>(qkv + tok + (size_t)(2 * heads + head) * hd + 2 * i);
    float2 q = __half22float2(q2), k = __half22float2(k2);
    if (rope) {
        // fp16 products and sums, like the framework expression t1*cos - t2*sin evaluated in fp16
        const __half c = cos_t[(size_t)p * (hd / 2) + i], s = sin_t[(size_t)p * (hd / 2) + i];
        const __half q0 = __hsub(__hmul(q2.x, c), __hmul(q2.y, s)), q1 = __hadd(__hmul(q2.x, s), __hmul(q2.y, c));
        const __half k0 = __hsub(__hmul(k2.x, c), __hmul(k2.y, s)), k1 = __hadd(__hmul(k2.x, s), __hmul(k2.y, c));
        q = make_float2(__half2float(q0), __half2float(q1));
        k = make_float2(__half2float(k0), __half2float(k1));
    }
    *reinterpret_cast<__half2*>(q_out + ((size_t)b * heads + head) * hd + 2 * i) = __floats2half2_rn(q.x, q.y);
    const size_t c_off = (((size_t)b * heads + head) * max_seq + p) * hd + 2 * i;
    *reinterpret_cast<__half2*>(k_cache + c_off) = __floats2half2_rn(k.x, k.y);
    *reinterpret_cast<__half2*>(v_cache + c_off) = v2;
}

__device__ __forceinline__ float ld_cluster_f32(const float* local_ptr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local_ptr)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Single-query attention over the cache positions 0..pos[0] (inclusive).  A cluster of kAttnSplit CTAs
// of 16 warps serves one (head, b); the 32-position chunks are dealt round-robin to all warps of the
// cluster, so a prompt of ~2000 tokens is still one chunk per warp.  Scores: each lane owns ONE position
// and reads that key row with 128-bit loads (all 32 rows in flight together); softmax statistics once per
// 32 positions; values: each lane owns HD/32 dims, the 32 probabilities are broadcast by shuffle and the
// 32 value rows are read coalesced.  Online softmax per warp; warps are combined through shared memory
// and the CTAs of the cluster through distributed shared memory by the cluster's first CTA.
//
// STEP = true is the whole attention part of a decode step in one launch: `q` is then qkv[b, 3, heads, hd] of the
// new token; every CTA rotates q and the new k itself (the same fp16 arithmetic as rope_cache_kernel), uses the new
// k and v from shared memory for position pos[0], and the cluster's first CTA writes them into the caches for the
// steps to come -- rope_cache_kernel + attn_decode_kernel without the launch in between.
//
// SPLIT CTAs (a cluster) of WARPS warps share one (sequence, head): the launcher picks the pair so that the whole grid
// is resident at once (128 registers per thread: 16 warps per SM) -- 4 x 16 for a single sequence, down to one CTA
// of 4 warps per (sequence, head) for a batch.
template <int HD, bool STEP, int SPLIT, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 16 / WARPS)
attn_decode_kernel(const __half* __restrict__ q, const __half* __restrict__ k_cache,
                   const __half* __restrict__ v_cache, const long long* __restrict__ pos, __half* __restrict__ out,
                   int heads, int max_seq, float scale, const __half* __restrict__ cos_t,
                   const __half* __restrict__ sin_t, int rope, __half* k_write, __half* v_write) {
    // k_write / v_write (STEP): the same caches, for the one row this kernel writes; that row is never read through
    // k_cache / v_cache here (position pos[0] is served from shared memory), so the read-only path stays valid.
    constexpr int PER = HD / 32;
    static_assert(WARPS * 32 >= HD / 2 && WARPS * 32 >= HD, "the prologue takes one thread per element");
    __shared__ __align__(16) __half q_sm[HD];
    __shared__ __align__(16) __half knew_sm[STEP ? HD : 8], vnew_sm[STEP ? HD : 8];
    __shared__ float sm_m[WARPS], sm_l[WARPS], sm_acc[WARPS][HD];
    __shared__ float cta_m, cta_l, cta_acc[HD];   // this CTA's partial result, read by the cluster's first CTA
    pdl_enter();
    const int split = blockIdx.x % SPLIT, head = blockIdx.x / SPLIT, b = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long p64 = pos[0];
    if (STEP && (p64 < 0 || p64 >= max_seq)) return;   // a position outside the caches: refused by the whole cluster
    const int P = STEP ? (int)p64 : -1;                // the position whose key and value are in shared memory
    // positions served from the caches: 0..pos[0] (never past their end); STEP: 0..pos[0]-1, the new one comes last
    const int L = STEP ? P : (p64 < 0 ? 0 : (p64 >= max_seq ? max_seq : (int)p64 + 1));
    const size_t base = ((size_t)b * heads + head) * (size_t)max_seq * HD;
    if constexpr (STEP) {
        if (threadIdx.x < HD / 2) {
            const int i = threadIdx.x;   // pair index
            const size_t tok = (size_t)b * 3 * heads * HD;
            const __half2 q2 = *reinterpret_cast<const __half2*>(q + tok + (size_t)head * HD + 2 * i);
            const __half2 k2 = *reinterpret_cast<const __half2*>(q + tok + (size_t)(heads + head) * HD + 2 * i);
            const __half2 v2 = *reinterpret_cast<const __half2*>(q + tok + (size_t)(2 * heads + head) * HD + 2 * i);
            float2 qf = __half22float2(q2), kf = __half22float2(k2);
            if (rope) {
                const __half c = cos_t[(size_t)P * (HD / 2) + i], sn = sin_t[(size_t)P * (HD / 2) + i];
                const __half q0 = __hsub(__hmul(q2.x, c), __hmul(q2.y, sn)), q1 = __hadd(__hmul(q2.x, sn), __hmul(q2.y, c));
                const __half k0 = __hsub(__hmul(k2.x, c), __hmul(k2.y, sn)), k1 = __hadd(__hmul(k2.x, sn), __hmul(k2.y, c));
                qf = make_float2(__half2float(q0), __half2float(q1));
                kf = make_float2(__half2float(k0), __half2float(k1));
            }
            const __half2 kr = __floats2half2_rn(kf.x, kf.y);
            *reinterpret_cast<__half2*>(q_sm + 2 * i) = __floats2half2_rn(qf.x, qf.y);
            *reinterpret_cast<__half2*>(knew_sm + 2 * i) = kr;
            *reinterpret_cast<__half2*>(vnew_sm + 2 * i) = v2;
            if (split == 0) {
                const size_t c_off = base + (size_t)P * HD + 2 * i;
                *reinterpret_cast<__half2*>(k_write + c_off) = kr;
                *reinterpret_cast<__half2*>(v_write + c_off) = v2;
            }
        }
    } else {
        if (threadIdx.x < HD) q_sm[threadIdx.x] = q[((size_t)b * heads + head) * HD + threadIdx.x];
    }
    __syncthreads();
    float acc[PER];
#pragma unroll
    for (int d = 0; d < PER; ++d) acc[d] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int t0 = (warp * SPLIT + split) * 32; t0 < L; t0 += WARPS * SPLIT * 32) {
        const int t = t0 + lane;
        // ---- score of this lane's position ----
        float dot = -INFINITY;
        if (t < L) {
            const uint4* kp = reinterpret_cast<const uint4*>(k_cache + base + (size_t)t * HD);
            uint4 kv[HD / 8];
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) kv[i] = kp[i];
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < HD / 8; ++i) {
                const __half2* k2 = reinterpret_cast<const __half2*>(&kv[i]);
                const __half2* q2 = reinterpret_cast<const __half2*>(q_sm + 8 * i);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 kf = __half22float2(k2[e]), qf = __half22float2(q2[e]);
                    s = fmaf(kf.x, qf.x, s);
                    s = fmaf(kf.y, qf.y, s);
                }
            }
            dot = s * scale;
        }
        const float m_new = fmaxf(m, warp_max(dot));
        const float pexp = (t < L) ? __expf(dot - m_new) : 0.f;
        const float corr = __expf(m - m_new);
        l = l * corr + warp_sum(pexp);
        m = m_new;
#pragma unroll
        for (int d = 0; d < PER; ++d) acc[d] *= corr;
        // ---- values: lanes own dims, positions are walked together ----
        const int n = min(32, L - t0);
        const __half* vp = v_cache + base + (size_t)t0 * HD + lane * PER;
#pragma unroll 8
        for (int i = 0; i < n; ++i) {
            const float p = __shfl_sync(0xffffffffu, pexp, i);
            if constexpr (PER == 4) {
                const uint2 raw = *reinterpret_cast<const uint2*>(vp + (size_t)i * HD);
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
                const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
                acc[0] = fmaf(p, a.x, acc[0]); acc[1] = fmaf(p, a.y, acc[1]);
                acc[2] = fmaf(p, c.x, acc[2]); acc[3] = fmaf(p, c.y, acc[3]);
            } else {
                const float2 a = __half22float2(*reinterpret_cast<const __half2*>(vp + (size_t)i * HD));
                acc[0] = fmaf(p, a.x, acc[0]); acc[1] = fmaf(p, a.y, acc[1]);
            }
        }
    }
    if (STEP && split == 0 && warp == 0) {
        // the new position: key and value are in shared memory; one more step of the online softmax for this warp
        float part = 0.f;
#pragma unroll
        for (int d = 0; d < PER; ++d)
            part = fmaf(__half2float(knew_sm[lane * PER + d]), __half2float(q_sm[lane * PER + d]), part);
        const float dot = warp_sum(part) * scale;
        const float m_new = fmaxf(m, dot);
        const float pexp = __expf(dot - m_new), corr = __expf(m - m_new);
        l = l * corr + pexp;
        m = m_new;
#pragma unroll
        for (int d = 0; d < PER; ++d) acc[d] = fmaf(pexp, __half2float(vnew_sm[lane * PER + d]), acc[d] * corr);
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int d = 0; d < PER; ++d) sm_acc[warp][lane * PER + d] = acc[d];
    __syncthreads();
    if (warp == 0) {   // combine the 16 warps of this CTA
        float gm = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) gm = fmaxf(gm, sm_m[w]);
        float gl = 0.f, wgt[WARPS];
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            wgt[w] = (sm_m[w] == -INFINITY) ? 0.f : __expf(sm_m[w] - gm);
            gl += sm_l[w] * wgt[w];
        }
        if (lane == 0) { cta_m = gm; cta_l = gl; }
#pragma unroll
        for (int d = 0; d < PER; ++d) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += sm_acc[w][lane * PER + d] * wgt[w];
            cta_acc[lane * PER + d] = v;
        }
    }
    if constexpr (SPLIT == 1) {
        __syncwarp();
        if (warp == 0) {
#pragma unroll
            for (int d = 0; d < PER; ++d)
                out[((size_t)b * heads + head) * HD + lane * PER + d] = __float2half_rn(cta_acc[lane * PER + d] / cta_l);
        }
        return;
    }
    cluster_sync_all();   // every CTA's (cta_m, cta_l, cta_acc) is visible to the cluster
    if (split == 0 && warp == 0) {
        float pm[SPLIT], pl[SPLIT], pa[SPLIT][PER];
#pragma unroll
        for (int r = 0; r < SPLIT; ++r) {   // all remote reads in flight together
            pm[r] = ld_cluster_f32(&cta_m, r);
            pl[r] = ld_cluster_f32(&cta_l, r);
#pragma unroll
            for (int d = 0; d < PER; ++d) pa[r][d] = ld_cluster_f32(&cta_acc[lane * PER + d], r);
        }
        float gm = -INFINITY;
#pragma unroll
        for (int r = 0; r < SPLIT; ++r) gm = fmaxf(gm, pm[r]);
        float gl = 0.f, wgt[SPLIT];
#pragma unroll
        for (int r = 0; r < SPLIT; ++r) {
            wgt[r] = (pm[r] == -INFINITY) ? 0.f : __expf(pm[r] - gm);
            gl += pl[r] * wgt[r];
        }
#pragma unroll
        for (int d = 0; d < PER; ++d) {
            float v = 0.f;
#pragma unroll
            for (int r = 0; r < SPLIT; ++r) v += pa[r][d] * wgt[r];
            out[((size_t)b * heads + head) * HD + lane * PER + d] = __float2half_rn(v / gl);
        }
    }
    cluster_sync_all();   // keep every CTA's shared memory alive until it has been read
}

// act[b, i] = silu(u[b, i]) * u[b, I + i]  (gated != 0)   or   relu(u[b, i])  (gated == 0)
__global__ void __launch_bounds__(256)
act_kernel(const __half* __restrict__ u, __half* __restrict__ act, int I, int gated, size_t total) {
    pdl_enter();
    const size_t idx = ((size_t)blockIdx.x * 256 + threadIdx.x) * 2;
    if (idx >= total) return;
    const size_t b = idx / I, i = idx % I;
    const size_t row = b * (size_t)(gated ? 2 * I : I);
    const float2 g = __half22float2(*reinterpret_cast<const __half2*>(u + row + i));
    float2 r;
    if (gated) {
        const float2 up = __half22float2(*reinterpret_cast<const __half2*>(u + row + I + i));
        // silu rounded to fp16 before the product, like the framework's two element-wise kernels
        const float s0 = __half2float(__float2half_rn(g.x / (1.f + __expf(-g.x))));
        const float s1 = __half2float(__float2half_rn(g.y / (1.f + __expf(-g.y))));
        r = make_float2(s0 * up.x, s1 * up.y);
    } else {
        r = make_float2(fmaxf(g.x, 0.f), fmaxf(g.y, 0.f));
    }
    *reinterpret_cast<__half2*>(act + idx) = __floats2half2_rn(r.x, r.y);
}

// y[m, n] = sum_k x[m, k] * w[n, k]: the dense fp16 vocabulary projection of a decode step (up to 8 rows of x),
// a pure stream of w.  x is staged in shared memory; a warp takes four rows of w at a time, a lane 16 bytes of
// each per step; eight products are accumulated in half2 (four HFMA2), then widened and summed in fp32.
template <int MM>
__global__ void __launch_bounds__(256)
dense_gemv_kernel(const __half* __restrict__ x, const __half* __restrict__ w, __half* __restrict__ y, int M, int K,
                  int N) {
    extern __shared__ __align__(16) unsigned char dense_smem[];
    __half* xs = reinterpret_cast<__half*>(dense_smem);
    pdl_enter();
    const int tid = threadIdx.x, lane = tid & 31;
    for (int i = tid; i < M * K / 8; i += 256) reinterpret_cast<uint4*>(xs)[i] = reinterpret_cast<const uint4*>(x)[i];
    __syncthreads();
    const int gw = blockIdx.x * 8 + (tid >> 5), nw = gridDim.x * 8;
    for (int n0 = gw * 4; n0 < N; n0 += nw * 4) {
        float acc[4][MM];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int m = 0; m < MM; ++m) acc[r][m] = 0.f;
        for (int k = lane * 8; k < K; k += 256) {
            uint4 wv[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                wv[r] = make_uint4(0u, 0u, 0u, 0u);
                if (n0 + r < N) wv[r] = __ldcs(reinterpret_cast<const uint4*>(w + (size_t)(n0 + r) * K + k));
            }
#pragma unroll
            for (int m = 0; m < MM; ++m) {
                if (m >= M) break;
                const uint4 xv = *reinterpret_cast<const uint4*>(xs + (size_t)m * K + k);
                const __half2* xh = reinterpret_cast<const __half2*>(&xv);
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const __half2* wh = reinterpret_cast<const __half2*>(&wv[r]);
                    __half2 p = __hmul2(wh[0], xh[0]);
                    p = __hfma2(wh[1], xh[1], p);
                    p = __hfma2(wh[2], xh[2], p);
                    p = __hfma2(wh[3], xh[3], p);
                    const float2 f = __half22float2(p);
                    acc[r][m] += f.x + f.y;
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int m = 0; m < MM; ++m) {
                const float v = warp_sum(acc[r][m]);
                if (lane == 0 && m < M && n0 + r < N) y[(size_t)m * N + n0 + r] = __float2half_rn(v);
            }
    }
}

// Greedy pick, first half: the largest of one row's logits (the lowest column on a tie, like the framework's argmax)
// over columns [0, valid).  One rank: the token goes straight to `tokens[row]`.  Several ranks: the row's slots of the
// exchange vector are written -- {logit, 0, index / 256, index % 256} as fp16 (all exact) in this rank's four slots,
// zeros in the others, so that the sum over ranks is a gather.
__global__ void __launch_bounds__(1024)
pick_local_kernel(const __half* __restrict__ logits, int ld, int valid, long long base_index, int world, int rank,
                  __half* __restrict__ slots, long long* __restrict__ tokens, long long max_token,
                  long long* __restrict__ pos_inc) {
    pdl_enter();
    __shared__ float sm_v[32];
    __shared__ int sm_i[32];
    const int row = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const __half* lr = logits + (size_t)row * ld;
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int c0 = threadIdx.x * 8; c0 < valid; c0 += 1024 * 8) {   // ld % 8 == 0: whole 16-byte pieces
        const uint4 raw = *reinterpret_cast<const uint4*>(lr + c0);
        const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float v = __half2float(h[i]);
            if (c0 + i < valid && (v > best || at == 0x7fffffff)) { best = v; at = c0 + i; }
        }
    }
    auto better = [](float v, int i, float bv, int bi) { return v > bv || (v == bv && i < bi); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float v = __shfl_xor_sync(0xffffffffu, best, o);
        const int i = __shfl_xor_sync(0xffffffffu, at, o);
        if (i != 0x7fffffff && (at == 0x7fffffff || better(v, i, best, at))) { best = v; at = i; }
    }
    if (lane == 0) { sm_v[warp] = best; sm_i[warp] = at; }
    __syncthreads();
    if (warp == 0) {
        best = sm_v[lane]; at = sm_i[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float v = __shfl_xor_sync(0xffffffffu, best, o);
            const int i = __shfl_xor_sync(0xffffffffu, at, o);
            if (i != 0x7fffffff && (at == 0x7fffffff || better(v, i, best, at))) { best = v; at = i; }
        }
        const long long token = base_index + (at == 0x7fffffff ? 0 : at);
        if (world == 1) {
            if (lane == 0) tokens[row] = token < max_token ? token : max_token;
        } else {
            for (int j = lane; j < 4 * world; j += 32) {
                float v = 0.f;
                if (j == 4 * rank) v = best;
                if (j == 4 * rank + 2) v = (float)(token >> 8);
                if (j == 4 * rank + 3) v = (float)(token & 255);
                slots[(size_t)row * 4 * world + j] = __float2half_rn(v);
            }
        }
        if (lane == 0 && row == 0 && pos_inc) *pos_inc += 1;
    }
}

// Second half (several ranks): the summed slots hold every rank's {logit, 0, index / 256, index % 256}; the best logit
// wins, the lowest rank on a tie (its columns come first).
__global__ void __launch_bounds__(32)
pick_final_kernel(const __half* __restrict__ slots, int world, long long* __restrict__ tokens, long long max_token,
                  long long* __restrict__ pos_inc) {
    pdl_enter();
    const int row = blockIdx.x;
    if (threadIdx.x == 0) {
        const __half* s = slots + (size_t)row * 4 * world;
        float best = -INFINITY;
        long long token = 0;
        for (int r = 0; r < world; ++r) {
            const float v = __half2float(s[4 * r]) + __half2float(s[4 * r + 1]);
            if (r == 0 || v > best) {
                best = v;
                token = (long long)__half2float(s[4 * r + 2]) * 256 + (long long)__half2float(s[4 * r + 3]);
            }
        }
        tokens[row] = token < max_token ? token : max_token;
        if (row == 0 && pos_inc) *pos_inc += 1;
    }
}

}  // namespace
}  // namespace b200gptq

using namespace b200gptq;

namespace {
// One launch of the attention kernel.  A (sequence, head) gets as many warps as keep the whole grid resident at once:
// the kernel takes 128 registers per thread, so an SM holds 16 warps.
template <int HD, bool STEP>
cudaError_t launch_attention(const __half* q, const __half* k_cache, const __half* v_cache, const long long* pos,
                             __half* out, int batch, int heads, int max_seq, float scale, const __half* cos_t,
                             const __half* sin_t, int rope, __half* k_write, __half* v_write, void* stream) {
    const long long pairs = (long long)batch * heads;
    const long long warps_each = (16LL * sm_count()) / pairs;
#define B200GPTQ_ATTN(SPLIT, WARPS)                                                                                    \
    launch_pdl(attn_decode_kernel<HD, STEP, SPLIT, WARPS>, dim3(heads * SPLIT, batch), dim3(WARPS * 32), 0, stream,    \
               SPLIT, q, k_cache, v_cache, pos, out, heads, max_seq, scale, cos_t, sin_t, rope, k_write, v_write)
    if (warps_each >= 64) return B200GPTQ_ATTN(4, 16);
    if (warps_each >= 32) return B200GPTQ_ATTN(4, 8);
    if (warps_each >= 16) return B200GPTQ_ATTN(4, 4);
    if (warps_each >= 8) return B200GPTQ_ATTN(1, 8);
    return B200GPTQ_ATTN(1, 4);
#undef B200GPTQ_ATTN
}
}  // namespace

extern "C" {

B200GPTQ_API int b200gptq_add_norm(void* x, const void* add, const void* w, const void* beta, void* h, int rows,
                                   int H, float eps, int rms, void* stream) {
    if (!x || !w || !h) return B200GPTQ_ERR_NULL_POINTER;
    if (rows <= 0 || H <= 0 || H % 8 != 0 || H > 12288) return B200GPTQ_ERR_SHAPE;
    B200GPTQ_CUDA_TRY(launch_pdl(add_norm_kernel, dim3(rows), dim3(256), H * sizeof(float), stream, 1,
                                 static_cast<__half*>(x), static_cast<const __half*>(add),
                                 static_cast<const __half*>(w), static_cast<const __half*>(beta),
                                 static_cast<__half*>(h), H, eps, rms));
    return B200GPTQ_OK;
}

B200GPTQ_API int b200gptq_rope_cache(const void* qkv, const void* cos_t, const void* sin_t, const void* pos,
                                     void* q_out, void* k_cache, void* v_cache, int batch, int heads, int hd,
                                     int max_seq, int rope, void* stream) {
    if (!qkv || !pos || !q_out || !k_cache || !v_cache || (rope && (!cos_t || !sin_t))) return B200GPTQ_ERR_NULL_POINTER;
    if (batch <= 0 || heads <= 0 || hd % 2 != 0 || hd > 2048) return B200GPTQ_ERR_SHAPE;
    B200GPTQ_CUDA_TRY(launch_pdl(rope_cache_kernel, dim3(heads, batch), dim3(hd / 2), 0, stream, 1,
                                 static_cast<const __half*>(qkv), static_cast<const __half*>(cos_t),
                                 static_cast<const __half*>(sin_t), static_cast<const long long*>(pos),
                                 static_cast<__half*>(q_out), static_cast<__half*>(k_cache),
                                 static_cast<__half*>(v_cache), heads, hd, max_seq, rope));
    return B200GPTQ_OK;
}

B200GPTQ_API int b200gptq_attn_decode(const void* q, const void* k_cache, const void* v_cache, const void* pos,
                                      void* out, int batch, int heads, int hd, int max_seq, float scale,
                                      void* stream) {
    if (!q || !k_cache || !v_cache || !pos || !out) return B200GPTQ_ERR_NULL_POINTER;
    if (batch <= 0 || heads <= 0 || (hd != 64 && hd != 128)) return B200GPTQ_ERR_SHAPE;
    const __half* qh = static_cast<const __half*>(q);
    const __half* kh = static_cast<const __half*>(k_cache);
    const __half* vh = static_cast<const __half*>(v_cache);
    const long long* ph = static_cast<const long long*>(pos);
    __half* oh = static_cast<__half*>(out);
    if (hd == 128) {
        B200GPTQ_CUDA_TRY((launch_attention<128, false>(qh, kh, vh, ph, oh, batch, heads, max_seq, scale, nullptr, nullptr,
                                                        0, nullptr, nullptr, stream)));
    } else {
        B200GPTQ_CUDA_TRY((launch_attention<64, false>(qh, kh, vh, ph, oh, batch, heads, max_seq, scale, nullptr, nullptr,
                                                       0, nullptr, nullptr, stream)));
    }
    B200GPTQ_CUDA_TRY(cudaGetLastError());
    return B200GPTQ_OK;
}

B200GPTQ_API int b200gptq_attn_step(const void* qkv, const void* cos_t, const void* sin_t, const void* pos,
                                    void* k_cache, void* v_cache, void* out, int batch, int heads, int hd,
                                    int max_seq, int rope, float scale, void* stream) {
    if (!qkv || !k_cache || !v_cache || !pos || !out || (rope && (!cos_t || !sin_t))) return B200GPTQ_ERR_NULL_POINTER;
    if (batch <= 0 || heads <= 0 || (hd != 64 && hd != 128)) return B200GPTQ_ERR_SHAPE;
    const __half* qh = static_cast<const __half*>(qkv);
    const __half* kh = static_cast<const __half*>(k_cache);
    const __half* vh = static_cast<const __half*>(v_cache);
    const __half* ch = static_cast<const __half*>(cos_t);
    const __half* sh = static_cast<const __half*>(sin_t);
    const long long* ph = static_cast<const long long*>(pos);
    __half* oh = static_cast<__half*>(out);
    if (hd == 128) {
        B200GPTQ_CUDA_TRY((launch_attention<128, true>(qh, kh, vh, ph, oh, batch, heads, max_seq, scale, ch, sh, rope,
                                                       static_cast<__half*>(k_cache), static_cast<__half*>(v_cache),
                                                       stream)));
    } else {
        B200GPTQ_CUDA_TRY((launch_attention<64, true>(qh, kh, vh, ph, oh, batch, heads, max_seq, scale, ch, sh, rope,
                                                      static_cast<__half*>(k_cache), static_cast<__half*>(v_cache),
                                                      stream)));
    }
    B200GPTQ_CUDA_TRY(cudaGetLastError());
    return B200GPTQ_OK;
}

B200GPTQ_API int b200gptq_act(const void* u, void* act, int rows, int I, int gated, void* stream) {
    if (!u || !act) return B200GPTQ_ERR_NULL_POINTER;
    if (rows <= 0 || I <= 0 || I % 2 != 0) return B200GPTQ_ERR_SHAPE;
    const size_t total = (size_t)rows * I;
    const unsigned blocks = (unsigned)((total / 2 + 255) / 256);
    B200GPTQ_CUDA_TRY(launch_pdl(act_kernel, dim3(blocks), dim3(256), 0, stream, 1, static_cast<const __half*>(u),
                                 static_cast<__half*>(act), I, gated, total));
    return B200GPTQ_OK;
}

B200GPTQ_API int b200gptq_dense_gemv(const void* x, const void* w, void* y, int rows, int K, int N, void* stream) {
    if (!x || !w || !y) return B200GPTQ_ERR_NULL_POINTER;
    if (rows < 1 || rows > 8 || K <= 0 || N <= 0 || K % 8 != 0 || (size_t)rows * K * 2 > 96 * 1024) return B200GPTQ_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15u) return B200GPTQ_ERR_ALIGNMENT;
    const size_t smem = (size_t)rows * K * 2;
    int blocks = (N + 31) / 32;                     // a CTA's eight warps take 32 rows of w per round
    if (blocks > 4 * sm_count()) blocks = 4 * sm_count();
    const __half* xh = static_cast<const __half*>(x);
    const __half* wh = static_cast<const __half*>(w);
    __half* yh = static_cast<__half*>(y);
    if (rows == 1) {
        static std::once_flag once[64];
        int dev = 0;
        B200GPTQ_CUDA_TRY(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64)
            std::call_once(once[dev], [] {
                cudaFuncSetAttribute(dense_gemv_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            });
        B200GPTQ_CUDA_TRY(launch_pdl(dense_gemv_kernel<1>, dim3(blocks), dim3(256), smem, stream, 1, xh, wh, yh, rows, K, N));
    } else {
        static std::once_flag once8[64];
        int dev = 0;
        B200GPTQ_CUDA_TRY(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64)
            std::call_once(once8[dev], [] {
                cudaFuncSetAttribute(dense_gemv_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
            });
        B200GPTQ_CUDA_TRY(launch_pdl(dense_gemv_kernel<8>, dim3(blocks), dim3(256), smem, stream, 1, xh, wh, yh, rows, K, N));
    }
    return B200GPTQ_OK;
}

B200GPTQ_API int b200gptq_pick_local(const void* logits, int rows, int ld, int valid, long long base_index, int world,
                                     int rank, void* slots, long long* tokens, long long max_token, long long* pos_inc,
                                     void* stream) {
    if (!logits || (world == 1 ? !tokens : !slots)) return B200GPTQ_ERR_NULL_POINTER;
    if (rows < 1 || ld < 8 || ld % 8 != 0 || valid < 1 || valid > ld || world < 1 || rank < 0 || rank >= world)
        return B200GPTQ_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(logits) & 15u) return B200GPTQ_ERR_ALIGNMENT;
    B200GPTQ_CUDA_TRY(launch_pdl(pick_local_kernel, dim3(rows), dim3(1024), 0, stream, 1,
                                 static_cast<const __half*>(logits), ld, valid, base_index, world, rank,
                                 static_cast<__half*>(slots), tokens, max_token, pos_inc));
    return B200GPTQ_OK;
}

B200GPTQ_API int b200gptq_pick_final(const void* slots, int rows, int world, long long* tokens, long long max_token,
                                     long long* pos_inc, void* stream) {
    if (!slots || !tokens) return B200GPTQ_ERR_NULL_POINTER;
    if (rows < 1 || world < 1) return B200GPTQ_ERR_SHAPE;
    B200GPTQ_CUDA_TRY(launch_pdl(pick_final_kernel, dim3(rows), dim3(32), 0, stream, 1,
                                 static_cast<const __half*>(slots), world, tokens, max_token, pos_inc));
    return B200GPTQ_OK;
}

}  // extern "C"
