// Decoder glue around the quantized linears, fp16, batch-1 decode, sm_100a.
//
// Replaces the reference runtime's per-token ops between two linears
// (called from C++/examples/models/llama.cpp:193-215, 396-476, 554, 646, 717, 763):
//   C++/ops/src/arm/arm_rmsnorm.cpp:25-41, 68-85      RMSNorm and residual-add + RMSNorm
//   C++/ops/src/arm/arm_rotary.cpp:4-88               RoPE on q and k (half-split pairs j, j + d/2)
//   C++/ops/src/arm/arm_cache.cpp:3-22                append k, v at the token's position
//   C++/ops/src/arm/arm_attention.cpp:196-270         single-token attention, grouped heads
//   C++/ops/src/arm/arm_activation.cpp:22-52          silu(gate) * up
//   C++/ops/src/arm/arm_argmax.cpp:3-29               greedy token
// RoPE, the cache append and the attention are one kernel; the others one kernel each.  All
// are launched with programmatic dependent launch and wait for their producers first, so in a
// stream (or a captured graph) of such kernels only the waits are serialized, not the launches.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>

#include <stdint.h>

#include "hlq_attn_dev.cuh"
#include "hlq_internal.h"

namespace hlq {
namespace {

__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename KernelT, typename... Args>
int launch_glue(KernelT kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    HLQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, args...));
    count_launch();
    return HLQ_OK;
}

// ---- RMSNorm (+ residual add) -------------------------------------------------------------
// One CTA per row.  With a residual: t = x + residual in fp32, the sum of squares is taken
// over t, t is stored rounded to fp16 (res_out) and the ROUNDED value is normalized, as the
// reference does (arm_rmsnorm.cpp:70-83).  out may alias x, res_out may alias residual.
constexpr int kNormThreads = 1024;

__global__ void __launch_bounds__(kNormThreads) rmsnorm_kernel(const __half *x, const __half *residual,
                                                               __half *res_out, const __half *gamma, float eps,
                                                               __half *out, int n) {
    __shared__ float part[kNormThreads / 32];
    __shared__ float inv_rms;
    pdl_enter();
    const size_t row = (size_t)blockIdx.x * n;
    const int nv = n >> 3;
    float sum = 0.f;
    for (int i = threadIdx.x; i < nv; i += kNormThreads) {
        uint4 a = *(const uint4 *)(x + row + 8 * (size_t)i);
        const __half2 *ah = (const __half2 *)&a;
        if (residual) {
            const uint4 b = *(const uint4 *)(residual + row + 8 * (size_t)i);
            const __half2 *bh = (const __half2 *)&b;
            uint4 o;
            __half2 *oh = (__half2 *)&o;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 fa = __half22float2(ah[e]), fb = __half22float2(bh[e]);
                const float t0 = fa.x + fb.x, t1 = fa.y + fb.y;
                sum += t0 * t0 + t1 * t1;
                oh[e] = __floats2half2_rn(t0, t1);
            }
            *(uint4 *)(res_out + row + 8 * (size_t)i) = o;
        } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 fa = __half22float2(ah[e]);
                sum += fa.x * fa.x + fa.y * fa.y;
            }
        }
    }
    sum = warp_sum(sum);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < kNormThreads / 32 ? part[threadIdx.x] : 0.f;
        v = warp_sum(v);
        if (threadIdx.x == 0) inv_rms = 1.0f / sqrtf(v / (float)n + eps);
    }
    __syncthreads();
    const float inv = inv_rms;
    const __half *src = residual ? res_out : x;
    for (int i = threadIdx.x; i < nv; i += kNormThreads) {
        const uint4 a = *(const uint4 *)(src + row + 8 * (size_t)i);
        const uint4 g = *(const uint4 *)(gamma + 8 * (size_t)i);
        const __half2 *ah = (const __half2 *)&a, *gh = (const __half2 *)&g;
        uint4 o;
        __half2 *oh = (__half2 *)&o;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 fa = __half22float2(ah[e]), fg = __half22float2(gh[e]);
            oh[e] = __floats2half2_rn(fa.x * fg.x * inv, fa.y * fg.y * inv);
        }
        *(uint4 *)(out + row + 8 * (size_t)i) = o;
    }
}

// ---- silu(gate) * up ----------------------------------------------------------------------
__global__ void __launch_bounds__(256) gated_silu_kernel(const __half *gate, const __half *up, __half *out,
                                                         long long nv) {
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nv;
         i += (long long)gridDim.x * blockDim.x) {
        const uint4 a = ((const uint4 *)gate)[i], b = ((const uint4 *)up)[i];
        const __half2 *ah = (const __half2 *)&a, *bh = (const __half2 *)&b;
        uint4 o;
        __half2 *oh = (__half2 *)&o;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 g = __half22float2(ah[e]), u = __half22float2(bh[e]);
            oh[e] = __floats2half2_rn(u.x * (g.x / (1.0f + expf(-g.x))), u.y * (g.y / (1.0f + expf(-g.y))));
        }
        ((uint4 *)out)[i] = o;
    }
}

// ---- argmax -------------------------------------------------------------------------------
// First index of the largest value (the reference keeps the first: strict >, arm_argmax.cpp:22).
template <typename T>
__global__ void __launch_bounds__(1024) argmax_kernel(const T *v, int n, int *index_out, float *value_out) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    pdl_enter();
    float best = -INFINITY;
    int idx = 0x7fffffff;
    auto take = [&](float f, int i) {
        if (f > best || (f == best && i < idx)) {
            best = f;
            idx = i;
        }
    };
    // 16-byte loads, four of them in flight per thread; scalar head and tail
    constexpr int kPer = 16 / (int)sizeof(T);
    const int head = min(n, (int)(((16 - ((uintptr_t)v & 15)) & 15) / sizeof(T)));
    const int nvec = (n - head) / kPer;
    const uint4 *vv = (const uint4 *)(v + head);
    for (int i0 = threadIdx.x; i0 < nvec; i0 += 4 * blockDim.x) {
        uint4 w[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * (int)blockDim.x < nvec) w[u] = vv[i0 + u * blockDim.x];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * (int)blockDim.x;
            if (i < nvec) {
                const T *e = (const T *)&w[u];
#pragma unroll
                for (int k = 0; k < kPer; ++k) take((float)e[k], head + i * kPer + k);
            }
        }
    }
    for (int i = threadIdx.x; i < head; i += blockDim.x) take((float)v[i], i);
    for (int i = head + nvec * kPer + threadIdx.x; i < n; i += blockDim.x) take((float)v[i], i);
    auto merge = [&](float ov, int oi) { take(ov, oi); };
#pragma unroll
    for (int d = 16; d; d >>= 1) merge(__shfl_xor_sync(0xffffffffu, best, d), __shfl_xor_sync(0xffffffffu, idx, d));
    if ((threadIdx.x & 31) == 0) {
        bv[threadIdx.x >> 5] = best;
        bi[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = (blockDim.x + 31) >> 5;
        best = threadIdx.x < nw ? bv[threadIdx.x] : -INFINITY;
        idx = threadIdx.x < nw ? bi[threadIdx.x] : 0x7fffffff;
#pragma unroll
        for (int d = 16; d; d >>= 1)
            merge(__shfl_xor_sync(0xffffffffu, best, d), __shfl_xor_sync(0xffffffffu, idx, d));
        if (threadIdx.x == 0) {
            *index_out = idx == 0x7fffffff ? 0 : idx;
            if (value_out) *value_out = best;
        }
    }
}

// ---- RoPE + cache append + single-token attention -----------------------------------------
// Grid (head_kv, splits), D * S threads: every CTA runs one unit of hlq_attn_dev.cuh.
template <int D, int S>
__global__ void __launch_bounds__(D *S) attention_decode_kernel(const AttnArgs a) {
    __shared__ AttnSmem<D> sm;
    pdl_enter();
    attention_unit<D, S>(a, blockIdx.x, blockIdx.y, gridDim.y, sm, threadIdx.x, [] { __syncthreads(); });
}

}  // namespace

// splits per kv head for a cache of max_ctx positions: about one CTA per SM, at least 128
// positions each, at most kMaxSplits
int attention_splits(int head_kv, int max_ctx) {
    int s = (148 + head_kv - 1) / head_kv;
    const int most = (max_ctx + 127) / 128;
    if (s > most) s = most;
    if (s < 1) s = 1;
    if (s > kMaxSplits) s = kMaxSplits;
    return s;
}

}  // namespace hlq

using namespace hlq;

extern "C" {

int hlq_rmsnorm(int rows, int n, const void *d_x, const void *d_residual, void *d_res_out, const void *d_gamma,
                float eps, void *d_out, void *stream) {
    if (rows < 0 || n <= 0 || !d_x || !d_gamma || !d_out) return HLQ_ERR_INVALID_ARGUMENT;
    if (d_residual && !d_res_out) return HLQ_ERR_INVALID_ARGUMENT;
    if (n % 8) return HLQ_ERR_SHAPE;
    if (((uintptr_t)d_x | (uintptr_t)d_out | (uintptr_t)d_gamma | (uintptr_t)d_residual | (uintptr_t)d_res_out) & 15)
        return HLQ_ERR_ALIGNMENT;
    if (rows == 0) return HLQ_OK;
    return launch_glue(rmsnorm_kernel, dim3(rows), dim3(kNormThreads), 0, (cudaStream_t)stream, (const __half *)d_x,
                       (const __half *)d_residual, (__half *)d_res_out, (const __half *)d_gamma, eps, (__half *)d_out,
                       n);
}

int hlq_gated_silu(int rows, int n, const void *d_gate, const void *d_up, void *d_out, void *stream) {
    if (rows < 0 || n <= 0 || !d_gate || !d_up || !d_out) return HLQ_ERR_INVALID_ARGUMENT;
    const long long total = (long long)rows * n;
    if (total % 8) return HLQ_ERR_SHAPE;
    if (((uintptr_t)d_gate | (uintptr_t)d_up | (uintptr_t)d_out) & 15) return HLQ_ERR_ALIGNMENT;
    if (total == 0) return HLQ_OK;
    const long long nv = total / 8;
    long long blocks = (nv + 255) / 256;
    if (blocks > 1184) blocks = 1184;
    return launch_glue(gated_silu_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream,
                       (const __half *)d_gate, (const __half *)d_up, (__half *)d_out, nv);
}

int hlq_argmax(int n, const void *d_values, int dtype, int *d_index_out, float *d_value_out, void *stream) {
    if (n <= 0 || !d_values || !d_index_out) return HLQ_ERR_INVALID_ARGUMENT;
    if (dtype == HLQ_F16)
        return launch_glue(argmax_kernel<__half>, dim3(1), dim3(1024), 0, (cudaStream_t)stream,
                           (const __half *)d_values, n, d_index_out, d_value_out);
    if (dtype == HLQ_F32)
        return launch_glue(argmax_kernel<float>, dim3(1), dim3(1024), 0, (cudaStream_t)stream,
                           (const float *)d_values, n, d_index_out, d_value_out);
    return HLQ_ERR_UNSUPPORTED;
}

size_t hlq_attention_workspace_bytes(int head_q, int head_kv, int dhead, int max_ctx) {
    if (head_q <= 0 || head_kv <= 0 || head_q % head_kv || dhead <= 0 || max_ctx <= 0) return 0;
    const int splits = attention_splits(head_kv, max_ctx);
    const size_t partial = (size_t)head_kv * splits * (head_q / head_kv) * (dhead + 2) * sizeof(float);
    return kWsHeader + ((partial + 255) & ~(size_t)255) + (((size_t)head_kv * 4 + 255) & ~(size_t)255);
}

int hlq_rope_cache_attention(const void *d_q, const void *d_k, const void *d_v, void *d_kcache, void *d_vcache,
                             const int *d_position, int head_q, int head_kv, int dhead, int max_ctx,
                             int kv_layout, float rotary_base, float scale, void *d_out, void *d_workspace,
                             size_t workspace_bytes, void *stream) {
    if (!d_q || !d_k || !d_v || !d_kcache || !d_vcache || !d_position || !d_out || !d_workspace)
        return HLQ_ERR_INVALID_ARGUMENT;
    if (head_q <= 0 || head_kv <= 0 || max_ctx <= 0 || head_q % head_kv) return HLQ_ERR_SHAPE;
    if (head_q / head_kv > kMaxGroup) return HLQ_ERR_UNSUPPORTED;
    if (dhead != 128 && dhead != 64) return HLQ_ERR_UNSUPPORTED;
    if (kv_layout != HLQ_KV_POSITION_MAJOR && kv_layout != HLQ_KV_HEAD_MAJOR) return HLQ_ERR_INVALID_ARGUMENT;
    if (((uintptr_t)d_kcache | (uintptr_t)d_vcache | (uintptr_t)d_workspace) & 15) return HLQ_ERR_ALIGNMENT;
    const size_t need = hlq_attention_workspace_bytes(head_q, head_kv, dhead, max_ctx);
    if (workspace_bytes < need) return HLQ_ERR_WORKSPACE;
    const int splits = attention_splits(head_kv, max_ctx);
    const size_t partial = (size_t)head_kv * splits * (head_q / head_kv) * (dhead + 2) * sizeof(float);
    AttnArgs a;
    a.q = (const __half *)d_q;
    a.k = (const __half *)d_k;
    a.v = (const __half *)d_v;
    a.kcache = (__half *)d_kcache;
    a.vcache = (__half *)d_vcache;
    a.position = d_position;
    a.out = (__half *)d_out;
    a.status = (int *)d_workspace;
    a.partial = (float *)((char *)d_workspace + kWsHeader);
    a.counters = (unsigned *)((char *)d_workspace + kWsHeader + ((partial + 255) & ~(size_t)255));
    a.head_q = head_q;
    a.head_kv = head_kv;
    a.group = head_q / head_kv;
    a.max_ctx = max_ctx;
    a.pos_stride = kv_layout == HLQ_KV_HEAD_MAJOR ? dhead : (long long)head_kv * dhead;
    a.head_stride = kv_layout == HLQ_KV_HEAD_MAJOR ? (long long)max_ctx * dhead : dhead;
    a.rotary_base = rotary_base;
    a.scale = scale;
    if (dhead == 128)
        return launch_glue(attention_decode_kernel<128, 4>, dim3(head_kv, splits), dim3(512), 0, (cudaStream_t)stream,
                           a);
    return launch_glue(attention_decode_kernel<64, 4>, dim3(head_kv, splits), dim3(256), 0, (cudaStream_t)stream, a);
}

}  // extern "C"
