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

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int d = 16; d; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int d = 16; d; d >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, d));
    return v;
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
// Grid (head_kv, splits); D threads (one per channel of a head).  A CTA owns one kv head, its
// G = head_q / head_kv query heads and a contiguous share of the positions 0..pos.  Per tile of
// D positions: one thread per position forms the G scores (its K row against the roped,
// pre-scaled queries in shared memory), the warps update the running max/sum per head and turn
// scores into weights in shared memory, then one thread per channel adds weight * V.  Partial
// (max, sum, unnormalized output) go to the workspace; the CTA that arrives last for its kv
// head (a counter that it re-zeroes) merges the splits and writes fp16 output.
constexpr int kMaxGroup = 8;
constexpr int kMaxSplits = 64;      // kMaxGroup * kMaxSplits floats fit the tile buffers (D >= 64)

struct AttnArgs {
    const __half *q, *k, *v;      // this token's projections: [head_q][D], [head_kv][D], [head_kv][D]
    __half *kcache, *vcache;      // [max_ctx][head_kv][D] or [head_kv][max_ctx][D]
    long long pos_stride, head_stride;   // elements between two positions / two kv heads of a cache
    const int *position;          // device: position of this token = number of cached tokens
    __half *out;                  // [head_q][D]
    float *partial;               // [head_kv][splits][G][D + 2]
    unsigned *counters;           // [head_kv]
    int *status;
    int head_q, head_kv, group, max_ctx;
    float rotary_base, scale;
};

// S threads share a position in the score phase (each takes D/S channels of the K row) and
// S groups of threads share the positions of a tile in the weighted sum of V: with one warp
// per scheduler the kernel was bound by the latency of its own instruction chains.
template <int D, int S>
__global__ void __launch_bounds__(D *S) attention_decode_kernel(const AttnArgs a) {
    constexpr int T = D * S;               // threads
    constexpr int KV = D / 8 / S;          // 16-byte loads per thread for its part of a K row / of the V tile
    static_assert(S == 1 || S == 2 || S == 4, "threads per position");
    static_assert(KV >= 1 && (S - 1) * kMaxGroup * D * 4 <= D * D * 2, "the partial sums reuse the V tile");
    __shared__ __align__(16) float qs[kMaxGroup][D];       // roped queries times scale
    __shared__ __align__(16) float pw[D][kMaxGroup];       // scores, then weights, of a tile
    __shared__ __align__(16) __half vs[D * D];             // the V tile: [position][channel]
    __shared__ float alpha[kMaxGroup], m_run[kMaxGroup], l_run[kMaxGroup];
    __shared__ int is_last;
    pdl_enter();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int hk = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y;
    const int G = a.group;
    int pos = *a.position;
    if (pos < 0 || pos >= a.max_ctx) {           // refuse to write outside the cache
        if (tid == 0) atomicExch(a.status, 3);
        pos = pos < 0 ? 0 : a.max_ctx - 1;
    }
    const int nkv = pos + 1;
    const int per = (nkv + nsplit - 1) / nsplit;
    const int t0 = split * per, t1 = min(nkv, t0 + per);
    const size_t row_stride = (size_t)a.pos_stride;
    const size_t head_off = (size_t)hk * (size_t)a.head_stride;

    // RoPE: pair (j, j + D/2), angle = pos * base^(-2j/D), results rounded to fp16 as stored
    if (tid < D / 2) {
        const float ang = (float)pos * powf(a.rotary_base, -(float)(2 * tid) / (float)D);
        float sn, cs;
        sincosf(ang, &sn, &cs);
        float q1[kMaxGroup], q2[kMaxGroup];        // all loads first: they do not wait for one another
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            const __half *qp = a.q + (size_t)(hk * G + (g < G ? g : 0)) * D;
            q1[g] = __half2float(qp[tid]);
            q2[g] = __half2float(qp[tid + D / 2]);
        }
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            if (g < G) {
                qs[g][tid] = __half2float(__float2half_rn(q1[g] * cs - q2[g] * sn)) * a.scale;
                qs[g][tid + D / 2] = __half2float(__float2half_rn(q1[g] * sn + q2[g] * cs)) * a.scale;
            }
        }
        if (pos >= t0 && pos < t1) {             // this CTA's share holds the new position: append
            const __half *kp = a.k + (size_t)hk * D;
            const float k1 = __half2float(kp[tid]), k2 = __half2float(kp[tid + D / 2]);
            __half *kc = a.kcache + (size_t)pos * row_stride + head_off;
            kc[tid] = __float2half_rn(k1 * cs - k2 * sn);
            kc[tid + D / 2] = __float2half_rn(k1 * sn + k2 * cs);
        }
    } else if (tid < D && pos >= t0 && pos < t1) {
        const int j = tid - D / 2;
        __half *vc = a.vcache + (size_t)pos * row_stride + head_off;
        const __half *vp = a.v + (size_t)hk * D;
        vc[j] = vp[j];
        vc[j + D / 2] = vp[j + D / 2];
    }
    if (tid < kMaxGroup) {
        m_run[tid] = -INFINITY;
        l_run[tid] = 0.f;
        alpha[tid] = 0.f;
    }
    float acc[kMaxGroup];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) acc[g] = 0.f;
    __syncthreads();

    const int sp = tid / S, part = tid % S;      // score phase: position of the tile, part of its row
    const int ch = tid % D, pg = tid / D;        // V phase: channel, group of positions
    for (int tile = t0; tile < t1; tile += D) {
        const int ntile = min(D, t1 - tile);
        // All global loads of the tile are issued before anything is computed: this thread's
        // part of a K row and its share of the V tile (both coalesced).
        uint4 kreg[KV], vreg[KV];
        if (sp < ntile) {
            // the S threads of a position take every S-th 16-byte chunk of the row: their loads
            // coalesce, and their reads of the queries below fall into different banks
            const uint4 *kr = (const uint4 *)(a.kcache + (size_t)(tile + sp) * row_stride + head_off) + part;
#pragma unroll
            for (int c = 0; c < KV; ++c) kreg[c] = kr[c * S];
        }
#pragma unroll
        for (int u = 0; u < KV; ++u) {
            const int idx = tid + u * T, t = idx / (D / 8), c8 = idx % (D / 8);
            vreg[u] = make_uint4(0u, 0u, 0u, 0u);
            if (t < ntile)
                vreg[u] = *(const uint4 *)(a.vcache + (size_t)(tile + t) * row_stride + head_off + 8 * c8);
        }
        // scores: S threads per position, then a shuffle reduction among them
        {
            float s[kMaxGroup];
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) s[g] = 0.f;
            if (sp < ntile) {
#pragma unroll
                for (int c = 0; c < KV; ++c) {
                    const __half2 *kh = (const __half2 *)&kreg[c];
                    float kf[8];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 f = __half22float2(kh[e]);
                        kf[2 * e] = f.x;
                        kf[2 * e + 1] = f.y;
                    }
                    const int c0 = 8 * (c * S + part);
#pragma unroll
                    for (int g = 0; g < kMaxGroup; ++g) {
                        if (g < G) {
                            const float4 qa = *(const float4 *)&qs[g][c0], qb = *(const float4 *)&qs[g][c0 + 4];
                            s[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x +
                                    kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
                        }
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) {
#pragma unroll
                for (int dd = 1; dd < S; dd <<= 1) s[g] += __shfl_xor_sync(0xffffffffu, s[g], dd);
                if (sp >= ntile) s[g] = -INFINITY;
            }
            if (part == 0) {
#pragma unroll
                for (int g = 0; g < kMaxGroup; ++g) pw[sp][g] = s[g];
            }
        }
#pragma unroll
        for (int u = 0; u < KV; ++u) ((uint4 *)vs)[tid + u * T] = vreg[u];
        __syncthreads();
        // running max and sum per head; scores become weights
        for (int g = warp; g < G; g += T / 32) {
            float sv[D / 32], tmax = -INFINITY;
#pragma unroll
            for (int i = 0; i < D / 32; ++i) {
                sv[i] = pw[lane + 32 * i][g];
                tmax = fmaxf(tmax, sv[i]);
            }
            tmax = warp_max(tmax);
            const float mold = m_run[g], mnew = fmaxf(mold, tmax);
            float psum = 0.f;
#pragma unroll
            for (int i = 0; i < D / 32; ++i) {
                const float p = expf(sv[i] - mnew);       // exp(-inf) = 0 for the positions past the tile
                pw[lane + 32 * i][g] = p;
                psum += p;
            }
            psum = warp_sum(psum);
            if (lane == 0) {
                const float al = expf(mold - mnew);        // 0 on the first tile (mold = -inf)
                alpha[g] = al;
                m_run[g] = mnew;
                l_run[g] = l_run[g] * al + psum;
            }
        }
        __syncthreads();
        // weighted sum of V from shared memory: thread = (channel, group of positions)
        {
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) acc[g] *= alpha[g];
            const int tb = pg * (D / S), te = min(ntile, tb + D / S);
#pragma unroll 8
            for (int t = tb; t < te; ++t) {
                const float v = __half2float(vs[t * D + ch]);
                const float4 pa = *(const float4 *)&pw[t][0], pb = *(const float4 *)&pw[t][4];
                acc[0] += pa.x * v; acc[1] += pa.y * v; acc[2] += pa.z * v; acc[3] += pa.w * v;
                acc[4] += pb.x * v; acc[5] += pb.y * v; acc[6] += pb.z * v; acc[7] += pb.w * v;
            }
        }
        __syncthreads();
    }
    // the S groups' sums of a channel meet in shared memory (the V tile is free now)
    if (S > 1) {
        float *part_acc = (float *)vs;           // [S - 1][kMaxGroup][D]
        if (pg > 0) {
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) part_acc[((pg - 1) * kMaxGroup + g) * D + ch] = acc[g];
        }
        __syncthreads();
        if (pg == 0) {
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g)
#pragma unroll
                for (int o = 0; o < S - 1; ++o) acc[g] += part_acc[(o * kMaxGroup + g) * D + ch];
        }
    }
    // publish this split (threads of the first group: one per channel)
    float *mine = a.partial + ((size_t)hk * nsplit + split) * G * (D + 2);
    if (tid < D) {
        for (int g = 0; g < G; ++g) {
            mine[(size_t)g * (D + 2) + tid] = acc[g];
            if (tid == 0) {
                mine[(size_t)g * (D + 2) + D] = m_run[g];
                mine[(size_t)g * (D + 2) + D + 1] = l_run[g];
            }
        }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned old = atomicAdd(&a.counters[hk], 1u);
        is_last = (old + 1u == (unsigned)nsplit);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // merge of the splits: thread = (channel, head phase), the heads are dealt out over the S
    // groups.  A thread loads its channel's partial sums and the (max, sum) pairs of all splits
    // at once (one round trip), forms the weights exp(max_s - max) itself and writes fp16.
    const float *base = a.partial + (size_t)hk * nsplit * G * (D + 2);
    for (int g = pg; g < G; g += S) {
        float M = -INFINITY;
        for (int s0 = 0; s0 < nsplit; s0 += 16) {
            float ov[16], mv[16], lv[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int s = min(s0 + u, nsplit - 1);
                const float *p = base + ((size_t)s * G + g) * (D + 2);
                ov[u] = __ldcg(p + ch);
                mv[u] = __ldcg(p + D);
                lv[u] = s0 + u < nsplit ? __ldcg(p + D + 1) : 0.f;
            }
            float Mc = M;
#pragma unroll
            for (int u = 0; u < 16; ++u) Mc = fmaxf(Mc, mv[u]);
            // running rescale across chunks of 16 splits (one chunk for caches up to 2048 positions)
            const float r = s0 ? expf(M - Mc) : 0.f;
            if (s0 == 0) {
                acc[0] = 0.f;
                acc[1] = 0.f;
            }
            acc[0] *= r;
            acc[1] *= r;
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const float w = s0 + u < nsplit ? expf(mv[u] - Mc) : 0.f;
                acc[0] += ov[u] * w;          // weighted output of this channel
                acc[1] += lv[u] * w;          // weighted sum of the softmax denominators
            }
            M = Mc;
        }
        a.out[(size_t)(hk * G + g) * D + ch] = __float2half_rn(acc[0] / acc[1]);
    }
    if (tid == 0) a.counters[hk] = 0u;
}

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

}  // namespace
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
