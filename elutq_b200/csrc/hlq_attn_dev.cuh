// RoPE + KV-cache append + single-token attention for one (kv head, split of the context) unit,
// as a device function: the stand-alone kernel of hlq_glue.cu and the decode chain kernel of
// hlq_chain.cu both run it.
//
// Replaces, for one token:
//   C++/ops/src/arm/arm_rotary.cpp:4-88               RoPE on q and k (half-split pairs j, j + d/2)
//   C++/ops/src/arm/arm_cache.cpp:3-22                append k, v at the token's position
//   C++/ops/src/arm/arm_attention.cpp:196-270         single-token attention, grouped heads
#pragma once
#include <cuda_fp16.h>
#include <math.h>
#include <stdint.h>

namespace hlq {

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

// Work unit (kv head, split); D * S threads.  A unit owns one kv head, its
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

// Shared memory of one unit (41 KB at D = 128).
template <int D>
struct AttnSmem {
    __align__(16) float qs[kMaxGroup][D];       // roped queries times scale
    __align__(16) float pw[D][kMaxGroup];       // scores, then weights, of a tile
    __align__(16) __half vs[D * D];             // the V tile: [position][channel]
    float alpha[kMaxGroup], m_run[kMaxGroup], l_run[kMaxGroup];
    int is_last;
    __align__(16) __half knew[D], vnew[D];      // the new token's roped k row and v row (attention_partial_unit)
};

// S threads share a position in the score phase (each takes D/S channels of the K row) and
// S groups of threads share the positions of a tile in the weighted sum of V: with one warp
// per scheduler the kernel was bound by the latency of its own instruction chains.
// `sync` is a barrier over the D * S threads that run the unit (thread index `tid`); `rope`, if
// given, holds {cos, sin} of the D/2 rotary angles of the token's (clamped) position.  Returns
// true in the unit that arrived last for its kv head, merged the splits and wrote the output.
template <int D, int S, typename Sync>
__device__ __forceinline__ bool attention_unit(const AttnArgs &a, int hk, int split, int nsplit, AttnSmem<D> &sm,
                                               int tid, Sync sync, const float2 *rope = nullptr,
                                               unsigned long long *stamps = nullptr) {

    constexpr int T = D * S;               // threads
    constexpr int KV = D / 8 / S;          // 16-byte loads per thread for its part of a K row / of the V tile
    static_assert(S == 1 || S == 2 || S == 4, "threads per position");
    static_assert(KV >= 1 && (S - 1) * kMaxGroup * D * 4 <= D * D * 2, "the partial sums reuse the V tile");
    auto &qs = sm.qs;
    auto &pw = sm.pw;
    __half *vs = sm.vs;
    float *alpha = sm.alpha, *m_run = sm.m_run, *l_run = sm.l_run;
    int &is_last = sm.is_last;
    const int lane = tid & 31, warp = tid >> 5;
    auto mark = [&](int k) {
        if (stamps && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            stamps[k] = t;
        }
    };
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
        float sn, cs;
        if (rope) {                               // {cos, sin} of this position, prepared by the caller
            cs = rope[tid].x;
            sn = rope[tid].y;
        } else {
            const float ang = (float)pos * powf(a.rotary_base, -(float)(2 * tid) / (float)D);
            sincosf(ang, &sn, &cs);
        }
        float q1[kMaxGroup], q2[kMaxGroup];        // all loads first: they do not wait for one another
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            const __half *qp = a.q + (size_t)(hk * G + (g < G ? g : 0)) * D;
            q1[g] = __half2float(__ldcg(qp + tid));          // through L2: another SM wrote them, possibly
            q2[g] = __half2float(__ldcg(qp + tid + D / 2));  // inside this very kernel (decode chain)
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
            const float k1 = __half2float(__ldcg(kp + tid)), k2 = __half2float(__ldcg(kp + tid + D / 2));
            __half *kc = a.kcache + (size_t)pos * row_stride + head_off;
            kc[tid] = __float2half_rn(k1 * cs - k2 * sn);
            kc[tid + D / 2] = __float2half_rn(k1 * sn + k2 * cs);
        }
    } else if (tid < D && pos >= t0 && pos < t1) {
        const int j = tid - D / 2;
        __half *vc = a.vcache + (size_t)pos * row_stride + head_off;
        const __half *vp = a.v + (size_t)hk * D;
        vc[j] = __ldcg(vp + j);
        vc[j + D / 2] = __ldcg(vp + j + D / 2);
    }
    if (tid < kMaxGroup) {
        m_run[tid] = -INFINITY;
        l_run[tid] = 0.f;
        alpha[tid] = 0.f;
    }
    float acc[kMaxGroup];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) acc[g] = 0.f;
    sync();
    mark(0);

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
        sync();
        mark(1);
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
        sync();
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
        sync();
        mark(2);
    }
    // the S groups' sums of a channel meet in shared memory (the V tile is free now)
    if (S > 1) {
        float *part_acc = (float *)vs;           // [S - 1][kMaxGroup][D]
        if (pg > 0) {
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) part_acc[((pg - 1) * kMaxGroup + g) * D + ch] = acc[g];
        }
        sync();
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
    sync();
    mark(3);
    if (tid == 0) {
        const unsigned old = atomicAdd(&a.counters[hk], 1u);
        is_last = (old + 1u == (unsigned)nsplit);
    }
    sync();
    mark(4);
    if (!is_last) return false;
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
    return true;
}

// The same unit for a caller that merges the splits itself (the decode chain: the linear that
// consumes the attention output merges them while it loads its activations).  Differences from
// attention_unit: the token's position `pos` (already clamped to the cache) and the rotary table
// `rope` come from the caller; the loads of the first K/V tile are issued BEFORE `wait_inputs()`
// returns (the cache does not depend on this token's q, k, v; the row of the new position is
// taken from the new k and v instead of from the prefetched tile); the unit ends when its
// partial (unnormalized output, running max and sum per head) is written to a.partial: no
// counter, no merge, a.out is not written.  `wait_inputs()` is called by all threads, returns
// the same value in all of them once q, k, v may be read, false to abandon the unit.
template <int D, int S, typename Sync, typename Wait>
__device__ __forceinline__ void attention_partial_unit(const AttnArgs &a, int hk, int split, int nsplit,
                                                       AttnSmem<D> &sm, int tid, Sync sync, const float2 *rope,
                                                       int pos, Wait wait_inputs, unsigned long long *stamps = nullptr) {
    constexpr int T = D * S;
    constexpr int KV = D / 8 / S;
    static_assert(S == 1 || S == 2 || S == 4, "threads per position");
    static_assert(KV >= 1 && (S - 1) * kMaxGroup * D * 4 <= D * D * 2, "the partial sums reuse the V tile");
    auto &qs = sm.qs;
    auto &pw = sm.pw;
    __half *vs = sm.vs;
    float *alpha = sm.alpha, *m_run = sm.m_run, *l_run = sm.l_run;
    const int lane = tid & 31, warp = tid >> 5;
    auto mark = [&](int k) {
        if (stamps && tid == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            stamps[k] = t;
        }
    };
    const int G = a.group;
    const int nkv = pos + 1;
    const int per = (nkv + nsplit - 1) / nsplit;
    const int t0 = split * per, t1 = min(nkv, t0 + per);
    const size_t row_stride = (size_t)a.pos_stride;
    const size_t head_off = (size_t)hk * (size_t)a.head_stride;
    const int sp = tid / S, part = tid % S;      // score phase: position of the tile, part of its row
    const int ch = tid % D, pg = tid / D;        // V phase: channel, group of positions

    // the first tile's loads, before the inputs are there
    uint4 kreg[KV], vreg[KV];
    auto load_tile_regs = [&](int tile, int ntile) {
        if (sp < ntile) {
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
    };
    if (t0 < t1) load_tile_regs(t0, min(D, t1 - t0));
    if (!wait_inputs()) return;
    mark(0);

    // RoPE: pair (j, j + D/2); q, k and v of this token are loaded together
    if (tid < D / 2) {
        const float cs = rope[tid].x, sn = rope[tid].y;
        float q1[kMaxGroup], q2[kMaxGroup];
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            const __half *qp = a.q + (size_t)(hk * G + (g < G ? g : 0)) * D;
            q1[g] = __half2float(__ldcg(qp + tid));
            q2[g] = __half2float(__ldcg(qp + tid + D / 2));
        }
        const __half *kp = a.k + (size_t)hk * D;
        const float k1 = __half2float(__ldcg(kp + tid)), k2 = __half2float(__ldcg(kp + tid + D / 2));
#pragma unroll
        for (int g = 0; g < kMaxGroup; ++g) {
            if (g < G) {
                qs[g][tid] = __half2float(__float2half_rn(q1[g] * cs - q2[g] * sn)) * a.scale;
                qs[g][tid + D / 2] = __half2float(__float2half_rn(q1[g] * sn + q2[g] * cs)) * a.scale;
            }
        }
        const __half ka = __float2half_rn(k1 * cs - k2 * sn), kb = __float2half_rn(k1 * sn + k2 * cs);
        sm.knew[tid] = ka;
        sm.knew[tid + D / 2] = kb;
        if (pos >= t0 && pos < t1) {             // this unit's share holds the new position: append
            __half *kc = a.kcache + (size_t)pos * row_stride + head_off;
            kc[tid] = ka;
            kc[tid + D / 2] = kb;
        }
    } else if (tid < D) {
        const int j = tid - D / 2;
        const __half *vp = a.v + (size_t)hk * D;
        const __half va = __ldcg(vp + j), vb = __ldcg(vp + j + D / 2);
        sm.vnew[j] = va;
        sm.vnew[j + D / 2] = vb;
        if (pos >= t0 && pos < t1) {
            __half *vc = a.vcache + (size_t)pos * row_stride + head_off;
            vc[j] = va;
            vc[j + D / 2] = vb;
        }
    }
    if (tid < kMaxGroup) {
        m_run[tid] = -INFINITY;
        l_run[tid] = 0.f;
        alpha[tid] = 0.f;
    }
    float acc[kMaxGroup];
#pragma unroll
    for (int g = 0; g < kMaxGroup; ++g) acc[g] = 0.f;
    sync();
    mark(1);

    for (int tile = t0; tile < t1; tile += D) {
        const int ntile = min(D, t1 - tile);
        if (tile != t0) load_tile_regs(tile, ntile);
        // the new position's row: from the new k / v, not from the (possibly prefetched) cache
        if (tile + sp == pos) {
#pragma unroll
            for (int c = 0; c < KV; ++c) kreg[c] = *(const uint4 *)(sm.knew + 8 * (c * S + part));
        }
#pragma unroll
        for (int u = 0; u < KV; ++u) {
            const int idx = tid + u * T, t = idx / (D / 8), c8 = idx % (D / 8);
            if (tile + t == pos) vreg[u] = *(const uint4 *)(sm.vnew + 8 * c8);
        }
        // scores, one query head at a time (one accumulator live instead of eight): S threads
        // per position, then a shuffle reduction among them
#pragma unroll 1
        for (int g = 0; g < G; ++g) {
            float s = 0.f;
            if (sp < ntile) {
#pragma unroll
                for (int c = 0; c < KV; ++c) {
                    const __half2 *kh = (const __half2 *)&kreg[c];
                    const int c0 = 8 * (c * S + part);
                    const float4 qa = *(const float4 *)&qs[g][c0], qb = *(const float4 *)&qs[g][c0 + 4];
                    const float2 f0 = __half22float2(kh[0]), f1 = __half22float2(kh[1]);
                    const float2 f2 = __half22float2(kh[2]), f3 = __half22float2(kh[3]);
                    s += f0.x * qa.x + f0.y * qa.y + f1.x * qa.z + f1.y * qa.w + f2.x * qb.x + f2.y * qb.y +
                         f3.x * qb.z + f3.y * qb.w;
                }
            }
#pragma unroll
            for (int dd = 1; dd < S; dd <<= 1) s += __shfl_xor_sync(0xffffffffu, s, dd);
            if (sp >= ntile) s = -INFINITY;
            if (part == 0) pw[sp][g] = s;
        }
#pragma unroll
        for (int u = 0; u < KV; ++u) ((uint4 *)vs)[tid + u * T] = vreg[u];
        sync();
        mark(2);
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
        sync();
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
        sync();
    }
    mark(3);
    if (S > 1) {
        float *part_acc = (float *)vs;           // [S - 1][kMaxGroup][D]
        if (pg > 0) {
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g) part_acc[((pg - 1) * kMaxGroup + g) * D + ch] = acc[g];
        }
        sync();
        if (pg == 0) {
#pragma unroll
            for (int g = 0; g < kMaxGroup; ++g)
#pragma unroll
                for (int o = 0; o < S - 1; ++o) acc[g] += part_acc[(o * kMaxGroup + g) * D + ch];
        }
    }
    // this split's partial: a share without positions (t0 >= t1) publishes max = -inf, sum = 0
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
    mark(4);
}

// Merge of the splits for `nheads` (<= 4) consecutive query heads, by the T = 128 * nheads...512
// threads of a CTA that then need the merged values (one channel per thread):
//   1. every thread issues the loads of its channel's unnormalized outputs of all splits;
//   2. warp h (h < nheads) turns the splits' (max, sum) pairs of head h into normalized weights
//      exp(max_s - max) / sum_s(...) in shared memory `wn` [4][64];
//   3. after `sync`, out = sum_s output_s * weight_s.
// `first_head` = local index of the first head, `partial` = [head_kv][nsplit][group][D + 2] floats.
// Returns the merged value of thread `tid`'s channel (0 for tid >= 128 * nheads).  nsplit <= 64.
template <int D, typename Sync>
__device__ __forceinline__ float attention_merge_heads(const float *partial, int group, int nsplit, int first_head,
                                                       int nheads, int tid, float *wn, Sync sync) {
    const int lane = tid & 31, warp = tid >> 5;
    const int hl = tid / D, ch = tid % D;                       // head of this thread's channel
    const bool live = hl < nheads;
    const int h = first_head + (live ? hl : 0), hk = h / group, g = h - hk * group;
    const float *base = partial + ((size_t)hk * nsplit * group + g) * (D + 2);
    const size_t stride = (size_t)group * (D + 2);
    float ov[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) ov[u] = (live && u < nsplit) ? __ldcg(base + (size_t)u * stride + ch) : 0.f;
    if (warp < nheads) {
        const int hh = first_head + warp, hk2 = hh / group, g2 = hh - hk2 * group;
        const float *b2 = partial + ((size_t)hk2 * nsplit * group + g2) * (D + 2);
        float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
        if (lane < nsplit) {
            m0 = __ldcg(b2 + (size_t)lane * stride + D);
            l0 = __ldcg(b2 + (size_t)lane * stride + D + 1);
        }
        if (lane + 32 < nsplit) {
            m1 = __ldcg(b2 + (size_t)(lane + 32) * stride + D);
            l1 = __ldcg(b2 + (size_t)(lane + 32) * stride + D + 1);
        }
        const float M = warp_max(fmaxf(m0, m1));
        const float w0 = m0 > -INFINITY ? expf(m0 - M) : 0.f, w1 = m1 > -INFINITY ? expf(m1 - M) : 0.f;
        const float den = warp_sum(l0 * w0 + l1 * w1);
        wn[warp * 64 + lane] = w0 / den;
        wn[warp * 64 + lane + 32] = w1 / den;
    }
    sync();
    float out = 0.f;
    if (live) {
#pragma unroll
        for (int u = 0; u < 16; ++u) out += ov[u] * wn[hl * 64 + u];
        for (int s0 = 16; s0 < nsplit; s0 += 16) {
#pragma unroll
            for (int u = 0; u < 16; ++u)
                if (s0 + u < nsplit) out += __ldcg(base + (size_t)(s0 + u) * stride + ch) * wn[hl * 64 + s0 + u];
        }
    }
    return out;
}

}  // namespace hlq
