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

// The unit for a caller that merges the splits itself (the decode chain: the linear that consumes
// the attention output merges them while it loads its activations), heads of 128 channels, 512
// threads, on the tensor cores.  Differences from attention_unit:
//   * the token's position `pos` (already clamped to the cache) and the rotary table `rope` come
//     from the caller; the loads of the first K/V tile are issued BEFORE `wait_inputs()` returns
//     (the cache does not depend on this token's q, k, v; the row of the new position is taken
//     from the new k and v instead of from the prefetched tile);
//   * scores: K rows go from global memory straight into A fragments of mma.sync.m16n8k16 (warp w
//     < 8 owns positions 16w .. 16w+15 of the tile; a lane's 16-byte loads are channels
//     8 (tig + 4j) .. +7 of rows gid and gid + 8 - the instruction's k index is only a label, the
//     roped queries in shared memory are read in the same order), B = the group's query heads
//     (n = 8 = kMaxGroup), D = [position][head] fp32, scaled afterwards;
//   * weighted sum: the V tile comes into shared memory by cp.async, its transposed 16 x 16 blocks
//     are A fragments (ldmatrix.trans), B = the fp16 weights [position][head], D = [channel][head];
//     warps w and w + 8 share the positions of a tile for channels 16 (w & 7) .. +15;
//   * the unit ends when its partial (unnormalized output, running max and sum per head) is
//     written to a.partial: no counter, no merge, a.out is not written.
// `sync` is a barrier over the 512 threads; `wait_inputs()` is called by all threads, returns the
// same value in all of them once q, k, v may be read, false to abandon the unit.
struct AttnMmaSmem {
    static constexpr int kPad = 136;                 // halves per padded row of 128: 272 bytes
    __align__(16) __half q16[kMaxGroup][kPad];       // roped queries (rows >= group: zero)
    __align__(16) float pw[128][kMaxGroup];          // scores of a tile
    __align__(16) __half pt[kMaxGroup][kPad];        // weights of a tile, [head][position]
    __align__(16) __half vs[128 * kPad];             // the V tile: [position][channel], rows 272 bytes apart
    __align__(16) float red[8][32][4];               // accumulators of warps 8..15
    float alpha[kMaxGroup], m_run[kMaxGroup], l_run[kMaxGroup];
    __align__(16) __half knew[128], vnew[128];       // the new token's roped k row and v row
};

__device__ __forceinline__ void attn_cp_async_16(void *dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst_smem)), "l"(src)
                 : "memory");
}
__device__ __forceinline__ void attn_cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void attn_mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void attn_ldmatrix_x4_trans(uint32_t (&r)[4], const void *row_smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"((uint32_t)__cvta_generic_to_shared(row_smem)));
}

template <typename Sync, typename Wait>
__device__ __forceinline__ void attention_partial_unit(const AttnArgs &a, int hk, int split, int nsplit, AttnMmaSmem &sm,
                                                       int tid, Sync sync, const float2 *rope, int pos,
                                                       Wait wait_inputs, unsigned long long *stamps = nullptr) {
    constexpr int D = 128, P = AttnMmaSmem::kPad;
    const int lane = tid & 31, warp = tid >> 5, gid = lane >> 2, tig = lane & 3;
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

    uint4 kf[2][4];      // warps 0..7: rows gid, gid + 8 of the warp's 16 positions, channels 8 (tig + 4j) .. +7
    auto load_tile = [&](int tile, int ntile) {
        if (warp < 8) {
#pragma unroll
            for (int rr = 0; rr < 2; ++rr) {
                const int p = 16 * warp + gid + 8 * rr;
                if (p < ntile) {
                    const uint4 *kr = (const uint4 *)(a.kcache + (size_t)(tile + p) * row_stride + head_off);
#pragma unroll
                    for (int j = 0; j < 4; ++j) kf[rr][j] = kr[tig + 4 * j];
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) kf[rr][j] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
        }
        // 128 rows x 16 chunks of 16 bytes, four per thread; rows past the tile are zero (a weight of
        // zero must not meet a NaN)
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int idx = tid + 512 * u, t = idx >> 4, c = idx & 15;
            __half *dst = sm.vs + t * P + 8 * c;
            if (t < ntile) attn_cp_async_16(dst, a.vcache + (size_t)(tile + t) * row_stride + head_off + 8 * c);
            else *(uint4 *)dst = make_uint4(0u, 0u, 0u, 0u);
        }
    };
    sync();            // the shared memory may still be in use by whatever ran before the unit
    if (t0 < t1) load_tile(t0, min(D, t1 - t0));
    if (!wait_inputs()) {
        attn_cp_async_wait_all();
        return;
    }
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
            sm.q16[g][tid] = g < G ? __float2half_rn(q1[g] * cs - q2[g] * sn) : __float2half_rn(0.f);
            sm.q16[g][tid + D / 2] = g < G ? __float2half_rn(q1[g] * sn + q2[g] * cs) : __float2half_rn(0.f);
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
    } else if (tid < D + kMaxGroup) {
        const int g = tid - D;
        sm.m_run[g] = -INFINITY;
        sm.l_run[g] = 0.f;
        sm.alpha[g] = 0.f;
    } else if (tid >= 256) {
        // weights of heads the group does not have stay zero
        for (int i = tid - 256; i < kMaxGroup * P; i += 256) (&sm.pt[0][0])[i] = __float2half_rn(0.f);
    }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};       // channels 16 (warp & 7) + gid (+ 8), heads 2 tig, 2 tig + 1
    attn_cp_async_wait_all();
    sync();
    mark(1);

    for (int tile = t0; tile < t1; tile += D) {
        const int ntile = min(D, t1 - tile);
        if (tile != t0) {
            load_tile(tile, ntile);
            attn_cp_async_wait_all();
        }
        // the new position's row: from the new k / v, not from the (possibly prefetched) cache
        if (warp < 8) {
#pragma unroll
            for (int rr = 0; rr < 2; ++rr)
                if (tile + 16 * warp + gid + 8 * rr == pos) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) kf[rr][j] = *(const uint4 *)(sm.knew + 8 * (tig + 4 * j));
                }
        }
        if (pos >= tile && pos < tile + ntile && tid >= 256 && tid < 256 + 16)
            *(uint4 *)(sm.vs + (pos - tile) * P + 8 * (tid - 256)) = *(const uint4 *)(sm.vnew + 8 * (tid - 256));
        // scores of the warp's 16 positions for all heads of the group
        if (warp < 8) {
            float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t k0[4] = {kf[0][j].x, kf[0][j].y, kf[0][j].z, kf[0][j].w};
                const uint32_t k1[4] = {kf[1][j].x, kf[1][j].y, kf[1][j].z, kf[1][j].w};
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const uint2 b = *(const uint2 *)(&sm.q16[gid][8 * (tig + 4 * j) + 4 * e]);
                    attn_mma_16816(c, k0[2 * e], k1[2 * e], k0[2 * e + 1], k1[2 * e + 1], b.x, b.y);
                }
            }
            const int p0 = 16 * warp + gid;
            const float sc = a.scale;
            *(float2 *)&sm.pw[p0][2 * tig] = p0 < ntile ? make_float2(c[0] * sc, c[1] * sc) : make_float2(-INFINITY, -INFINITY);
            *(float2 *)&sm.pw[p0 + 8][2 * tig] =
                p0 + 8 < ntile ? make_float2(c[2] * sc, c[3] * sc) : make_float2(-INFINITY, -INFINITY);
        }
        sync();
        mark(2);
        // running max and sum per head; scores become fp16 weights [head][position]
        for (int g = warp; g < G; g += 16) {
            float sv[D / 32], tmax = -INFINITY;
#pragma unroll
            for (int i = 0; i < D / 32; ++i) {
                sv[i] = sm.pw[lane + 32 * i][g];
                tmax = fmaxf(tmax, sv[i]);
            }
            tmax = warp_max(tmax);
            const float mold = sm.m_run[g], mnew = fmaxf(mold, tmax);
            float psum = 0.f;
#pragma unroll
            for (int i = 0; i < D / 32; ++i) {
                const float p = expf(sv[i] - mnew);       // exp(-inf) = 0 for the positions past the tile
                const __half ph = __float2half_rn(p);
                sm.pt[g][lane + 32 * i] = ph;
                psum += __half2float(ph);                 // the sum of what the weighted sum will use
            }
            psum = warp_sum(psum);
            if (lane == 0) {
                const float al = expf(mold - mnew);        // 0 on the first tile (mold = -inf)
                sm.alpha[g] = al;
                sm.m_run[g] = mnew;
                sm.l_run[g] = sm.l_run[g] * al + psum;
            }
        }
        sync();
        {
            const int dw = warp & 7, kh = warp >> 3;
            const float a0 = sm.alpha[2 * tig], a1 = sm.alpha[2 * tig + 1];
            acc[0] *= a0; acc[1] *= a1; acc[2] *= a0; acc[3] *= a1;
            const int mi = lane >> 3;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const int base = 16 * (4 * kh + ks);
                if (base < ntile) {                 // uniform in the warp
                    uint32_t vf[4];
                    attn_ldmatrix_x4_trans(vf, sm.vs + (base + (lane & 7) + 8 * (mi >> 1)) * P + 16 * dw + 8 * (mi & 1));
                    const uint32_t b0 = *(const uint32_t *)&sm.pt[gid][base + 2 * tig];
                    const uint32_t b1 = *(const uint32_t *)&sm.pt[gid][base + 2 * tig + 8];
                    attn_mma_16816(acc, vf[0], vf[1], vf[2], vf[3], b0, b1);
                }
            }
        }
        sync();
    }
    mark(3);
    // warps w + 8 hand their half of the positions to warps w
    if (warp >= 8) *(float4 *)&sm.red[warp - 8][lane][0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    sync();
    // This split's partial: outputs [head][split][D] (a head's splits lie side by side, every row a
    // whole number of 128-byte lines), then the (max, sum) pairs [head][split][2].  A share without
    // positions (t0 >= t1) publishes max = -inf, sum = 0.
    if (warp < 8) {
        const float4 o = *(const float4 *)&sm.red[warp][lane][0];
        const int d0 = 16 * warp + gid;
        float *mine = a.partial + ((size_t)(hk * G) * nsplit + split) * D + d0;
        const size_t hs = (size_t)nsplit * D;
        if (2 * tig < G) {
            mine[(size_t)(2 * tig) * hs] = acc[0] + o.x;
            mine[(size_t)(2 * tig) * hs + 8] = acc[2] + o.z;
        }
        if (2 * tig + 1 < G) {
            mine[(size_t)(2 * tig + 1) * hs] = acc[1] + o.y;
            mine[(size_t)(2 * tig + 1) * hs + 8] = acc[3] + o.w;
        }
    } else if (tid - 256 < G) {
        const int g = tid - 256;
        float2 *ml = (float2 *)(a.partial + (size_t)a.head_q * nsplit * D) + (size_t)(hk * G + g) * nsplit + split;
        *ml = make_float2(sm.m_run[g], sm.l_run[g]);
    }
    mark(4);
}

// Merge of the splits for `nheads` (<= 4) consecutive query heads, by the T = 128 * nheads...512
// threads of a CTA that then need the merged values (one channel per thread):
//   1. every thread issues the loads of its channel's unnormalized outputs of all splits;
//   2. warp h (h < nheads) turns the splits' (max, sum) pairs of head h into normalized weights
//      exp(max_s - max) / sum_s(...) in shared memory `wn` [4][64];
//   3. after `sync`, out = sum_s output_s * weight_s.
// `first_head` = index of the first head, `partial` = [head][nsplit][D] floats, `ml` = [head][nsplit][2]
// (as attention_partial_unit writes them).  Returns the merged value of thread `tid`'s channel (0
// for tid >= 128 * nheads).  nsplit <= 64.
template <int D, typename Sync>
__device__ __forceinline__ float attention_merge_heads(const float *partial, const float *ml, int nsplit, int first_head,
                                                       int nheads, int tid, float *wn, Sync sync) {
    const int lane = tid & 31, warp = tid >> 5;
    const int hl = tid / D, ch = tid % D;                       // head of this thread's channel
    const bool live = hl < nheads;
    const float *base = partial + (size_t)(first_head + (live ? hl : 0)) * nsplit * D + ch;
    float ov[16];
#pragma unroll
    for (int u = 0; u < 16; ++u) ov[u] = (live && u < nsplit) ? __ldcg(base + (size_t)u * D) : 0.f;
    if (warp < nheads) {
        const float2 *b2 = (const float2 *)ml + (size_t)(first_head + warp) * nsplit;
        float2 p0 = make_float2(-INFINITY, 0.f), p1 = make_float2(-INFINITY, 0.f);
        if (lane < nsplit) p0 = __ldcg(b2 + lane);
        if (lane + 32 < nsplit) p1 = __ldcg(b2 + lane + 32);
        const float M = warp_max(fmaxf(p0.x, p1.x));
        const float w0 = p0.x > -INFINITY ? expf(p0.x - M) : 0.f, w1 = p1.x > -INFINITY ? expf(p1.x - M) : 0.f;
        const float den = warp_sum(p0.y * w0 + p1.y * w1);
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
                if (s0 + u < nsplit) out += __ldcg(base + (size_t)(s0 + u) * D) * wn[hl * 64 + s0 + u];
        }
    }
    return out;
}

}  // namespace hlq
