// Device-side building blocks of the LUT GEMV kernels (shared by hlq_gemv.cu and hlq_chain.cu):
// shared-memory and streaming loads, mbarrier + TMA bulk copy with bounded waits, the register
// tile of one duo (16 output rows x 512 input channels x Q planes) and its table lookups.
//
// Replaces the inner loops of the reference's kernel:
//   C++/ops/src/arm/arm_t_mac_kernal.cpp:364-469  (per-plane table lookups, alpha scaling)
//   C++/ops/src/arm/arm_gemm.cpp:259-286          (zero term)
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hlq_internal.h"

namespace hlq {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ float lds_f32_hi(uint32_t addr) {   // second bank-row of the table row
    float v;
    asm volatile("ld.shared.f32 %0, [%1+128];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32_hi(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+128];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts_u32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void sts_f32(uint32_t addr, float v) {
    asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// byte `SEL` of word -> bits 8..15 of base (bytes 0, 2, 3 of base are kept)
template <int SEL>
__device__ __forceinline__ uint32_t byte_into_base(uint32_t word, uint32_t base) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(word), "r"(base), "n"(0x7604 | (SEL << 4)));
    return r;
}
__device__ __forceinline__ uint4 ldg_stream_v4(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ldg_stream_v2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void *p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned ldcg_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float ldcg_f32(const float *p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}
// traffic of the fused all-reduce: ONE naturally aligned 64-bit scalar carries a value (low
// word) and the launch number that validates it (high word).  A 64-bit scalar access is
// single-copy atomic, so a reader sees both halves of one store or neither, and neither side
// needs a fence (a system-scope fence or release per block costs 5-15 us while the
// accumulators' reductions are in flight)
__device__ __forceinline__ void st_relaxed_sys_b64(unsigned long long *p, uint32_t value, uint32_t tag) {
    const unsigned long long v = ((unsigned long long)tag << 32) | value;
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_sys_b64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float x_to_float(uint16_t bits, int dtype) {
    if (dtype == HLQ_BF16) return __uint_as_float((uint32_t)bits << 16);
    return __half2float(__ushort_as_half(bits));
}
__device__ __forceinline__ void store_y(void *y, int64_t idx, float v, int dtype) {
    if (dtype == HLQ_F16) ((__half *)y)[idx] = __float2half_rn(v);
    else if (dtype == HLQ_BF16) ((__nv_bfloat16 *)y)[idx] = __float2bfloat16_rn(v);
    else ((float *)y)[idx] = v;
}

// ---- mbarrier + TMA bulk copy (non-tensor form), all waits bounded -----------------------
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t mbar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(mbar), "r"(parity)
        : "memory");
    return ok != 0;
}
// false when the wait gave up.  `fail` is the CTA-wide failure flag in shared memory: the
// wait that runs out sets it, and once it is set every later wait of the CTA tries once and
// gives up, so that a kernel whose peer or copy never arrives drains in microseconds instead
// of spinning its full limit again at every wait.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity, volatile int *fail, int limit) {
    if (mbar_try_wait(mbar, parity)) return true;
    if (!*fail) {
        for (int i = 0; i < limit; ++i) {
            if (mbar_try_wait(mbar, parity)) return true;
            if ((i & 255) == 255 && *fail) break;
        }
    }
    *fail = 1;
    return false;
}
__device__ __forceinline__ void tma_bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                             uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(mbar)
        : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
template <int ID, int COUNT>
__device__ __forceinline__ void named_bar_sync() {
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(COUNT) : "memory");
}
__device__ __forceinline__ void named_bar_sync_dyn(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void named_bar_arrive_dyn(int id, int count) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ---- per-lane registers of one duo (2 octs x Q planes) -----------------------------------
template <int Q, int GPW>
struct Tile {
    uint4 w[2][Q];
    uint32_t mt[Q + 1][GPW];  // 2*GPW fp16 values per plane-or-zero: [oct & 1][u]
};

template <int Q, int GPW>
__device__ __forceinline__ void load_tile(Tile<Q, GPW> &t, const uint8_t *pl, const uint16_t *mp) {
#pragma unroll
    for (int ou = 0; ou < 2; ++ou)
#pragma unroll
        for (int p = 0; p < Q; ++p) t.w[ou][p] = ldg_stream_v4(pl + (ou * Q + p) * kCellBytes);
#pragma unroll
    for (int pp = 0; pp <= Q; ++pp) {
        const uint16_t *m = mp + pp * (32 * 2 * GPW);
        if (GPW == 1) {
            t.mt[pp][0] = ldg_stream_u32(m);
        } else if (GPW == 2) {
            const uint2 v = ldg_stream_v2(m);
            t.mt[pp][0] = v.x;
            t.mt[pp][GPW - 1] = v.y;
        } else {
            const uint4 v = ldg_stream_v4(m);
            t.mt[pp][0] = v.x;
            t.mt[pp][1 % GPW] = v.y;
            t.mt[pp][2 % GPW] = v.z;
            t.mt[pp][3 % GPW] = v.w;
        }
    }
}

// fp16 value h (h = ou * GPW + u) of a meta entry
template <int GPW>
__device__ __forceinline__ float meta_value(const uint32_t (&m)[GPW], int h) {
    const uint32_t word = m[h >> 1];
    return __half2float(__ushort_as_half((h & 1) ? (uint16_t)(word >> 16) : (uint16_t)(word & 0xffffu)));
}

// 16 lookups of one 128-bit word; sums per positional sub-group (16 / GPW bytes each).
template <int GPW>
__device__ __forceinline__ void lookup_word(const uint4 &w, const uint32_t (&rt)[8], float (&sum)[GPW]) {
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    constexpr int kWordsPerSub = 4 / GPW;   // 32-bit words per sub-group: 4, 2 or 1
#pragma unroll
    for (int u = 0; u < GPW; ++u) {
        float a0 = 0.f, a1 = 0.f;
#pragma unroll
        for (int q = 0; q < kWordsPerSub; ++q) {
            const int wi = u * kWordsPerSub + q;
            const uint32_t word = words[wi];
            const float v0 = lds_f32(byte_into_base<0>(word, rt[2 * wi]));
            const float v1 = lds_f32_hi(byte_into_base<1>(word, rt[2 * wi]));
            const float v2 = lds_f32(byte_into_base<2>(word, rt[2 * wi + 1]));
            const float v3 = lds_f32_hi(byte_into_base<3>(word, rt[2 * wi + 1]));
            if (q == 0) {
                a0 = v0 + v2;
                a1 = v1 + v3;
            } else {
                a0 += v0;
                a1 += v1;
                a0 += v2;
                a1 += v3;
            }
        }
        sum[u] = a0 + a1;
    }
}

// Two rows of x at once: a table entry is a half2 {row 0, row 1} of the same subset sum, so one
// lookup serves both rows (entries are rounded to fp16 as the reference's tables are; the sums
// are taken in fp32).
template <int GPW>
__device__ __forceinline__ void lookup_word2(const uint4 &w, const uint32_t (&rt)[8], float (&s0)[GPW],
                                             float (&s1)[GPW]) {
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
    constexpr int kWordsPerSub = 4 / GPW;
#pragma unroll
    for (int u = 0; u < GPW; ++u) {
        float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f;
#pragma unroll
        for (int q = 0; q < kWordsPerSub; ++q) {
            const int wi = u * kWordsPerSub + q;
            const uint32_t word = words[wi];
            const uint32_t e0 = lds_u32(byte_into_base<0>(word, rt[2 * wi]));
            const uint32_t e1 = lds_u32_hi(byte_into_base<1>(word, rt[2 * wi]));
            const uint32_t e2 = lds_u32(byte_into_base<2>(word, rt[2 * wi + 1]));
            const uint32_t e3 = lds_u32_hi(byte_into_base<3>(word, rt[2 * wi + 1]));
            // two entries are added as half2 (one more fp16 rounding), then widened: the sums
            // of 16 activations still sit far inside the fp16 range for any input the
            // reference's fp16 accumulation over whole groups can handle
            const float2 f0 = __half22float2(__hadd2(*(const __half2 *)&e0, *(const __half2 *)&e2));
            const float2 f1 = __half22float2(__hadd2(*(const __half2 *)&e1, *(const __half2 *)&e3));
            a0 += f0.x; b0 += f0.y;
            a1 += f1.x; b1 += f1.y;
        }
        s0[u] = a0 + a1;
        s1[u] = b0 + b1;
    }
}

// One duo for two rows of x: four totals (row, oct) per lane; after the exchange lane j of a
// row's four lanes holds the total of (x row j >> 1, oct j & 1) and adds it to that
// accumulator.  `prow` as in compute_tile; `row_stride` = accumulator elements per row of x.
template <int Q, int GPW>
__device__ __forceinline__ void compute_tile2(const Tile<Q, GPW> &t, const uint32_t (&rt)[8],
                                              const float (&xsu0)[GPW], const float (&xsu1)[GPW], float *prow,
                                              int row_stride, int lane) {
    float v[2][2];   // [x row][oct]
#pragma unroll
    for (int ou = 0; ou < 2; ++ou) {
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (int u = 0; u < GPW; ++u) {
            const float z = meta_value<GPW>(t.mt[Q], ou * GPW + u);
            t0 += z * xsu0[u];
            t1 += z * xsu1[u];
        }
#pragma unroll
        for (int p = 0; p < Q; ++p) {
            float s0[GPW], s1[GPW];
            lookup_word2<GPW>(t.w[ou][p], rt, s0, s1);
#pragma unroll
            for (int u = 0; u < GPW; ++u) {
                const float al = meta_value<GPW>(t.mt[p], ou * GPW + u);
                t0 += al * s0[u];
                t1 += al * s1[u];
            }
        }
        v[0][ou] = t0;
        v[1][ou] = t1;
    }
    const int j = lane & 3;
    const bool odd = j & 1, hi = j & 2;
    float k0 = odd ? v[0][1] : v[0][0], k1 = odd ? v[1][1] : v[1][0];       // this lane's oct, both rows
    k0 += __shfl_xor_sync(0xffffffffu, odd ? v[0][0] : v[0][1], 1);
    k1 += __shfl_xor_sync(0xffffffffu, odd ? v[1][0] : v[1][1], 1);
    float keep = hi ? k1 : k0;
    keep += __shfl_xor_sync(0xffffffffu, hi ? k0 : k1, 2);
    atomicAdd(prow + (hi ? row_stride : 0) + (odd ? kOctRows : 0), keep);
}

// One duo: both octs' totals, the 4-lane reduction, and the add into the row's fp32
// accumulator (a reduction without return value: the slices of a row come from different
// CTAs).  `prow` points at acc[row of (first oct, this lane's r)].
template <int Q, int GPW>
__device__ __forceinline__ void compute_tile(const Tile<Q, GPW> &t, const uint32_t (&rt)[8],
                                             const float (&xsu)[GPW], float *prow, int lane) {
    float v[2];
#pragma unroll
    for (int ou = 0; ou < 2; ++ou) {
        float tot = 0.f;
#pragma unroll
        for (int u = 0; u < GPW; ++u) tot += meta_value<GPW>(t.mt[Q], ou * GPW + u) * xsu[u];
#pragma unroll
        for (int p = 0; p < Q; ++p) {
            float sum[GPW];
            lookup_word<GPW>(t.w[ou][p], rt, sum);
#pragma unroll
            for (int u = 0; u < GPW; ++u) tot += meta_value<GPW>(t.mt[p], ou * GPW + u) * sum[u];
        }
        v[ou] = tot;
    }
    // lanes j = 0..3 of a row: after the exchange lane j < 2 holds oct j of the duo
    const int j = lane & 3;
    const bool odd = j & 1;
    float keep = odd ? v[1] : v[0];
    const float send = odd ? v[0] : v[1];
    keep += __shfl_xor_sync(0xffffffffu, send, 1);
    keep += __shfl_xor_sync(0xffffffffu, keep, 2);
    if (j < 2) atomicAdd(prow + j * kOctRows, keep);
}

}  // namespace hlq
