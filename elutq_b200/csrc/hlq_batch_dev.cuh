// Register-level dequantization of HLQ weights in the streaming layout, shared by the small-batch
// kernels (hlq_batch.cu: mma.sync; hlq_batch_umma.cu: tcgen05): the layout's byte-pair permutation
// undone, the q bits of a weight gathered into a nibble, the 2^q values of a (row, group) as byte
// tables for prmt.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

#include "hlq_gemv_dev.cuh"

namespace hlq {

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
// bits of a where the mask is set, bits of b elsewhere
__device__ __forceinline__ uint32_t merge_bits(uint32_t a, uint32_t b, uint32_t mask) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(r) : "r"(mask), "r"(a), "r"(b));   // mask ? a : b
    return r;
}


// The four words of a lane's 16 bytes in SOURCE order: position pair i holds source pair i ^ r, so
// source word c sits in position word c ^ (r >> 1), its halves swapped when r is odd.  Bit 2 of r
// picks between words two apart (a select); bit 1 and the swap are one byte permute over a pair of
// words with the lane's selector `usel` (see unpermute_selector).
__device__ __forceinline__ uint32_t unpermute_selector(int r) {
    return (r & 2) ? ((r & 1) ? 0x5476u : 0x7654u) : ((r & 1) ? 0x1032u : 0x3210u);
}
__device__ __forceinline__ void source_order(const uint4 &w, bool far, uint32_t usel, uint32_t (&out)[4]) {
    const uint32_t q0 = far ? w.z : w.x, q1 = far ? w.w : w.y, q2 = far ? w.x : w.z, q3 = far ? w.y : w.w;
    out[0] = prmt(q0, q1, usel);
    out[1] = prmt(q1, q0, usel);
    out[2] = prmt(q2, q3, usel);
    out[3] = prmt(q3, q2, usel);
}

// fp16 scale or zero of (plane-or-zero pp, oct ou, positional sub-group u) of a tile
template <int GPW>
__device__ __forceinline__ float tile_meta(const uint32_t (&m)[GPW], int ou, int u) {
    uint32_t word;
    bool hi;
    if (GPW == 1) {
        word = m[0];
        hi = ou;
    } else if (GPW == 2) {
        word = m[ou];
        hi = u & 1;
    } else {
        word = (u & 2) ? m[(2 * ou + 1) % GPW] : m[(2 * ou) % GPW];
        hi = u & 1;
    }
    return __half2float(__ushort_as_half(hi ? (uint16_t)(word >> 16) : (uint16_t)(word & 0xffffu)));
}

// Byte tables of one (row, group): lo[h] / hi[h] hold the low / high bytes of the fp16 values of
// codes 4h .. 4h + 3 (code = bits of the planes, plane 0 lowest).
template <int Q>
struct ByteTables {
    uint32_t lo[2], hi[2];
};
template <int Q, int GPW>
__device__ __forceinline__ void build_tables(const uint32_t (&mt)[Q + 1][GPW], int ou, int u, ByteTables<Q> &bt) {
    const float z = tile_meta<GPW>(mt[Q], ou, u);
    float al[Q];
#pragma unroll
    for (int p = 0; p < Q; ++p) al[p] = tile_meta<GPW>(mt[p], ou, u);
    float v[1 << Q];
    v[0] = z;
#pragma unroll
    for (int p = 0; p < Q; ++p)
#pragma unroll
        for (int e = 0; e < (1 << p); ++e) v[(1 << p) + e] = v[e] + al[p];
    uint32_t pr[(1 << Q) / 2];
#pragma unroll
    for (int e = 0; e < (1 << Q) / 2; ++e) {
        const __half2 h = __floats2half2_rn(v[2 * e], v[2 * e + 1]);
        pr[e] = *(const uint32_t *)&h;
    }
    bt.lo[0] = prmt(pr[0], pr[1], 0x6420u);
    bt.hi[0] = prmt(pr[0], pr[1], 0x7531u);
    if (Q == 3) {
        bt.lo[1] = prmt(pr[2 % ((1 << Q) / 2)], pr[3 % ((1 << Q) / 2)], 0x6420u);
        bt.hi[1] = prmt(pr[2 % ((1 << Q) / 2)], pr[3 % ((1 << Q) / 2)], 0x7531u);
    } else {
        bt.lo[1] = 0u;
        bt.hi[1] = 0u;
    }
}


// The code words of word c of a lane's rows from its planes in source order: xs[oct][s].
template <int Q>
__device__ __forceinline__ void code_words(const uint32_t (&pw)[2][Q][4], int c, uint32_t (&xs)[2][4]) {
    // planes 1 and 2 rotated (not shifted: the top nibble's bits wrap and come back) so that
    // bit p of plane 0, bit p + 1 of plane 1', bit p + 2 of plane 2' belong to one channel
#pragma unroll
    for (int ou = 0; ou < 2; ++ou) {
        const uint32_t w0 = pw[ou][0][c];
        const uint32_t w1 = __funnelshift_l(pw[ou][1 % Q][c], pw[ou][1 % Q][c], 1);
        const uint32_t w2 = __funnelshift_l(pw[ou][2 % Q][c], pw[ou][2 % Q][c], 2);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            constexpr uint32_t kOne = 0x11111111u, kTwo = 0x33333333u;
            const uint32_t m1 = s ? ((kOne << s) | (kOne >> (32 - s))) : kOne;
            const uint32_t m2 = s ? ((kTwo << s) | (kTwo >> (32 - s))) : kTwo;
            uint32_t m = merge_bits(w0, w1, m1);
            if (Q == 3) m = merge_bits(m, w2, m2);
            if (s) m = __funnelshift_r(m, m, s);
            xs[ou][s] = m & (Q == 3 ? 0x77777777u : 0x33333333u);
        }
    }
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

}  // namespace hlq
