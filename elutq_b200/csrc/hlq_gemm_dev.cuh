// Shared by the two prefill kernels (hlq_gemm.cu, hlq_gemm_pair.cu): launch arguments, mbarrier /
// TMA / tcgen05 wrappers, what a dequantizer thread loads from the streaming layout for one K step
// and how it turns those bits into fp16 weights.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hlq_internal.h"

namespace hlq {
namespace gemm {

constexpr int kTileK = 64;        // channels per K step: 128 bytes of 16-bit operands
constexpr int kMaxTileM = 256;    // tokens per CTA at most (UMMA N)
constexpr uint32_t kXBytes = kMaxTileM * kTileK * 2;   // 32 KB reserved per stage
constexpr uint32_t kLutBytes = 8192;        // nibble tables (256 bytes), byte tables of the pair kernel (4 KB)
constexpr uint32_t kBarBytes = 256;
constexpr int kSpinLimit = 1 << 24;

struct GemmArgs {
    const uint8_t *planes;
    const uint16_t *meta;
    const uint16_t *bias;
    void *y;
    int *status;
    int m, n, k, np, kp, octs, duos, gpw, gshift;
    int tile_m;          // tokens per CTA: multiple of 32, <= 256
    int tok_group;       // pair kernel: token tiles walked together (their activations share L2)
    int ksplit;          // pair kernel: parts K is split into (1: outputs are stored; > 1: sums go to acc)
    float *acc;          // pair kernel, ksplit > 1: ksplit fp32 slabs [m][n] in the workspace
    int y_dtype;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t mbar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(mbar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
    for (int i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(mbar, parity)) return true;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int c0, int c1, uint32_t mbar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(mbar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row atoms of 1024 bytes.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3fff);   // start address, 16-byte units
    d |= (uint64_t)1 << 16;                        // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;              // stride between 8-row atoms
    d |= (uint64_t)1 << 46;                        // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}
// kind::f16 instruction descriptor: fp32 accumulator, A and B fp16, both K-major, M = 128,
// N = tokens per tile.
__device__ __forceinline__ uint32_t umma_idesc(int tile_m) {
    return (1u << 4) | ((uint32_t)(tile_m >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar)
                 : "memory");
}

// What a dequantizer thread fetches for one K step: the 4 bytes per plane that hold its 32
// channels of its row, and the fp16 scales / zero of the group they fall into.
template <int Q>
struct Raw {
    uint32_t w[Q];
    uint16_t al[Q];
    uint16_t z;
};

// hh = which 32-channel half of the 64-channel K step this thread owns
template <int Q>
__device__ __forceinline__ void load_raw(Raw<Q> &rw, const GemmArgs &a, int kt, int oct, int r, int hh,
                                         bool row_ok) {
    const int k0 = kt * kTileK;
    const int sl = k0 >> 9, j = (k0 >> 7) & 3, h = (k0 >> 6) & 1;
    const int ln = r * 4 + j;
    const int half = h ^ (r >> 2);            // which 8 bytes of the lane word hold the 64 channels
    const int word = hh ^ ((r & 3) >> 1);     // and which 4 of those hold this thread's two byte pairs
#pragma unroll
    for (int p = 0; p < Q; ++p) {
        rw.w[p] = 0u;
        if (row_ok)
            rw.w[p] = __ldg((const uint32_t *)(a.planes + (((int64_t)sl * a.octs + oct) * Q + p) * kCellBytes +
                                               ln * 16 + 8 * half + 4 * word));
    }
    // source sub-group inside the lane's 128 channels: g = 128 -> 0, g = 64 -> h, g = 32 -> 2h + hh
    const int su = a.gpw == 1 ? 0 : (a.gpw == 2 ? h : 2 * h + hh);
    const int u = su ^ (r >> a.gshift);
    const int64_t mbase = ((((int64_t)sl * a.duos + (oct >> 1)) * (Q + 1)) * 32 + ln) * 2 * a.gpw +
                          (oct & 1) * a.gpw + u;
    const int64_t pstride = (int64_t)32 * 2 * a.gpw;
#pragma unroll
    for (int p = 0; p < Q; ++p) rw.al[p] = row_ok ? __ldg(a.meta + mbase + p * pstride) : (uint16_t)0;
    rw.z = row_ok ? __ldg(a.meta + mbase + Q * pstride) : (uint16_t)0;
}

// The fp16 weights of CH = 16 or 32 consecutive channels of one row, two per word in channel order,
// from `bits[p]`: the CH bits of plane p in source order (bit c = channel c).  `lut` is the
// nibble -> four 16-bit masks table, `sel_lut` the two nibble -> prmt selector tables of the
// two-plane form (both in shared memory, filled by fill_dequant_tables).
template <int Q, int CH>
__device__ __forceinline__ void dequant_channels(const uint32_t (&bits)[Q], const uint16_t (&alpha)[Q], uint16_t zero,
                                                 const uint2 *lut, const uint32_t *sel_lut, uint32_t (&o)[CH / 2]) {
    if constexpr (Q == 2) {
        // the four values a weight of this group can take, each rounded once to fp16
        const float zf = __half2float(__ushort_as_half(zero));
        const float a0 = __half2float(__ushort_as_half(alpha[0]));
        const float a1 = __half2float(__ushort_as_half(alpha[1]));
        uint32_t t01, t23;
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(t01) : "f"(zf + a0), "f"(zf));
        asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(t23) : "f"(zf + a0 + a1), "f"(zf + a1));
#pragma unroll
        for (int nb = 0; nb < CH / 4; ++nb) {           // a nibble of each plane: 4 weights
            const uint32_t sel = sel_lut[(bits[0] >> (4 * nb)) & 0xfu] | sel_lut[16 + ((bits[1] >> (4 * nb)) & 0xfu)];
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(o[2 * nb]) : "r"(t01), "r"(t23), "r"(sel));
            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(o[2 * nb + 1]) : "r"(t01), "r"(t23), "r"(sel >> 16));
        }
    } else {
        uint32_t al[Q];                                 // fp16x2 alpha per plane
#pragma unroll
        for (int p = 0; p < Q; ++p) al[p] = (uint32_t)alpha[p] * 0x10001u;
        const uint32_t zz = (uint32_t)zero * 0x10001u;
#pragma unroll
        for (int e = 0; e < CH / 2; ++e) o[e] = zz;
#pragma unroll
        for (int p = 0; p < Q; ++p)
#pragma unroll
            for (int nb = 0; nb < CH / 4; ++nb) {
                const uint2 mk = lut[(bits[p] >> (4 * nb)) & 0xfu];
                const uint32_t t0 = mk.x & al[p], t1 = mk.y & al[p];
                asm("add.rn.f16x2 %0, %0, %1;" : "+r"(o[2 * nb]) : "r"(t0));
                asm("add.rn.f16x2 %0, %0, %1;" : "+r"(o[2 * nb + 1]) : "r"(t1));
            }
    }
}

// nibble -> four 16-bit masks (two words).  16 entries x 8 bytes = 128 bytes = one row of all 32
// banks: lanes with different nibbles hit different banks, equal nibbles broadcast.  Two-plane
// weights: nibble of plane 0 / plane 1 -> one selector byte per weight for prmt: byte t =
// 0x10 + 0x22 * bit_t (plane 0), 0x44 * bit_t (plane 1); their OR selects the fp16 value of index
// b0 + 2 * b1 out of the 8 bytes {v0, v1, v2, v3}.  Called by threads 0..15 of the CTA.
__device__ __forceinline__ void fill_dequant_tables(int e, uint2 *lut, uint32_t *sel_lut) {
    uint2 v;
    v.x = ((e & 1) ? 0xffffu : 0u) | ((e & 2) ? 0xffff0000u : 0u);
    v.y = ((e & 4) ? 0xffffu : 0u) | ((e & 8) ? 0xffff0000u : 0u);
    lut[e] = v;
    uint32_t sa = 0x10101010u, sb = 0u;
    for (int t2 = 0; t2 < 4; ++t2)
        if (e >> t2 & 1) {
            sa += 0x22u << (8 * t2);
            sb += 0x44u << (8 * t2);
        }
    sel_lut[e] = sa;
    sel_lut[16 + e] = sb;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// The same problem on CTA pairs (hlq_gemm_pair.cu); `x` is fp16.  HLQ_ERR_UNSUPPORTED: use the
// single-CTA kernel.
// `acc`: room for fp32 slabs [m][n] in the workspace, one per part of a split K (nullptr or fewer than
// two slabs: K is not split).
int launch_dequant_gemm_pair(const GemmArgs &a, int q, const void *x, int sms, float *acc, size_t acc_bytes,
                             cudaStream_t stream);
// tokens per pair tile and (optionally) waves x tokens as a cost to compare tilings by
int pair_tile_tokens(int n, int m, int sms, double *cost);

}  // namespace gemm
}  // namespace hlq
