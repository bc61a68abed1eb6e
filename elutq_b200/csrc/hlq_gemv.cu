// Bit-serial LUT GEMV over HLQ weights for decode (m = 1..16), sm_100a.
//
// Replaces the reference's GEMV worker and kernel:
//   C++/ops/src/arm/arm_gemm.cpp:248-308          (group sums, zero term, planes, bias)
//   C++/ops/src/arm/arm_t_mac_kernal.cpp:95-138   (16-entry partial-sum table per 4 channels)
//   C++/ops/src/arm/arm_t_mac_kernal.cpp:364-469  (per-plane table lookups, alpha scaling)
//
// lut8_gemv_kernel (streaming layout, see hlq_layout.h)
//   One CTA per SM walks a contiguous range of (slice, oct) units.  Per slice it
//     1. copies the 512 activations of the slice into shared memory with one TMA bulk copy,
//     2. builds, for every 8 activations, the 256-entry fp32 table of subset sums.  Each
//        table is the sum of the two 16-entry tables of its 4-activation halves, so one
//        lookup consumes a whole packed byte (two nibbles of the reference's scheme).
//        The 64 tables of a slice are interleaved so that entry e of every table sits in
//        the same 256-byte row: address = base + 256*e + offset(table).  With the table
//        block aligned to 64 KB, the address of a lookup is ONE byte-permute (prmt) that
//        drops the packed byte into bits 8..15 of a per-lane base register.
//     3. streams its cells with 128-bit loads (one cell = 8 rows x 512 channels of one
//        plane; a lane's 16 bytes are one row's 128 channels = one group at g = 128) and
//        per byte does prmt + ld.shared + fadd.  The byte-pair permutation of the layout
//        makes the 32 lanes of every lookup hit 32 different banks.
//     4. scales each plane's group sum by its fp16 alpha, adds z * (sum of the group's
//        activations), reduces the four lanes of a row with warp shuffles and writes the
//        row's fp32 partial for this slice.
//   The last CTA to finish a block of 32 rows (one atomic counter per block) adds the
//   partials of all slices in slice order, adds the bias and writes y: the result does not
//   depend on scheduling.
//
// lut4_gemv_kernel (exported layout, any group size that is a multiple of 8)
//   The reference's scheme as it stands: a 16-entry table per 4 activations in shared
//   memory, two lookups per packed byte, warp-shuffle reduction per output row.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "hlq_internal.h"

namespace hlq {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr uint32_t kTableBytes = 65536;
constexpr uint32_t kAuxBytes = 8192;   // activations, group sums, mbarrier, completion list
constexpr int kListCap = 512;
constexpr int kSpinLimit = 1 << 22;

// aux region layout (bytes from its start)
constexpr uint32_t kAuxX = 0;          // 512 x 16-bit activations (1 KB)
constexpr uint32_t kAuxXsum = 1024;    // up to 16 group sums (fp32)
constexpr uint32_t kAuxMbar = 1152;    // one 8-byte mbarrier
constexpr uint32_t kAuxListN = 1160;   // int: entries in the completion list
constexpr uint32_t kAuxFlag = 1164;    // int: CTA-wide failure flag
constexpr uint32_t kAuxList = 2048;    // kListCap ints

struct GemvArgs {
    const uint8_t *planes;
    const uint16_t *meta;
    const void *x;
    void *y;
    const uint16_t *bias;
    float *partial;
    unsigned *counters;
    int *status;
    int n, k, np, slices, octs, blocks;
    int x_dtype, y_dtype;
    uint32_t dyn_smem;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ float lds_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
// the constant offset folds into the instruction's immediate field
template <int IMM>
__device__ __forceinline__ float lds_f32_imm(uint32_t addr) {
    return lds_f32(addr + (uint32_t)IMM);
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
__device__ __forceinline__ float ldcg_f32(const float *p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
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
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
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
// false when the wait gave up
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t mbar, uint32_t parity) {
    for (int i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(mbar, parity)) return true;
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

// ---- per-lane registers of one prefetched group of OU octs -------------------------------
template <int Q, int GPW, int OU>
struct Tile {
    uint4 w[OU][Q];
    uint32_t mt[OU][Q + 1][(GPW + 1) / 2];  // GPW fp16 values per (oct, plane-or-zero)
};

template <int Q, int GPW, int OU>
__device__ __forceinline__ void load_tile(Tile<Q, GPW, OU> &t, const GemvArgs &a, int s, int oct0,
                                          int oct_end, int lane) {
#pragma unroll
    for (int ou = 0; ou < OU; ++ou) {
        const int oct = oct0 + ou;
        if (oct < oct_end) {
            const int64_t cell = (int64_t)s * a.octs + oct;
            const uint8_t *pp = a.planes + cell * (Q * kCellBytes) + lane * 16;
#pragma unroll
            for (int p = 0; p < Q; ++p) t.w[ou][p] = ldg_stream_v4(pp + p * kCellBytes);
            const uint16_t *mp = a.meta + (cell * (Q + 1) * 32 + lane) * GPW;
#pragma unroll
            for (int p = 0; p <= Q; ++p) {
                const uint16_t *m = mp + p * 32 * GPW;
                if (GPW == 1) {
                    t.mt[ou][p][0] = __ldg(m);
                } else if (GPW == 2) {
                    t.mt[ou][p][0] = __ldg((const uint32_t *)m);
                } else {
                    uint2 v = __ldg((const uint2 *)m);
                    t.mt[ou][p][0] = v.x;
                    t.mt[ou][p][(GPW + 1) / 2 - 1] = v.y;
                }
            }
        } else {
#pragma unroll
            for (int p = 0; p < Q; ++p) t.w[ou][p] = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int p = 0; p <= Q; ++p)
#pragma unroll
                for (int h = 0; h < (GPW + 1) / 2; ++h) t.mt[ou][p][h] = 0;
        }
    }
}

template <int GPW>
__device__ __forceinline__ float meta_value(const uint32_t (&m)[(GPW + 1) / 2], int u) {
    const uint32_t word = m[u >> 1];
    const uint16_t h = (u & 1) ? (uint16_t)(word >> 16) : (uint16_t)(word & 0xffffu);
    return __half2float(__ushort_as_half(h));
}

// 16 lookups of one 128-bit word; sums per positional sub-group (16 / GPW bytes each).
template <int GPW>
__device__ __forceinline__ void lookup_word(const uint4 &w, const uint32_t (&rt)[8],
                                            float (&sum)[GPW]) {
    float acc[GPW][2];
#pragma unroll
    for (int u = 0; u < GPW; ++u) acc[u][0] = acc[u][1] = 0.f;
    const uint32_t words[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int wi = 0; wi < 4; ++wi) {
        const uint32_t word = words[wi];
        constexpr int kPerSub = 16 / GPW;
        const int u0 = (4 * wi) / kPerSub;  // all four bytes of a word share a sub-group
        acc[u0][0] += lds_f32_imm<0>(byte_into_base<0>(word, rt[2 * wi]));
        acc[u0][1] += lds_f32_imm<128>(byte_into_base<1>(word, rt[2 * wi]));
        acc[u0][0] += lds_f32_imm<0>(byte_into_base<2>(word, rt[2 * wi + 1]));
        acc[u0][1] += lds_f32_imm<128>(byte_into_base<3>(word, rt[2 * wi + 1]));
    }
#pragma unroll
    for (int u = 0; u < GPW; ++u) sum[u] = acc[u][0] + acc[u][1];
}

template <int Q, int GPW, int OU>
__device__ __forceinline__ void compute_tile(const Tile<Q, GPW, OU> &t, const GemvArgs &a,
                                             const uint32_t (&rt)[8], const float (&xsu)[GPW],
                                             int s, int oct0, int oct_end, int lane, int mrow) {
    float v[OU];
#pragma unroll
    for (int ou = 0; ou < OU; ++ou) {
        float tot = 0.f;
#pragma unroll
        for (int u = 0; u < GPW; ++u) tot += meta_value<GPW>(t.mt[ou][Q], u) * xsu[u];
#pragma unroll
        for (int p = 0; p < Q; ++p) {
            float sum[GPW];
            lookup_word<GPW>(t.w[ou][p], rt, sum);
#pragma unroll
            for (int u = 0; u < GPW; ++u) tot += meta_value<GPW>(t.mt[ou][p], u) * sum[u];
        }
        v[ou] = tot;
    }
    // reduce the four lanes (j = lane & 3) of each row; with OU > 1 the reduction also
    // transposes, so that lane j ends up with oct oct0 + j
    const int j = lane & 3;
    float res;
    int my_oct;
    if (OU == 4) {
        const bool odd = j & 1;
        float k0 = odd ? v[1] : v[0], k1 = odd ? v[3] : v[2];
        float s0 = odd ? v[0] : v[1], s1 = odd ? v[2] : v[3];
        k0 += __shfl_xor_sync(0xffffffffu, s0, 1);
        k1 += __shfl_xor_sync(0xffffffffu, s1, 1);
        const bool hi = j & 2;
        float keep = hi ? k1 : k0, send = hi ? k0 : k1;
        keep += __shfl_xor_sync(0xffffffffu, send, 2);
        res = keep;
        my_oct = oct0 + j;
    } else if (OU == 2) {
        const bool odd = j & 1;
        float keep = odd ? v[OU - 1] : v[0], send = odd ? v[0] : v[OU - 1];
        keep += __shfl_xor_sync(0xffffffffu, send, 1);
        keep += __shfl_xor_sync(0xffffffffu, keep, 2);
        res = keep;
        my_oct = (j < 2) ? oct0 + j : oct_end;  // lanes j >= 2 hold duplicates
    } else {
        float keep = v[0];
        keep += __shfl_xor_sync(0xffffffffu, keep, 1);
        keep += __shfl_xor_sync(0xffffffffu, keep, 2);
        res = keep;
        my_oct = (j == 0) ? oct0 : oct_end;
    }
    if (my_oct < oct_end) {
        const int row = my_oct * kOctRows + (lane >> 2);
        a.partial[((int64_t)mrow * a.slices + s) * a.np + row] = res;
    }
}

template <int Q, int GPW, int OU>
__global__ void __launch_bounds__(kThreads, 1) lut8_gemv_kernel(const GemvArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mrow = blockIdx.y;

    // The table block must start on a 64 KB boundary of the shared window.
    const uint32_t sbase = smem_u32(smem_raw);
    const uint32_t tbl = (sbase + 0xffffu) & ~0xffffu;
    const uint32_t aux_u32 = (tbl - sbase >= kAuxBytes) ? sbase : tbl + kTableBytes;
    if (tbl + kTableBytes > sbase + a.dyn_smem || aux_u32 + kAuxBytes > sbase + a.dyn_smem) {
        if (tid == 0) atomicExch(a.status, 2);
        return;
    }
    unsigned char *aux = smem_raw + (aux_u32 - sbase);
    uint16_t *xs = (uint16_t *)(aux + kAuxX);
    float *xsum = (float *)(aux + kAuxXsum);
    const uint32_t mbar = aux_u32 + kAuxMbar;
    int *list_n = (int *)(aux + kAuxListN);
    int *fail = (int *)(aux + kAuxFlag);
    int *list = (int *)(aux + kAuxList);

    pdl_launch_dependents();

    if (tid == 0) {
        mbar_init(mbar, 1);
        *fail = 0;
    }

    // per-lane lookup bases: bank 8*j + (t ^ r) of the table row
    const int r = lane >> 2, j = lane & 3;
    uint32_t rt[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) rt[t] = tbl + 4u * (8u * j + (uint32_t)(t ^ r));

    // contiguous range of (slice, oct) units of this CTA
    const int64_t units = (int64_t)a.slices * a.octs;
    int64_t u = units * blockIdx.x / gridDim.x;
    const int64_t u_end = units * (blockIdx.x + 1) / gridDim.x;

    constexpr int gshift = GPW == 1 ? 3 : (GPW == 2 ? 2 : 1);
    uint32_t phase = 0;
    bool first = true;

    __syncthreads();

    while (u < u_end) {
        const int s = (int)(u / a.octs);
        const int oa = (int)(u % a.octs);
        const int ob = (int)min((int64_t)a.octs, oa + (u_end - u));

        // 1. start streaming weights (they do not depend on the activations)
        Tile<Q, GPW, OU> ta, tb;
        int o = oa + warp * OU;
        constexpr int ostride = kWarps * OU;
        if (o < ob) load_tile<Q, GPW, OU>(ta, a, s, o, ob, lane);

        // 2. activations of this slice: TMA bulk copy + zero padding
        if (first) {
            pdl_wait();
            first = false;
        }
        const int valid = min(kSliceK, a.k - s * kSliceK);
        if (tid == 0) {
            fence_proxy_async();
            mbar_expect_tx(mbar, (uint32_t)valid * 2u);
            const uint16_t *src = (const uint16_t *)a.x + (int64_t)mrow * a.k + (int64_t)s * kSliceK;
            tma_bulk_g2s(aux_u32 + kAuxX, src, (uint32_t)valid * 2u, mbar);
        }
        if (tid >= valid && tid < kSliceK) xs[tid] = 0;
        const bool ok = mbar_wait_bounded(mbar, phase);
        phase ^= 1u;
        if (!ok) *fail = 1;
        __syncthreads();
        if (*fail) {
            if (tid == 0) atomicExch(a.status, 1);
            return;  // the copy was given 2^22 polls; nothing else of this CTA is in flight
        }

        // 3. group sums (warp 0) and the 64 tables of 256 subset sums (all warps)
        if (warp == 0) {
            float part = 0.f;
#pragma unroll
            for (int i = 0; i < 16; ++i) part += x_to_float(xs[lane * 16 + i], a.x_dtype);
            // a group is g / 16 consecutive lanes: 8, 4 or 2
#pragma unroll
            for (int d = 1; d < (8 >> (3 - gshift)); d <<= 1)
                part += __shfl_xor_sync(0xffffffffu, part, d);
            constexpr int lanes_per_group = 8 >> (3 - gshift);
            if ((lane & (lanes_per_group - 1)) == 0) xsum[lane / lanes_per_group] = part;
        }
        {
            const int h = warp & 1, ehi = warp >> 1;  // bank-row, top three index bits
            const int c = 16 * (lane >> 3) + 2 * (lane & 7) + h;
            const uint4 raw = *(const uint4 *)(xs + 8 * c);
            const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
            float xv[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                xv[2 * i] = x_to_float((uint16_t)(rw[i] & 0xffffu), a.x_dtype);
                xv[2 * i + 1] = x_to_float((uint16_t)(rw[i] >> 16), a.x_dtype);
            }
            float base = 0.f;
            if (ehi & 1) base += xv[5];
            if (ehi & 2) base += xv[6];
            if (ehi & 4) base += xv[7];
            float tv[32];
            tv[0] = base;
#pragma unroll
            for (int b = 0; b < 5; ++b)
#pragma unroll
                for (int e = 0; e < (1 << b); ++e) tv[(1 << b) + e] = tv[e] + xv[b];
            const uint32_t dst = tbl + (uint32_t)ehi * (32u * 256u) + 4u * lane + 128u * h;
#pragma unroll
            for (int e = 0; e < 32; ++e) sts_f32(dst + (uint32_t)e * 256u, tv[e]);
        }
        __syncthreads();
        asm volatile("" ::: "memory");

        float xsu[GPW];
#pragma unroll
        for (int uu = 0; uu < GPW; ++uu) xsu[uu] = xsum[GPW * j + (uu ^ (r >> gshift))];

        // 4. stream: ping-pong between two register tiles
        while (o < ob) {
            int on = o + ostride;
            if (on < ob) load_tile<Q, GPW, OU>(tb, a, s, on, ob, lane);
            compute_tile<Q, GPW, OU>(ta, a, rt, xsu, s, o, ob, lane, mrow);
            o = on;
            if (o >= ob) break;
            on = o + ostride;
            if (on < ob) load_tile<Q, GPW, OU>(ta, a, s, on, ob, lane);
            compute_tile<Q, GPW, OU>(tb, a, rt, xsu, s, o, ob, lane, mrow);
            o = on;
        }

        // 5. publish: count finished octs per 32-row block; whoever completes a block sums it
        __threadfence();
        __syncthreads();
        const int bfirst = oa >> 2, blast = (ob - 1) >> 2;
        const unsigned total = (unsigned)a.slices * 4u;
        for (int b0 = bfirst; b0 <= blast; b0 += kListCap) {
            if (tid == 0) *list_n = 0;
            __syncthreads();
            const int blk = b0 + tid;
            if (tid < kListCap && blk <= blast) {
                const int lo = max(oa, 4 * blk), hi = min(ob, 4 * blk + 4);
                const unsigned cnt = (unsigned)(hi - lo);
                __threadfence();
                const unsigned old = atomicAdd(&a.counters[(int64_t)mrow * a.blocks + blk], cnt);
                if (old + cnt == total) list[atomicAdd(list_n, 1)] = blk;
            }
            __syncthreads();
            const int nlist = *list_n;
            if (nlist > 0) {
                __threadfence();
                for (int li = warp; li < nlist; li += kWarps) {
                    const int blk2 = list[li];
                    const int row = blk2 * kBlockRows + lane;
                    const float *pp = a.partial + (int64_t)mrow * a.slices * a.np + row;
                    float acc = 0.f;
                    for (int ss = 0; ss < a.slices; ++ss) acc += ldcg_f32(pp + (int64_t)ss * a.np);
                    if (row < a.n) {
                        if (a.bias) acc += __half2float(__ushort_as_half(a.bias[row]));
                        store_y(a.y, (int64_t)mrow * a.n + row, acc, a.y_dtype);
                    }
                    if (lane == 0) a.counters[(int64_t)mrow * a.blocks + blk2] = 0;
                }
            }
            __syncthreads();
        }
        u += ob - oa;
    }
}

// ------------------------------------------------------------------------------------------
// Generic kernel on the exported layout.
// ------------------------------------------------------------------------------------------
constexpr int kGenThreads = 256;
constexpr int kGenTileK = 2048;      // activations per shared-memory tile
constexpr int kGenMaxRows = 2048;    // output rows one CTA may own

struct GenArgs {
    const uint8_t *planes;   // [q][n][k/8]
    const uint16_t *scale;   // [q][n][k/g]
    const uint16_t *zero;    // [n][k/g]
    const uint16_t *bias;
    const void *x;
    void *y;
    int *status;
    int n, k, g, rows_per_cta;
    int x_dtype, y_dtype;
};

template <int Q, bool PER_BYTE>
__global__ void __launch_bounds__(kGenThreads) lut4_gemv_kernel(const GenArgs a) {
    __shared__ __align__(16) uint16_t xs[kGenTileK];
    __shared__ __align__(16) float lut[kGenTileK / 4][16];
    __shared__ float xword[kGenTileK / 32];
    __shared__ float yacc[kGenMaxRows];
    __shared__ __align__(8) unsigned long long mbar_store;
    __shared__ int fail;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mrow = blockIdx.y;
    const int row0 = blockIdx.x * a.rows_per_cta;
    const int rows = min(a.rows_per_cta, a.n - row0);
    if (rows <= 0) return;
    const uint32_t mbar = smem_u32(&mbar_store);
    pdl_launch_dependents();
    if (tid == 0) {
        mbar_init(mbar, 1);
        fail = 0;
    }
    for (int i = tid; i < rows; i += kGenThreads) yacc[i] = 0.f;
    __syncthreads();
    pdl_wait();

    const int kb = a.k / 8, ng = a.k / a.g;
    uint32_t phase = 0;
    for (int kt = 0; kt < a.k; kt += kGenTileK) {
        const int valid = min(kGenTileK, a.k - kt);
        if (tid == 0) {
            fence_proxy_async();
            mbar_expect_tx(mbar, (uint32_t)valid * 2u);
            tma_bulk_g2s(smem_u32(xs), (const uint16_t *)a.x + (int64_t)mrow * a.k + kt,
                         (uint32_t)valid * 2u, mbar);
        }
        for (int i = valid + tid; i < kGenTileK; i += kGenThreads) xs[i] = 0;
        const bool ok = mbar_wait_bounded(mbar, phase);
        phase ^= 1u;
        if (!ok) fail = 1;
        __syncthreads();
        if (fail) {
            if (tid == 0) atomicExch(a.status, 1);
            return;
        }
        // 16 subset sums per 4 activations (entry e adds x[b] for each set bit b of e)
        for (int c = tid; c < kGenTileK / 4; c += kGenThreads) {
            float xv[4];
#pragma unroll
            for (int b = 0; b < 4; ++b) xv[b] = x_to_float(xs[4 * c + b], a.x_dtype);
            float tv[16];
            tv[0] = 0.f;
#pragma unroll
            for (int b = 0; b < 4; ++b)
#pragma unroll
                for (int e = 0; e < (1 << b); ++e) tv[(1 << b) + e] = tv[e] + xv[b];
#pragma unroll
            for (int e = 0; e < 16; ++e) lut[c][e] = tv[e];
        }
        __syncthreads();
        for (int wd = tid; wd < kGenTileK / 32; wd += kGenThreads) {
            float sacc = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) sacc += lut[8 * wd + c][15];
            xword[wd] = sacc;
        }
        __syncthreads();

        const int words = (valid + 31) / 32;  // 32-bit words of packed bits per row in this tile
        for (int rl = warp; rl < rows; rl += kGenThreads / 32) {
            const int row = row0 + rl;
            float tot = 0.f;
            for (int wd = lane; wd < words; wd += 32) {
                const int kbyte = kt / 8 + 4 * wd;  // first byte of the word within the row
                const int nbytes = min(4, kb - kbyte);
                uint32_t bitsw[Q];
#pragma unroll
                for (int p = 0; p < Q; ++p) {
                    const uint8_t *src = a.planes + ((int64_t)p * a.n + row) * kb + kbyte;
                    uint32_t v = 0;
                    if (nbytes == 4 && ((uintptr_t)src & 3) == 0) {
                        v = __ldg((const uint32_t *)src);
                    } else {
                        for (int b = 0; b < nbytes; ++b) v |= (uint32_t)__ldg(src + b) << (8 * b);
                    }
                    bitsw[p] = v;
                }
                if (!PER_BYTE) {
                    const int grp = (kt + 32 * wd) / a.g;
                    float acc = __half2float(__ushort_as_half(__ldg(a.zero + (int64_t)row * ng + grp))) *
                                xword[wd];
#pragma unroll
                    for (int p = 0; p < Q; ++p) {
                        float sp = 0.f;
#pragma unroll
                        for (int nb = 0; nb < 8; ++nb)
                            sp += lut[8 * wd + nb][(bitsw[p] >> (4 * nb)) & 15u];
                        const float al = __half2float(__ushort_as_half(
                            __ldg(a.scale + ((int64_t)p * a.n + row) * ng + grp)));
                        acc += al * sp;
                    }
                    tot += acc;
                } else {
                    for (int b = 0; b < nbytes; ++b) {
                        const int grp = (kt + 32 * wd + 8 * b) / a.g;
                        const float xb = lut[8 * wd + 2 * b][15] + lut[8 * wd + 2 * b + 1][15];
                        float acc = __half2float(__ushort_as_half(
                                        __ldg(a.zero + (int64_t)row * ng + grp))) * xb;
#pragma unroll
                        for (int p = 0; p < Q; ++p) {
                            const uint32_t by = (bitsw[p] >> (8 * b)) & 255u;
                            const float sp = lut[8 * wd + 2 * b][by & 15u] + lut[8 * wd + 2 * b + 1][by >> 4];
                            const float al = __half2float(__ushort_as_half(
                                __ldg(a.scale + ((int64_t)p * a.n + row) * ng + grp)));
                            acc += al * sp;
                        }
                        tot += acc;
                    }
                }
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, d);
            if (lane == 0) yacc[rl] += tot;
        }
        __syncthreads();
    }
    for (int rl = tid; rl < rows; rl += kGenThreads) {
        float v = yacc[rl];
        if (a.bias) v += __half2float(__ushort_as_half(a.bias[row0 + rl]));
        store_y(a.y, (int64_t)mrow * a.n + row0 + rl, v, a.y_dtype);
    }
}

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
size_t workspace_bytes_for(int m, const StreamDims &d) {
    const int mm = m < kLutMaxM ? m : kLutMaxM;
    size_t counters = ((size_t)mm * d.blocks * sizeof(unsigned) + 255) / 256 * 256;
    size_t partial = (size_t)mm * d.slices * d.np * sizeof(float);
    return kWsHeader + counters + partial;
}

Workspace carve_workspace(void *base, int m, const StreamDims &d) {
    const int mm = m < kLutMaxM ? m : kLutMaxM;
    Workspace w;
    unsigned char *p = (unsigned char *)base;
    w.status = (int *)p;
    w.counters = (unsigned *)(p + kWsHeader);
    size_t counters = ((size_t)mm * d.blocks * sizeof(unsigned) + 255) / 256 * 256;
    w.partial = (float *)(p + kWsHeader + counters);
    return w;
}

struct DeviceInfo {
    int sms = 0;
    int max_dyn_smem = 0;
    bool ok = false;
};
static DeviceInfo g_dev[64];

static int device_info(int device, DeviceInfo **out) {
    if (device < 0 || device >= 64) return HLQ_ERR_INVALID_ARGUMENT;
    DeviceInfo &d = g_dev[device];
    if (!d.ok) {
        int major = 0;
        HLQ_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
        if (major != 10) return HLQ_ERR_NO_DEVICE;
        HLQ_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, device));
        HLQ_CUDA(cudaDeviceGetAttribute(&d.max_dyn_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin,
                                        device));
        d.ok = true;
    }
    *out = &d;
    return HLQ_OK;
}

template <typename KernelT, typename ArgsT>
static int launch_pdl(KernelT kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                      const ArgsT &args) {
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
    HLQ_CUDA(cudaLaunchKernelEx(&cfg, kernel, args));
    count_launch();
    return HLQ_OK;
}

// dynamic shared memory that always contains a 64 KB-aligned 64 KB block plus the aux area,
// wherever the window starts: 64 KB of slack, the table, the aux area.
constexpr uint32_t kLut8DynSmem = 65536 - 1024 + kTableBytes + kAuxBytes;

template <int Q, int GPW, int OU>
static int launch_lut8_inst(const GemvArgs &args, dim3 grid, cudaStream_t stream) {
    static bool configured[64] = {};
    int dev = 0;
    HLQ_CUDA(cudaGetDevice(&dev));
    auto kernel = lut8_gemv_kernel<Q, GPW, OU>;
    if (!configured[dev & 63]) {
        HLQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)kLut8DynSmem));
        configured[dev & 63] = true;
    }
    return launch_pdl(kernel, grid, dim3(kThreads), kLut8DynSmem, stream, args);
}

template <int Q, int GPW>
static int launch_lut8_ou(int ou, const GemvArgs &args, dim3 grid, cudaStream_t stream) {
    if (Q <= 2 && ou >= 4) return launch_lut8_inst<Q, GPW, (Q <= 2 ? 4 : 2)>(args, grid, stream);
    if (ou >= 2) return launch_lut8_inst<Q, GPW, 2>(args, grid, stream);
    return launch_lut8_inst<Q, GPW, 1>(args, grid, stream);
}

template <int Q>
static int launch_lut8_gpw(int gpw, int ou, const GemvArgs &args, dim3 grid, cudaStream_t stream) {
    if (gpw == 1) return launch_lut8_ou<Q, 1>(ou, args, grid, stream);
    if (gpw == 2) return launch_lut8_ou<Q, 2>(ou, args, grid, stream);
    return launch_lut8_ou<Q, 4>(ou, args, grid, stream);
}

static int env_int(const char *name, int dflt) {
    const char *v = getenv(name);
    return v && *v ? atoi(v) : dflt;
}

int launch_lut8_gemv(const hlq_weight *w, int m, const void *x, int x_dtype, void *y, int y_dtype,
                     void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (w->layout != HLQ_LAYOUT_STREAM) return HLQ_ERR_UNSUPPORTED;
    if (x_dtype != HLQ_F16 && x_dtype != HLQ_BF16) return HLQ_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)y & 3)) return HLQ_ERR_ALIGNMENT;
    const StreamDims d = stream_dims(w->n, w->k, w->g, w->q);
    if (!workspace || workspace_bytes < workspace_bytes_for(m, d)) return HLQ_ERR_WORKSPACE;
    DeviceInfo *di;
    int rc = device_info(w->device, &di);
    if (rc) return rc;
    if ((uint32_t)di->max_dyn_smem < kLut8DynSmem) return HLQ_ERR_NO_DEVICE;

    static const int force_ou = env_int("HLQ_GEMV_OU", 0);
    static const int force_ctas = env_int("HLQ_GEMV_CTAS", 0);
    const size_t xsz = 2, ysz = y_dtype == HLQ_F32 ? 4 : 2;
    for (int m0 = 0; m0 < m; m0 += kLutMaxM) {
        const int mc = (m - m0) < kLutMaxM ? (m - m0) : kLutMaxM;
        const Workspace ws = carve_workspace(workspace, mc, d);
        GemvArgs a;
        a.planes = w->d_planes;
        a.meta = w->d_meta;
        a.x = (const char *)x + (size_t)m0 * w->k * xsz;
        a.y = (char *)y + (size_t)m0 * w->n * ysz;
        a.bias = w->d_bias;
        a.partial = ws.partial;
        a.counters = ws.counters;
        a.status = ws.status;
        a.n = w->n; a.k = w->k; a.np = d.np; a.slices = d.slices; a.octs = d.octs;
        a.blocks = d.blocks;
        a.x_dtype = x_dtype; a.y_dtype = y_dtype;
        a.dyn_smem = kLut8DynSmem;
        const int64_t units = (int64_t)d.slices * d.octs;
        int ctas = force_ctas > 0 ? force_ctas : di->sms;
        if (units < ctas) ctas = (int)units;
        const int64_t per_cta = units / ctas;
        int ou = force_ou > 0 ? force_ou : (per_cta >= 10 * kWarps ? 4 : (per_cta >= 3 * kWarps ? 2 : 1));
        dim3 grid(ctas, mc);
        switch (w->q) {
            case 1: rc = launch_lut8_gpw<1>(d.gpw, ou, a, grid, stream); break;
            case 2: rc = launch_lut8_gpw<2>(d.gpw, ou, a, grid, stream); break;
            case 3: rc = launch_lut8_gpw<3>(d.gpw, ou, a, grid, stream); break;
            case 4: rc = launch_lut8_gpw<4>(d.gpw, ou, a, grid, stream); break;
            default: rc = HLQ_ERR_SHAPE;
        }
        if (rc) return rc;
    }
    return HLQ_OK;
}

// Status word used by the generic kernel when the caller gave no workspace.
static int *generic_status_word(int device) {
    static int *words[64] = {};
    if (!words[device & 63]) {
        int *p = nullptr;
        if (cudaMalloc(&p, 256) != cudaSuccess) return nullptr;
        cudaMemset(p, 0, 256);
        words[device & 63] = p;
    }
    return words[device & 63];
}

int launch_lut4_gemv(const hlq_weight *w, int m, const void *x, int x_dtype, void *y, int y_dtype,
                     cudaStream_t stream) {
    if (w->layout != HLQ_LAYOUT_EXPORT) return HLQ_ERR_UNSUPPORTED;
    if (x_dtype != HLQ_F16 && x_dtype != HLQ_BF16) return HLQ_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)y & 3)) return HLQ_ERR_ALIGNMENT;
    DeviceInfo *di;
    int rc = device_info(w->device, &di);
    if (rc) return rc;
    GenArgs a;
    a.planes = w->d_planes;
    a.scale = w->d_meta;
    a.zero = w->d_meta + (int64_t)w->q * w->n * (w->k / w->g);
    a.bias = w->d_bias;
    a.x = x;
    a.y = y;
    a.status = generic_status_word(w->device);
    if (!a.status) return note_cuda(cudaErrorMemoryAllocation);
    a.n = w->n; a.k = w->k; a.g = w->g;
    a.x_dtype = x_dtype; a.y_dtype = y_dtype;
    int rows_per_cta = (w->n + 4 * di->sms - 1) / (4 * di->sms);
    if (rows_per_cta < 8) rows_per_cta = 8;
    if (rows_per_cta > kGenMaxRows) rows_per_cta = kGenMaxRows;
    a.rows_per_cta = rows_per_cta;
    const int gx = (w->n + rows_per_cta - 1) / rows_per_cta;
    const bool per_byte = (w->g % 32) != 0;
    for (int m0 = 0; m0 < m; m0 += 65535) {
        const int mc = (m - m0) < 65535 ? (m - m0) : 65535;
        GenArgs b = a;
        b.x = (const char *)x + (size_t)m0 * w->k * 2;
        b.y = (char *)y + (size_t)m0 * w->n * (y_dtype == HLQ_F32 ? 4 : 2);
        dim3 grid(gx, mc);
#define HLQ_GEN_CASE(QV)                                                                       \
    case QV:                                                                                   \
        rc = per_byte ? launch_pdl(lut4_gemv_kernel<QV, true>, grid, dim3(kGenThreads), 0, stream, b) \
                      : launch_pdl(lut4_gemv_kernel<QV, false>, grid, dim3(kGenThreads), 0, stream, b); \
        break;
        switch (w->q) {
            HLQ_GEN_CASE(1)
            HLQ_GEN_CASE(2)
            HLQ_GEN_CASE(3)
            HLQ_GEN_CASE(4)
            default: rc = HLQ_ERR_SHAPE;
        }
#undef HLQ_GEN_CASE
        if (rc) return rc;
    }
    return HLQ_OK;
}

}  // namespace hlq
