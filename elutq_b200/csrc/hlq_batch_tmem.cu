// Small batches (3..16 rows of activations) with the weight operand in TENSOR MEMORY, sm_100a.
//
// Replaces, for small m, the reference's batched path
//   C++/ops/src/arm/arm_gemm.cpp:362-387   (GEMM worker: a table per row of x, all rows re-walk the planes)
// The two kernels beside it keep the streaming layout: batch_mma_kernel (hlq_batch.cu) pays 8 cycles
// of a sub-partition per mma.sync on top of the integer work, batch_umma_kernel (hlq_batch_umma.cu)
// pays shared-memory bandwidth for an fp16 operand that is written once and read once.  Here the
// dequantized weights go from registers straight into tensor memory (tcgen05.st) and tcgen05.mma
// reads its A operand there; shared memory carries only the activations.
//
// That wants a lane to own a whole ROW of the operand (a thread can write only its own lane of
// tensor memory), which the streaming layout does not give (there four lanes share a row).  The
// kernel therefore reads the optional "row codes" of a weight (hlq_weight_build_batch_codes; 2- and
// 3-bit weights with g = 128 and rows a multiple of 128): per slice and tile of 128 rows, for
// every quarter kp of the slice and row, 128 four-bit codes in channel order (64 bytes, as four
// 16-byte chunks laid out [kp][chunk][row] so that a warp's loads are contiguous) and the group's
// scales and zero as four fp16 [kp][row].
//
//   warps 0..15   dequantizers: warp w owns rows 32 (w & 3) .. +31 of the tile (its quarter of the
//                 lanes of tensor memory) and quarter kp = w >> 2 of the slice: one (row, group)
//                 per lane, so one pair of byte tables per lane and tile; 8 prmt per word of 8
//                 codes, 16 registers per tcgen05.st.32x32b.x16.  The operand buffers (one per
//                 quarter of a slice, 64 columns) form a ring of seven: the tensor cores read
//                 one tile while the next is written.
//   warp 21       one thread issues tcgen05.mma (A in tensor memory, B = the rows of x in shared
//                 memory, 128 x 16 x 16, fp32 accumulation in two alternating 16-column accumulators).
//   warp 24       one thread brings a tile's row codes and scales (36 KB, contiguous) into a ring of
//                 three shared-memory slots by bulk copies: loads in flight do not cost registers.
//   warps 16..19  epilogue, warp 20 control, warps 22..23 completion of blocks: as batch_umma_kernel.
//
// What bounds it (measured on the 8B projection set, 3-bit): a product of 128 rows x 16 channels
// costs the tensor pipe about 95 cycles whatever the number of activation rows (16 columns are the
// smallest product there is, and most of it is bringing in the 128 x 16 operand), 32 products per
// tile: 1.2 ms for the model at 4..16 rows.  Without the products the kernel runs in 0.75 ms
// (4 rows), without the dequantization or without the stores in the same 1.2 ms.  So it matches
// batch_mma_kernel with code words at 16 rows and loses below; it is selectable
// (hlq_select_batch_kernel) and not the default.
//
// Every wait is an mbarrier wait with a poll limit; the first one that runs out sets the CTA's
// failure flag, after which all waits give up at once and the roles run out of work.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hlq_batch_dev.cuh"
#include "hlq_gemv_args.cuh"
#include "hlq_gemv_dev.cuh"
#include "hlq_internal.h"

namespace hlq {

namespace {

constexpr int kBuThreads = 25 * 32;                  // 16 dequantizer warps and 9 others
constexpr int kBuEpiWarp0 = 16, kBuCtlWarp = 20, kBuMmaWarp = 21, kBuFinWarp0 = 22, kBuFinWarps = 2, kBuLoadWarp = 24;
constexpr int kLoadRing = 3;                         // tiles of row codes in flight in shared memory
constexpr uint32_t kLoadTileBytes = kRowCodeTileBytes + kRowMetaTileBytes;
constexpr int kBtTileDuos = 8;                       // duos per tile of 128 rows
constexpr int kBuStageBlocks = 8;                    // blocks a completing warp stages at once
constexpr int kBuListMax = 64;                       // blocks one segment can complete (128 duos)
// tensor memory columns: per tile in flight (two) kAccSplit accumulators of 16, then a ring of operand
// buffers of 64 columns (one quarter of a slice: 128 channels as fp16 pairs).  Products into one
// accumulator follow one another; spreading them over four accumulators that the epilogue adds was
// measured and is slower (the epilogue's four loads cost more than the chain), so kAccSplit is 1.
constexpr int kAccSplit = 1;
constexpr uint32_t kTmAcc = 0, kTmAccTile = 16 * kAccSplit, kTmA = 2 * kTmAccTile, kTmABuf = 64, kTmCols = 512;
constexpr int kRing = 7;
static_assert(kTmA + kRing * kTmABuf <= kTmCols, "tensor memory of one SM");

// What the control warp hands the completing warps for one segment.
struct FinJob {
    float *acc;
    unsigned *counters;
    void *y;
    const uint16_t *bias;
    int n, y_dtype;
    int count;                 // blocks in the list; -1: no more segments
    int blocks[kBuListMax];
};

// shared memory (bytes from the 1 KB-aligned base)
constexpr uint32_t kBuB = 0;                                   // 2 slots x 8 K steps x [16 rows of x][128 bytes]
constexpr uint32_t kBuBSlotBytes = 8 * 2048;
constexpr uint32_t kBuRaw = kBuB + 2 * kBuBSlotBytes;          // [16][512] 16-bit activations as they come
constexpr uint32_t kBuStage = kBuRaw + 16384;                  // per completing warp: accumulators of finished blocks
constexpr uint32_t kBuList = kBuStage + kBuFinWarps * kBuStageBlocks * 2048;     // 2 x FinJob
constexpr uint32_t kBuListSlot = 512;
constexpr uint32_t kBuSeg = kBuList + 2 * kBuListSlot;         // 2 x Seg
constexpr uint32_t kBuSegSlot = 192;
constexpr uint32_t kBuLoad = ((kBuSeg + 2 * kBuSegSlot + 127) / 128) * 128;     // kLoadRing x (row codes, scales) of a tile
constexpr uint32_t kBuBars = kBuLoad + kLoadRing * kLoadTileBytes;                // mbarriers, 8 bytes each
constexpr uint32_t kBuTmemSlot = kBuBars + 8 * 40;
constexpr uint32_t kBuFlag = kBuTmemSlot + 8;
constexpr uint32_t kBuSmem = kBuFlag + 8 + 1024;               // + slack for the alignment
static_assert(sizeof(Seg) <= kBuSegSlot, "Seg must fit its slot");
static_assert(sizeof(FinJob) <= kBuListSlot, "FinJob must fit its slot");
static_assert(kBuSmem <= 227 * 1024, "shared memory of one CTA");
// mbarrier indices
enum { kBarDesc = 0, kBarXraw = 2, kBarBfull = 3, kBarAccFull = 5, kBarAccEmpty = 7, kBarSegDone = 9, kBarListFull = 11,
       kBarListEmpty = 13, kBarAfull = 15, kBarAempty = 15 + kRing, kBarLfull = 15 + 2 * kRing,
       kBarLempty = 15 + 2 * kRing + kLoadRing };

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
// kind::f16: fp32 accumulator, A and B fp16, both K-major, M = 128, N = 16
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(16 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
// A operand in tensor memory (lane = row, a column = two consecutive channels), B in shared memory
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(kIdesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar)
                 : "memory");
}
__device__ __forceinline__ void bu_cp_async_16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void bu_cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// What a dequantizer lane holds of a tile: the 128 codes of its row and quarter, the group's scales and zero.
struct RowTile {
    uint4 w[4];
    uint2 mt;       // fp16: alpha 0, alpha 1 | alpha 2 (or 0), zero
};

template <int Q, int NT>
__global__ void __launch_bounds__(kBuThreads, 1) batch_tmem_kernel(const __grid_constant__ GemvArgs a) {
    static_assert(Q == 2 || Q == 3, "byte tables hold at most eight codes");
    constexpr int GPW = 1;                          // g = 128: one group per quarter of a slice
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int MT = 8 * NT;                     // rows of x the global accumulators hold
    constexpr int kBlockBytes = kBlockRows * MT * 4;
    const int m = a.batch_rows;

    const uint32_t sraw = smem_u32(smem_dyn);
    const uint32_t sbase = (sraw + 1023u) & ~1023u;
    unsigned char *sm = smem_dyn + (sbase - sraw);
    if (sbase + kBuSmem - 1024 > sraw + a.dyn_smem) {
        if (tid == 0) atomicExch(a.status, 2);
        return;
    }
    volatile int *fail = (volatile int *)(sm + kBuFlag);
    const int spin = a.spin_limit;
    Seg *ring = (Seg *)(sm + kBuSeg);
    uint32_t *tmem_slot = (uint32_t *)(sm + kBuTmemSlot);
    auto bar = [&](int index) { return sbase + kBuBars + 8u * (uint32_t)index; };

    pdl_launch_dependents();
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar(kBarDesc + i), 1);
            mbar_init(bar(kBarBfull + i), 1);
            mbar_init(bar(kBarAccFull + i), 1);
            mbar_init(bar(kBarAccEmpty + i), 4);
            mbar_init(bar(kBarSegDone + i), 4);
            mbar_init(bar(kBarListFull + i), 1);
            mbar_init(bar(kBarListEmpty + i), kBuFinWarps);
        }
        for (int i = 0; i < kRing; ++i) {
            mbar_init(bar(kBarAfull + i), 4);        // the four warps of a quarter
            mbar_init(bar(kBarAempty + i), 1);
        }
        for (int i = 0; i < kLoadRing; ++i) {
            mbar_init(bar(kBarLfull + i), 1);
            mbar_init(bar(kBarLempty + i), 16);      // every dequantizer warp has taken its share
        }
        mbar_init(bar(kBarXraw), 1);
        mbar_init_fence();
        *fail = 0;
    }
    if (warp == kBuMmaWarp) {      // all of tensor memory: one CTA per SM
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // tiles of a segment (its duos are a multiple of 8: GemvArgs::unit_align)
    auto tiles_of = [](const Seg &sg) { return (sg.duo_b - sg.duo_a) / kBtTileDuos; };
    constexpr bool CODES = true;
    (void)CODES;

    if (warp == kBuCtlWarp) {
        // ============== control: descriptors, activations as the B operand ====================
        Walker wk;
        bool waited = false;
        int xuse = 0;             // bulk copies of activations issued so far (parity of their barrier)
        auto emit = [&](int slot, int use) {
            Seg sg;
            int valid;
            const uint16_t *src = walker_next<Q, GPW>(wk, sg, valid);
            if (lane == 0) ring[slot] = sg;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarDesc + slot));
            if (!sg.live) return;
            if (!waited) {
                pdl_wait();
                waited = true;
            }
            uint16_t *xs = (uint16_t *)(sm + kBuRaw);
            if (valid < kSliceK)
                for (int rr = 0; rr < m; ++rr)
                    for (int i = valid + lane; i < kSliceK; i += 32) xs[rr * kSliceK + i] = 0;
            __syncwarp();
            if (lane == 0) {
                fence_proxy_async();
                const uint32_t bytes = (uint32_t)valid * 2u;
                mbar_expect_tx(bar(kBarXraw), bytes * (uint32_t)m);
                for (int rr = 0; rr < m; ++rr)
                    tma_bulk_g2s(sbase + kBuRaw + rr * kSliceK * 2, src + (long long)rr * sg.k, bytes, bar(kBarXraw));
            }
            mbar_wait_bounded(bar(kBarXraw), xuse & 1, fail, spin);
            ++xuse;
            // B operand: row of x t, K step ks of 64 channels, 16-byte chunk c8 of its 128 bytes, in
            // channel order; 128-byte swizzle: chunk ^ (t & 7)
            const int x_dtype = sg.x_dtype;
            unsigned char *dst = sm + kBuB + slot * kBuBSlotBytes;
            for (int u = lane; u < 16 * 64; u += 32) {
                const int t = u >> 6, ks = (u >> 3) & 7, c8 = u & 7;
                uint4 w4 = make_uint4(0u, 0u, 0u, 0u);
                if (t < m) w4 = *(const uint4 *)(xs + t * kSliceK + 64 * ks + 8 * c8);
                if (x_dtype != HLQ_F16) {
                    uint32_t in[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const __half2 h2 = __floats2half2_rn(x_to_float((uint16_t)(in[e] & 0xffffu), x_dtype),
                                                             x_to_float((uint16_t)(in[e] >> 16), x_dtype));
                        in[e] = *(const uint32_t *)&h2;
                    }
                    w4 = make_uint4(in[0], in[1], in[2], in[3]);
                }
                *(uint4 *)(dst + ks * 2048 + t * 128 + ((c8 ^ (t & 7)) << 4)) = w4;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarBfull + slot));
            (void)use;
        };
        int lists = 0;            // lists handed to the completing warps so far
        walker_init(wk, a, 0);
        emit(0, 0);
        emit(1, 1);
        pdl_wait();
        for (int i = 0;; ++i) {
            const int slot = i & 1;
            const bool have = mbar_wait_bounded(bar(kBarDesc + slot), (i >> 1) & 1, fail, spin);
            if (!have || !ring[slot].live) break;
            const Seg sg = ring[slot];
            // the segment's last sums have been added by all four epilogue warps: its slot is free
            // for segment i + 2; then count finished duos per block of 32 rows - the blocks this
            // segment completes become outputs (as in batch_mma_kernel)
            if (!mbar_wait_bounded(bar(kBarSegDone + slot), (i >> 1) & 1, fail, spin)) break;
            emit(slot, i + 2);
            // counters: the blocks this segment completes go to the completing warps
            const int bfirst = sg.duo_a >> 1, blast = (sg.duo_b - 1) >> 1;
            const unsigned total = (unsigned)sg.slices * 2u;
            if (i >= 2 && !mbar_wait_bounded(bar(kBarListEmpty + slot), ((i >> 1) - 1) & 1, fail, spin)) break;
            FinJob *job = (FinJob *)(sm + kBuList + slot * kBuListSlot);
            int nlist = 0;
            __threadfence();
#pragma unroll
            for (int e = 0; e < kBuListMax / 32; ++e) {
                const int bi = bfirst + 32 * e + lane;
                bool mine = false;
                if (bi <= blast) {
                    const int lo = max(sg.duo_a, 2 * bi), hi = min(sg.duo_b, 2 * bi + 2);
                    const unsigned cnt = (unsigned)(hi - lo);
                    mine = atomicAdd(&sg.counters[bi], cnt) + cnt == total;
                }
                const unsigned mask = __ballot_sync(0xffffffffu, mine);
                if (mine) job->blocks[nlist + __popc(mask & ((1u << lane) - 1u))] = bi;
                nlist += __popc(mask);
            }
            if (lane == 0) {
                job->acc = sg.acc; job->counters = sg.counters; job->y = sg.y; job->bias = sg.bias;
                job->n = sg.n; job->y_dtype = sg.y_dtype; job->count = nlist;
            }
            if (nlist) __threadfence();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarListFull + slot));
            ++lists;
        }
        // tell the completing warps that nothing follows
        {
            const int slot = lists & 1;
            if (lists < 2 || mbar_wait_bounded(bar(kBarListEmpty + slot), ((lists >> 1) - 1) & 1, fail, spin)) {
                FinJob *job = (FinJob *)(sm + kBuList + slot * kBuListSlot);
                if (lane == 0) job->count = -1;
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kBarListFull + slot));
            }
        }
    } else if (warp >= kBuFinWarp0 && warp < kBuFinWarp0 + kBuFinWarps) {
        // ==================== completion of blocks of 32 rows ==================================
        const int fwi = warp - kBuFinWarp0;
        const uint32_t stage = kBuStage + fwi * kBuStageBlocks * 2048;
        pdl_wait();
        for (int i = 0;; ++i) {
            const int slot = i & 1;
            if (!mbar_wait_bounded(bar(kBarListFull + slot), (i >> 1) & 1, fail, spin)) break;
            const FinJob *job = (const FinJob *)(sm + kBuList + slot * kBuListSlot);
            const int count = job->count;
            if (count < 0) break;
            float *acc = job->acc;
            for (int l0 = fwi * kBuStageBlocks; l0 < count; l0 += kBuFinWarps * kBuStageBlocks) {
                const int nb = min(kBuStageBlocks, count - l0);
                for (int e = 0; e < nb; ++e) {
                    const unsigned char *src = (const unsigned char *)acc + (long long)job->blocks[l0 + e] * kBlockBytes;
#pragma unroll
                    for (int c = 0; c < kBlockBytes / 512; ++c)
                        bu_cp_async_16(sbase + stage + e * kBlockBytes + (c * 32 + lane) * 16, src + (c * 32 + lane) * 16);
                }
                bu_cp_async_wait_all();
                __syncwarp();
                for (int e = 0; e < nb; ++e) {
                    const int blk = job->blocks[l0 + e];
                    const int row = blk * kBlockRows + lane;
                    const float4 *sp = (const float4 *)(sm + stage + e * kBlockBytes + lane * (MT * 4));
                    float o[MT];
#pragma unroll
                    for (int qd = 0; qd < MT / 4; ++qd) {
                        const float4 f = sp[qd];
                        o[4 * qd] = f.x; o[4 * qd + 1] = f.y; o[4 * qd + 2] = f.z; o[4 * qd + 3] = f.w;
                    }
                    float4 *ap = (float4 *)((unsigned char *)acc + (long long)blk * kBlockBytes);
#pragma unroll
                    for (int c = 0; c < kBlockBytes / 512; ++c) ap[c * 32 + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (row < job->n) {
                        const float bias = job->bias ? __half2float(__ushort_as_half(job->bias[row])) : 0.f;
#pragma unroll
                        for (int rr = 0; rr < MT; ++rr)
                            if (rr < m) store_y(job->y, (long long)rr * job->n + row, o[rr] + bias, job->y_dtype);
                    }
                    if (lane == 0) job->counters[blk] = 0;
                }
                __syncwarp();
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarListEmpty + slot));
        }
    } else if (warp == kBuLoadWarp) {
        // ============== producer: a tile's row codes and scales by bulk copies ================
        if (lane == 0) {
            int T = 0, ls = 0, luse = 0;      // tiles so far; slot of the ring; rounds of the ring completed
            for (int i = 0;; ++i) {
                const int slot = i & 1;
                const bool have = mbar_wait_bounded(bar(kBarDesc + slot), (i >> 1) & 1, fail, spin);
                if (!have || !ring[slot].live) break;
                const Seg &sg = ring[slot];
                const int nt = tiles_of(sg);
                const uint8_t *rc = sg.rcodes;
                const uint8_t *rm = (const uint8_t *)sg.rmeta;
                bool ok = true;
                for (int t = 0; t < nt && ok; ++t, ++T) {
                    if (luse >= 1) ok = mbar_wait_bounded(bar(kBarLempty + ls), (uint32_t)(luse - 1) & 1u, fail, spin);
                    if (!ok) break;
                    const uint32_t dst = sbase + kBuLoad + ls * kLoadTileBytes;
                    mbar_expect_tx(bar(kBarLfull + ls), kLoadTileBytes);
                    tma_bulk_g2s(dst, rc + (long long)t * kRowCodeTileBytes, kRowCodeTileBytes, bar(kBarLfull + ls));
                    tma_bulk_g2s(dst + kRowCodeTileBytes, rm + (long long)t * kRowMetaTileBytes, kRowMetaTileBytes,
                                 bar(kBarLfull + ls));
                    if (++ls == kLoadRing) {
                        ls = 0;
                        ++luse;
                    }
                }
                if (!ok) break;
            }
        }
    } else if (warp == kBuMmaWarp) {
        // ============================ tensor-core issue =======================================
        if (lane == 0) {
            // One thread issues everything, so its own instruction count is what a tile costs here:
            // descriptors are formed once per segment and advanced by constants, the ring position
            // is counted, not divided.
            int T = 0;            // tiles so far, over all segments
            int rs = 0;           // next buffer of the ring
            uint32_t rpar = 0;    // parity of its "full" barrier
            for (int i = 0;; ++i) {
                const int slot = i & 1;
                const bool have = mbar_wait_bounded(bar(kBarDesc + slot), (i >> 1) & 1, fail, spin);
                if (!have || !ring[slot].live) break;
                const int nt = tiles_of(ring[slot]);
                if (!mbar_wait_bounded(bar(kBarBfull + slot), (i >> 1) & 1, fail, spin)) break;
                const uint64_t bdesc0 = umma_desc(sbase + kBuB + slot * kBuBSlotBytes);
                bool ok = true;
                for (int t = 0; t < nt && ok; ++t, ++T) {
                    const int ab = T & 1;
                    if (T >= 2 && !mbar_wait_bounded(bar(kBarAccEmpty + ab), ((T >> 1) - 1) & 1, fail, spin)) {
                        ok = false;
                        break;
                    }
                    const uint32_t dcol = tmem_base + kTmAcc + kTmAccTile * (uint32_t)ab;
#pragma unroll
                    for (int kp = 0; kp < 4; ++kp) {
                        if (!mbar_wait_bounded(bar(kBarAfull + rs), rpar, fail, spin)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t acol = tmem_base + kTmA + (uint32_t)rs * kTmABuf;
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk)         // 16 channels = 8 columns of A, 32 bytes of B
                            umma_f16_ts(dcol + (uint32_t)(16 * (kk % kAccSplit)), acol + (uint32_t)(8 * kk),
                                        bdesc0 + (uint64_t)(((2 * kp + (kk >> 2)) * 2048 >> 4) + 2 * (kk & 3)),
                                        (kp > 0 || kk >= kAccSplit) ? 1u : 0u);
                        umma_commit(bar(kBarAempty + rs));
                        if (++rs == kRing) {
                            rs = 0;
                            rpar ^= 1u;
                        }
                    }
                    if (ok) umma_commit(bar(kBarAccFull + ab));
                }
                if (!ok || *fail) break;
            }
        }
    } else if (warp >= kBuEpiWarp0) {
        // ====================== epilogue and completion of blocks =============================
        const int q4 = warp - kBuEpiWarp0;             // TMEM lanes 32 q4 .. +31
        int T = 0;
        bool first = true;
        for (int i = 0;; ++i) {
            const int slot = i & 1;
            const bool have = mbar_wait_bounded(bar(kBarDesc + slot), (i >> 1) & 1, fail, spin);
            if (!have || !ring[slot].live) break;
            const Seg sg = ring[slot];
            const int nt = tiles_of(sg);
            if (first) {
                pdl_wait();       // before this warp's first global write
                first = false;
            }
            bool ok = true;
            for (int t = 0; t < nt && ok; ++t, ++T) {
                const int ab = T & 1;
                ok = mbar_wait_bounded(bar(kBarAccFull + ab), (T >> 1) & 1, fail, spin);
                if (!ok) break;
                tc_fence_after();
                uint32_t v[16];
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * q4) << 16) + kTmAcc + kTmAccTile * (uint32_t)ab;
                auto load16 = [&](uint32_t *r, uint32_t addr) {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                        : "r"(addr) : "memory");
                };
                load16(v, taddr);
#pragma unroll
                for (int c = 1; c < kAccSplit; ++c) {
                    uint32_t u[16];
                    load16(u, taddr + (uint32_t)(16 * c));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(u[e]));
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kBarAccEmpty + ab));
                const int row = (sg.duo_a + t * kBtTileDuos) * 16 + 32 * q4 + lane;     // row of the linear
                if (row < sg.duo_b * 16) {
                    float4 *dstp = (float4 *)(sg.acc + (long long)row * MT);
#pragma unroll
                    for (int qd = 0; qd < MT / 4; ++qd)
                        atomicAdd(dstp + qd, make_float4(__uint_as_float(v[4 * qd]), __uint_as_float(v[4 * qd + 1]),
                                                         __uint_as_float(v[4 * qd + 2]), __uint_as_float(v[4 * qd + 3])));
                }
            }
            if (!ok) break;
            __threadfence();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(kBarSegDone + slot));
        }
    } else {
        // ================================ dequantizers =========================================
        const int q4 = warp & 3, kp = warp >> 2;         // lanes 32 q4 .. +31 of tensor memory, quarter kp of the slice
        const uint32_t tlane = tmem_base + ((uint32_t)(32 * q4) << 16) + kTmA;
        // this lane's part of a tile in the ring of row codes: 16 bytes per chunk, 8 bytes of scales
        const uint32_t lrow = (uint32_t)(((kp * 4) * 128 + 32 * q4 + lane) * 16);
        const uint32_t lmeta = kRowCodeTileBytes + (uint32_t)((kp * 128 + 32 * q4 + lane) * 8);
        int ls = 0, luse = 0;       // slot of the ring of loads, rounds completed
        int T = 0;
        int rs = kp, use = 0;       // buffer of the ring this warp writes next, and how often it has been used
        bool first = true;
        for (int i = 0;; ++i) {
            const int slot = i & 1;
            const bool have = mbar_wait_bounded(bar(kBarDesc + slot), (i >> 1) & 1, fail, spin);
            if (!have || !ring[slot].live) break;
            const Seg &sg = ring[slot];
            const int nt = tiles_of(sg);
            if (first) {
                pdl_wait();
                first = false;
            }
            bool ok = true;
            for (int t = 0; t < nt && ok; ++t) {
                // the tile's codes and scales from shared memory; the slot goes back to the producer at once
                RowTile cur;
                ok = mbar_wait_bounded(bar(kBarLfull + ls), (uint32_t)luse & 1u, fail, spin);
                if (!ok) break;
                {
                    const unsigned char *lp = sm + kBuLoad + ls * kLoadTileBytes;
#pragma unroll
                    for (int c = 0; c < 4; ++c) cur.w[c] = *(const uint4 *)(lp + lrow + c * 128 * 16);
                    cur.mt = *(const uint2 *)(lp + lmeta);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kBarLempty + ls));
                if (++ls == kLoadRing) {
                    ls = 0;
                    ++luse;
                }
                // the 2^q values of this lane's (row, group) as byte tables
                ByteTables<Q> bt;
                {
                    const float z = __half2float(__ushort_as_half((uint16_t)(cur.mt.y >> 16)));
                    float al[3];
                    al[0] = __half2float(__ushort_as_half((uint16_t)(cur.mt.x & 0xffffu)));
                    al[1] = __half2float(__ushort_as_half((uint16_t)(cur.mt.x >> 16)));
                    al[2] = __half2float(__ushort_as_half((uint16_t)(cur.mt.y & 0xffffu)));
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
                    bt.lo[1] = Q == 3 ? prmt(pr[2 % ((1 << Q) / 2)], pr[3 % ((1 << Q) / 2)], 0x6420u) : 0u;
                    bt.hi[1] = Q == 3 ? prmt(pr[2 % ((1 << Q) / 2)], pr[3 % ((1 << Q) / 2)], 0x7531u) : 0u;
                }
                // this quarter's buffer of the ring: 4 T + kp, counted modulo kRing
                if (use >= 1) ok = mbar_wait_bounded(bar(kBarAempty + rs), (uint32_t)(use - 1) & 1u, fail, spin);
                if (ok) {
                    tc_fence_after();
                    const uint32_t tcol = tlane + (uint32_t)rs * kTmABuf;
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t words[4] = {cur.w[c].x, cur.w[c].y, cur.w[c].z, cur.w[c].w};
                        uint32_t o[16];
#pragma unroll
                        for (int wi = 0; wi < 4; ++wi)
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                const uint32_t sel = h ? (words[wi] >> 16) : words[wi];
                                const uint32_t lb = prmt(bt.lo[0], bt.lo[1], sel);
                                const uint32_t hb = prmt(bt.hi[0], bt.hi[1], sel);
                                o[4 * wi + 2 * h] = prmt(lb, hb, 0x5140u);         // channels 8 wi + 4 h, + 1
                                o[4 * wi + 2 * h + 1] = prmt(lb, hb, 0x7362u);     // channels 8 wi + 4 h + 2, + 3
                            }
                        asm volatile(
                            "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                            "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                            ::"r"(tcol + (uint32_t)(16 * c)), "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "r"(o[4]), "r"(o[5]),
                              "r"(o[6]), "r"(o[7]), "r"(o[8]), "r"(o[9]), "r"(o[10]), "r"(o[11]), "r"(o[12]), "r"(o[13]),
                              "r"(o[14]), "r"(o[15]) : "memory");
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(kBarAfull + rs));
                }
                ++T;
                rs += 4;
                if (rs >= kRing) {
                    rs -= kRing;
                    ++use;
                }
            }
            if (!ok) break;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kBuMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmCols) : "memory");
    }
    if (tid == 0 && *fail) atomicExch(a.status, 1);
}

// Row codes from the streaming layout: one thread per (slice, tile of 128 rows, quarter, chunk, row).
template <int Q>
__global__ void build_row_codes_kernel(const uint8_t *__restrict__ planes, const uint16_t *__restrict__ meta,
                                       uint8_t *__restrict__ rcodes, uint16_t *__restrict__ rmeta, StreamDims d) {
    const long long tiles = d.np / 128;
    const long long total = (long long)d.slices * tiles * 4 * 4 * 128;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
        const int rowt = (int)(idx % 128);
        const int chunk = (int)((idx / 128) % 4), kp = (int)((idx / 512) % 4);
        const long long st = idx / 2048;                      // slice * tiles + tile
        const int s = (int)(st / tiles);
        const int row = (int)(st % tiles) * 128 + rowt;
        const int oct = row / kOctRows, r = row % kOctRows;
        uint32_t words[4];
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
            const int b = 4 * chunk + wi;                     // source byte of the quarter: channels 8 b .. +7
            uint32_t bytes[Q];
#pragma unroll
            for (int p = 0; p < Q; ++p) bytes[p] = planes[stream_plane_offset(d, s, oct, p, r * 4 + kp, stream_pos_of_src(b, r))];
            uint32_t w = 0;
#pragma unroll
            for (int t = 0; t < 8; ++t) {
                uint32_t code = 0;
#pragma unroll
                for (int p = 0; p < Q; ++p) code |= ((bytes[p] >> t) & 1u) << p;
                w |= code << (4 * t);
            }
            words[wi] = w;
        }
        *(uint4 *)(rcodes + st * kRowCodeTileBytes + (((long long)kp * 4 + chunk) * 128 + rowt) * 16) =
            make_uint4(words[0], words[1], words[2], words[3]);
        if (chunk == 0) {
            uint16_t mv[4] = {0, 0, 0, 0};
#pragma unroll
            for (int p = 0; p < Q; ++p) mv[p] = meta[stream_meta_offset(d, s, oct, p, r * 4 + kp, 0)];
            mv[3] = meta[stream_meta_offset(d, s, oct, Q, r * 4 + kp, 0)];
            *(uint2 *)((uint8_t *)rmeta + st * kRowMetaTileBytes + (kp * 128 + rowt) * 8) =
                make_uint2((uint32_t)mv[0] | ((uint32_t)mv[1] << 16), (uint32_t)mv[2] | ((uint32_t)mv[3] << 16));
        }
    }
}

template <int Q, int NT>
int launch_tmem_inst(const GemvArgs &args, int ctas, cudaStream_t stream) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    HLQ_CUDA(cudaGetDevice(&dev));
    auto kernel = batch_tmem_kernel<Q, NT>;
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_first_use);
        HLQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBuSmem));
        configured[dev & 63].store(true, std::memory_order_release);
    }
    return launch_pdl(kernel, dim3(ctas), dim3(kBuThreads), kBuSmem, stream, args);
}

}  // namespace

// All `m` rows of x of the launch in one pass, as launch_batch_mma (same accumulators, counters and
// walk, a CTA's share cut on tiles of 8 duos); every job must have row codes.
int launch_batch_tmem(int q, int gpw, const GemvArgs &a_in, int ctas, int m, cudaStream_t stream) {
    if (!batch_mma_supported(q, m) || gpw != 1 || !a_in.use_rcodes) return HLQ_ERR_UNSUPPORTED;
    GemvArgs a = a_in;
    a.batch_rows = m;
    a.row_base = 0;
    a.dyn_smem = kBuSmem;
    a.chunk_duos = kChunkDuos;
    a.seg_cost = kChunkSegCost;
    a.unit_align = 8;
    a.total_units = a_in.total_units_chunked;
    if (q == 2) return m <= 8 ? launch_tmem_inst<2, 1>(a, ctas, stream) : launch_tmem_inst<2, 2>(a, ctas, stream);
    return m <= 8 ? launch_tmem_inst<3, 1>(a, ctas, stream) : launch_tmem_inst<3, 2>(a, ctas, stream);
}

int launch_build_row_codes(int q, const uint8_t *planes, const uint16_t *meta, uint8_t *rcodes, uint16_t *rmeta,
                           const StreamDims &d, cudaStream_t stream) {
    if (d.g != 128 || d.np % 128 || (q != 2 && q != 3)) return HLQ_ERR_UNSUPPORTED;
    const long long total = (long long)d.slices * (d.np / 128) * 2048;
    unsigned grid = (unsigned)((total + 255) / 256);
    if (grid > 148u * 64u) grid = 148u * 64u;
    if (q == 2) build_row_codes_kernel<2><<<grid, 256, 0, stream>>>(planes, meta, rcodes, rmeta, d);
    else build_row_codes_kernel<3><<<grid, 256, 0, stream>>>(planes, meta, rcodes, rmeta, d);
    HLQ_CUDA(cudaGetLastError());
    count_launch();
    return HLQ_OK;
}

}  // namespace hlq
