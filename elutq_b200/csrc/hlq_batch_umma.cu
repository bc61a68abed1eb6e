// Small batches (3..16 rows of activations) over HLQ weights in the streaming layout on the
// tcgen05 tensor cores, sm_100a: the weights are streamed once per call, dequantized in registers
// (hlq_batch_dev.cuh), written to shared memory as the A operand of tcgen05.mma, accumulated in
// tensor memory.
//
// Replaces, for small m, the reference's batched path
//   C++/ops/src/arm/arm_gemm.cpp:362-387   (GEMM worker: a table per row of x, all rows re-walk the planes)
// beside batch_mma_kernel (hlq_batch.cu), whose register-fed mma.sync costs the sub-partitions 8
// cycles per instruction ON TOP of the integer work of the dequantization.  Here the matrix work
// leaves the sub-partitions altogether:
//
//   warps 0..15   dequantizers.  A tile is 128 output rows (8 duos) x one slice of 512 channels;
//                 warp o owns oct o of it (8 rows: lane (r, j) row r, quarter j of the slice, as the
//                 layout gives them).  A lane's 128 weights go out as sixteen 16-byte chunks, one per
//                 (word c, s): the 8 channels 32 c + s + 4 i, i = 0..7.  The k index of the
//                 instruction is only a label, so a chunk is 8 consecutive "k" of a 64-wide K step:
//                 K step 2 j + (c >> 1), chunk ((c & 1) * 4 + s) ^ 2 j (the XOR with 2 j keeps the
//                 four quarters' stores of a row off one bank), in the 128-byte-swizzled K-major
//                 layout.  The tile is written in two halves (c = 0, 1 -> K steps 0, 2, 4, 6;
//                 c = 2, 3 -> 1, 3, 5, 7) of 64 KB each, so that the tensor cores work on one half
//                 while the other is written.
//   warp 21       one thread issues tcgen05.mma (128 x 16 x 16, kind::f16, fp32 accumulation in
//                 tensor memory; two accumulators of 16 columns used alternately) and commits the
//                 halves free / the accumulators full.
//   warps 16..19  epilogue: tcgen05.ld of the tile's 128 x 16 accumulators (one TMEM lane = one
//                 output row), 128-bit reductions into the global accumulators [row][8 or 16 rows
//                 of x].
//   warp 20       control: walks the CTA's share of the launch (chunked walk, hlq_gemv_args.cuh), brings
//                 a slice's rows of x in by bulk copies and rearranges them into the B operand
//                 (K-major, 128-byte swizzle, the same k labels), one segment ahead; completes blocks
//                 of 32 rows as batch_mma_kernel does.
//
// Status: bit-for-bit the same tables and selectors as batch_mma_kernel and the same results, but
// at present SLOWER (8B projection set at w3g128: 1.65 / 1.95 ms for 4 / 16 rows against 1.02 /
// 1.34), so the dispatcher keeps batch_mma_kernel and this kernel runs only when selected
// (hlq_select_batch_kernel).  On 8 layers with 4 rows: the whole 0.43 ms; without the dequantization
// 0.28, without the tcgen05.mma 0.40, without the proxy fences 0.43, and without the stores of the
// dequantized weights 0.28 - the integer work hides completely, what costs is shared memory: an
// fp16 weight is written once (2 bytes) and read once by the tensor cores (2 bytes), 256 KB per
// tile of 128 rows against 128 bytes per clock.  The way out is a weight operand that never
// passes shared memory (tcgen05.st into tensor memory, which wants a lane to own a whole row,
// i.e. another weight layout); not built.
//
// Every wait is an mbarrier wait with a poll limit; the first one that runs out sets the CTA's
// failure flag, after which all waits give up at once and the roles run out of work.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <type_traits>

#include "hlq_batch_dev.cuh"
#include "hlq_gemv_args.cuh"
#include "hlq_gemv_dev.cuh"
#include "hlq_internal.h"

namespace hlq {

namespace {

constexpr int kBuDeqWarps = 16;
constexpr int kBuThreads = 24 * 32;
constexpr int kBuEpiWarp0 = 16, kBuCtlWarp = 20, kBuMmaWarp = 21, kBuFinWarp0 = 22, kBuFinWarps = 2;
constexpr int kBuTileDuos = 8;                       // duos per tile of 128 rows
constexpr int kBuStageBlocks = 8;                    // blocks a completing warp stages at once
constexpr int kBuListMax = 64;                       // blocks one segment can complete (128 duos)

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
constexpr uint32_t kBuA = 0;                                   // 2 halves x 4 K steps x [128 rows][128 bytes]
constexpr uint32_t kBuHalfBytes = 4 * 16384;
constexpr uint32_t kBuB = 2 * kBuHalfBytes;                    // 2 slots x 8 K steps x [16 rows of x][128 bytes]
constexpr uint32_t kBuBSlotBytes = 8 * 2048;
constexpr uint32_t kBuRaw = kBuB + 2 * kBuBSlotBytes;          // [16][512] 16-bit activations as they come
constexpr uint32_t kBuStage = kBuRaw + 16384;                  // per completing warp: accumulators of finished blocks (up to 2 KB each)
constexpr uint32_t kBuList = kBuStage + kBuFinWarps * kBuStageBlocks * 2048;     // 2 x FinJob
constexpr uint32_t kBuListSlot = 512;
constexpr uint32_t kBuSeg = kBuList + 2 * kBuListSlot;         // 2 x Seg
constexpr uint32_t kBuSegSlot = 192;
constexpr uint32_t kBuBars = kBuSeg + 2 * kBuSegSlot;          // mbarriers, 8 bytes each
constexpr uint32_t kBuTmemSlot = kBuBars + 8 * 20;
constexpr uint32_t kBuFlag = kBuTmemSlot + 8;
constexpr uint32_t kBuSmem = kBuFlag + 8 + 1024;               // + slack for the alignment
static_assert(sizeof(Seg) <= kBuSegSlot, "Seg must fit its slot");
static_assert(sizeof(FinJob) <= kBuListSlot, "FinJob must fit its slot");
static_assert(kBuSmem <= 227 * 1024, "shared memory of one CTA");
// mbarrier indices
enum { kBarDesc = 0, kBarXraw = 2, kBarBfull = 3, kBarAfull = 5, kBarAempty = 7, kBarAccFull = 9, kBarAccEmpty = 11,
       kBarSegDone = 13, kBarListFull = 15, kBarListEmpty = 17 };

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
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kIdesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar)
                 : "memory");
}
// asks the L2 for `bytes` (a multiple of 16, from a 16-byte boundary) of global memory; nothing waits for it
__device__ __forceinline__ void bulk_prefetch_l2(const void *src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bu_cp_async_16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void bu_cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// What a dequantizer lane holds of its oct of a tile: the planes (or, CODES, the code words) of its
// row and quarter, and the duo's scales and zeros.
template <int Q, int GPW, bool CODES>
struct OctTile {
    uint4 w[CODES ? 4 : Q];
    uint32_t mt[Q + 1][GPW];
};

template <int Q, int GPW, int NT, bool CODES>
__global__ void __launch_bounds__(kBuThreads, 1) batch_umma_kernel(const __grid_constant__ GemvArgs a) {
    static_assert(Q == 2 || Q == 3, "byte tables hold at most eight codes");
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
            mbar_init(bar(kBarAfull + i), kBuDeqWarps);
            mbar_init(bar(kBarAempty + i), 1);
            mbar_init(bar(kBarAccFull + i), 1);
            mbar_init(bar(kBarAccEmpty + i), 4);
            mbar_init(bar(kBarSegDone + i), 4);
            mbar_init(bar(kBarListFull + i), 1);
            mbar_init(bar(kBarListEmpty + i), kBuFinWarps);
        }
        mbar_init(bar(kBarXraw), 1);
        mbar_init_fence();
        *fail = 0;
    }
    if (warp == kBuMmaWarp) {      // tensor memory: two accumulators of 16 fp32 columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(32)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // tiles of a segment
    auto tiles_of = [](const Seg &sg) { return (sg.duo_b - sg.duo_a + kBuTileDuos - 1) / kBuTileDuos; };

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
            {
                // The segment's weights into the L2, one segment ahead of the dequantizers: a warp
                // keeps only one oct of loads in flight, which covers the L2's latency, not HBM's.
                constexpr uint32_t kDuoBytes = CODES ? kCodeDuoBytes : 2 * Q * kCellBytes;
                constexpr uint32_t kMetaBytes = (Q + 1) * 32 * 2 * GPW * 2;
                const int nd = sg.duo_b - sg.duo_a;
                const uint8_t *pl = CODES ? sg.codes : sg.planes;
                for (int d0 = 8 * lane; d0 < nd; d0 += 8 * 32) {
                    const uint32_t cnt = (uint32_t)min(8, nd - d0);
                    bulk_prefetch_l2(pl + (long long)d0 * kDuoBytes, cnt * kDuoBytes);
                    bulk_prefetch_l2((const uint8_t *)sg.meta + (long long)d0 * kMetaBytes, cnt * kMetaBytes);
                }
            }
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
            // B operand: row of x t, K step ks = 2 j + (c >> 1), chunk ((c & 1) * 4 + s) ^ 2 j holds the
            // channels 128 j + 32 c + s + 4 i, i = 0..7; 128-byte swizzle: chunk ^ (t & 7).  A lane
            // takes one word c of a row and quarter (32 channels) and turns it into its four chunks.
            const int x_dtype = sg.x_dtype;
            unsigned char *dst = sm + kBuB + slot * kBuBSlotBytes;
            for (int u = lane; u < 16 * 16; u += 32) {
                const int t = u >> 4, j = (u >> 2) & 3, c = u & 3;
                uint32_t in[16];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    uint4 w4 = make_uint4(0u, 0u, 0u, 0u);
                    if (t < m) w4 = *(const uint4 *)(xs + t * kSliceK + 128 * j + 32 * c + 8 * q4);
                    in[4 * q4] = w4.x; in[4 * q4 + 1] = w4.y; in[4 * q4 + 2] = w4.z; in[4 * q4 + 3] = w4.w;
                }
                if (x_dtype != HLQ_F16) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const __half2 h2 = __floats2half2_rn(x_to_float((uint16_t)(in[e] & 0xffffu), x_dtype),
                                                             x_to_float((uint16_t)(in[e] >> 16), x_dtype));
                        in[e] = *(const uint32_t *)&h2;
                    }
                }
                const int ks = 2 * j + (c >> 1);
#pragma unroll
                for (int s2 = 0; s2 < 4; ++s2) {
                    // element i of chunk s2 = channel s2 + 4 i = half (s2 & 1) of word 2 i + (s2 >> 1)
                    uint32_t o[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t lo = in[4 * e + (s2 >> 1)], hi = in[4 * e + 2 + (s2 >> 1)];
                        o[e] = (s2 & 1) ? prmt(lo, hi, 0x7632u) : prmt(lo, hi, 0x5410u);
                    }
                    const int chunk = (((c & 1) * 4 + s2) ^ (2 * j)) ^ (t & 7);
                    *(uint4 *)(dst + ks * 2048 + t * 128 + chunk * 16) = make_uint4(o[0], o[1], o[2], o[3]);
                }
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
    } else if (warp >= kBuFinWarp0) {
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
    } else if (warp == kBuMmaWarp) {
        // ============================ tensor-core issue =======================================
        if (lane == 0) {
            int T = 0;            // tiles so far, over all segments
            for (int i = 0;; ++i) {
                const int slot = i & 1;
                const bool have = mbar_wait_bounded(bar(kBarDesc + slot), (i >> 1) & 1, fail, spin);
                if (!have || !ring[slot].live) break;
                const int nt = tiles_of(ring[slot]);
                if (!mbar_wait_bounded(bar(kBarBfull + slot), (i >> 1) & 1, fail, spin)) break;
                for (int t = 0; t < nt; ++t, ++T) {
                    const int ab = T & 1;
                    if (T >= 2 && !mbar_wait_bounded(bar(kBarAccEmpty + ab), ((T >> 1) - 1) & 1, fail, spin)) break;
                    const uint32_t dcol = tmem_base + (uint32_t)(16 * ab);
#pragma unroll 1
                    for (int hf = 0; hf < 2; ++hf) {
                        if (!mbar_wait_bounded(bar(kBarAfull + hf), T & 1, fail, spin)) break;
                        tc_fence_after();
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            const uint64_t adesc = umma_desc(sbase + kBuA + hf * kBuHalfBytes + jj * 16384);
                            const uint64_t bdesc = umma_desc(sbase + kBuB + slot * kBuBSlotBytes + (2 * jj + hf) * 2048);
#pragma unroll
                            for (int kk = 0; kk < 4; ++kk)
                                umma_f16(dcol, adesc + 2 * kk, bdesc + 2 * kk, (hf | jj | kk) ? 1u : 0u);
                        }
                        umma_commit(bar(kBarAempty + hf));
                    }
                    umma_commit(bar(kBarAccFull + ab));
                }
                if (*fail) break;
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
                const uint32_t taddr = tmem_base + ((uint32_t)(32 * q4) << 16) + (uint32_t)(16 * ab);
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                    : "r"(taddr) : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(kBarAccEmpty + ab));
                const int row = (sg.duo_a + t * kBuTileDuos) * 16 + 32 * q4 + lane;     // row of the linear
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
        const int r = lane >> 2, j = lane & 3;
        const int ou = warp & 1, dw = warp >> 1;           // this warp's oct: duo dw of the tile, oct ou of the duo
        constexpr long long kDuoPlaneBytes = CODES ? kCodeDuoBytes : 2 * Q * kCellBytes;
        constexpr int kWords = CODES ? 4 : Q;
        constexpr long long kDuoMetaElems = (Q + 1) * 32 * 2 * GPW;
        constexpr int kWordsPerGroup = 4 / GPW;
        constexpr int gshift = GPW == 1 ? 3 : (GPW == 2 ? 2 : 1);
        const uint32_t usel = unpermute_selector(r);
        // this lane's 16-byte slot in a K step's tile: row 8 warp + r, swizzled chunk
        // (rows are 128 bytes apart and 128-byte aligned: the lane's chunk XOR pattern (2 j ^ r) << 4
        // can sit in the base, a chunk's address is then one XOR with a constant)
        const uint32_t arow = (sbase + kBuA + (uint32_t)j * 16384u + (uint32_t)(8 * warp + r) * 128u) |
                              (uint32_t)(((2 * j) ^ r) & 7) << 4;
        OctTile<Q, GPW, CODES> t0, t1;
        auto load_oct = [&](OctTile<Q, GPW, CODES> &t, const Seg &sg, int duo) {
            const uint8_t *pl = (CODES ? sg.codes : sg.planes) + (long long)(duo - sg.duo_a) * kDuoPlaneBytes +
                                (long long)ou * kWords * kCellBytes + lane * 16;
            const uint16_t *mp = sg.meta + (long long)(duo - sg.duo_a) * kDuoMetaElems + lane * (2 * GPW);
#pragma unroll
            for (int p = 0; p < kWords; ++p) t.w[p] = ldg_stream_v4(pl + p * kCellBytes);
#pragma unroll
            for (int pp = 0; pp <= Q; ++pp) {
                const uint16_t *mm = mp + pp * (32 * 2 * GPW);
                if (GPW == 1) {
                    t.mt[pp][0] = ldg_stream_u32(mm);
                } else if (GPW == 2) {
                    const uint2 v = ldg_stream_v2(mm);
                    t.mt[pp][0] = v.x;
                    t.mt[pp][GPW - 1] = v.y;
                } else {
                    const uint4 v = ldg_stream_v4(mm);
                    t.mt[pp][0] = v.x;
                    t.mt[pp][1 % GPW] = v.y;
                    t.mt[pp][2 % GPW] = v.z;
                    t.mt[pp][3 % GPW] = v.w;
                }
            }
        };
        // one half of the tile (words c = 2 hf, 2 hf + 1) of this lane's row into shared memory
        ByteTables<Q> bt;
        auto write_half = [&](const OctTile<Q, GPW, CODES> &t, const uint32_t (&pw)[Q][4], auto hf_tag) {
            constexpr int hf = decltype(hf_tag)::value;
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
                constexpr int c0 = 2 * hf;
                const int c = c0 + cc;
                if (c % kWordsPerGroup == 0) {
                    const int u = (c / kWordsPerGroup) ^ ((r >> gshift) & (GPW - 1));
                    build_tables<Q, GPW>(t.mt, ou, u, bt);
                }
                uint32_t xs[4];
                if constexpr (CODES) {
                    xs[0] = t.w[c].x; xs[1] = t.w[c].y; xs[2] = t.w[c].z; xs[3] = t.w[c].w;
                } else {
                    const uint32_t w0 = pw[0][c];
                    const uint32_t w1 = __funnelshift_l(pw[1 % Q][c], pw[1 % Q][c], 1);
                    const uint32_t w2 = __funnelshift_l(pw[2 % Q][c], pw[2 % Q][c], 2);
#pragma unroll
                    for (int s = 0; s < 4; ++s) {
                        constexpr uint32_t kOne = 0x11111111u, kTwo = 0x33333333u;
                        const uint32_t m1 = s ? ((kOne << s) | (kOne >> (32 - s))) : kOne;
                        const uint32_t m2 = s ? ((kTwo << s) | (kTwo >> (32 - s))) : kTwo;
                        uint32_t mm = merge_bits(w0, w1, m1);
                        if (Q == 3) mm = merge_bits(mm, w2, m2);
                        if (s) mm = __funnelshift_r(mm, mm, s);
                        xs[s] = mm & (Q == 3 ? 0x77777777u : 0x33333333u);
                    }
                }
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    uint32_t o[4];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t sel = h ? (xs[s] >> 16) : xs[s];
                        const uint32_t lb = prmt(bt.lo[0], bt.lo[1], sel);
                        const uint32_t hb = prmt(bt.hi[0], bt.hi[1], sel);
                        o[2 * h] = prmt(lb, hb, 0x5140u);        // channels s + 4 (4h), s + 4 (4h + 1)
                        o[2 * h + 1] = prmt(lb, hb, 0x7362u);    // channels s + 4 (4h + 2), s + 4 (4h + 3)
                    }
                    asm volatile("st.shared.v4.u32 [%0+%5], {%1, %2, %3, %4};" ::"r"(arow ^ (uint32_t)((cc * 4 + s) << 4)),
                                 "r"(o[0]), "r"(o[1]), "r"(o[2]), "r"(o[3]), "n"(hf * (int)kBuHalfBytes) : "memory");
                }
            }
        };
        int T = 0;
        bool first = true;
        for (int i = 0;; ++i) {
            const int slot = i & 1;
            const bool have = mbar_wait_bounded(bar(kBarDesc + slot), (i >> 1) & 1, fail, spin);
            if (!have || !ring[slot].live) break;
            const Seg &sg = ring[slot];
            const int nt = tiles_of(sg);
            const int dlast = sg.duo_b;
            if (first) {
                pdl_wait();
                first = false;
            }
            int duo = sg.duo_a + dw;
            if (duo < dlast) load_oct(t0, sg, duo);
            bool ok = true;
            // one tile: this oct's rows into both halves of the A operand (a warp whose oct lies
            // past the segment's last duo only takes part in the hand-offs)
            auto tile = [&](const OctTile<Q, GPW, CODES> &cur) {
                const bool mine = duo < dlast;
                uint32_t pw[Q][4];
                if (!CODES && mine) {
#pragma unroll
                    for (int p = 0; p < Q; ++p) source_order(cur.w[p], r & 4, usel, pw[p]);
                }
                auto half = [&](auto hf_tag) {
                    constexpr int hf = decltype(hf_tag)::value;
                    if (T >= 1) ok = mbar_wait_bounded(bar(kBarAempty + hf), (T - 1) & 1, fail, spin);
                    if (!ok) return;
                    if (mine) write_half(cur, pw, hf_tag);
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar(kBarAfull + hf));
                };
                half(std::integral_constant<int, 0>());
                if (ok) half(std::integral_constant<int, 1>());
                ++T;
                duo += kBuTileDuos;
            };
            for (int t = 0; t < nt && ok; t += 2) {
                if (duo + kBuTileDuos < dlast) load_oct(t1, sg, duo + kBuTileDuos);
                tile(t0);
                if (t + 1 >= nt || !ok) break;
                if (duo + kBuTileDuos < dlast) load_oct(t0, sg, duo + kBuTileDuos);
                tile(t1);
            }
            if (!ok) break;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kBuMmaWarp) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32) : "memory");
    }
    if (tid == 0 && *fail) atomicExch(a.status, 1);
}

template <int Q, int GPW, int NT, bool CODES>
int launch_umma_inst(const GemvArgs &args, int ctas, cudaStream_t stream) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    HLQ_CUDA(cudaGetDevice(&dev));
    auto kernel = batch_umma_kernel<Q, GPW, NT, CODES>;
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_first_use);
        HLQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBuSmem));
        configured[dev & 63].store(true, std::memory_order_release);
    }
    return launch_pdl(kernel, dim3(ctas), dim3(kBuThreads), kBuSmem, stream, args);
}

}  // namespace

// All `m` rows of x of the launch in one pass, as launch_batch_mma (same accumulators, counters and walk).
int launch_batch_umma(int q, int gpw, const GemvArgs &a_in, int ctas, int m, cudaStream_t stream) {
    if (!batch_mma_supported(q, m)) return HLQ_ERR_UNSUPPORTED;
    GemvArgs a = a_in;
    a.batch_rows = m;
    a.row_base = 0;
    a.dyn_smem = kBuSmem;
    a.chunk_duos = kChunkDuos;
    a.seg_cost = kChunkSegCost;
    a.total_units = a_in.total_units_chunked;
#define HLQ_CASE(QV, GV)                                                                                            \
    if (q == QV && gpw == GV) {                                                                                     \
        if (a.use_codes)                                                                                            \
            return m <= 8 ? launch_umma_inst<QV, GV, 1, true>(a, ctas, stream) : launch_umma_inst<QV, GV, 2, true>(a, ctas, stream); \
        return m <= 8 ? launch_umma_inst<QV, GV, 1, false>(a, ctas, stream) : launch_umma_inst<QV, GV, 2, false>(a, ctas, stream);   \
    }
    HLQ_CASE(2, 1) HLQ_CASE(2, 2) HLQ_CASE(2, 4)
    HLQ_CASE(3, 1) HLQ_CASE(3, 2) HLQ_CASE(3, 4)
#undef HLQ_CASE
    return HLQ_ERR_SHAPE;
}

}  // namespace hlq
