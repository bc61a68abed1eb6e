// Small batches (3..16 rows of activations) over HLQ weights in the streaming layout, sm_100a:
// the weights are streamed ONCE per call, whatever the number of rows.
//
// Replaces, for small m, the reference's batched path
//   C++/ops/src/arm/arm_gemm.cpp:362-387   (GEMM worker: a table per row of x, all rows re-walk the planes)
// A table lookup serves one row of x (two with half2 entries), so the LUT kernel's cost grows
// with the rows.  Here a lane turns its bits into fp16 weights in registers and the rows of x
// share them through the tensor cores:
//
//   * Lane (r, j) of a warp owns, per duo of 16 output rows, the 128 channels of quarter j of the
//     slice for rows r and r + 8 (hlq_layout.h) - exactly the rows and the column pairs lane
//     (group r, thread-in-group j) feeds into the A operand of mma.sync.m16n8k16.  The k index of
//     the instruction is only a label: any assignment of channels to it is right as long as the
//     activations in the B operand follow it.  One instruction therefore takes four channels from
//     each of the four quarters of the slice.
//   * Dequantization is a byte permute: per (row, group) the 2^q possible values z + sum(alpha_p * bit_p)
//     are formed once in fp32, rounded to fp16 and kept as a table of low bytes and a table of
//     high bytes (two registers each).  Masked merges of the plane words give, for every fourth
//     channel, a nibble with the channel's q bits; one prmt per byte table looks up four weights,
//     two more interleave them into half2 pairs.
//   * The byte pairs of the layout are permuted by the row (for the LUT kernel's bank spread);
//     the lanes undo that in registers first, so that all rows of an instruction hold the same
//     channels.
//   * The slice's activations (all rows of x) are brought into shared memory by bulk copies one
//     segment ahead, then rearranged into the order the B fragments want (one 64-bit load per
//     fragment, conflict-free by an XOR of the unit index with the lane's position).
//   * fp32 accumulators of a duo (16 rows x up to 16 rows of x) are added to global accumulators
//     [output row][row of x] with 128-bit reductions; completion counters per block of 32 rows
//     and the finalizing pass are those of the LUT kernel, run by one warp.
//
// What bounds it: the integer pipe.  A sub-partition issues one prmt / lop3 / shf every two cycles,
// and a duo costs each lane about 540 of them (256 table permutes, 160 for the selectors, the
// rest for the layout's permutation, the tables and addressing).  The register-fed
// mma.sync.m16n8k16 takes 8 more cycles of the same sub-partition per instruction on this part
// and does not overlap with the integer work (measured: 8.0 cycles back to back; 12 / 19 / 36
// with 4 / 8 / 16 permutes between two of them), i.e. another 256 or 512 cycles per duo for up
// to 8 or 16 rows of x.  Measured duo rates match that sum (342 and 438 cycles per duo and SM).
// tcgen05 would take the matrix work off the sub-partitions but wants its weight operand in
// shared memory or TMEM, i.e. one more store per dequantized register.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "hlq_batch_dev.cuh"
#include "hlq_gemv_args.cuh"
#include "hlq_gemv_dev.cuh"
#include "hlq_internal.h"

namespace hlq {

namespace {

constexpr int kBmWarps = 15;                 // consumer warps
constexpr int kBmConsumers = kBmWarps * 32;
constexpr int kBmThreads = kBmConsumers + 32;   // + the control warp
constexpr int kBmBarSegDone = 2;             // + slot: consumers arrive, the control warp syncs

// Activations in fragment order: per row of x four quarters of 32 units of 8 bytes.  Rows are
// 1056 bytes apart and quarters 264, so that the 16 lanes of a half-warp (4 rows x 4 quarters,
// same unit) read 16 different 8-byte bank slots.
constexpr uint32_t kBmRowStride = 1056, kBmQuarterStride = 264;
constexpr uint32_t kBmBBytes = 16 * kBmRowStride;    // one buffer: 16 rows of x
constexpr int kBmStageBlocks = 16;                   // blocks of 32 rows whose accumulators are staged at once

// shared memory (bytes from the 1 KB-aligned base)
constexpr uint32_t kBmB = 0;                                   // 2 buffers of fragment-ordered activations
constexpr uint32_t kBmRaw = 2 * kBmBBytes;                     // 2 slots x [16][512] 16-bit activations as they come
constexpr uint32_t kBmStage = kBmRaw + 2 * 16384;              // accumulators of finished blocks (up to 2 KB each)
constexpr int kBmListBlocks = 128;                             // candidates looked at per round of counter updates
constexpr uint32_t kBmList = kBmStage + kBmStageBlocks * 2048; // finished blocks among them
constexpr uint32_t kBmSeg = kBmList + kBmListBlocks * 4;       // 2 x Seg
constexpr uint32_t kBmSegSlot = 192;
constexpr uint32_t kBmMbarDesc = kBmSeg + 2 * kBmSegSlot;
constexpr uint32_t kBmMbarX = kBmMbarDesc + 16;
constexpr uint32_t kBmMbarB = kBmMbarX + 16;
constexpr uint32_t kBmNext = kBmMbarB + 16;                    // 2 ints: next duo of the segment in a slot
constexpr uint32_t kBmFlag = kBmNext + 8;
constexpr uint32_t kBmSmem = kBmFlag + 8 + 1024;               // + slack for the alignment
static_assert(sizeof(Seg) <= kBmSegSlot, "Seg must fit its slot");
static_assert(kBmBBytes % 16 == 0 && kBmRaw % 16 == 0 && kBmStage % 16 == 0, "bulk copies and cp.async want 16-byte alignment");

__device__ __forceinline__ uint2 lds_v2(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// What the consumers hold of one duo: the planes as they are stored, or (CODES) the code words -
// per lane rows r and r + 8, word (c, s) = eight nibbles, nibble i the q bits of channel
// 32 c + 4 i + s of the lane's quarter (planes 0.. from the low bit) - plus the scales and zeros.
template <int Q, int GPW, bool CODES>
struct BatchTile {
    uint4 w[2][CODES ? 4 : Q];      // planes: [oct][plane]; codes: [oct][word c] = {s = 0, 1, 2, 3}
    uint32_t mt[Q + 1][GPW];
};
template <int Q, int GPW, bool CODES>
__device__ __forceinline__ void load_batch_tile(BatchTile<Q, GPW, CODES> &t, const uint8_t *pl, const uint16_t *mp) {
    constexpr int W = CODES ? 4 : Q;
#pragma unroll
    for (int ou = 0; ou < 2; ++ou)
#pragma unroll
        for (int p = 0; p < W; ++p) t.w[ou][p] = ldg_stream_v4(pl + (ou * W + p) * kCellBytes);
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
// One duo (16 rows x the slice's 512 channels) times the rows of x in shared memory.
// `bs`: this lane's base into the fragment-ordered activations (its row of x and quarter).
template <int Q, int GPW, int NT, bool CODES>
__device__ __forceinline__ void mma_tile(const BatchTile<Q, GPW, CODES> &t, uint32_t bs, int r, uint32_t usel,
                                         float (&acc)[4 / NT][NT][4]) {
    constexpr int kChains = 4 / NT;     // independent accumulators per block of 8 rows of x
    uint32_t pw[2][Q][4];
    if constexpr (!CODES) {
#pragma unroll
        for (int ou = 0; ou < 2; ++ou)
#pragma unroll
            for (int p = 0; p < Q; ++p) source_order(t.w[ou][p], r & 4, usel, pw[ou][p]);
    }
    constexpr int kWordsPerGroup = 4 / GPW;
    constexpr int gshift = GPW == 1 ? 3 : (GPW == 2 ? 2 : 1);
    ByteTables<Q> bt[2];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        if (c % kWordsPerGroup == 0) {
            // source group c / kWordsPerGroup sits at positional sub-group (that) ^ (r >> gshift)
            const int u = (c / kWordsPerGroup) ^ ((r >> gshift) & (GPW - 1));
#pragma unroll
            for (int ou = 0; ou < 2; ++ou) build_tables<Q, GPW>(t.mt, ou, u, bt[ou]);
        }
        uint32_t xs[2][4];       // nibble i of xs[oct][s]: the code of channel 4 * i + s of this word
        if constexpr (CODES) {
#pragma unroll
            for (int ou = 0; ou < 2; ++ou) {
                xs[ou][0] = t.w[ou][c].x; xs[ou][1] = t.w[ou][c].y; xs[ou][2] = t.w[ou][c].z; xs[ou][3] = t.w[ou][c].w;
            }
        } else {
            code_words<Q>(pw, c, xs);
        }
#pragma unroll
        for (int s = 0; s < 4; ++s) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                uint32_t a[2][2];
#pragma unroll
                for (int ou = 0; ou < 2; ++ou) {
                    const uint32_t sel = h ? (xs[ou][s] >> 16) : xs[ou][s];
                    const uint32_t lb = prmt(bt[ou].lo[0], bt[ou].lo[1], sel);
                    const uint32_t hb = prmt(bt[ou].hi[0], bt[ou].hi[1], sel);
                    a[ou][0] = prmt(lb, hb, 0x5140u);    // channels 4 * (4h) + s, 4 * (4h + 1) + s
                    a[ou][1] = prmt(lb, hb, 0x7362u);    // channels 4 * (4h + 2) + s, 4 * (4h + 3) + s
                }
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint2 b = lds_v2(bs + (uint32_t)((c * 8 + s * 2 + h) * 8) + nt * 8 * kBmRowStride);
                    // consecutive instructions add into different accumulators: one whose input is
                    // the result of the one before would wait out the tensor pipe's latency
                    mma_16816(acc[(2 * s + h) % kChains][nt], a[0][0], a[1][0], a[0][1], a[1][1], b.x, b.y);
                }
            }
        }
    }
}

// Writes the code words of a weight from its planes: one warp per duo.
template <int Q>
__global__ void __launch_bounds__(256) build_codes_kernel(const uint8_t *__restrict__ planes, uint8_t *__restrict__ codes,
                                                          long long nduos) {
    const int lane = threadIdx.x & 31, r = lane >> 2;
    const long long d = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (d >= nduos) return;
    const uint32_t usel = unpermute_selector(r);
    const uint8_t *pl = planes + d * (2 * Q * kCellBytes) + lane * 16;
    uint32_t pw[2][Q][4];
#pragma unroll
    for (int ou = 0; ou < 2; ++ou)
#pragma unroll
        for (int p = 0; p < Q; ++p) source_order(*(const uint4 *)(pl + (ou * Q + p) * kCellBytes), r & 4, usel, pw[ou][p]);
    uint8_t *out = codes + d * kCodeDuoBytes + lane * 16;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t xs[2][4];
        code_words<Q>(pw, c, xs);
#pragma unroll
        for (int ou = 0; ou < 2; ++ou)
            *(uint4 *)(out + (ou * 4 + c) * kCellBytes) = make_uint4(xs[ou][0], xs[ou][1], xs[ou][2], xs[ou][3]);
    }
}

template <int Q, int GPW, int NT, bool CODES>
__global__ void __launch_bounds__(kBmThreads, 1) batch_mma_kernel(const __grid_constant__ GemvArgs a) {
    static_assert(Q == 2 || Q == 3, "byte tables hold at most eight codes");
    extern __shared__ __align__(1024) unsigned char smem_dyn[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int MT = 8 * NT;                     // rows of x the accumulators hold
    constexpr int kBlockBytes = kBlockRows * MT * 4;
    const int m = a.batch_rows;

    const uint32_t sraw = smem_u32(smem_dyn);
    const uint32_t sbase = (sraw + 1023u) & ~1023u;
    unsigned char *sm = smem_dyn + (sbase - sraw);
    if (sbase + kBmSmem - 1024 > sraw + a.dyn_smem) {
        if (tid == 0) atomicExch(a.status, 2);
        return;
    }
    volatile int *fail = (volatile int *)(sm + kBmFlag);
    const int spin = a.spin_limit;
    Seg *ring = (Seg *)(sm + kBmSeg);
    int *next_duo = (int *)(sm + kBmNext);
    const uint32_t mb_desc = sbase + kBmMbarDesc, mb_x = sbase + kBmMbarX, mb_b = sbase + kBmMbarB;

    pdl_launch_dependents();
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(mb_desc + 8 * i, 1);
            mbar_init(mb_x + 8 * i, 1);
            mbar_init(mb_b + 8 * i, 1);
        }
        mbar_init_fence();
        *fail = 0;
    }
    __syncthreads();

    if (warp == kBmWarps) {
        // ======= control warp: descriptors, activations in fragment order, completion =========
        Walker wk;
        bool waited = false;
        int emitted = 0;          // segments whose descriptor is out
        // descriptor of the next segment into `slot`, and the bulk copies of its activations
        auto emit = [&](int slot) {
            Seg sg;
            int valid;
            const uint16_t *src = walker_next<Q, GPW>(wk, sg, valid);
            if (lane == 0) {
                ring[slot] = sg;
                next_duo[slot] = sg.duo_a + kBmWarps;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(mb_desc + 8 * slot);
            if (sg.live) {
                if (!waited) {
                    pdl_wait();
                    waited = true;
                }
                uint16_t *xs = (uint16_t *)(sm + kBmRaw) + slot * (16 * kSliceK);
                if (valid < kSliceK)
                    for (int rr = 0; rr < m; ++rr)
                        for (int i = valid + lane; i < kSliceK; i += 32) xs[rr * kSliceK + i] = 0;
                __syncwarp();
                if (lane == 0) {
                    fence_proxy_async();
                    const uint32_t bytes = (uint32_t)valid * 2u;
                    mbar_expect_tx(mb_x + 8 * slot, bytes * (uint32_t)m);
                    for (int rr = 0; rr < m; ++rr)
                        tma_bulk_g2s(sbase + kBmRaw + (slot * 16 + rr) * kSliceK * 2, src + (long long)rr * sg.k, bytes,
                                     mb_x + 8 * slot);
                }
            }
            ++emitted;
            return sg.live != 0;
        };
        // The slice's activations, as they came, into the order the B fragments read them:
        // unit (row of x, quarter, word c, s, h) = channels 128 quarter + 32 c + 4 (4 h + e) + s, e = 0..3.
        auto arrange = [&](int slot, int use, int x_dtype) {
            mbar_wait_bounded(mb_x + 8 * slot, (use >> 1) & 1, fail, spin);
            const uint16_t *raw = (const uint16_t *)(sm + kBmRaw) + slot * (16 * kSliceK);
            unsigned char *dst = sm + kBmB + slot * kBmBBytes;
            for (int u = lane; u < MT * 128; u += 32) {
                const int row = u >> 7, un = u & 127;
                const int qtr = un >> 5, c = (un >> 3) & 3, s = (un >> 1) & 3, h = un & 1;
                uint32_t lo = 0u, hi = 0u;
                if (row < m) {
                    const uint16_t *src = raw + row * kSliceK + 128 * qtr + 32 * c + 16 * h + s;
                    uint16_t e[4];
#pragma unroll
                    for (int q2 = 0; q2 < 4; ++q2) {
                        e[q2] = src[4 * q2];
                        if (x_dtype != HLQ_F16) e[q2] = __half_as_ushort(__float2half_rn(x_to_float(e[q2], x_dtype)));
                    }
                    lo = (uint32_t)e[0] | ((uint32_t)e[1] << 16);
                    hi = (uint32_t)e[2] | ((uint32_t)e[3] << 16);
                }
                *(uint2 *)(dst + row * kBmRowStride + qtr * kBmQuarterStride + (un & 31) * 8) = make_uint2(lo, hi);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(mb_b + 8 * slot);      // releases the buffer to the consumers
        };
        walker_init(wk, a, 0);
        {
            const bool l0 = emit(0);
            const bool l1 = emit(1);
            if (l0) arrange(0, 0, ring[0].x_dtype);
            if (l1) arrange(1, 1, ring[1].x_dtype);
        }
        pdl_wait();       // before this warp's first global write
        int *list = (int *)(sm + kBmList);
        for (int i = 0;; ++i) {
            const int slot = i & 1;
            const bool have = mbar_wait_bounded(mb_desc + 8 * slot, (i >> 1) & 1, fail, spin);
            const Seg sg = ring[slot];
            if (!have || !sg.live) break;
            named_bar_sync_dyn(kBmBarSegDone + slot, kBmThreads);      // the consumers are done with it
            const bool live2 = emit(slot);                             // segment i + 2
            // its activations first, then publish: count finished duos per block of 32 rows; the
            // blocks this segment completes are collected (128 candidates at a time), then turned
            // into outputs (and cleared, with their counters, for the next launch) through a
            // staging area, 16 blocks per round trip
            if (live2) arrange(slot, i + 2, ring[slot].x_dtype);
            const int bfirst = sg.duo_a >> 1, blast = (sg.duo_b - 1) >> 1;
            const unsigned total = (unsigned)sg.slices * 2u;
            __threadfence();
            for (int b0 = bfirst; b0 <= blast; b0 += kBmListBlocks) {
                int nlist = 0;
                bool mine[kBmListBlocks / 32];
#pragma unroll
                for (int e = 0; e < kBmListBlocks / 32; ++e) {
                    const int bi = b0 + 32 * e + lane;
                    mine[e] = false;
                    if (bi <= blast) {
                        const int lo = max(sg.duo_a, 2 * bi), hi = min(sg.duo_b, 2 * bi + 2);
                        const unsigned cnt = (unsigned)(hi - lo);
                        mine[e] = atomicAdd(&sg.counters[bi], cnt) + cnt == total;
                    }
                }
#pragma unroll
                for (int e = 0; e < kBmListBlocks / 32; ++e) {
                    const unsigned mask = __ballot_sync(0xffffffffu, mine[e]);
                    if (mine[e]) list[nlist + __popc(mask & ((1u << lane) - 1u))] = b0 + 32 * e + lane;
                    nlist += __popc(mask);
                }
                __syncwarp();
                if (nlist) __threadfence();
                for (int l0 = 0; l0 < nlist; l0 += kBmStageBlocks) {
                    const int nb = min(kBmStageBlocks, nlist - l0);
                    for (int e = 0; e < nb; ++e) {
                        const unsigned char *src = (const unsigned char *)sg.acc + (long long)list[l0 + e] * kBlockBytes;
#pragma unroll
                        for (int c = 0; c < kBlockBytes / 512; ++c)
                            cp_async_16(sbase + kBmStage + e * kBlockBytes + (c * 32 + lane) * 16, src + (c * 32 + lane) * 16);
                    }
                    cp_async_wait_all();
                    __syncwarp();
                    for (int e = 0; e < nb; ++e) {
                        const int blk = list[l0 + e];
                        const int row = blk * kBlockRows + lane;
                        const float4 *sp = (const float4 *)(sm + kBmStage + e * kBlockBytes + lane * (MT * 4));
                        float v[MT];
#pragma unroll
                        for (int qd = 0; qd < MT / 4; ++qd) {
                            const float4 f = sp[qd];
                            v[4 * qd] = f.x; v[4 * qd + 1] = f.y; v[4 * qd + 2] = f.z; v[4 * qd + 3] = f.w;
                        }
                        float4 *ap = (float4 *)((unsigned char *)sg.acc + (long long)blk * kBlockBytes);
#pragma unroll
                        for (int c = 0; c < kBlockBytes / 512; ++c) ap[c * 32 + lane] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (row < sg.n) {
                            const float bias = sg.bias ? __half2float(__ushort_as_half(sg.bias[row])) : 0.f;
#pragma unroll
                            for (int rr = 0; rr < MT; ++rr)
                                if (rr < m) store_y(sg.y, (long long)rr * sg.n + row, v[rr] + bias, sg.y_dtype);
                        }
                        if (lane == 0) sg.counters[blk] = 0;
                    }
                    __syncwarp();
                }
            }
        }
        if (*fail && lane == 0) atomicExch(a.status, 1);
        return;
    }

    // =============================== consumer warps =======================================
    const int r = lane >> 2, j = lane & 3;
    constexpr long long kDuoPlaneBytes = CODES ? kCodeDuoBytes : 2 * Q * kCellBytes;
    constexpr long long kDuoMetaElems = (Q + 1) * 32 * 2 * GPW;
    // B fragments: lane (r, j) reads row of x (r + 8 nt), quarter j
    const uint32_t bs0 = sbase + kBmB + (uint32_t)r * kBmRowStride + (uint32_t)j * kBmQuarterStride;
    const uint32_t usel = unpermute_selector(r);

    BatchTile<Q, GPW, CODES> t0, t1;
    const uint8_t *planes;        // the planes, or the code words
    const uint16_t *meta;
    float *accb;
    int cur, dend;
    auto load_duo = [&](BatchTile<Q, GPW, CODES> &t, int d) {
        load_batch_tile<Q, GPW, CODES>(t, planes + (long long)d * kDuoPlaneBytes, meta + (long long)d * kDuoMetaElems);
    };
    // the next duo of the segment that nobody has taken yet
    auto take = [&](int slot) {
        int d = 0;
        if (lane == 0) d = atomicAdd(next_duo + slot, 1);
        return __shfl_sync(0xffffffffu, d, 0);
    };
    auto open_segment = [&](const Seg &sg) {
        cur = sg.duo_a + warp;
        dend = sg.duo_b;
        planes = (CODES ? sg.codes : sg.planes) - (long long)sg.duo_a * kDuoPlaneBytes + lane * 16;
        meta = sg.meta - (long long)sg.duo_a * kDuoMetaElems + lane * (2 * GPW);
        // reduction target of this lane: even j: row r, odd j: row r + 8; rows of x 4 (j >> 1) ..
        accb = sg.acc + (long long)(r + ((j & 1) ? 8 : 0)) * MT + 4 * (j >> 1);
        if (cur < dend) load_duo(t0, cur);
    };
    {
        const bool have = mbar_wait_bounded(mb_desc, 0, fail, spin);
        if (!have || !ring[0].live) return;
        open_segment(ring[0]);
    }
    auto run_tile = [&](const BatchTile<Q, GPW, CODES> &t, int d, uint32_t bs) {
        float accs[4 / NT][NT][4] = {};
        mma_tile<Q, GPW, NT, CODES>(t, bs, r, usel, accs);
        float acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                acc[nt][e] = accs[0][nt][e];
#pragma unroll
                for (int ch = 1; ch < 4 / NT; ++ch) acc[nt][e] += accs[ch][nt][e];
            }
        // lanes j, j ^ 1 hold rows of x (2j, 2j + 1) of output rows r and r + 8: after the exchange
        // the even lane owns four rows of x of output row r, the odd lane those of row r + 8
        float *dst = accb + (long long)d * (16 * MT);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const bool odd = j & 1;
            const float s0 = odd ? acc[nt][0] : acc[nt][2], s1 = odd ? acc[nt][1] : acc[nt][3];
            const float g0 = __shfl_xor_sync(0xffffffffu, s0, 1), g1 = __shfl_xor_sync(0xffffffffu, s1, 1);
            const float4 v = odd ? make_float4(g0, g1, acc[nt][2], acc[nt][3]) : make_float4(acc[nt][0], acc[nt][1], g0, g1);
            atomicAdd((float4 *)(dst + 8 * nt), v);
        }
    };
    for (int i = 0;; ++i) {
        const int slot = i & 1;
        mbar_wait_bounded(mb_b + 8 * slot, (i >> 1) & 1, fail, spin);      // the activations are arranged
        if (i == 0) pdl_wait();
        const uint32_t bs = bs0 + slot * kBmBBytes;
        // stream: two register tiles, the next duo's loads in flight behind the one in use; duos
        // beyond each warp's first are taken from a counter, so no warp idles at the segment's end
        while (cur < dend) {
            int nxt = take(slot);
            if (nxt < dend) load_duo(t1, nxt);
            run_tile(t0, cur, bs);
            cur = nxt;
            if (cur >= dend) break;
            nxt = take(slot);
            if (nxt < dend) load_duo(t0, nxt);
            run_tile(t1, cur, bs);
            cur = nxt;
        }
        // hand this segment to the control warp, then the first loads of the next one (an
        // arrival waits for the loads its thread has in flight)
        const bool have = mbar_wait_bounded(mb_desc + 8 * (slot ^ 1), ((i + 1) >> 1) & 1, fail, spin);
        named_bar_arrive_dyn(kBmBarSegDone + slot, kBmThreads);
        const Seg &nx = ring[slot ^ 1];
        if (!have || !nx.live) break;
        open_segment(nx);
    }
}

template <int Q, int GPW, int NT, bool CODES>
int launch_inst(const GemvArgs &args, int ctas, cudaStream_t stream) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    HLQ_CUDA(cudaGetDevice(&dev));
    auto kernel = batch_mma_kernel<Q, GPW, NT, CODES>;
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_first_use);
        HLQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBmSmem));
        configured[dev & 63].store(true, std::memory_order_release);
    }
    return launch_pdl(kernel, dim3(ctas), dim3(kBmThreads), kBmSmem, stream, args);
}

}  // namespace

// Two rows of x are cheaper as one pass of the LUT kernel with half2 table entries (0.65 of this
// kernel's time on the Llama-3-8B projection set); from three rows on this kernel wins.
bool batch_mma_supported(int q, int m) { return (q == 2 || q == 3) && m >= 3 && m <= kLutMaxM; }

// All `m` rows of x of the launch in one pass.  The accumulators of a job are [np][8 or 16] fp32
// (rows of x innermost), the counters those of its first row.
int launch_batch_mma(int q, int gpw, const GemvArgs &a_in, int ctas, int m, cudaStream_t stream) {
    if (!batch_mma_supported(q, m)) return HLQ_ERR_UNSUPPORTED;
    GemvArgs a = a_in;
    a.batch_rows = m;
    a.row_base = 0;
    a.dyn_smem = kBmSmem;
    a.chunk_duos = kChunkDuos;
    a.seg_cost = kChunkSegCost;
    a.total_units = a_in.total_units_chunked;
#define HLQ_CASE(QV, GV)                                                                                       \
    if (q == QV && gpw == GV) {                                                                                \
        if (a.use_codes)                                                                                       \
            return m <= 8 ? launch_inst<QV, GV, 1, true>(a, ctas, stream) : launch_inst<QV, GV, 2, true>(a, ctas, stream); \
        return m <= 8 ? launch_inst<QV, GV, 1, false>(a, ctas, stream) : launch_inst<QV, GV, 2, false>(a, ctas, stream);   \
    }
    HLQ_CASE(2, 1) HLQ_CASE(2, 2) HLQ_CASE(2, 4)
    HLQ_CASE(3, 1) HLQ_CASE(3, 2) HLQ_CASE(3, 4)
#undef HLQ_CASE
    return HLQ_ERR_SHAPE;
}

int launch_build_codes(int q, const uint8_t *planes, uint8_t *codes, int slices, int duos, cudaStream_t stream) {
    const long long nduos = (long long)slices * duos;
    if (nduos <= 0) return HLQ_OK;
    const unsigned grid = (unsigned)((nduos + 7) / 8);
    if (q == 2) build_codes_kernel<2><<<grid, 256, 0, stream>>>(planes, codes, nduos);
    else if (q == 3) build_codes_kernel<3><<<grid, 256, 0, stream>>>(planes, codes, nduos);
    else return HLQ_ERR_UNSUPPORTED;
    HLQ_CUDA(cudaGetLastError());
    count_launch();
    return HLQ_OK;
}

}  // namespace hlq
