// Bit-serial LUT GEMV over HLQ weights for decode (m = 1..16), sm_100a.
//
// Replaces the reference's GEMV worker and kernel:
//   C++/ops/src/arm/arm_gemm.cpp:248-308          (group sums, zero term, planes, bias)
//   C++/ops/src/arm/arm_t_mac_kernal.cpp:95-138   (16-entry partial-sum table per 4 channels)
//   C++/ops/src/arm/arm_t_mac_kernal.cpp:364-469  (per-plane table lookups, alpha scaling)
//
// lut8_gemv_kernel (streaming layout, see hlq_layout.h) is a persistent kernel: one CTA per
// SM walks a contiguous range of (job, slice, duo) units, where a job is one linear of a
// group (or the single linear of hlq_linear_forward), a slice is 512 input channels and a
// duo is 16 output rows.  A maximal run of units inside one slice of one job is a SEGMENT.
//
// Per segment the 16 CONSUMER warps
//   1. build, for every 8 activations of the slice, the 256-entry fp32 table of subset sums.
//      Each table is the sum of the two 16-entry tables of its 4-activation halves, so one
//      lookup consumes a whole packed byte (two nibbles of the reference's scheme).  The 64
//      tables of a slice are interleaved so that entry e of every table sits in the same
//      256-byte row: address = base + 256*e + offset(table).  With the table block aligned to
//      64 KB, the address of a lookup is ONE byte-permute (prmt) that drops the packed byte
//      into bits 8..15 of a per-lane base register;
//   2. stream their duos with 128-bit loads through a ring of three register tiles (a lane's
//      16 bytes are one row's 128 channels = one group at g = 128) and per byte do
//      prmt + ld.shared + fadd.  The byte-pair permutation of the layout makes the 32 lanes
//      of every lookup hit 32 different banks;
//   3. scale each plane's group sum by its fp16 alpha, add z * (sum of the group's
//      activations), reduce the four lanes of a row with warp shuffles and add the row's
//      sum for this slice into the row's fp32 accumulator in global memory (red.add.f32);
//   4. issue the first loads of the NEXT segment before handing this one over.
// Four FINALIZER warps run beside them: warp 16 walks the unit range one segment ahead,
// publishes segment descriptors in shared memory and brings each slice's 512 activations in
// with a TMA bulk copy (double buffered); all four then publish finished segments: one
// atomic counter per block of 32 rows counts finished (slice, duo) units, and whoever
// completes a block reads its 32 accumulators, adds the bias, writes y and clears the
// accumulators and the counter for the next launch.  The consumers never wait for this
// completion pass.  The slices of a row are added in the order their CTAs finish, so fp32
// results can differ in the last bit between runs.
//
// lut4_gemv_kernel (exported layout, any group size that is a multiple of 8)
//   The reference's scheme as it stands: a 16-entry table per 4 activations in shared
//   memory, two lookups per packed byte, warp-shuffle reduction per output row.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "hlq_gemv_args.cuh"
#include "hlq_gemv_dev.cuh"
#include "hlq_internal.h"

namespace hlq {

constexpr int kConsumerWarps = 16;
constexpr int kFinalWarps = 4;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kFinalizers = kFinalWarps * 32;
constexpr int kThreads = kConsumers + kFinalizers;
constexpr uint32_t kTableBytes = 65536;
constexpr uint32_t kAuxBytes = 8192;

// named barriers (0 is __syncthreads)
constexpr int kBarConsumers = 1;   // 512 consumer threads
constexpr int kBarSegDone = 2;     // +slot: consumers arrive, finalizers sync (640)
constexpr int kBarFinalizers = 6;  // 128 finalizer threads

// aux region layout (bytes from its start)
constexpr uint32_t kAuxX = 0;          // 2 x 512 16-bit activations
constexpr uint32_t kAuxXsum = 2048;    // up to 16 group sums (fp32)
constexpr uint32_t kAuxMbarDesc = 2112;  // 2 mbarriers
constexpr uint32_t kAuxMbarX = 2128;     // 2 mbarriers
constexpr uint32_t kAuxFlag = 2144;    // int: CTA-wide failure flag
constexpr uint32_t kAuxRed = 2944;     // 16 partial sums of an RMS over a row of x
constexpr uint32_t kAuxSeg = 3072;     // 2 x Seg (<= 192 bytes each)
constexpr uint32_t kAuxSegSlot = 192;
constexpr uint32_t kAuxX2 = 4096;      // two-row passes: 2 slots x 2 rows x 512 activations; one-row
                                       // passes with an input transform: 2 slots x 512 of the second input
constexpr uint32_t kAuxGamma = 6144;   // input transform: 2 slots x 512 RMSNorm weights
constexpr uint32_t kAuxTp = 2560;      // copy of the TpDev of a fused all-reduce (<= 256 bytes)
constexpr uint32_t kAuxXsum2 = 2816;   // two-row passes: 2 x 16 group sums
static_assert(sizeof(TpDev) <= 256, "TpDev must fit its slot");
static_assert(sizeof(Seg) <= kAuxSegSlot, "Seg must fit its slot");
static_assert(kAuxGamma + 2048 <= kAuxBytes, "aux area");

// R = rows of x one pass serves: 1, or 2 with half2 table entries {row, row + 1}.
// XOP: the instantiation that applies the jobs' input transforms (one-row passes only), kept
// apart so that the plain kernel does not carry its registers.
template <int Q, int GPW, int R, bool XOP>
__global__ void __launch_bounds__(kThreads, 1) lut8_gemv_kernel(const __grid_constant__ GemvArgs a) {
    static_assert(R == 1 || R == 2, "rows per pass");
    static_assert(!XOP || R == 1, "input transforms run in one-row passes");
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int mrow = a.row_base + blockIdx.y * R;
    constexpr uint32_t kX = R == 2 ? kAuxX2 : kAuxX;          // activation slices: [slot][row][512]

    // The table block must start on a 64 KB boundary of the shared window.
    const uint32_t sbase = smem_u32(smem_raw);
    const uint32_t tbl = (sbase + 0xffffu) & ~0xffffu;
    const uint32_t aux_u32 = (tbl - sbase >= kAuxBytes) ? sbase : tbl + kTableBytes;
    if (tbl + kTableBytes > sbase + a.dyn_smem || aux_u32 + kAuxBytes > sbase + a.dyn_smem) {
        if (tid == 0) atomicExch(a.status, 2);
        return;
    }
    unsigned char *aux = smem_raw + (aux_u32 - sbase);
    float *xsum = (float *)(aux + (R == 2 ? kAuxXsum2 : kAuxXsum));    // [row][16]
    volatile int *fail = (volatile int *)(aux + kAuxFlag);
    const int spin = a.spin_limit;
    Seg *ring = (Seg *)(aux + kAuxSeg);
    const uint32_t mb_desc = aux_u32 + kAuxMbarDesc, mb_x = aux_u32 + kAuxMbarX;

    pdl_launch_dependents();
    if (tid == 0) {
        mbar_init(mb_desc, 1);
        mbar_init(mb_desc + 8, 1);
        mbar_init(mb_x, 1);
        mbar_init(mb_x + 8, 1);
        mbar_init_fence();
        *fail = 0;
    }
    __syncthreads();

    if (warp >= kConsumerWarps) {
        // =========================== finalizer warps ======================================
        const int fw = warp - kConsumerWarps, ftid = tid - kConsumers;
        Walker wk;
        bool waited = false;
        auto emit = [&](int slot) {   // control warp only
            Seg sg;
            int valid;
            const uint16_t *src = walker_next<Q, GPW>(wk, sg, valid);
            if (lane == 0) ring[slot] = sg;
            __syncwarp();
            if (lane == 0) mbar_arrive(mb_desc + 8 * slot);
            if (sg.live) {
                if (!waited) {
                    pdl_wait();
                    waited = true;
                }
                uint16_t *xs = (uint16_t *)(aux + kX) + slot * (R * kSliceK);
                for (int rr = 0; rr < R; ++rr)
                    for (int i = valid + lane; i < kSliceK; i += 32) xs[rr * kSliceK + i] = 0;
                __syncwarp();
                // input transform (one-row passes): the slice of the second input and of gamma
                const Job *jb = sg.jb;
                const int xop = XOP ? jb->xop : 0;
                const uint16_t *src2 = nullptr, *srcg = nullptr;
                if (xop) {
                    uint16_t *xs2 = (uint16_t *)(aux + kAuxX2) + slot * kSliceK;
                    uint16_t *gs = (uint16_t *)(aux + kAuxGamma) + slot * kSliceK;
                    const long long off = (long long)sg.mrow * sg.k + (long long)sg.slice * kSliceK;
                    if (jb->x2) src2 = (const uint16_t *)jb->x2 + off;
                    if (xop == HLQ_INPUT_ADD_RMSNORM) srcg = jb->gamma + (long long)sg.slice * kSliceK;
                    for (int i = (src2 ? valid : 0) + lane; i < kSliceK; i += 32) xs2[i] = 0;
                    for (int i = (srcg ? valid : 0) + lane; i < kSliceK; i += 32) gs[i] = 0;
                }
                __syncwarp();
                if (lane == 0) {
                    fence_proxy_async();
                    const uint32_t bytes = (uint32_t)valid * 2u;
                    mbar_expect_tx(mb_x + 8 * slot, bytes * (R + (src2 ? 1 : 0) + (srcg ? 1 : 0)));
                    for (int rr = 0; rr < R; ++rr)
                        tma_bulk_g2s(aux_u32 + kX + (slot * R + rr) * kSliceK * 2, src + (long long)rr * sg.k, bytes,
                                     mb_x + 8 * slot);
                    if (src2) tma_bulk_g2s(aux_u32 + kAuxX2 + slot * kSliceK * 2, src2, bytes, mb_x + 8 * slot);
                    if (srcg) tma_bulk_g2s(aux_u32 + kAuxGamma + slot * kSliceK * 2, srcg, bytes, mb_x + 8 * slot);
                }
            }
        };
        if (fw == 0) {
            walker_init(wk, a, mrow);
            emit(0);
            emit(1);
        }
        pdl_wait();       // before this warp's first global write (and before reading `seq`)
        // fused all-reduce: this launch's number; its parity picks the half of the peer buffers
        // (the descriptor is copied to shared memory once: it is read for every block)
        const TpDev *tp = nullptr;
        unsigned epoch = 0, par = 0;
        Seg last_sg;
        last_sg.live = 0;
        if (a.tp) {
            // the second phase needs the (single) job's output even in a CTA whose unit range
            // holds no duo
            const Job &jb = a.single;
            last_sg.live = 1;
            last_sg.y = jb.y;
            last_sg.y_base = (long long)mrow * jb.n;
            last_sg.n = jb.n;
            last_sg.y_dtype = jb.y_dtype;
            last_sg.mrow = mrow;
            last_sg.blocks = jb.blocks;
            uint32_t *dst = (uint32_t *)(aux + kAuxTp);
            const uint32_t *src = (const uint32_t *)a.tp;
            for (int i = ftid; i < (int)(sizeof(TpDev) / 4); i += kFinalizers) dst[i] = __ldg(src + i);
            named_bar_sync<kBarFinalizers, kFinalizers>();
            tp = (const TpDev *)(aux + kAuxTp);
            epoch = ldcg_u32(tp->seq) + 1u;
            par = epoch & 1u;
        }
        for (int i = 0;; ++i) {
            const int slot = i & 1;
            const bool have = mbar_wait_bounded(mb_desc + 8 * slot, (i >> 1) & 1, fail, spin);
            const Seg sg = ring[slot];
            if (!have || !sg.live) break;     // no descriptor: nothing may be read from the ring slot
            last_sg = sg;
            named_bar_sync_dyn(kBarSegDone + slot, kThreads);      // consumers are done with it
            named_bar_sync<kBarFinalizers, kFinalizers>();         // every finalizer holds its copy
            if (fw == 0) emit(slot);                               // segment i + 2
            // publish: count finished duos per 32-row block; whoever completes a block sums it
            const int bfirst = sg.duo_a >> 1, blast = (sg.duo_b - 1) >> 1;
            const unsigned total = (unsigned)sg.slices * 2u;
            constexpr int kPub = 4;      // counter updates a thread keeps in flight
            for (int b0 = bfirst; b0 <= blast; b0 += kFinalizers * kPub) {
                unsigned minebits = 0;
                if (b0 + ftid <= blast) __threadfence();
#pragma unroll
                for (int i = 0; i < kPub; ++i) {
                    const int bi = b0 + i * kFinalizers + ftid;
                    if (bi <= blast) {
                        const int lo = max(sg.duo_a, 2 * bi), hi = min(sg.duo_b, 2 * bi + 2);
                        const unsigned cnt = (unsigned)(hi - lo);
                        const unsigned old = atomicAdd(&sg.counters[bi], cnt);
                        minebits |= (old + cnt == total ? 1u : 0u) << i;
                    }
                }
#pragma unroll 1
                for (int i = 0; i < kPub; ++i) {
                const int blk = b0 + i * kFinalizers + ftid;
                unsigned mask = __ballot_sync(0xffffffffu, (minebits >> i) & 1u);
                if (mask) __threadfence();
                // lane = row of a finished block; several blocks per round trip
                while (mask) {
                    float v[8], v2[R == 2 ? 8 : 1];
                    int rows[8];
                    unsigned mm = mask;
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        rows[b] = -1;
                        if (mm) {
                            const int src_lane = __ffs(mm) - 1;
                            mm &= mm - 1;
                            rows[b] = __shfl_sync(0xffffffffu, blk, src_lane) * kBlockRows + lane;
                            v[b] = ldcg_f32(sg.acc + rows[b]);
                            if constexpr (R == 2) v2[b] = ldcg_f32(sg.acc + sg.np + rows[b]);
                        }
                    }
#pragma unroll
                    for (int b = 0; b < 8; ++b) {
                        if (rows[b] >= 0) {
                            sg.acc[rows[b]] = 0.f;
                            float o = v[b];
                            if (sg.bias && rows[b] < sg.n) o += __half2float(__ushort_as_half(sg.bias[rows[b]]));
                            if constexpr (R == 2) {       // the second row of x of this pass
                                sg.acc[sg.np + rows[b]] = 0.f;
                                float o2 = v2[b];
                                if (sg.bias && rows[b] < sg.n) o2 += __half2float(__ushort_as_half(sg.bias[rows[b]]));
                                if (rows[b] < sg.n) store_y(sg.y, sg.y_base + sg.n + rows[b], o2, sg.y_dtype);
                            }
                            if (!tp) {
                                if (rows[b] < sg.n) store_y(sg.y, sg.y_base + rows[b], o, sg.y_dtype);
                            } else {
                                // push this rank's sum of the block to every rank (itself included)
                                const long long slot_row =
                                    (((long long)par * tp->world + tp->rank) * tp->max_m + sg.mrow) * tp->np_cap + rows[b];
                                for (int p = 0; p < tp->world; ++p)
                                    st_relaxed_sys_b64(tp->recv[p] + slot_row, __float_as_uint(o), epoch);
                            }
                            if (lane == 0) sg.counters[rows[b] / kBlockRows] = 0;
                        }
                    }
                    mask = mm;
                }
                }
            }
        }
        if (tp && last_sg.live) {
            // Second phase of the fused all-reduce.  Pushing never waits; summing is split
            // statically over the CTAs: poll every rank's slot of a row until it carries this
            // launch's number, add the ranks' sums in rank order, write y.
            const Seg &sg = last_sg;
            const int nwarps = gridDim.x * kFinalWarps;
            for (int blk = blockIdx.x * kFinalWarps + fw; blk < sg.blocks; blk += nwarps) {
                const int row = blk * kBlockRows + lane;
                float sum = 0.f;
                bool ok = true;
                for (int src = 0; src < tp->world; ++src) {
                    const unsigned long long *slot =
                        tp->recv[tp->rank] + (((long long)par * tp->world + src) * tp->max_m + sg.mrow) * tp->np_cap + row;
                    unsigned long long v = ld_relaxed_sys_b64(slot);
                    // a peer that never arrives: the first wait that runs out ends all later ones
                    const int lim = *fail ? 0 : spin;
                    for (int it = 0; it < lim && (uint32_t)(v >> 32) != epoch; ++it) {
                        v = ld_relaxed_sys_b64(slot);
                        if ((it & 255) == 255 && *fail) break;
                    }
                    ok = ok && ((uint32_t)(v >> 32) == epoch);
                    sum += __uint_as_float((uint32_t)v);
                }
                if (!ok) *fail = 1;
                if (row < sg.n) store_y(sg.y, sg.y_base + row, sum, sg.y_dtype);
                __syncwarp();
                if (lane == 0) {
                    const unsigned old = atomicAdd(tp->done, 1u);
                    if (old + 1u == (unsigned)sg.blocks * gridDim.y) {     // last block of the launch
                        *tp->done = 0u;
                        __threadfence();
                        *tp->seq = epoch;
                    }
                }
            }
        }
        if (*fail && ftid == 0) atomicExch(a.status, 1);
        return;
    }

    // =============================== consumer warps =======================================
    const int r = lane >> 2, j = lane & 3;
    uint32_t rt[8];   // per-lane lookup bases: bank 8*j + (t ^ r) of the table row
#pragma unroll
    for (int t = 0; t < 8; ++t) rt[t] = tbl + 4u * (8u * j + (uint32_t)(t ^ r));
    constexpr int gshift = GPW == 1 ? 3 : (GPW == 2 ? 2 : 1);
    constexpr long long kDuoPlaneBytes = 2 * Q * kCellBytes;
    constexpr long long kDuoMetaElems = (Q + 1) * 32 * 2 * GPW;

    // Register tiles in flight: three where a tile is small enough, else two.
    constexpr int kRing = (8 * Q + (Q + 1) * GPW < 22) ? 3 : 2;
    Tile<Q, GPW> t0, t1, t2;
    // running state of the current segment
    const uint8_t *pl;
    const uint16_t *mp;
    float *prow;
    int d, dend, x_dtype, acc_stride = 0;
    // input transform of the current segment's job
    const Job *cur_job = nullptr, *rms_job = nullptr;
    int cur_slice = 0, cur_xop = 0, cur_k = 0;
    bool cur_first = false;            // the segment starts its slice: it writes res_out
    float inv_rms = 0.f;

    auto open_segment = [&](const Seg &sg) {
        d = sg.duo_a + warp;
        dend = sg.duo_b;
        x_dtype = sg.x_dtype;
        acc_stride = sg.np;
        if (XOP) {
            cur_job = sg.jb;
            cur_slice = sg.slice;
            cur_k = sg.k;
            cur_first = sg.duo_a == 0;
        }
        cur_xop = XOP ? sg.jb->xop : 0;
        pl = sg.planes + (long long)warp * kDuoPlaneBytes + lane * 16;
        mp = sg.meta + (long long)warp * kDuoMetaElems + lane * (2 * GPW);
        prow = sg.acc + (long long)d * 16 + r;
        if (d < dend) load_tile<Q, GPW>(t0, pl, mp);
        if (kRing == 3 && d + kConsumerWarps < dend)
            load_tile<Q, GPW>(t1, pl + kConsumerWarps * kDuoPlaneBytes, mp + kConsumerWarps * kDuoMetaElems);
    };

    {
        const bool have = mbar_wait_bounded(mb_desc, 0, fail, spin);
        const Seg sg = ring[0];
        if (!have || !sg.live) return;
        open_segment(sg);
    }
    for (int i = 0;; ++i) {
        const int slot = i & 1;
        named_bar_sync<kBarConsumers, kConsumers>();     // everyone is done with the old table
        if (i == 0) pdl_wait();   // orders this thread's reads and writes after the previous grid
        if (XOP && cur_xop == HLQ_INPUT_ADD_RMSNORM && cur_job != rms_job) {
            // 1 / rms of the whole row t = x + x2, once per job and CTA (the rows sit in L2)
            const uint4 *xr = (const uint4 *)((const uint16_t *)cur_job->x + (long long)mrow * cur_k);
            const uint4 *x2r = cur_job->x2 ? (const uint4 *)((const uint16_t *)cur_job->x2 + (long long)mrow * cur_k)
                                           : nullptr;
            float ss = 0.f;
            for (int v = tid; v < cur_k / 8; v += kConsumers) {
                const uint4 av = xr[v];
                uint4 bv = make_uint4(0u, 0u, 0u, 0u);
                if (x2r) bv = x2r[v];
                const __half2 *ah = (const __half2 *)&av, *bh = (const __half2 *)&bv;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 fa = __half22float2(ah[e]), fb = __half22float2(bh[e]);
                    const float t0 = fa.x + fb.x, t1 = fa.y + fb.y;
                    ss += t0 * t0 + t1 * t1;
                }
            }
#pragma unroll
            for (int dd = 16; dd; dd >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, dd);
            float *red = (float *)(aux + kAuxRed);
            if (lane == 0) red[warp] = ss;
            named_bar_sync<kBarConsumers, kConsumers>();
            float tot = 0.f;
#pragma unroll
            for (int w2 = 0; w2 < kConsumerWarps; ++w2) tot += red[w2];
            inv_rms = 1.0f / sqrtf(tot / (float)cur_k + cur_job->eps);
            rms_job = cur_job;
            named_bar_sync<kBarConsumers, kConsumers>();     // red[] may be rewritten by the next job
        }
        mbar_wait_bounded(mb_x + 8 * slot, (i >> 1) & 1, fail, spin);
        const uint16_t *xs = (const uint16_t *)(aux + kX) + slot * (R * kSliceK);
        // group sums (warps 0..R-1) and the 64 tables of 256 subset sums (all consumer warps)
        const uint16_t *xs2 = (const uint16_t *)(aux + kAuxX2) + slot * kSliceK;     // input transform only
        const uint16_t *gs = (const uint16_t *)(aux + kAuxGamma) + slot * kSliceK;
        // transformed activation: the value the tables are built from (rounded to fp16 like
        // the tensor the unfused kernels would have written)
        auto x_eff = [&](float xv, int ch) {
            if (!XOP || cur_xop == 0) return xv;
            const float sv = __half2float(__ushort_as_half(xs2[ch]));
            if (cur_xop == HLQ_INPUT_GATED_SILU)
                return __half2float(__float2half_rn(sv * (xv / (1.0f + expf(-xv)))));
            const float t16 = __half2float(__float2half_rn(xv + sv));
            return __half2float(__float2half_rn(t16 * __half2float(__ushort_as_half(gs[ch])) * inv_rms));
        };
        if (warp < R) {
            float part = 0.f;
#pragma unroll
            for (int q2 = 0; q2 < 16; ++q2)
                part += x_eff(x_to_float(xs[warp * kSliceK + lane * 16 + q2], x_dtype), lane * 16 + q2);
            constexpr int lanes_per_group = 8 >> (3 - gshift);   // g / 16 lanes: 8, 4 or 2
#pragma unroll
            for (int dd = 1; dd < lanes_per_group; dd <<= 1) part += __shfl_xor_sync(0xffffffffu, part, dd);
            if ((lane & (lanes_per_group - 1)) == 0) xsum[warp * 16 + lane / lanes_per_group] = part;
        }
        {
            const int h = warp & 1, ehi = warp >> 1;   // bank-row, top three index bits
            const int c = 16 * (lane >> 3) + 2 * (lane & 7) + h;
            const uint32_t dst = tbl + (uint32_t)ehi * (32u * 256u) + 4u * lane + 128u * h;
            uint32_t packed[R == 2 ? 32 : 1];    // two-row passes: row 0's entries as fp16 bits
#pragma unroll
            for (int rr = 0; rr < R; ++rr) {
                const uint4 raw = *(const uint4 *)(xs + rr * kSliceK + 8 * c);
                const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w};
                float xv[8];
#pragma unroll
                for (int q2 = 0; q2 < 4; ++q2) {
                    xv[2 * q2] = x_to_float((uint16_t)(rw[q2] & 0xffffu), x_dtype);
                    xv[2 * q2 + 1] = x_to_float((uint16_t)(rw[q2] >> 16), x_dtype);
                }
                if (XOP && cur_xop) {
                    if (cur_xop == HLQ_INPUT_ADD_RMSNORM && ehi == 0 && cur_first && cur_job->res_out &&
                        cur_slice * kSliceK + 8 * c < cur_k) {
                        // the residual stream's new value: written once per slice, by the
                        // segment that starts it
                        const uint4 sraw = *(const uint4 *)(xs2 + 8 * c);
                        const __half2 *xh = (const __half2 *)&raw, *sh = (const __half2 *)&sraw;
                        uint4 o;
                        __half2 *oh = (__half2 *)&o;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 fa = __half22float2(xh[e]), fb = __half22float2(sh[e]);
                            oh[e] = __floats2half2_rn(fa.x + fb.x, fa.y + fb.y);
                        }
                        *(uint4 *)(cur_job->res_out + (long long)mrow * cur_k + cur_slice * kSliceK + 8 * c) = o;
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e) xv[e] = x_eff(xv[e], 8 * c + e);
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
                if constexpr (R == 1) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) sts_f32(dst + (uint32_t)e * 256u, tv[e]);
                } else if (rr == 0) {
#pragma unroll
                    for (int e = 0; e < 32; ++e) packed[e] = __half_as_ushort(__float2half_rn(tv[e]));
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e)
                        sts_u32(dst + (uint32_t)e * 256u,
                                packed[e] | ((uint32_t)__half_as_ushort(__float2half_rn(tv[e])) << 16));
                }
            }
        }
        named_bar_sync<kBarConsumers, kConsumers>();
        asm volatile("" ::: "memory");

        float xsu[GPW], xsu1[GPW];
#pragma unroll
        for (int uu = 0; uu < GPW; ++uu) {
            xsu[uu] = xsum[GPW * j + (uu ^ (r >> gshift))];
            xsu1[uu] = R == 2 ? xsum[16 + GPW * j + (uu ^ (r >> gshift))] : 0.f;
        }
        auto compute = [&](const Tile<Q, GPW> &t, float *row) {
            if constexpr (R == 2)
                compute_tile2<Q, GPW>(t, rt, xsu, xsu1, row, acc_stride, lane);
            else
                compute_tile<Q, GPW>(t, rt, xsu, row, lane);
        };

        // stream: ring of three register tiles, two loads in flight behind the one in use
        constexpr long long kStepP = kConsumerWarps * kDuoPlaneBytes;
        constexpr long long kStepM = kConsumerWarps * kDuoMetaElems;
        constexpr int kStepRow = kConsumerWarps * 16;
        if (kRing == 3) {
            while (d < dend) {
                if (d + 2 * kConsumerWarps < dend) load_tile<Q, GPW>(t2, pl + 2 * kStepP, mp + 2 * kStepM);
                compute(t0, prow);
                d += kConsumerWarps;
                if (d >= dend) break;
                if (d + 2 * kConsumerWarps < dend) load_tile<Q, GPW>(t0, pl + 3 * kStepP, mp + 3 * kStepM);
                compute(t1, prow + kStepRow);
                d += kConsumerWarps;
                if (d >= dend) break;
                if (d + 2 * kConsumerWarps < dend) load_tile<Q, GPW>(t1, pl + 4 * kStepP, mp + 4 * kStepM);
                compute(t2, prow + 2 * kStepRow);
                d += kConsumerWarps;
                pl += 3 * kStepP;
                mp += 3 * kStepM;
                prow += 3 * kStepRow;
            }
        } else {
            while (d < dend) {
                if (d + kConsumerWarps < dend) load_tile<Q, GPW>(t1, pl + kStepP, mp + kStepM);
                compute(t0, prow);
                d += kConsumerWarps;
                if (d >= dend) break;
                if (d + kConsumerWarps < dend) load_tile<Q, GPW>(t0, pl + 2 * kStepP, mp + 2 * kStepM);
                compute(t1, prow + kStepRow);
                d += kConsumerWarps;
                pl += 2 * kStepP;
                mp += 2 * kStepM;
                prow += 2 * kStepRow;
            }
        }

        // first loads of the next segment, then hand this one to the finalizers
        const bool have = mbar_wait_bounded(mb_desc + 8 * (slot ^ 1), ((i + 1) >> 1) & 1, fail, spin);
        const Seg nx = ring[slot ^ 1];
        const bool more = have && nx.live;
        if (more) open_segment(nx);
        named_bar_arrive_dyn(kBarSegDone + slot, kThreads);
        if (!more) break;
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
        mbar_init_fence();
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
        mbar_wait_bounded(mbar, phase, (volatile int *)&fail, kDefaultSpinLimit);
        phase ^= 1u;
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
// scratch of the LUT GEMV alone: header, counters, accumulators for up to 16 rows of x
// rows of accumulators a launch of m rows of x needs: the small-batch kernel keeps 8 or 16 per output row
static int acc_rows(int m) { return m < 2 ? m : (m + 7) / 8 * 8; }

static size_t lut_scratch_bytes(int m, const StreamDims &d) {
    const int mm = m < kLutMaxM ? m : kLutMaxM;
    size_t counters = ((size_t)mm * d.blocks * sizeof(unsigned) + 255) / 256 * 256;
    size_t partial = (size_t)acc_rows(mm) * d.np * sizeof(float);
    return kWsHeader + counters + partial;
}

// Where the tensor-core GEMM may put its fp16 copy of bf16 activations: behind everything a LUT
// launch of any number of rows keeps in the workspace (counters and accumulators that are zero
// between calls), so that one workspace serves prefill and decode calls in any order.
size_t gemm_scratch_offset(const StreamDims &d) { return (lut_scratch_bytes(kLutMaxM, d) + 255) / 256 * 256; }

// ... and behind that copy the fp32 slabs [m][n] of a GEMM whose K is split (at most kGemmSplitMaxM rows of x).
size_t gemm_acc_offset(int m, const StreamDims &d) {
    return gemm_scratch_offset(d) + ((size_t)m * d.k * 2 + 255) / 256 * 256;
}

size_t workspace_bytes_for(int m, const StreamDims &d) {
    size_t need = lut_scratch_bytes(m, d);
    if (m > kLutMaxM) {
        need = gemm_acc_offset(m, d);
        // slabs for a split K: only problems of fewer tiles (256 rows each) than a B200 has SM pairs
        // split, and only calls of at most kGemmSplitMaxM rows; counted for every m above 16 so that
        // the size grows with m (a workspace for m rows serves every call with fewer)
        if ((d.n + 255) / 256 < 74) {
            const size_t slab = (size_t)(m < kGemmSplitMaxM ? m : kGemmSplitMaxM) * d.n * sizeof(float);
            need += 8 * slab < kGemmSlabBytes ? 8 * slab : kGemmSlabBytes;
        }
    }
    return need;
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

static DeviceInfo g_dev[64];
std::mutex g_first_use;
std::atomic<int> g_batch_kernel{0};

int device_info(int device, DeviceInfo **out) {
    if (device < 0 || device >= 64) return HLQ_ERR_INVALID_ARGUMENT;
    DeviceInfo &d = g_dev[device];
    if (!d.ok.load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_first_use);
        if (!d.ok.load(std::memory_order_relaxed)) {
            int major = 0;
            HLQ_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
            if (major != 10) return HLQ_ERR_NO_DEVICE;
            HLQ_CUDA(cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, device));
            HLQ_CUDA(cudaDeviceGetAttribute(&d.max_dyn_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin,
                                            device));
            d.ok.store(true, std::memory_order_release);
        }
    }
    *out = &d;
    return HLQ_OK;
}

// dynamic shared memory that always contains a 64 KB-aligned 64 KB block plus the aux area,
// wherever the window starts: 64 KB of slack, the table, the aux area.
constexpr uint32_t kLut8DynSmem = 65536 - 1024 + kTableBytes + kAuxBytes;

template <int Q, int GPW, int R, bool XOP>
static int launch_lut8_inst(const GemvArgs &args, dim3 grid, cudaStream_t stream) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    HLQ_CUDA(cudaGetDevice(&dev));
    auto kernel = lut8_gemv_kernel<Q, GPW, R, XOP>;
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(g_first_use);
        HLQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)kLut8DynSmem));
        configured[dev & 63].store(true, std::memory_order_release);
    }
    return launch_pdl(kernel, grid, dim3(kThreads), kLut8DynSmem, stream, args);
}

template <int R, bool XOP>
static int launch_lut8_rows(int q, int gpw, const GemvArgs &a, dim3 grid, cudaStream_t stream) {
#define HLQ_CASE(QV, GV) \
    if (q == QV && gpw == GV) return launch_lut8_inst<QV, GV, R, XOP>(a, grid, stream);
    HLQ_CASE(1, 1) HLQ_CASE(1, 2) HLQ_CASE(1, 4)
    HLQ_CASE(2, 1) HLQ_CASE(2, 2) HLQ_CASE(2, 4)
    HLQ_CASE(3, 1) HLQ_CASE(3, 2) HLQ_CASE(3, 4)
    HLQ_CASE(4, 1) HLQ_CASE(4, 2) HLQ_CASE(4, 4)
#undef HLQ_CASE
    return HLQ_ERR_SHAPE;
}


// grid.y = rows of x.  Two or more rows go through passes of two rows each (half2 table
// entries: one lookup serves both) plus a single-row pass for an odd last row.  The table
// entries of such a pass are rounded to fp16 (2^-11, as the reference's tables are), which is
// below the rounding of a 16-bit output; fp32 outputs therefore keep one row per pass and
// fp32 entries, and so does the fused all-reduce.
//
// Plain launches of 3 <= m <= 16 rows at q = 2 or 3 with 16-bit outputs go to the small-batch kernel
// instead (hlq_batch.cu: one pass over the weights for all rows; its weights are rounded to fp16,
// which is below the rounding of a 16-bit output but not of an fp32 one), unless `lut_only` (a
// weight whose extra bit-plane has already been added into accumulators of the LUT kernel's layout).
static int launch_lut8_any(int q, int gpw, const GemvArgs &a_in, dim3 grid, cudaStream_t stream,
                           bool lut_only = false) {
    const int m = (int)grid.y;
    GemvArgs a = a_in;
    a.row_base = 0;
    if (a.one_row_passes) return launch_lut8_rows<1, true>(q, gpw, a, grid, stream);
    if (!lut_only && !a.tp && !a.y_is_f32 && batch_mma_supported(q, m)) {
        // by measurement: the mma.sync kernel is the faster of the two at every m <= 16 (hlq_batch_umma.cu)
        const int which = g_batch_kernel.load(std::memory_order_relaxed);
        if (which == 3 && a.use_rcodes && gpw == 1) return launch_batch_tmem(q, gpw, a, (int)grid.x, m, stream);
        if (which == 2) return launch_batch_umma(q, gpw, a, (int)grid.x, m, stream);
        return launch_batch_mma(q, gpw, a, (int)grid.x, m, stream);
    }
    if (m < 2 || a.tp || a.y_is_f32) return launch_lut8_rows<1, false>(q, gpw, a, grid, stream);
    int rc = launch_lut8_rows<2, false>(q, gpw, a, dim3(grid.x, m / 2), stream);
    if (rc || !(m & 1)) return rc;
    a.row_base = m - 1;
    return launch_lut8_rows<1, false>(q, gpw, a, dim3(grid.x, 1), stream);
}

static void fill_job(Job &j, const hlq_weight *w, const StreamDims &d, const void *x, int x_dtype,
                     void *y, int y_dtype, float *partial, unsigned *counters, long long unit_begin) {
    j.planes = w->d_planes;
    j.meta = w->d_meta;
    j.codes = w->d_codes;
    j.rcodes = w->d_rcodes;
    j.rmeta = w->d_rmeta;
    j.bias = w->d_bias;
    j.acc = partial;
    j.counters = counters;
    j.x = x;
    j.y = y;
    j.n = w->n; j.k = w->k; j.np = d.np; j.slices = d.slices; j.duos = d.duos; j.blocks = d.blocks;
    j.x_dtype = x_dtype; j.y_dtype = y_dtype;
    j.unit_begin = unit_begin;
    j.unit_begin_chunked = unit_begin;      // a single job starts at 0 either way; groups set their own
    j.xop = HLQ_INPUT_PLAIN;
    j.eps = 0.f;
    j.x2 = nullptr;
    j.gamma = nullptr;
    j.res_out = nullptr;
}

// Checks an input transform and copies it into a job (row offset `m0` of a chunked call).
static int apply_input_op(Job &j, const hlq_input_op *op, int x_dtype, int m0) {
    j.xop = HLQ_INPUT_PLAIN;
    j.eps = 0.f;
    j.x2 = nullptr;
    j.gamma = nullptr;
    j.res_out = nullptr;
    if (!op || op->kind == HLQ_INPUT_PLAIN) return HLQ_OK;
    if (op->kind != HLQ_INPUT_GATED_SILU && op->kind != HLQ_INPUT_ADD_RMSNORM) return HLQ_ERR_INVALID_ARGUMENT;
    if (x_dtype != HLQ_F16) return HLQ_ERR_UNSUPPORTED;
    if (j.k % 8) return HLQ_ERR_SHAPE;
    if (op->kind == HLQ_INPUT_GATED_SILU && !op->d_second) return HLQ_ERR_INVALID_ARGUMENT;
    if (op->kind == HLQ_INPUT_ADD_RMSNORM && !op->d_gamma) return HLQ_ERR_INVALID_ARGUMENT;
    if (((uintptr_t)op->d_second | (uintptr_t)op->d_gamma | (uintptr_t)op->d_res_out) & 15) return HLQ_ERR_ALIGNMENT;
    if (op->d_res_out && (op->d_res_out == j.x || op->d_res_out == op->d_second)) return HLQ_ERR_INVALID_ARGUMENT;
    const size_t row = (size_t)m0 * j.k * 2;
    j.xop = op->kind;
    j.eps = op->eps;
    j.x2 = op->d_second ? (const char *)op->d_second + row : nullptr;
    j.gamma = (const uint16_t *)op->d_gamma;
    j.res_out = op->kind == HLQ_INPUT_ADD_RMSNORM && op->d_res_out ? (uint16_t *)((char *)op->d_res_out + row) : nullptr;
    return HLQ_OK;
}

int launch_lut8_gemv(const hlq_weight *w, int m, const void *x, int x_dtype, void *y, int y_dtype,
                     void *workspace, size_t workspace_bytes, cudaStream_t stream, const hlq_input_op *op) {
    if (w->layout != HLQ_LAYOUT_STREAM) return HLQ_ERR_UNSUPPORTED;
    if (x_dtype != HLQ_F16 && x_dtype != HLQ_BF16) return HLQ_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)y & 3)) return HLQ_ERR_ALIGNMENT;
    const StreamDims d = stream_dims(w->n, w->k, w->g, w->q);
    if (!workspace || workspace_bytes < lut_scratch_bytes(m, d)) return HLQ_ERR_WORKSPACE;
    DeviceInfo *di;
    int rc = device_info(w->device, &di);
    if (rc) return rc;
    if ((uint32_t)di->max_dyn_smem < kLut8DynSmem) return HLQ_ERR_NO_DEVICE;

    const size_t xsz = 2, ysz = y_dtype == HLQ_F32 ? 4 : 2;
    for (int m0 = 0; m0 < m; m0 += kLutMaxM) {
        const int mc = (m - m0) < kLutMaxM ? (m - m0) : kLutMaxM;
        const Workspace ws = carve_workspace(workspace, mc, d);
        GemvArgs a = {};
        a.jobs = nullptr;
        a.njobs = 0;
        a.total_units = launch_units(d.slices, d.duos, 0);
        a.total_units_chunked = launch_units_chunked(d.slices, d.duos, kChunkDuos, kChunkSegCost);
        a.status = ws.status;
        a.dyn_smem = kLut8DynSmem;
        a.spin_limit = kDefaultSpinLimit;
        a.y_is_f32 = y_dtype == HLQ_F32;
        a.use_codes = w->d_codes != nullptr;
        a.use_rcodes = w->d_rcodes != nullptr;
        fill_job(a.single, w, d, (const char *)x + (size_t)m0 * w->k * xsz, x_dtype,
                 (char *)y + (size_t)m0 * w->n * ysz, y_dtype, ws.partial, ws.counters, 0);
        rc = apply_input_op(a.single, op, x_dtype, m0);
        if (rc) return rc;
        a.one_row_passes = a.single.xop != HLQ_INPUT_PLAIN;
        int ctas = di->sms;
        if ((long long)d.slices * d.duos < ctas) ctas = d.slices * d.duos;
        // a weight with the extra bit-plane: its blocks' sums go into the accumulators first
        rc = launch_sparse_plane(w, mc, a.single.x, x_dtype, ws.partial, d.np, nullptr, y_dtype, stream);
        if (rc) return rc;
        rc = launch_lut8_any(w->q, d.gpw, a, dim3(ctas, mc), stream, w->sp_pairs != 0);
        if (rc) return rc;
    }
    return HLQ_OK;
}

// ---- forward without any allocation: scratch in a fixed device array -------------------------
//
// Some callers may not allocate device memory around a forward call: a serving process that
// handed all of HBM to its own cache manager at start-up has nothing left to cudaMalloc from,
// and a latency-critical section cannot afford the device-wide synchronization cudaMalloc and
// cudaFree imply.  For them the LUT GEMV can keep its scratch (status word, completion
// counters, fp32 row accumulators) in the array below instead of a caller-provided workspace.
// Every GPU that loads this library holds the array until the process exits.  The first 256
// bytes hold the kernels' status word; the calls never clear it (hlq_static_scratch_status
// reads and clears it), so a failure stays visible until somebody has looked.
constexpr size_t kStaticScratchBytes = 1u << 20;   // 1 MiB, must match HLQ_STATIC_SCRATCH_BYTES
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address.
// The address is looked up once per device, with that device current.
static int static_scratch_address(int device, void **out) {
    static std::atomic<void *> addr[64];
    if (device < 0 || device >= 64) return HLQ_ERR_INVALID_ARGUMENT;
    void *p = addr[device].load(std::memory_order_acquire);
    if (!p) {
        std::lock_guard<std::mutex> lock(g_first_use);
        HLQ_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
        if (!p) return HLQ_ERR_CUDA;
        addr[device].store(p, std::memory_order_release);
    }
    *out = p;
    return HLQ_OK;
}

int launch_lut8_gemv_static(const hlq_weight *w, int m, const void *x, int x_dtype, void *y,
                            int y_dtype, cudaStream_t stream) {
    if (w->layout != HLQ_LAYOUT_STREAM || w->sp_pairs) return HLQ_ERR_UNSUPPORTED;
    if (x_dtype != HLQ_F16 && x_dtype != HLQ_BF16) return HLQ_ERR_UNSUPPORTED;
    if (((uintptr_t)x & 15) || ((uintptr_t)y & 3)) return HLQ_ERR_ALIGNMENT;
    const StreamDims d = stream_dims(w->n, w->k, w->g, w->q);
    const size_t need = lut_scratch_bytes(m, d);
    if (need > kStaticScratchBytes) return HLQ_ERR_WORKSPACE;   // beyond the fixed maximum
    DeviceInfo *di;
    int rc = device_info(w->device, &di);
    if (rc) return rc;
    if ((uint32_t)di->max_dyn_smem < kLut8DynSmem) return HLQ_ERR_NO_DEVICE;
    void *scratch = nullptr;
    rc = static_scratch_address(w->device, &scratch);
    if (rc) return rc;

    const size_t xsz = 2, ysz = y_dtype == HLQ_F32 ? 4 : 2;
    for (int m0 = 0; m0 < m; m0 += kLutMaxM) {
        const int mc = (m - m0) < kLutMaxM ? (m - m0) : kLutMaxM;
        // The array keeps whatever the previous call left; counters and accumulators must
        // start at zero, so clear the part this launch uses (a memset node, no allocation).
        // The header with the status word is left alone: see hlq_static_scratch_status.
        HLQ_CUDA(cudaMemsetAsync((unsigned char *)scratch + kWsHeader, 0, lut_scratch_bytes(mc, d) - kWsHeader,
                                 stream));
        const Workspace ws = carve_workspace(scratch, mc, d);
        GemvArgs a = {};
        a.jobs = nullptr;
        a.njobs = 0;
        a.total_units = launch_units(d.slices, d.duos, 0);
        a.total_units_chunked = launch_units_chunked(d.slices, d.duos, kChunkDuos, kChunkSegCost);
        a.status = ws.status;
        a.dyn_smem = kLut8DynSmem;
        a.spin_limit = kDefaultSpinLimit;
        a.y_is_f32 = y_dtype == HLQ_F32;
        a.use_codes = w->d_codes != nullptr;
        a.use_rcodes = w->d_rcodes != nullptr;
        fill_job(a.single, w, d, (const char *)x + (size_t)m0 * w->k * xsz, x_dtype,
                 (char *)y + (size_t)m0 * w->n * ysz, y_dtype, ws.partial, ws.counters, 0);
        int ctas = di->sms;
        if ((long long)d.slices * d.duos < ctas) ctas = d.slices * d.duos;
        rc = launch_lut8_any(w->q, d.gpw, a, dim3(ctas, mc), stream);
        if (rc) return rc;
    }
    return HLQ_OK;
}

}  // namespace hlq

extern "C" int hlq_linear_forward_static(int m, int k, int n, const void *d_x, int x_dtype, void *d_y,
                                         int y_dtype, const hlq_weight *w, void *stream) {
    if (!w || m < 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (k != w->k || n != w->n) return HLQ_ERR_SHAPE;
    if (m == 0) return HLQ_OK;
    if (!d_x || !d_y) return HLQ_ERR_INVALID_ARGUMENT;
    if (y_dtype != HLQ_F16 && y_dtype != HLQ_BF16 && y_dtype != HLQ_F32) return HLQ_ERR_UNSUPPORTED;
    int cur = -1;
    HLQ_CUDA(cudaGetDevice(&cur));
    if (cur != w->device) return HLQ_ERR_INVALID_ARGUMENT;   // the weight's device must be current
    return hlq::launch_lut8_gemv_static(w, m, d_x, x_dtype, d_y, y_dtype, (cudaStream_t)stream);
}

extern "C" int hlq_select_batch_kernel(int which) {
    if (which < 0 || which > 3) return HLQ_ERR_INVALID_ARGUMENT;
    hlq::g_batch_kernel.store(which, std::memory_order_relaxed);
    return HLQ_OK;
}

extern "C" int hlq_static_scratch_status(int device, void *stream, int *kernel_status) {
    if (!kernel_status) return HLQ_ERR_INVALID_ARGUMENT;
    int cur = -1;
    HLQ_CUDA(cudaGetDevice(&cur));
    if (cur != device) return HLQ_ERR_INVALID_ARGUMENT;       // the device must be current
    void *scratch = nullptr;
    const int rc = hlq::static_scratch_address(device, &scratch);
    if (rc) return rc;
    HLQ_CUDA(cudaMemcpyAsync(kernel_status, scratch, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    HLQ_CUDA(cudaMemsetAsync(scratch, 0, sizeof(int), (cudaStream_t)stream));    // read once, then clear
    HLQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return *kernel_status ? HLQ_ERR_KERNEL : HLQ_OK;
}

// ---- fused all-reduce for row-parallel linears ----------------------------------------------
// Fills the device-side descriptor once every rank's buffer address is known.
static int tp_comm_publish(hlq_tp_comm *c) {
    hlq::TpDev t = {};
    for (int p = 0; p < c->world; ++p) t.recv[p] = (unsigned long long *)c->peer[p];
    t.seq = (unsigned *)(c->local + c->seq_off);
    t.done = t.seq + 1;
    t.rank = c->rank; t.world = c->world; t.max_m = c->max_m; t.np_cap = c->np_cap;
    return hlq::note_cuda(cudaMemcpy(c->d_tp, &t, sizeof(t), cudaMemcpyHostToDevice));
}

extern "C" {

int hlq_tp_comm_create(hlq_tp_comm **out, int rank, int world, int max_n, int max_m, int device) {
    if (!out) return HLQ_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (world < 1 || world > 8 || rank < 0 || rank >= world || max_n <= 0 || max_m < 1 || max_m > hlq::kLutMaxM)
        return HLQ_ERR_INVALID_ARGUMENT;
    hlq_tp_comm *c = new (std::nothrow) hlq_tp_comm();
    if (!c) return HLQ_ERR_INVALID_ARGUMENT;
    c->device = device; c->rank = rank; c->world = world; c->max_m = max_m;
    c->np_cap = (max_n + hlq::kBlockRows - 1) / hlq::kBlockRows * hlq::kBlockRows;
    const size_t recv = (size_t)2 * world * max_m * c->np_cap * sizeof(unsigned long long);
    c->seq_off = (recv + 255) / 256 * 256;
    c->bytes = c->seq_off + 256;
    int prev = -1;
    cudaGetDevice(&prev);
    int rc = HLQ_OK;
    if (cudaSetDevice(device) != cudaSuccess) rc = HLQ_ERR_NO_DEVICE;
    if (!rc && cudaMalloc((void **)&c->local, c->bytes) != cudaSuccess) rc = hlq::note_cuda(cudaErrorMemoryAllocation);
    if (!rc) rc = hlq::note_cuda(cudaMemset(c->local, 0, c->bytes));
    if (!rc && cudaMalloc((void **)&c->d_tp, sizeof(hlq::TpDev)) != cudaSuccess)
        rc = hlq::note_cuda(cudaErrorMemoryAllocation);
    if (prev >= 0) cudaSetDevice(prev);
    if (rc) {
        if (c->local) cudaFree(c->local);
        if (c->d_tp) cudaFree(c->d_tp);
        delete c;
        return rc;
    }
    *out = c;
    return HLQ_OK;
}

int hlq_tp_comm_handle(const hlq_tp_comm *c, void *handle64) {
    if (!c || !handle64) return HLQ_ERR_INVALID_ARGUMENT;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are exchanged as 64 bytes");
    cudaIpcMemHandle_t h;
    HLQ_CUDA(cudaIpcGetMemHandle(&h, c->local));
    memcpy(handle64, &h, 64);
    return HLQ_OK;
}

int hlq_tp_comm_connect(hlq_tp_comm *c, const void *handles) {
    if (!c || (!handles && c->world > 1)) return HLQ_ERR_INVALID_ARGUMENT;
    if (c->connected) return HLQ_ERR_INVALID_ARGUMENT;
    int prev = -1;
    cudaGetDevice(&prev);
    if (cudaSetDevice(c->device) != cudaSuccess) return HLQ_ERR_NO_DEVICE;
    int rc = HLQ_OK;
    for (int p = 0; p < c->world && !rc; ++p) {
        if (p == c->rank) {
            c->peer[p] = c->local;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const char *)handles + 64 * p, 64);
        rc = hlq::note_cuda(cudaIpcOpenMemHandle(&c->peer[p], h, cudaIpcMemLazyEnablePeerAccess));
    }
    if (!rc) rc = tp_comm_publish(c);
    if (prev >= 0) cudaSetDevice(prev);
    if (!rc) {
        c->connected = true;
        c->ipc = true;
    }
    return rc;
}

int hlq_tp_comm_buffer_bytes(const hlq_tp_comm *c, size_t *bytes) {
    if (!c || !bytes) return HLQ_ERR_INVALID_ARGUMENT;
    *bytes = c->bytes;
    return HLQ_OK;
}

int hlq_tp_comm_connect_pointers(hlq_tp_comm *c, void *const *d_peer_buffers) {
    if (!c || (!d_peer_buffers && c->world > 1)) return HLQ_ERR_INVALID_ARGUMENT;
    if (c->connected) return HLQ_ERR_INVALID_ARGUMENT;
    for (int p = 0; p < c->world; ++p) {
        if (p == c->rank) {
            c->peer[p] = c->local;
            continue;
        }
        if (!d_peer_buffers[p] || ((uintptr_t)d_peer_buffers[p] & 255)) return HLQ_ERR_ALIGNMENT;
        c->peer[p] = d_peer_buffers[p];
    }
    int prev = -1;
    cudaGetDevice(&prev);
    if (cudaSetDevice(c->device) != cudaSuccess) return HLQ_ERR_NO_DEVICE;
    const int rc = tp_comm_publish(c);
    if (prev >= 0) cudaSetDevice(prev);
    if (!rc) c->connected = true;
    return rc;
}

int hlq_tp_comm_local_buffer(const hlq_tp_comm *c, void **d_buffer) {
    if (!c || !d_buffer) return HLQ_ERR_INVALID_ARGUMENT;
    *d_buffer = c->local;
    return HLQ_OK;
}

int hlq_tp_comm_set_spin_limit(hlq_tp_comm *c, int polls) {
    if (!c || polls < 1) return HLQ_ERR_INVALID_ARGUMENT;
    c->spin_limit = polls;
    return HLQ_OK;
}

int hlq_tp_comm_free(hlq_tp_comm *c) {
    if (!c) return HLQ_OK;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(c->device);
    for (int p = 0; p < c->world; ++p)
        if (c->ipc && p != c->rank && c->peer[p]) cudaIpcCloseMemHandle(c->peer[p]);
    if (c->local) cudaFree(c->local);
    if (c->d_tp) cudaFree(c->d_tp);
    if (prev >= 0) cudaSetDevice(prev);
    delete c;
    return HLQ_OK;
}

int hlq_linear_forward_allreduce(int m, int k, int n, const void *d_x, int x_dtype, void *d_y, int y_dtype,
                                 void *d_workspace, size_t workspace_bytes, const hlq_weight *w,
                                 hlq_tp_comm *comm, void *stream_) {
    return hlq_linear_forward_allreduce_op(m, k, n, d_x, x_dtype, d_y, y_dtype, d_workspace, workspace_bytes, w, comm,
                                           nullptr, stream_);
}

int hlq_linear_forward_allreduce_op(int m, int k, int n, const void *d_x, int x_dtype, void *d_y, int y_dtype,
                                    void *d_workspace, size_t workspace_bytes, const hlq_weight *w,
                                    hlq_tp_comm *comm, const hlq_input_op *op, void *stream_) {
    using namespace hlq;
    if (!w || !comm || m < 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (k != w->k || n != w->n) return HLQ_ERR_SHAPE;
    if (m == 0) return HLQ_OK;
    if (!d_x || !d_y) return HLQ_ERR_INVALID_ARGUMENT;
    if (!comm->connected || comm->device != w->device) return HLQ_ERR_INVALID_ARGUMENT;
    if (w->layout != HLQ_LAYOUT_STREAM || w->sp_pairs) return HLQ_ERR_UNSUPPORTED;
    if (x_dtype != HLQ_F16 && x_dtype != HLQ_BF16) return HLQ_ERR_UNSUPPORTED;
    if (y_dtype != HLQ_F16 && y_dtype != HLQ_BF16 && y_dtype != HLQ_F32) return HLQ_ERR_UNSUPPORTED;
    if (((uintptr_t)d_x & 15) || ((uintptr_t)d_y & 3)) return HLQ_ERR_ALIGNMENT;
    const StreamDims d = stream_dims(w->n, w->k, w->g, w->q);
    if (d.np > comm->np_cap || m > comm->max_m) return HLQ_ERR_WORKSPACE;
    if (!d_workspace || workspace_bytes < lut_scratch_bytes(m, d)) return HLQ_ERR_WORKSPACE;
    int cur = -1;
    HLQ_CUDA(cudaGetDevice(&cur));
    if (cur != w->device) return HLQ_ERR_INVALID_ARGUMENT;
    DeviceInfo *di;
    int rc = device_info(w->device, &di);
    if (rc) return rc;
    const Workspace ws = carve_workspace(d_workspace, m, d);
    GemvArgs a = {};
    a.tp = comm->d_tp;
    a.total_units = launch_units(d.slices, d.duos, 0);
    a.status = ws.status;
    a.dyn_smem = kLut8DynSmem;
    a.spin_limit = comm->spin_limit;
    fill_job(a.single, w, d, d_x, x_dtype, d_y, y_dtype, ws.partial, ws.counters, 0);
    rc = apply_input_op(a.single, op, x_dtype, 0);
    if (rc) return rc;
    a.one_row_passes = a.single.xop != HLQ_INPUT_PLAIN;
    int ctas = di->sms;
    if ((long long)d.slices * d.duos < ctas) ctas = d.slices * d.duos;
    return launch_lut8_any(w->q, d.gpw, a, dim3(ctas, m), (cudaStream_t)stream_);
}

}  // extern "C"

// ---- groups: many independent linears in one persistent launch -----------------------------
struct hlq_group {
    int device = 0;
    int count = 0, max_m = 1;
    int q = 0, gpw = 0;
    long long total_units = 0;    // with the per-slice set-up share (launch_units)
    long long total_units_chunked = 0;   // under the small-batch kernel's walk (launch_units_chunked)
    long long duo_units = 0;      // (slice, duo) pairs
    int seg_cost = 0;
    bool one_row_passes = false;  // a member has an input transform
    bool use_codes = false;       // every member had code words when the group was made
    bool use_rcodes = false;      // ... and row codes
    std::vector<const hlq_weight *> weights;
    std::vector<hlq::Job> jobs_host;
    hlq::Job *d_jobs = nullptr;
    unsigned char *d_scratch = nullptr;   // status word, counters and partial sums of all jobs
    size_t scratch_bytes = 0;
    bool bound = false;
};

using namespace hlq;

extern "C" {

int hlq_group_create(hlq_group **out, int count, const hlq_weight *const *weights, int max_m) {
    if (!out) return HLQ_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (count <= 0 || !weights || max_m < 1 || max_m > kLutMaxM) return HLQ_ERR_INVALID_ARGUMENT;
    for (int i = 0; i < count; ++i) {
        if (!weights[i]) return HLQ_ERR_INVALID_ARGUMENT;
        if (weights[i]->layout != HLQ_LAYOUT_STREAM || weights[i]->sp_pairs) return HLQ_ERR_UNSUPPORTED;
        if (weights[i]->q != weights[0]->q || weights[i]->g != weights[0]->g ||
            weights[i]->device != weights[0]->device)
            return HLQ_ERR_UNSUPPORTED;
    }
    hlq_group *g = new (std::nothrow) hlq_group();
    if (!g) return HLQ_ERR_INVALID_ARGUMENT;
    g->device = weights[0]->device;
    g->count = count;
    g->max_m = max_m;
    g->q = weights[0]->q;
    g->weights.assign(weights, weights + count);
    g->jobs_host.resize(count);
    // scratch: [status 256 B][per job: counters, partial]
    size_t off = kWsHeader;
    std::vector<size_t> coff(count), poff(count);
    long long units = 0;
    for (int i = 0; i < count; ++i) {
        const hlq_weight *w = weights[i];
        const StreamDims d = stream_dims(w->n, w->k, w->g, w->q);
        g->gpw = d.gpw;
        coff[i] = off;
        off += ((size_t)max_m * d.blocks * sizeof(unsigned) + 255) / 256 * 256;
        poff[i] = off;
        off += ((size_t)acc_rows(max_m) * d.np * sizeof(float) + 255) / 256 * 256;
        units += (long long)d.slices * d.duos;
    }
    g->scratch_bytes = off;
    int prev = -1;
    cudaGetDevice(&prev);
    int rc = HLQ_OK;
    if (cudaSetDevice(g->device) != cudaSuccess) rc = HLQ_ERR_NO_DEVICE;
    if (!rc && cudaMalloc((void **)&g->d_scratch, off) != cudaSuccess) rc = note_cuda(cudaErrorMemoryAllocation);
    if (!rc && cudaMalloc((void **)&g->d_jobs, sizeof(Job) * count) != cudaSuccess)
        rc = note_cuda(cudaErrorMemoryAllocation);
    if (!rc) rc = note_cuda(cudaMemset(g->d_scratch, 0, off));
    if (!rc) {
        g->seg_cost = count > 1 ? kSegCost : 0;
        long long ub = 0, ubc = 0;
        for (int i = 0; i < count; ++i) {
            const hlq_weight *w = weights[i];
            const StreamDims d = stream_dims(w->n, w->k, w->g, w->q);
            fill_job(g->jobs_host[i], w, d, nullptr, HLQ_F16, nullptr, HLQ_F16,
                     (float *)(g->d_scratch + poff[i]), (unsigned *)(g->d_scratch + coff[i]), ub);
            g->jobs_host[i].unit_begin_chunked = ubc;
            ub += launch_units(d.slices, d.duos, g->seg_cost);
            ubc += launch_units_chunked(d.slices, d.duos, kChunkDuos, kChunkSegCost);
            g->duo_units += (long long)d.slices * d.duos;
        }
        g->total_units = ub;
        g->total_units_chunked = ubc;
        g->use_codes = g->use_rcodes = true;
        for (int i = 0; i < count; ++i) {
            g->use_codes = g->use_codes && weights[i]->d_codes != nullptr;
            g->use_rcodes = g->use_rcodes && weights[i]->d_rcodes != nullptr;
        }
    }
    if (prev >= 0) cudaSetDevice(prev);
    if (rc) {
        if (g->d_scratch) cudaFree(g->d_scratch);
        if (g->d_jobs) cudaFree(g->d_jobs);
        delete g;
        return rc;
    }
    *out = g;
    return HLQ_OK;
}

int hlq_group_bind(hlq_group *g, const void *const *d_x, void *const *d_y, int x_dtype, int y_dtype,
                   void *stream) {
    return hlq_group_bind_op(g, d_x, d_y, x_dtype, y_dtype, nullptr, stream);
}

int hlq_group_bind_op(hlq_group *g, const void *const *d_x, void *const *d_y, int x_dtype, int y_dtype,
                      const hlq_input_op *ops, void *stream) {
    if (!g || !d_x || !d_y) return HLQ_ERR_INVALID_ARGUMENT;
    if (x_dtype != HLQ_F16 && x_dtype != HLQ_BF16) return HLQ_ERR_UNSUPPORTED;
    if (y_dtype != HLQ_F16 && y_dtype != HLQ_BF16 && y_dtype != HLQ_F32) return HLQ_ERR_UNSUPPORTED;
    g->one_row_passes = false;
    for (int i = 0; i < g->count; ++i) {
        if (!d_x[i] || !d_y[i]) return HLQ_ERR_INVALID_ARGUMENT;
        if (((uintptr_t)d_x[i] & 15) || ((uintptr_t)d_y[i] & 3)) return HLQ_ERR_ALIGNMENT;
        g->jobs_host[i].x = d_x[i];
        g->jobs_host[i].y = d_y[i];
        g->jobs_host[i].x_dtype = x_dtype;
        g->jobs_host[i].y_dtype = y_dtype;
        const int rc = hlq::apply_input_op(g->jobs_host[i], ops ? &ops[i] : nullptr, x_dtype, 0);
        if (rc) return rc;
        if (g->jobs_host[i].xop != HLQ_INPUT_PLAIN) g->one_row_passes = true;
    }
    // the table is small; a synchronous copy keeps the host vector free to change afterwards
    HLQ_CUDA(cudaMemcpyAsync(g->d_jobs, g->jobs_host.data(), sizeof(Job) * g->count, cudaMemcpyHostToDevice,
                             (cudaStream_t)stream));
    HLQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    g->bound = true;
    return HLQ_OK;
}

int hlq_group_forward(hlq_group *g, int m, void *stream) {
    if (!g || m < 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (m == 0) return HLQ_OK;
    if (!g->bound) return HLQ_ERR_INVALID_ARGUMENT;
    if (m > g->max_m) return HLQ_ERR_WORKSPACE;
    int cur = -1;
    HLQ_CUDA(cudaGetDevice(&cur));
    if (cur != g->device) return HLQ_ERR_INVALID_ARGUMENT;
    DeviceInfo *di;
    int rc = device_info(g->device, &di);
    if (rc) return rc;
    if ((uint32_t)di->max_dyn_smem < kLut8DynSmem) return HLQ_ERR_NO_DEVICE;
    GemvArgs a = {};
    a.jobs = g->d_jobs;
    a.njobs = g->count;
    a.total_units = g->total_units;
    a.total_units_chunked = g->total_units_chunked;
    a.use_codes = g->use_codes;
    a.use_rcodes = g->use_rcodes;
    a.seg_cost = g->seg_cost;
    a.status = (int *)g->d_scratch;
    a.dyn_smem = kLut8DynSmem;
    a.spin_limit = kDefaultSpinLimit;
    a.y_is_f32 = g->jobs_host[0].y_dtype == HLQ_F32;
    a.one_row_passes = g->one_row_passes;
    int ctas = di->sms;
    if (g->duo_units < ctas) ctas = (int)g->duo_units;
    return launch_lut8_any(g->q, g->gpw, a, dim3(ctas, m), (cudaStream_t)stream);
}

int hlq_group_status(const hlq_group *g, void *stream, int *kernel_status) {
    if (!g || !kernel_status) return HLQ_ERR_INVALID_ARGUMENT;
    HLQ_CUDA(cudaMemcpyAsync(kernel_status, g->d_scratch, sizeof(int), cudaMemcpyDeviceToHost,
                             (cudaStream_t)stream));
    HLQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return *kernel_status ? HLQ_ERR_KERNEL : HLQ_OK;
}

int hlq_group_info(const hlq_group *g, int *count, int64_t *scratch_bytes, int64_t *algorithmic_bytes) {
    if (!g) return HLQ_ERR_INVALID_ARGUMENT;
    if (count) *count = g->count;
    if (scratch_bytes) *scratch_bytes = (int64_t)g->scratch_bytes;
    if (algorithmic_bytes) {
        int64_t t = 0;
        for (const hlq_weight *w : g->weights)
            t += (int64_t)w->q * w->n * (w->k / 8) + 2 * (int64_t)(w->q + 1) * w->n * (w->k / w->g);
        *algorithmic_bytes = t;
    }
    return HLQ_OK;
}

int hlq_group_free(hlq_group *g) {
    if (!g) return HLQ_OK;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(g->device);
    if (g->d_scratch) cudaFree(g->d_scratch);
    if (g->d_jobs) cudaFree(g->d_jobs);
    if (prev >= 0) cudaSetDevice(prev);
    delete g;
    return HLQ_OK;
}

}  // extern "C"

namespace hlq {

// The kernel's status word is the caller's workspace header when there is one (so that
// hlq_workspace_status sees it, as for the other kernels), else the word the handle owns.
int launch_lut4_gemv(const hlq_weight *w, int m, const void *x, int x_dtype, void *y, int y_dtype,
                     void *workspace, size_t workspace_bytes, cudaStream_t stream) {
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
    a.status = (workspace && workspace_bytes >= kWsHeader) ? (int *)workspace : w->d_status;
    if (!a.status) return HLQ_ERR_WORKSPACE;
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


