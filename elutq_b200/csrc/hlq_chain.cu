// Decode chain: the per-token op chain of a decoder (all its layers) as ONE persistent kernel.
//
// Replaces the per-op call chain of the reference's model loop for one token,
//   C++/examples/models/llama.cpp:185-700
// (per layer: RMSNorm, q/k/v GEMV, RoPE, cache append, attention, o GEMV, residual add +
// RMSNorm, gate/up GEMV, gated SiLU, down GEMV), whose every op is a call that returns before
// the next starts.  Here the CTAs (one per SM) stay resident across all ops.  A chain is a
// list of STAGES; a stage is either a set of independent LUT GEMVs (as in lut8_gemv_kernel:
// tables of 256 subset sums per 8 activations, one lookup per packed byte, fp32 accumulation)
// or the attention of one token (hlq_attn_dev.cuh).  Stage s + 1 reads what stage s wrote, so
// the hand-off between two stages is a counter in global memory: whoever completes a block of
// 32 output rows (or a kv head) adds to done[s] after a fence, and the control warp of every
// CTA polls done[s] (bounded) before it brings the first activations of stage s + 1 in.
// While a CTA waits, its consumer warps already hold the first weight tiles of the next stage
// in registers: weights do not depend on activations.
//
// The elementwise ops between two linears live where the data already is:
//   RMSNorm      in the table build of the consuming GEMV: x_eff = fp16(x16 * gamma * inv_rms),
//                inv_rms from a sum of squares that the PRODUCING stage accumulated (one fp32
//                cell per norm) while it completed its rows;
//   residual add in the completion pass of o and down: t = resid + fp16(y), resid = fp16(t),
//                cell += sum t^2  (the order of arm_rmsnorm.cpp:68-85);
//   gated SiLU   in the completion pass of a fused gate/up weight whose rows alternate in
//                chunks of 16 (gate rows 16c.., up rows 16c..): lane j < 16 of a completed
//                32-row block pairs with lane j + 16  (arm_activation.cpp:36-49).
// With tensor parallelism the row-parallel stages (o, down) sum over the ranks exactly as
// lut8_gemv_kernel does (64-bit {value, tag} stores into every rank's slots, bounded polls),
// with one tag per stage and two slot sets used alternately.
//
// Every wait is bounded; the first one that runs out sets the CTA's failure flag and the
// status word (1), after which all roles skip their work, every later wait gives up at once and
// the control warp ends the item stream, so the kernel drains instead of hanging.
#include <cuda_fp16.h>

#include <atomic>
#include <mutex>
#include <new>
#include <algorithm>
#include <utility>
#include <vector>

#include "hlq_attn_dev.cuh"
#include "hlq_gemv_dev.cuh"
#include "hlq_internal.h"

namespace hlq {

constexpr int kChConsumerWarps = 16;
constexpr int kChFinalWarps = 4;
constexpr int kChConsumers = kChConsumerWarps * 32;
constexpr int kChFinalizers = kChFinalWarps * 32;
constexpr int kChThreads = kChConsumers + kChFinalizers;
constexpr uint32_t kChTableBytes = 65536;
constexpr uint32_t kChAuxBytes = 8192;

constexpr int kChBarConsumers = 1;   // 512 consumer threads
constexpr int kChBarItemDone = 2;    // +slot: consumers arrive, finalizers sync (640)
constexpr int kChBarFinalizers = 6;  // 128 finalizer threads

enum { CH_IN_PLAIN = 0, CH_IN_NORM = 1, CH_IN_ATTENTION = 2, CH_IN_GATED_ACC = 3 };   // the last one is set by the host, not by callers
enum { CH_OUT_STORE = 0, CH_OUT_RESIDUAL = 1, CH_OUT_GATED_SILU = 2 };
enum { CH_STAGE_GEMV = 0, CH_STAGE_ATTENTION = 1 };
enum { CH_ITEM_END = 0, CH_ITEM_SEGMENT = 1, CH_ITEM_ATTENTION = 2, CH_ITEM_NOTHING = 3 };

// One linear of a GEMV stage.
struct ChainJob {
    const uint8_t *planes;
    const uint16_t *meta;
    const uint16_t *bias;
    float *acc;              // [np] fp32 accumulators, zero between uses
    const uint16_t *x;       // fp16 [k]: the activations (PLAIN) or the residual stream (NORM); ATTENTION: the
                             // splits' partials of the attention stage before (float [head][nsplit][128], then [head][nsplit][2])
    __half *y;               // STORE: [n]; RESIDUAL: the residual stream [n], updated in place; GATED_SILU: [n / 2]
    const uint16_t *gamma;   // NORM: fp16 [k]
    const float *ss_in;      // NORM: sum of squares of the residual stream
    float *ss_out;           // RESIDUAL: receives the sum of squares of the updated stream
    float eps, inv_k;        // NORM: inv_rms = 1 / sqrt(*ss_in * inv_k + eps)
    int n, k, np, slices, duos, blocks;
    int in_kind, out_kind;
    int attn_nsplit, attn_group;   // ATTENTION input: splits per kv head, query heads per kv head
    int attn_heads;                // ATTENTION input: query heads of the attention stage
};

struct ChainStage {
    int kind;
    int job_begin, job_count;
    unsigned target;         // done[this stage] when complete: blocks of all jobs, or kv heads
    int tp_ordinal;          // > 0: the (single) job's rows are summed over the ranks; tag = base + ordinal
    int attn, nsplit;        // attention: index into the table of AttnArgs, splits per kv head
};

struct ChainItem;
struct ChainArgs {
    const ChainItem *items;  // every CTA's items, one CTA after the other, each list ended by an END item
    const int *first;        // [ctas + 1]: index of a CTA's first item
    const ChainJob *jobs;
    const AttnArgs *attn;
    unsigned *done;          // [nstages], zero at launch: finished blocks (kv heads) per stage
    unsigned *raw;           // [nstages], zero at launch: CTAs that have added all their partial sums
    int *status;
    const TpDev *tp;         // nullptr: no rank sums
    int nstages, n_tp_stages;
    uint32_t dyn_smem;
    int spin_limit;
    const int *rope_position;    // the attention stages share position, base and cache length: cos/sin are built once
    float rope_base;
    int rope_max_ctx;
    unsigned long long *trace;   // optional timeline: [cta][item][16] nanosecond stamps, or nullptr
    int trace_items;
};

// One unit of work of one CTA: a run of duos inside one slice of one linear (SEGMENT), one
// (kv head, split) of an attention (ATTENTION), or nothing (a stage that holds no work for the
// CTA still gives it one item, so that every CTA passes every stage).  The host lays every
// CTA's items out when the chain is finished; the control warp of a CTA copies them one by
// one into a ring of two slots in shared memory, two items ahead of the consumers.
struct __align__(16) ChainItem {
    const uint8_t *planes;   // SEGMENT: first cell
    const uint16_t *meta;
    // SEGMENT: the fields of its job that the roles use (copied here so that nobody reads a
    // descriptor from global memory between two stages)
    const uint16_t *x, *gamma, *bias;
    const float *ss_in;
    float *ss_out, *acc;
    __half *y;
    const float *attn_ml;    // SEGMENT with ATTENTION input: the splits' (max, sum) pairs, [head][split][2]
    float eps, inv_k;
    int n, job_slices, in_kind, out_kind;
    int kind, stage;
    int last_of_stage;       // this CTA's last item of the stage: the stage's rank sum follows
    int duo_a, duo_b, slice, valid;
    int hk, split, nsplit, attn;   // ATTENTION
    int tp_ordinal;
    int job_index;           // SEGMENT or rank sum: index of the job
    unsigned dep_target;     // done[stage - 1] when the stage before this one is complete
    int job_first, stage_jobs;   // the stage's linears (stage_jobs = 0: not a GEMV stage)
    unsigned stage_blocks;   // blocks of 32 rows of all the stage's linears = done[stage] when complete
    // A GEMV stage whose only input is the gated-SiLU output of the single linear of the stage before
    // (down after gate/up) skips that stage's completion pass: its consumers read the fp32 sums
    // themselves (x = those accumulators, gamma = that linear's bias, attn_ml = its fp16 output, which
    // they still write), gated by raw[] instead of done[]; the stage before only counts its CTAs
    // (defer_out), and this stage's completion pass clears the accumulators it read (clear_acc).
    int dep_raw, defer_out, clear_blocks;
    float *clear_acc;
};

// aux region layout (bytes from its start)
constexpr uint32_t kChAuxX = 0;           // 2 slots x 512 fp16 activations
constexpr uint32_t kChAuxXsum = 2048;     // up to 16 group sums (fp32)
constexpr uint32_t kChAuxMbarDesc = 2112; // 2 mbarriers
constexpr uint32_t kChAuxMbarX = 2128;    // 2 mbarriers
constexpr uint32_t kChAuxFlag = 2144;     // int: CTA-wide failure flag
constexpr uint32_t kChAuxDecide = 2152;   // 2 ints: whether the consumers run the item of a slot
constexpr uint32_t kChAuxInvRms = 2160;   // 2 floats: 1 / rms of the norm input of a slot's item
constexpr uint32_t kChAuxPos = 2168;      // int: the token's position, clamped to the cache
constexpr uint32_t kChAuxTp = 2560;       // copy of the TpDev (<= 256 bytes)
constexpr uint32_t kChAuxItem = 3072;     // 2 x ChainItem (<= 192 bytes each)
constexpr uint32_t kChAuxItemSlot = 192;
constexpr uint32_t kChAuxRope = 4096;     // 64 x {cos, sin} of the token's position (heads of 128 channels)
constexpr uint32_t kChAuxMerge = 4608;    // 4 x 64 floats: normalized weights of the attention splits of a slice's heads
constexpr uint32_t kChAuxGamma = 6144;    // 2 slots x 512 fp16 norm weights
static_assert(sizeof(ChainItem) == kChAuxItemSlot, "a ChainItem is one ring slot (and one bulk copy)");
static_assert(sizeof(AttnMmaSmem) <= kChTableBytes, "the attention unit borrows the table block");

__device__ __forceinline__ unsigned ld_acquire_gpu_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_relaxed_gpu_s32(const int *p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits of the chain are bounded in TIME (polls of different kinds take different times): a
// spin limit of p polls stands for p * 256 ns.  The control warp and the rank sums give up
// after that budget; the waits of the other roles ON the control warp get eight times as much,
// so that it is always the control warp that ends a chain whose inputs never arrive.
__device__ __forceinline__ unsigned long long budget_ns(int spin_limit) { return (unsigned long long)spin_limit << 8; }
// false when the wait gave up; sets the CTA's failure flag then
__device__ __forceinline__ bool mbar_wait_timed(uint32_t mbar, uint32_t parity, volatile int *fail,
                                                unsigned long long budget) {
    if (mbar_try_wait(mbar, parity)) return true;
    if (!*fail) {
        const unsigned long long t0 = global_ns();
        for (;;) {
#pragma unroll 1
            for (int k = 0; k < 32; ++k)
                if (mbar_try_wait(mbar, parity)) return true;
            if (*fail || global_ns() - t0 > budget) break;
        }
    }
    *fail = 1;
    return false;
}

// The attention unit as a function of its own: its registers (K rows, V tile shares, eight
// accumulators) are not the GEMV loop's.  Issues the first tile's loads, waits for the item's
// inputs (the stage before must be complete), computes the split's partial and writes it.
// Returns whether the unit ran.
struct ChainWait {
    uint32_t mbar;             // the item's input barrier
    uint32_t parity;
    volatile int *fail;
    unsigned long long budget;
    int *decide;               // the slot's decision cell
};
__device__ __noinline__ bool chain_attention(const AttnArgs *args, int hk, int split, int nsplit, unsigned char *smem,
                                             int tid, const float2 *rope, int pos, ChainWait w,
                                             unsigned long long *stamps) {
    AttnMmaSmem &sm = *(AttnMmaSmem *)smem;
    auto sync = [] { named_bar_sync<kChBarConsumers, kChConsumers>(); };
    auto wait_inputs = [&]() {
        const bool got = mbar_wait_timed(w.mbar, w.parity, w.fail, w.budget);
        if (tid == 0) *w.decide = (got && !*w.fail) ? 1 : 0;      // one thread decides for all
        named_bar_sync<kChBarConsumers, kChConsumers>();
        return *w.decide != 0;
    };
    attention_partial_unit(*args, hk, split, nsplit, sm, tid, sync, rope, pos, wait_inputs, stamps);
    return *w.decide != 0;
}

// The consumers' loop over SEGMENT / NOTHING items, from item `i` on, until the next item is an
// ATTENTION item (true; `i` is its index) or the END (false).
template <int Q, int GPW>
__device__ __forceinline__ bool chain_gemv_items(const ChainArgs &a, unsigned char *aux, uint32_t tbl, int &i) {
    // everything else is re-derived from `aux` where it is needed: the fewer values stay live across
    // the streaming loop, the fewer of its registers get spilled
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#define CH_AUX_U32 (smem_u32(aux))
#define CH_MB_DESC (CH_AUX_U32 + kChAuxMbarDesc)
#define CH_MB_X (CH_AUX_U32 + kChAuxMbarX)
#define CH_RING ((ChainItem *)(aux + kChAuxItem))
#define CH_FAIL ((volatile int *)(aux + kChAuxFlag))
#define CH_DECIDE ((int *)(aux + kChAuxDecide))
#define CH_BUDGET_LONG (budget_ns(a.spin_limit) << 3)
    auto stamp = [&](int it, int k) {
        if (a.trace && it < a.trace_items) a.trace[((size_t)blockIdx.x * a.trace_items + it) * 16 + k] = global_ns();
    };
    const int r = lane >> 2, j = lane & 3;
    uint32_t rt[8];   // per-lane lookup bases: bank 8*j + (t ^ r) of the table row
#pragma unroll
    for (int t = 0; t < 8; ++t) rt[t] = tbl + 4u * (8u * j + (uint32_t)(t ^ r));
    constexpr int gshift = GPW == 1 ? 3 : (GPW == 2 ? 2 : 1);
    constexpr long long kDuoPlaneBytes = 2 * Q * kCellBytes;
    constexpr long long kDuoMetaElems = (Q + 1) * 32 * 2 * GPW;
    constexpr int kRing = (8 * Q + (Q + 1) * GPW < 22) ? 3 : 2;
    Tile<Q, GPW> t0, t1, t2;
    const uint8_t *pl = nullptr;
    const uint16_t *mp = nullptr;
    float *prow = nullptr;
    int d = 0, dend = 0;

    int cur_kind = CH_ITEM_END;
    bool cur_norm = false, cur_attn = false, cur_gated = false;
    // first loads of an item (its descriptor stays in its ring slot until the consumers hand
    // the item over, so only what the streaming loop needs is kept in registers)
    auto open_item = [&](const ChainItem &it) {
        cur_kind = it.kind;
        if (it.kind != CH_ITEM_SEGMENT) return;
        cur_norm = it.in_kind == CH_IN_NORM;
        cur_attn = it.in_kind == CH_IN_ATTENTION;
        cur_gated = it.in_kind == CH_IN_GATED_ACC;
        d = it.duo_a + warp;
        dend = it.duo_b;
        pl = it.planes + (long long)warp * kDuoPlaneBytes + lane * 16;
        mp = it.meta + (long long)warp * kDuoMetaElems + lane * (2 * GPW);
        prow = it.acc + (long long)d * 16 + r;
        if (d < dend) load_tile<Q, GPW>(t0, pl, mp);
        if (kRing == 3 && d + kChConsumerWarps < dend)
            load_tile<Q, GPW>(t1, pl + kChConsumerWarps * kDuoPlaneBytes, mp + kChConsumerWarps * kDuoMetaElems);
    };
    open_item(CH_RING[i & 1]);
    for (;; ++i) {
        const int slot = i & 1;
        if (tid == 0) stamp(i, 2);
        const bool got = mbar_wait_timed(CH_MB_X + 8 * slot, (i >> 1) & 1, CH_FAIL, CH_BUDGET_LONG);
        if (tid == 0) stamp(i, 3);
        // one thread decides for all whether the item runs (the failure flag can be raised at
        // any moment by another role; the barriers below need one answer)
        if (tid == 0) CH_DECIDE[slot] = (got && !*CH_FAIL) ? 1 : 0;
        named_bar_sync<kChBarConsumers, kChConsumers>();     // also: everyone is done with the old table
        const bool run = CH_DECIDE[slot] != 0;
        if (tid == 0) stamp(i, 4);
        if (cur_kind == CH_ITEM_SEGMENT && run) {
            if (cur_attn) {
                // the activations are the attention output: merge the splits' partials of this slice's
                // channels here (one channel per thread) instead of in a pass of the attention's own
                const ChainItem &it = CH_RING[slot];
                const float *partial = (const float *)it.x;
                uint16_t *xw = (uint16_t *)(aux + kChAuxX) + slot * kSliceK;
                // a slice of 512 channels = up to four heads of 128; the weights of the splits are
                // formed once per head (in the group-sum area, free until the tables are built)
                const float val = attention_merge_heads<128>(
                    partial, it.attn_ml, it.nsplit, it.slice * (kSliceK / 128), (it.valid + 127) / 128, tid,
                    (float *)(aux + kChAuxMerge), [] { named_bar_sync<kChBarConsumers, kChConsumers>(); });
                if (tid == 0) stamp(i, 10);
                xw[tid] = __half_as_ushort(__float2half_rn(val));
                named_bar_sync<kChBarConsumers, kChConsumers>();
                if (tid == 0) stamp(i, 15);
            }
            if (cur_gated) {
                // the activations are the gated SiLU of the stage before, whose fp32 sums are complete
                // (raw[] gate) but not finished: one channel per thread, the roundings of the
                // completion pass (fp16 gate, fp16 up, fp16 product); rows 32 b .. + 15 are gate rows,
                // + 16 .. + 31 the up rows of channels 16 b .. + 15
                const ChainItem &it = CH_RING[slot];
                const float *sums = (const float *)it.x;
                uint16_t *xw = (uint16_t *)(aux + kChAuxX) + slot * kSliceK;
                uint16_t hb = 0;
                if (tid < it.valid) {
                    const int c = it.slice * kSliceK + tid;
                    const int row = 32 * (c >> 4) + (c & 15);
                    float gate = ldcg_f32(sums + row), up = ldcg_f32(sums + row + 16);
                    if (it.gamma) {
                        gate += __half2float(__ushort_as_half(it.gamma[row]));
                        up += __half2float(__ushort_as_half(it.gamma[row + 16]));
                    }
                    const float mine = __half2float(__float2half_rn(gate)), other = __half2float(__float2half_rn(up));
                    const __half h = __float2half_rn(other * (mine / (1.0f + expf(-mine))));
                    hb = __half_as_ushort(h);
                    ((__half *)it.attn_ml)[c] = h;       // the stage's output stays where callers expect it
                }
                xw[tid] = hb;
                named_bar_sync<kChBarConsumers, kChConsumers>();
            }
            const bool norm = cur_norm;
            const float inv_rms = norm ? ((const float *)(aux + kChAuxInvRms))[slot] : 1.f;
            const uint16_t *xs = (const uint16_t *)(aux + kChAuxX) + slot * kSliceK;
            const uint16_t *gs = (const uint16_t *)(aux + kChAuxGamma) + slot * kSliceK;
            // the value the tables are built from: rounded to fp16 where the separate norm kernel rounds
            auto x_eff = [&](uint16_t xb, uint16_t gb) {
                const float xv = __half2float(__ushort_as_half(xb));
                if (!norm) return xv;
                return __half2float(__float2half_rn(xv * __half2float(__ushort_as_half(gb)) * inv_rms));
            };
            if (warp == 0) {
                float part = 0.f;
#pragma unroll
                for (int q2 = 0; q2 < 16; ++q2) part += x_eff(xs[lane * 16 + q2], gs[lane * 16 + q2]);
                constexpr int lanes_per_group = 8 >> (3 - gshift);   // g / 16 lanes: 8, 4 or 2
#pragma unroll
                for (int dd = 1; dd < lanes_per_group; dd <<= 1) part += __shfl_xor_sync(0xffffffffu, part, dd);
                if ((lane & (lanes_per_group - 1)) == 0) ((float *)(aux + kChAuxXsum))[lane / lanes_per_group] = part;
            }
            {
                const int h = warp & 1, ehi = warp >> 1;   // bank-row, top three index bits
                const int c = 16 * (lane >> 3) + 2 * (lane & 7) + h;
                const uint32_t dst = tbl + (uint32_t)ehi * (32u * 256u) + 4u * lane + 128u * h;
                const uint4 raw = *(const uint4 *)(xs + 8 * c);
                const uint4 graw = *(const uint4 *)(gs + 8 * c);
                const uint32_t rw[4] = {raw.x, raw.y, raw.z, raw.w}, gw[4] = {graw.x, graw.y, graw.z, graw.w};
                float xv[8];
#pragma unroll
                for (int q2 = 0; q2 < 4; ++q2) {
                    xv[2 * q2] = x_eff((uint16_t)(rw[q2] & 0xffffu), (uint16_t)(gw[q2] & 0xffffu));
                    xv[2 * q2 + 1] = x_eff((uint16_t)(rw[q2] >> 16), (uint16_t)(gw[q2] >> 16));
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
#pragma unroll
                for (int e = 0; e < 32; ++e) sts_f32(dst + (uint32_t)e * 256u, tv[e]);
            }
            named_bar_sync<kChBarConsumers, kChConsumers>();
            asm volatile("" ::: "memory");
            if (tid == 0) stamp(i, 5);

            float xsu[GPW];
#pragma unroll
            for (int uu = 0; uu < GPW; ++uu) xsu[uu] = ((const float *)(aux + kChAuxXsum))[GPW * j + (uu ^ (r >> gshift))];

            // stream: ring of register tiles, loads in flight behind the one in use
            constexpr long long kStepP = kChConsumerWarps * kDuoPlaneBytes;
            constexpr long long kStepM = kChConsumerWarps * kDuoMetaElems;
            constexpr int kStepRow = kChConsumerWarps * 16;
            if (kRing == 3) {
                while (d < dend) {
                    if (d + 2 * kChConsumerWarps < dend) load_tile<Q, GPW>(t2, pl + 2 * kStepP, mp + 2 * kStepM);
                    compute_tile<Q, GPW>(t0, rt, xsu, prow, lane);
                    d += kChConsumerWarps;
                    if (d >= dend) break;
                    if (d + 2 * kChConsumerWarps < dend) load_tile<Q, GPW>(t0, pl + 3 * kStepP, mp + 3 * kStepM);
                    compute_tile<Q, GPW>(t1, rt, xsu, prow + kStepRow, lane);
                    d += kChConsumerWarps;
                    if (d >= dend) break;
                    if (d + 2 * kChConsumerWarps < dend) load_tile<Q, GPW>(t1, pl + 4 * kStepP, mp + 4 * kStepM);
                    compute_tile<Q, GPW>(t2, rt, xsu, prow + 2 * kStepRow, lane);
                    d += kChConsumerWarps;
                    pl += 3 * kStepP;
                    mp += 3 * kStepM;
                    prow += 3 * kStepRow;
                }
            } else {
                while (d < dend) {
                    if (d + kChConsumerWarps < dend) load_tile<Q, GPW>(t1, pl + kStepP, mp + kStepM);
                    compute_tile<Q, GPW>(t0, rt, xsu, prow, lane);
                    d += kChConsumerWarps;
                    if (d >= dend) break;
                    if (d + kChConsumerWarps < dend) load_tile<Q, GPW>(t0, pl + 2 * kStepP, mp + 2 * kStepM);
                    compute_tile<Q, GPW>(t1, rt, xsu, prow + kStepRow, lane);
                    d += kChConsumerWarps;
                    pl += 2 * kStepP;
                    mp += 2 * kStepM;
                    prow += 2 * kStepRow;
                }
            }
        }
        if (tid == 0) stamp(i, 6);
        // hand this item to the finalizers, THEN the first loads of the next one: a barrier
        // arrival waits for the loads a thread has in flight
        named_bar_arrive_dyn(kChBarItemDone + slot, kChThreads);
        if (tid == 0) stamp(i, 7);
        const bool have = mbar_wait_timed(CH_MB_DESC + 8 * (slot ^ 1), ((i + 1) >> 1) & 1, CH_FAIL, CH_BUDGET_LONG);
        if (!have || CH_RING[slot ^ 1].kind == CH_ITEM_END) return false;
        if (CH_RING[slot ^ 1].kind == CH_ITEM_ATTENTION) {
            ++i;
            return true;
        }
        open_item(CH_RING[slot ^ 1]);
    }
}

template <int Q, int GPW>
__global__ void __launch_bounds__(kChThreads, 1) decode_chain_kernel(const __grid_constant__ ChainArgs a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    // The table block must start on a 64 KB boundary of the shared window.
    const uint32_t sbase = smem_u32(smem_raw);
    const uint32_t tbl = (sbase + 0xffffu) & ~0xffffu;
    const uint32_t aux_u32 = (tbl - sbase >= kChAuxBytes) ? sbase : tbl + kChTableBytes;
    if (tbl + kChTableBytes > sbase + a.dyn_smem || aux_u32 + kChAuxBytes > sbase + a.dyn_smem) {
        if (tid == 0) atomicExch(a.status, 2);
        return;
    }
    unsigned char *aux = smem_raw + (aux_u32 - sbase);
    unsigned char *table_ptr = smem_raw + (tbl - sbase);
    float *xsum = (float *)(aux + kChAuxXsum);
    volatile int *fail = (volatile int *)(aux + kChAuxFlag);
    ChainItem *ring = (ChainItem *)(aux + kChAuxItem);
    const uint32_t mb_desc = aux_u32 + kChAuxMbarDesc, mb_x = aux_u32 + kChAuxMbarX;
    const unsigned long long budget = budget_ns(a.spin_limit), budget_long = budget << 3;
    int *decide = (int *)(aux + kChAuxDecide);
    // timeline for profiling: stamp k of item i of this CTA (see hlq_chain_trace)
    auto stamp = [&](int i, int k) {
        if (a.trace && i < a.trace_items) a.trace[((size_t)blockIdx.x * a.trace_items + i) * 16 + k] = global_ns();
    };
    float *inv_rms_s = (float *)(aux + kChAuxInvRms);

    float2 *rope_tab = (float2 *)(aux + kChAuxRope);
    int *pos_s = (int *)(aux + kChAuxPos);
    if (a.rope_position && tid >= 64 && tid < 128) {
        // the token's position and its rotary angles, once per CTA instead of once per attention unit
        const int jj = tid - 64;
        int pos = *a.rope_position;
        if (pos < 0 || pos >= a.rope_max_ctx) {      // refuse to write outside the cache
            if (jj == 0 && blockIdx.x == 0) atomicExch(a.attn[0].status, 3);
            pos = pos < 0 ? 0 : a.rope_max_ctx - 1;
        }
        if (jj == 0) *pos_s = pos;
        const float ang = (float)pos * powf(a.rope_base, -(float)(2 * jj) / 128.0f);
        float sn, cs;
        sincosf(ang, &sn, &cs);
        rope_tab[jj] = make_float2(cs, sn);
    }
    if (tid == 0) {
        mbar_init(mb_desc, 1);
        mbar_init(mb_desc + 8, 1);
        mbar_init(mb_x, 1);
        mbar_init(mb_x + 8, 1);
        mbar_init_fence();
        *fail = 0;
    }
    __syncthreads();

    if (warp >= kChConsumerWarps) {
        // =========================== finalizer warps ======================================
        const int fw = warp - kChConsumerWarps, ftid = tid - kChConsumers;
        // control state (warp 16 only)
        const int item_first = a.first[blockIdx.x], item_count = a.first[blockIdx.x + 1] - item_first;
        int emitted = 0;                // descriptor copies started (or END injected) so far
        int issued = 0;                 // items whose inputs have been released to the consumers
        int known_done = -1;            // highest stage known to be complete
        bool ended = false;             // the list's END item (or an injected one) is on its way

        // rank sums: descriptor in shared memory, base tag of this launch
        const TpDev *tp = nullptr;
        unsigned tag_base = 0;
        if (a.tp) {
            uint32_t *dst = (uint32_t *)(aux + kChAuxTp);
            const uint32_t *src = (const uint32_t *)a.tp;
            for (int i = ftid; i < (int)(sizeof(TpDev) / 4); i += kChFinalizers) dst[i] = __ldg(src + i);
            named_bar_sync<kChBarFinalizers, kChFinalizers>();
            tp = (const TpDev *)(aux + kChAuxTp);
            tag_base = ldcg_u32(tp->seq);
        }

        // releases the inputs of the item in `slot` to the consumers (control warp)
        auto release = [&](int slot) {
            const ChainItem &it = ring[slot];
            if (it.kind == CH_ITEM_SEGMENT && it.in_kind != CH_IN_ATTENTION && it.in_kind != CH_IN_GATED_ACC && !*fail) {
                const bool norm = it.in_kind == CH_IN_NORM;
                uint16_t *xs = (uint16_t *)(aux + kChAuxX) + slot * kSliceK;
                uint16_t *gs = (uint16_t *)(aux + kChAuxGamma) + slot * kSliceK;
                if (it.valid < kSliceK) {
                    for (int i = it.valid + lane; i < kSliceK; i += 32) {
                        xs[i] = 0;
                        gs[i] = 0;
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    fence_proxy_async_all();     // other SMs' (acquired) writes and the zero fill, before the bulk copies
                    const uint32_t bytes = (uint32_t)it.valid * 2u;
                    tma_bulk_g2s(aux_u32 + kChAuxX + slot * kSliceK * 2, it.x + (long long)it.slice * kSliceK, bytes,
                                 mb_x + 8 * slot);
                    if (norm) {
                        tma_bulk_g2s(aux_u32 + kChAuxGamma + slot * kSliceK * 2,
                                     it.gamma + (long long)it.slice * kSliceK, bytes, mb_x + 8 * slot);
                        // 1 / rms while the copies fly; the arrive below publishes it with them
                        inv_rms_s[slot] = 1.0f / sqrtf(ldcg_f32(it.ss_in) * it.inv_k + it.eps);
                    }
                    mbar_expect_tx(mb_x + 8 * slot, bytes * (norm ? 2u : 1u));
                }
            } else {
                if (lane == 0) mbar_arrive(mb_x + 8 * slot);
            }
            __syncwarp();
        };
        // waits (bounded) until the stage that gates `stage` is complete (control warp)
        auto wait_dep = [&](int dep, unsigned target, bool on_raw) {
            if (dep < 0 || dep <= known_done) return;
            int ok = 0;
            const unsigned *counter = on_raw ? a.raw + dep : a.done + dep;     // CTAs that streamed, or finished blocks
            if (on_raw) target = gridDim.x;
            if (lane == 0 && !*fail) {           // the lane that polls is the lane that issues the copies
                const unsigned long long t0 = global_ns();
                for (;;) {
#pragma unroll 1
                    for (int k = 0; k < 16 && !ok; ++k) ok = ld_acquire_gpu_u32(counter) >= target;
                    if (ok || *fail || ld_relaxed_gpu_s32(a.status) != 0 || global_ns() - t0 > budget) break;
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (ok) known_done = dep;
            else *fail = 1;
        };
        // starts the copy of this CTA's next item into `slot` (its arrival completes the slot's
        // descriptor barrier); after a failure an END item is written there instead
        auto emit = [&](int slot) {
            if (*fail || emitted >= item_count) {
                if (lane == 0) {
                    ring[slot].kind = CH_ITEM_END;
                    mbar_arrive(mb_desc + 8 * slot);
                }
                ended = true;
            } else {
                if (lane == 0) {
                    mbar_expect_tx(mb_desc + 8 * slot, (uint32_t)sizeof(ChainItem));
                    tma_bulk_g2s(aux_u32 + kChAuxItem + slot * kChAuxItemSlot, a.items + item_first + emitted,
                                 (uint32_t)sizeof(ChainItem), mb_desc + 8 * slot);
                }
                if (emitted + 1 == item_count) ended = true;      // the list's last item is its END
            }
            ++emitted;
            __syncwarp();
        };
        // Releases the inputs of the items whose descriptors are out, in order.  `done_upto`:
        // index of the last item this CTA has published.  An item that starts a stage may look
        // at its gate only when all of this CTA's earlier items are published (the stage before
        // it cannot complete otherwise); an item behind it waits with it.
        auto release_pending = [&](int done_upto) {
            while (issued < emitted) {
                const int ps = issued & 1;
                if (!mbar_wait_timed(mb_desc + 8 * ps, (issued >> 1) & 1, fail, budget_long)) break;
                const ChainItem &it = ring[ps];
                if (it.kind == CH_ITEM_END) break;
                const int dep = it.stage - 1;
                const bool gated = it.kind != CH_ITEM_NOTHING && dep > known_done;
                if (gated && issued > done_upto + 1) break;
                if (gated) wait_dep(dep, it.dep_target, it.dep_raw != 0);
                if (lane == 0) stamp(issued, 0);
                release(ps);
                if (lane == 0) stamp(issued, 1);
                ++issued;
            }
        };

        if (fw == 0) {
            emit(0);
            if (!ended) emit(1);
            release_pending(-1);
        }
        for (int i = 0;; ++i) {
            const int slot = i & 1;
            const bool have = mbar_wait_timed(mb_desc + 8 * slot, (i >> 1) & 1, fail, budget_long);
            const ChainItem it = ring[slot];
            if (!have || it.kind == CH_ITEM_END) break;
            named_bar_sync_dyn(kChBarItemDone + slot, kChThreads);      // consumers are done with it
            if (ftid == 0) stamp(i, 8);
            named_bar_sync<kChBarFinalizers, kChFinalizers>();          // every finalizer holds its copy
            if (fw == 0 && !ended) emit(slot);                           // item i + 2
            // ---- end of a GEMV stage for this CTA: the completion pass ------------------------
            // The CTA's partial sums of the stage sit in the linears' fp32 accumulators (added there
            // by the consumers).  1. fence, one addition to raw[stage]; 2. wait (bounded) until all
            // CTAs have added theirs; 3. the blocks of 32 rows are dealt out over the finalizer warps
            // of ALL CTAs: read the accumulators, run the linear's output op (or push the sums to the
            // ranks and add theirs), clear the accumulators; 4. fence, add the number of finished
            // blocks to done[stage].  Which CTA streamed last no longer matters for who completes what.
            if (it.last_of_stage && it.stage_jobs > 0 && it.defer_out) {
                // the next stage's consumers finish this stage's sums themselves: count this CTA, no more
                if (ftid == 0 && !*fail) {
                    __threadfence();
                    atomicAdd(a.raw + it.stage, 1u);
                }
            } else if (it.last_of_stage && it.stage_jobs > 0) {
                if (ftid == 0 && !*fail) {
                    __threadfence();
                    atomicAdd(a.raw + it.stage, 1u);
                }
                const ChainJob J0 = a.jobs[it.job_first];        // in flight while the others arrive
                if (fw == 0) {
                    int ok = 0;
                    if (lane == 0 && !*fail) {
                        const unsigned long long t0 = global_ns();
                        for (;;) {
#pragma unroll 1
                            for (int k = 0; k < 16 && !ok; ++k) ok = ld_acquire_gpu_u32(a.raw + it.stage) >= gridDim.x;
                            if (ok || *fail || ld_relaxed_gpu_s32(a.status) != 0 || global_ns() - t0 > budget) break;
                        }
                        if (!ok) *fail = 1;
                    }
                }
                named_bar_sync<kChBarFinalizers, kChFinalizers>();
                if (ftid == 0) stamp(i, 11);
                const bool failed = __any_sync(0xffffffffu, *fail != 0);      // one view per warp: collectives follow
                const bool push = tp && it.tp_ordinal > 0;
                const unsigned tag = tag_base + (unsigned)it.tp_ordinal;
                const int nwarps = gridDim.x * kChFinalWarps, wme = blockIdx.x * kChFinalWarps + fw;
                // every CTA has streamed this stage, so every CTA has read the sums of the stage before
                // that this one took unfinished: they are cleared here, for the next token
                if (it.clear_acc && !failed)
                    for (int blk = wme; blk < it.clear_blocks; blk += nwarps) it.clear_acc[blk * kBlockRows + lane] = 0.f;
                int ndone = 0;
                int off = 0;                               // blocks of the jobs before this one
                for (int jj = 0; jj < it.stage_jobs && !failed; ++jj) {
                    const ChainJob J = jj == 0 ? J0 : a.jobs[it.job_first + jj];
                    const bool resid = J.out_kind == CH_OUT_RESIDUAL;
                    float ssq = 0.f;
                    // first block of this job for this warp: the jobs' blocks form one sequence
                    int blk = (wme - off % nwarps + nwarps) % nwarps;
                    off += J.blocks;
                    constexpr int kPerRound = 8;
                    for (; blk < J.blocks; blk += nwarps * kPerRound) {
                        float v[kPerRound], rs[kPerRound];
#pragma unroll
                        for (int b = 0; b < kPerRound; ++b) {
                            const int row = (blk + b * nwarps) * kBlockRows + lane;
                            rs[b] = 0.f;
                            if (blk + b * nwarps < J.blocks) {
                                v[b] = ldcg_f32(J.acc + row);
                                if (resid && !push && row < J.n) rs[b] = __half2float(__ldcg(J.y + row));
                            }
                        }
#pragma unroll
                        for (int b = 0; b < kPerRound; ++b) {
                            if (blk + b * nwarps >= J.blocks) continue;          // uniform over the warp
                            const int row = (blk + b * nwarps) * kBlockRows + lane;
                            ++ndone;
                            J.acc[row] = 0.f;
                            float o = v[b];
                            if (J.bias && row < J.n) o += __half2float(__ushort_as_half(J.bias[row]));
                            if (push) {
                                // this rank's sum of the block to every rank (itself included)
                                const long long slot_row =
                                    (((long long)(tag & 1u) * tp->world + tp->rank) * tp->max_m) * tp->np_cap + row;
                                for (int r = 0; r < tp->world; ++r)
                                    st_relaxed_sys_b64(tp->recv[r] + slot_row, __float_as_uint(o), tag);
                            } else if (J.out_kind == CH_OUT_STORE) {
                                if (row < J.n) J.y[row] = __float2half_rn(o);
                            } else if (resid) {
                                if (row < J.n) {
                                    const float t = rs[b] + __half2float(__float2half_rn(o));
                                    J.y[row] = __float2half_rn(t);
                                    ssq += t * t;
                                }
                            } else {
                                // rows 32b .. 32b+15 are gate rows 16b.., rows 32b+16 .. are the up rows
                                const float mine = __half2float(__float2half_rn(o));
                                const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
                                if (lane < 16 && row < J.n)
                                    J.y[(row >> 5) * 16 + lane] = __float2half_rn(other * (mine / (1.0f + expf(-mine))));
                            }
                        }
                    }
                    if (push) {
                        // Rank sum.  Pushing never waits; every warp then polls, for the blocks it
                        // pushed, every rank's slot until it carries this stage's tag, adds the ranks'
                        // sums in rank order and runs the output op.
                        blk = (wme - (off - J.blocks) % nwarps + nwarps) % nwarps;
                        for (; blk < J.blocks; blk += nwarps) {
                            const int row = blk * kBlockRows + lane;
                            float sum = 0.f;
                            bool ok = true;
                            for (int src = 0; src < tp->world; ++src) {
                                const unsigned long long *sl =
                                    tp->recv[tp->rank] + (((long long)(tag & 1u) * tp->world + src) * tp->max_m) * tp->np_cap + row;
                                unsigned long long v = ld_relaxed_sys_b64(sl);
                                if ((uint32_t)(v >> 32) != tag && !*fail) {
                                    // a peer that never arrives: the first wait that runs out ends all later ones
                                    const unsigned long long t0 = global_ns();
                                    for (;;) {
#pragma unroll 1
                                        for (int k = 0; k < 16 && (uint32_t)(v >> 32) != tag; ++k) v = ld_relaxed_sys_b64(sl);
                                        if ((uint32_t)(v >> 32) == tag || *fail || global_ns() - t0 > budget) break;
                                    }
                                }
                                ok = ok && ((uint32_t)(v >> 32) == tag);
                                sum += __uint_as_float((uint32_t)v);
                            }
                            if (!ok) *fail = 1;
                            if (row < J.n) {
                                if (resid) {
                                    const float t = __half2float(__ldcg(J.y + row)) + __half2float(__float2half_rn(sum));
                                    J.y[row] = __float2half_rn(t);
                                    ssq += t * t;
                                } else {
                                    J.y[row] = __float2half_rn(sum);
                                }
                            }
                        }
                    }
                    if (resid) {
#pragma unroll
                        for (int dd = 16; dd; dd >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, dd);
                        if (lane == 0 && ssq != 0.f) atomicAdd(J.ss_out, ssq);
                    }
                }
                __syncwarp();
                if (lane == 0 && ndone) {
                    __threadfence();
                    const unsigned old = atomicAdd(a.done + it.stage, (unsigned)ndone);
                    // the launch's last rank sum: publish the tags this launch has used
                    if (push && it.tp_ordinal == a.n_tp_stages && old + (unsigned)ndone == it.stage_blocks) *tp->seq = tag;
                }
            }
            if (ftid == 0) stamp(i, 9);
            if (fw == 0) release_pending(i);
        }
        if (*fail && ftid == 0) atomicExch(a.status, 1);
        return;
    }

    // =============================== consumer warps =======================================
    // Two code regions: a loop over SEGMENT / NOTHING items (the register tiles of the weight
    // stream live across its iterations) and, outside of it, the ATTENTION items.  Kept apart
    // on purpose: with the attention call inside the streaming loop the compiler spilled the
    // loop's state around it and the stream ran at half its speed.
    {
        const bool have = mbar_wait_timed(mb_desc, 0, fail, budget_long);
        if (!have || ring[0].kind == CH_ITEM_END) return;
    }
    int i = 0;                              // index of the current item; its descriptor is in ring[i & 1]
    // hands the item to the finalizers and waits for the next descriptor; false at the end
    auto end_item = [&](int slot) {
        if (tid == 0) stamp(i, 6);
        named_bar_arrive_dyn(kChBarItemDone + slot, kChThreads);
        if (tid == 0) stamp(i, 7);
        const bool have = mbar_wait_timed(mb_desc + 8 * (slot ^ 1), ((i + 1) >> 1) & 1, fail, budget_long);
        ++i;
        return have && ring[slot ^ 1].kind != CH_ITEM_END;
    };
    for (;;) {
        if (ring[i & 1].kind == CH_ITEM_ATTENTION) {
            const int slot = i & 1;
            const ChainItem &cur = ring[slot];
            if (tid == 0) stamp(i, 2);
            ChainWait w = {mb_x + 8 * slot, (uint32_t)((i >> 1) & 1), fail, budget_long, decide + slot};
            const bool ran = chain_attention(a.attn + cur.attn, cur.hk, cur.split, cur.nsplit, table_ptr, tid, rope_tab,
                                             *pos_s, w,
                                             (a.trace && i < a.trace_items)
                                                 ? a.trace + ((size_t)blockIdx.x * a.trace_items + i) * 16 + 11
                                                 : nullptr);
            named_bar_sync<kChBarConsumers, kChConsumers>();   // the split's partial is written by all
            if (ran && tid == 0) {
                __threadfence();
                atomicAdd(a.done + cur.stage, 1u);
            }
            if (!end_item(slot)) return;
            continue;
        }
        if (!chain_gemv_items<Q, GPW>(a, aux, tbl, i)) return;
    }
}

}  // namespace hlq

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
using namespace hlq;

struct hlq_chain {
    int device = 0;
    int q = 0, g = 0, gpw = 0;
    int ss_cells = 0;
    std::vector<ChainStage> stages;
    std::vector<ChainJob> jobs;
    std::vector<AttnArgs> attn;
    std::vector<std::pair<int, int>> job_ss;      // per job: (ss_in cell, ss_out cell), -1: none
    hlq_tp_comm *comm = nullptr;
    int n_tp_stages = 0;
    int items_total = 0;
    // device
    ChainItem *d_items = nullptr;
    int *d_first = nullptr;
    ChainJob *d_jobs = nullptr;
    AttnArgs *d_attn = nullptr;
    unsigned char *d_state = nullptr;             // [256 B status][done: nstages][raw: nstages][ss: cells]  (cleared every forward)
    unsigned char *d_scratch = nullptr;           // fp32 accumulators of all jobs (self-cleaning)
    size_t state_bytes = 0, scratch_bytes = 0, done_off = 0, raw_off = 0, ss_off = 0;
    int sms = 0;
    bool finished = false;
    unsigned long long *d_trace = nullptr;        // set by hlq_chain_trace
    int trace_items = 0;
};

namespace {

constexpr uint32_t kChainDynSmem = 65536 - 1024 + kChTableBytes + kChAuxBytes;

template <int Q, int GPW>
int launch_chain_inst(const ChainArgs &args, int ctas, cudaStream_t stream) {
    static std::atomic<bool> configured[64];
    static std::mutex mu;
    int dev = 0;
    HLQ_CUDA(cudaGetDevice(&dev));
    auto kernel = decode_chain_kernel<Q, GPW>;
    if (!configured[dev & 63].load(std::memory_order_acquire)) {
        std::lock_guard<std::mutex> lock(mu);
        HLQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kChainDynSmem));
        configured[dev & 63].store(true, std::memory_order_release);
    }
    kernel<<<dim3(ctas), dim3(kChThreads), kChainDynSmem, stream>>>(args);
    HLQ_CUDA(cudaGetLastError());
    count_launch();
    return HLQ_OK;
}

int launch_chain(int q, int gpw, const ChainArgs &a, int ctas, cudaStream_t stream) {
#define HLQ_CASE(QV, GV) \
    if (q == QV && gpw == GV) return launch_chain_inst<QV, GV>(a, ctas, stream);
    HLQ_CASE(2, 1) HLQ_CASE(3, 1) HLQ_CASE(4, 1)
    HLQ_CASE(2, 2) HLQ_CASE(3, 2) HLQ_CASE(4, 2)
#undef HLQ_CASE
    return HLQ_ERR_UNSUPPORTED;
}

}  // namespace

extern "C" {

int hlq_chain_create(hlq_chain **out, int device, int ss_cells) {
    if (!out) return HLQ_ERR_INVALID_ARGUMENT;
    *out = nullptr;
    if (ss_cells < 0 || ss_cells > (1 << 20)) return HLQ_ERR_INVALID_ARGUMENT;
    int major = 0, sms = 0, smem = 0;
    HLQ_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) return HLQ_ERR_NO_DEVICE;
    HLQ_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
    HLQ_CUDA(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
    if ((uint32_t)smem < kChainDynSmem) return HLQ_ERR_NO_DEVICE;
    hlq_chain *c = new (std::nothrow) hlq_chain();
    if (!c) return HLQ_ERR_INVALID_ARGUMENT;
    c->device = device;
    c->ss_cells = ss_cells;
    c->sms = sms;
    *out = c;
    return HLQ_OK;
}

int hlq_chain_add_linears(hlq_chain *c, int count, const hlq_chain_linear *m, hlq_tp_comm *comm) {
    if (!c || c->finished || count <= 0 || !m) return HLQ_ERR_INVALID_ARGUMENT;
    if (comm && count != 1) return HLQ_ERR_INVALID_ARGUMENT;        // a rank sum covers one linear
    if (comm && c->comm && comm != c->comm) return HLQ_ERR_INVALID_ARGUMENT;
    for (int i = 0; i < count; ++i) {
        const hlq_weight *w = m[i].w;
        if (!w || !m[i].d_y) return HLQ_ERR_INVALID_ARGUMENT;
        if (!m[i].d_x && m[i].in_kind != HLQ_CHAIN_IN_ATTENTION) return HLQ_ERR_INVALID_ARGUMENT;
        if (w->layout != HLQ_LAYOUT_STREAM || w->device != c->device || w->sp_pairs) return HLQ_ERR_UNSUPPORTED;
        if (c->q == 0) {
            c->q = w->q;
            c->g = w->g;
        }
        if (w->q != c->q || w->g != c->g) return HLQ_ERR_UNSUPPORTED;
        if (((uintptr_t)m[i].d_x | (uintptr_t)m[i].d_gamma) & 15) return HLQ_ERR_ALIGNMENT;
        if ((uintptr_t)m[i].d_y & 1) return HLQ_ERR_ALIGNMENT;
        if (m[i].in_kind < HLQ_CHAIN_IN_PLAIN || m[i].in_kind > HLQ_CHAIN_IN_ATTENTION) return HLQ_ERR_INVALID_ARGUMENT;
        if (m[i].in_kind == HLQ_CHAIN_IN_ATTENTION) {
            // the stage before must be an attention whose output has this linear's input channels
            if (c->stages.empty() || c->stages.back().kind != CH_STAGE_ATTENTION) return HLQ_ERR_INVALID_ARGUMENT;
            if (c->attn[c->stages.back().attn].head_q * 128 != w->k) return HLQ_ERR_SHAPE;
        }
        if (m[i].out_kind < HLQ_CHAIN_OUT_STORE || m[i].out_kind > HLQ_CHAIN_OUT_GATED_SILU)
            return HLQ_ERR_INVALID_ARGUMENT;
        if (m[i].in_kind == HLQ_CHAIN_IN_NORM && (!m[i].d_gamma || m[i].ss_in < 0 || m[i].ss_in >= c->ss_cells))
            return HLQ_ERR_INVALID_ARGUMENT;
        if (m[i].out_kind == HLQ_CHAIN_OUT_RESIDUAL && (m[i].ss_out < 0 || m[i].ss_out >= c->ss_cells))
            return HLQ_ERR_INVALID_ARGUMENT;
        if (m[i].out_kind == HLQ_CHAIN_OUT_GATED_SILU && (w->n % 32 || comm)) return HLQ_ERR_SHAPE;
        if (w->k % 8) return HLQ_ERR_SHAPE;
    }
    if (comm && (!comm->connected || comm->device != c->device || comm->max_m < 1)) return HLQ_ERR_INVALID_ARGUMENT;
    ChainStage st = {};
    st.kind = CH_STAGE_GEMV;
    st.job_begin = (int)c->jobs.size();
    st.job_count = count;
    st.target = 0;
    for (int i = 0; i < count; ++i) {
        const hlq_weight *w = m[i].w;
        const StreamDims d = stream_dims(w->n, w->k, w->g, w->q);
        if (comm && d.np > comm->np_cap) return HLQ_ERR_WORKSPACE;
        c->gpw = d.gpw;
        ChainJob j = {};
        j.planes = w->d_planes;
        j.meta = w->d_meta;
        j.bias = w->d_bias;
        j.x = (const uint16_t *)m[i].d_x;
        if (m[i].in_kind == HLQ_CHAIN_IN_ATTENTION) {
            const AttnArgs &at = c->attn[c->stages.back().attn];
            j.x = (const uint16_t *)at.partial;
            j.attn_nsplit = c->stages.back().nsplit;
            j.attn_group = at.group;
            j.attn_heads = at.head_q;
        }
        j.y = (__half *)m[i].d_y;
        j.gamma = (const uint16_t *)m[i].d_gamma;
        j.eps = m[i].eps;
        j.inv_k = m[i].norm_channels > 0 ? 1.0f / (float)m[i].norm_channels : 1.0f / (float)w->k;
        j.n = w->n; j.k = w->k; j.np = d.np; j.slices = d.slices; j.duos = d.duos; j.blocks = d.blocks;
        j.in_kind = m[i].in_kind;
        j.out_kind = m[i].out_kind;
        st.target += (unsigned)d.blocks;
        c->jobs.push_back(j);
        c->job_ss.push_back({m[i].in_kind == HLQ_CHAIN_IN_NORM ? m[i].ss_in : -1,
                             m[i].out_kind == HLQ_CHAIN_OUT_RESIDUAL ? m[i].ss_out : -1});
    }
    if (comm) {
        c->comm = comm;
        st.tp_ordinal = ++c->n_tp_stages;
    }
    c->stages.push_back(st);
    return HLQ_OK;
}

int hlq_chain_add_attention(hlq_chain *c, const void *d_q, const void *d_k, const void *d_v, void *d_kcache,
                            void *d_vcache, const int *d_position, int head_q, int head_kv, int dhead, int max_ctx,
                            int kv_layout, float rotary_base, float scale, void *d_out, void *d_workspace,
                            size_t workspace_bytes) {
    if (!c || c->finished) return HLQ_ERR_INVALID_ARGUMENT;
    if (!d_q || !d_k || !d_v || !d_kcache || !d_vcache || !d_position || !d_out || !d_workspace)
        return HLQ_ERR_INVALID_ARGUMENT;
    if (head_q <= 0 || head_kv <= 0 || max_ctx <= 0 || head_q % head_kv) return HLQ_ERR_SHAPE;
    if (head_q / head_kv > kMaxGroup) return HLQ_ERR_UNSUPPORTED;
    if (dhead != 128) return HLQ_ERR_UNSUPPORTED;                   // the chain runs the 128-channel unit only
    if (kv_layout != HLQ_KV_POSITION_MAJOR && kv_layout != HLQ_KV_HEAD_MAJOR) return HLQ_ERR_INVALID_ARGUMENT;
    if (((uintptr_t)d_kcache | (uintptr_t)d_vcache | (uintptr_t)d_workspace) & 15) return HLQ_ERR_ALIGNMENT;
    if (workspace_bytes < hlq_attention_workspace_bytes(head_q, head_kv, dhead, max_ctx)) return HLQ_ERR_WORKSPACE;
    const int splits = attention_splits(head_kv, max_ctx);
    const size_t partial = (size_t)head_kv * splits * (head_q / head_kv) * (dhead + 2) * sizeof(float);
    // one token, one position: the attention stages of a chain share the position cell, the rotary
    // base and the cache length (the kernel prepares the rotary angles once)
    if (!c->attn.empty() && (c->attn[0].position != d_position || c->attn[0].rotary_base != rotary_base ||
                             c->attn[0].max_ctx != max_ctx))
        return HLQ_ERR_UNSUPPORTED;
    AttnArgs a;
    a.q = (const __half *)d_q;
    a.k = (const __half *)d_k;
    a.v = (const __half *)d_v;
    a.kcache = (__half *)d_kcache;
    a.vcache = (__half *)d_vcache;
    a.position = d_position;
    a.out = (__half *)d_out;
    a.status = (int *)d_workspace;
    a.partial = (float *)((char *)d_workspace + kWsHeader);
    a.counters = (unsigned *)((char *)d_workspace + kWsHeader + ((partial + 255) & ~(size_t)255));
    a.head_q = head_q;
    a.head_kv = head_kv;
    a.group = head_q / head_kv;
    a.max_ctx = max_ctx;
    a.pos_stride = kv_layout == HLQ_KV_HEAD_MAJOR ? dhead : (long long)head_kv * dhead;
    a.head_stride = kv_layout == HLQ_KV_HEAD_MAJOR ? (long long)max_ctx * dhead : dhead;
    a.rotary_base = rotary_base;
    a.scale = scale;
    ChainStage st = {};
    st.kind = CH_STAGE_ATTENTION;
    st.target = (unsigned)(head_kv * splits);      // one count per (kv head, split)
    st.attn = (int)c->attn.size();
    st.nsplit = splits;
    c->attn.push_back(a);
    c->stages.push_back(st);
    return HLQ_OK;
}

// Lays out every CTA's items.  A GEMV stage is cut along its (linear, slice) pairs: every pair
// gets a number of CTAs in proportion to its duos (at least one) and its duos are dealt out
// evenly among them, so that a CTA builds ONE set of tables per stage and all CTAs stream about
// the same number of duos.  (With more pairs than CTAs, whole pairs are dealt out in order of
// their cumulative duos.)  The units of an attention stage go round the CTAs.  A CTA without work
// in a stage gets a NOTHING item; the last item of a CTA in a stage is marked, for the rank sum.
static void chain_build_items(const hlq_chain *c, int ctas, int q, int gpw, std::vector<std::vector<ChainItem>> &out) {
    out.assign(ctas, {});
    unsigned prev_target = 0;
    for (size_t si = 0; si < c->stages.size(); ++si) {
        const ChainStage &st = c->stages[si];
        std::vector<size_t> before(ctas);
        for (int g = 0; g < ctas; ++g) before[g] = out[g].size();
        // Stage t hands its sums to stage t + 1 unfinished when it is ONE linear with gated-SiLU output
        // and no rank sum, and stage t + 1 is ONE linear that takes exactly that output as plain input.
        auto hands_over = [&](size_t t) {
            if (t + 1 >= c->stages.size()) return false;
            const ChainStage &sa = c->stages[t], &sb = c->stages[t + 1];
            if (sa.kind != CH_STAGE_GEMV || sb.kind != CH_STAGE_GEMV || sa.job_count != 1 || sb.job_count != 1) return false;
            if (sa.tp_ordinal != 0) return false;
            const ChainJob &ja = c->jobs[sa.job_begin], &jb = c->jobs[sb.job_begin];
            return ja.out_kind == CH_OUT_GATED_SILU && jb.in_kind == CH_IN_PLAIN && (const void *)jb.x == (const void *)ja.y &&
                   jb.k * 2 == ja.n;
        };
        const bool takes_sums = si >= 1 && hands_over(si - 1), gives_sums = hands_over(si);
        auto base_item = [&](int kind) {
            ChainItem it = {};
            it.kind = kind;
            it.stage = (int)si;
            it.defer_out = gives_sums ? 1 : 0;
            if (takes_sums) {
                const ChainJob &ja = c->jobs[c->stages[si - 1].job_begin];
                it.dep_raw = 1;
                it.clear_acc = ja.acc;
                it.clear_blocks = ja.blocks;
            }
            it.tp_ordinal = st.tp_ordinal;
            it.dep_target = prev_target;
            it.job_index = st.kind == CH_STAGE_GEMV ? st.job_begin : -1;
            it.job_first = st.kind == CH_STAGE_GEMV ? st.job_begin : 0;
            it.stage_jobs = st.kind == CH_STAGE_GEMV ? st.job_count : 0;
            it.stage_blocks = st.target;
            return it;
        };
        if (st.kind == CH_STAGE_ATTENTION) {
            const int units = (int)st.target;
            for (int u = 0; u < units; ++u) {
                ChainItem it = base_item(CH_ITEM_ATTENTION);
                it.attn = st.attn;
                it.nsplit = st.nsplit;
                it.hk = u / st.nsplit;
                it.split = u % st.nsplit;
                out[u % ctas].push_back(it);
            }
        } else {
            struct Pair { int job, slice, duos; };
            std::vector<Pair> pairs;
            long long total = 0;
            for (int j = st.job_begin; j < st.job_begin + st.job_count; ++j)
                for (int sl = 0; sl < c->jobs[j].slices; ++sl) {
                    pairs.push_back({j, sl, c->jobs[j].duos});
                    total += c->jobs[j].duos;
                }
            auto segment = [&](const Pair &p, int da, int db) {
                const ChainJob &jb = c->jobs[p.job];
                ChainItem it = base_item(CH_ITEM_SEGMENT);
                const long long cell = (long long)p.slice * jb.duos + da;           // in duos
                it.planes = jb.planes + cell * (2 * q * kCellBytes);
                it.meta = jb.meta + cell * ((q + 1) * 32 * 2 * gpw);
                it.job_index = p.job;
                it.x = jb.x; it.gamma = jb.gamma; it.bias = jb.bias;
                it.ss_in = jb.ss_in; it.ss_out = jb.ss_out; it.acc = jb.acc;
                it.y = jb.y;
                it.eps = jb.eps; it.inv_k = jb.inv_k;
                it.n = jb.n; it.job_slices = jb.slices; it.in_kind = jb.in_kind; it.out_kind = jb.out_kind;
                it.duo_a = da; it.duo_b = db; it.slice = p.slice;
                it.nsplit = jb.attn_nsplit; it.attn = jb.attn_group;     // ATTENTION input: splits, heads per kv head
                it.attn_ml = jb.in_kind == HLQ_CHAIN_IN_ATTENTION
                                 ? (const float *)jb.x + (size_t)jb.attn_heads * jb.attn_nsplit * 128 : nullptr;
                it.valid = jb.k - p.slice * kSliceK < kSliceK ? jb.k - p.slice * kSliceK : kSliceK;
                if (takes_sums) {
                    const ChainJob &ja = c->jobs[c->stages[si - 1].job_begin];
                    it.in_kind = CH_IN_GATED_ACC;
                    it.x = (const uint16_t *)ja.acc;
                    it.gamma = ja.bias;
                    it.attn_ml = (const float *)ja.y;
                }
                return it;
            };
            const int np = (int)pairs.size();
            if (np <= ctas) {
                // CTAs per pair: proportional to the pair's duos, at least one, summing to `ctas`
                std::vector<int> share(np);
                int used = 0;
                for (int p = 0; p < np; ++p) {
                    share[p] = (int)((long long)pairs[p].duos * ctas / total);
                    if (share[p] < 1) share[p] = 1;
                    if (share[p] > pairs[p].duos) share[p] = pairs[p].duos;
                    used += share[p];
                }
                while (used != ctas) {           // fix the rounding where it changes the load least
                    int best = -1;
                    double best_load = 0;
                    for (int p = 0; p < np; ++p) {
                        if (used < ctas) {
                            if (share[p] >= pairs[p].duos) continue;
                            const double load = (double)pairs[p].duos / share[p];
                            if (best < 0 || load > best_load) { best = p; best_load = load; }
                        } else {
                            if (share[p] <= 1) continue;
                            const double load = (double)pairs[p].duos / (share[p] - 1);
                            if (best < 0 || load < best_load) { best = p; best_load = load; }
                        }
                    }
                    if (best < 0) break;
                    share[best] += used < ctas ? 1 : -1;
                    used += used < ctas ? 1 : -1;
                }
                // What that costs: the largest share plus one set of tables (in duos: building the 64
                // tables of a slice takes as long as streaming kTableDuos duos).  Where whole CTAs per
                // pair fit badly (56 slices on 148 CTAs: 2 or 3 CTAs per slice, 256 or 171 duos each)
                // it is cheaper to cut the pairs' concatenated duos into `ctas` runs of equal COST and
                // let the CTAs whose run crosses a slice build two sets of tables: the smallest budget
                // per CTA for which that fits is found by bisection.
                constexpr int kTableDuos = 36;
                long long whole_cost = 0;
                for (int p = 0; p < np; ++p) {
                    const long long cst = (pairs[p].duos + share[p] - 1) / share[p] + kTableDuos;
                    if (cst > whole_cost) whole_cost = cst;
                }
                auto fits = [&](long long budget, std::vector<std::vector<std::pair<int, std::pair<int, int>>>> *runs) {
                    int g = 0, p = 0, at = 0;          // CTA, pair, first duo of the pair not yet dealt out
                    if (runs) runs->assign(ctas, {});
                    while (p < np) {
                        if (g >= ctas) return false;
                        long long left = budget;
                        while (p < np && left > kTableDuos) {
                            left -= kTableDuos;
                            const int d = (int)std::min<long long>(pairs[p].duos - at, left);
                            if (runs) (*runs)[g].push_back({p, {at, at + d}});
                            left -= d;
                            at += d;
                            if (at < pairs[p].duos) break;       // the CTA is full
                            ++p;
                            at = 0;
                        }
                        ++g;
                    }
                    return true;
                };
                long long lo = total / ctas + kTableDuos, hi = whole_cost;      // lo may not fit, hi is tried below
                bool cut_fits = fits(hi, nullptr);
                if (cut_fits) {
                    while (lo < hi) {
                        const long long mid = (lo + hi) / 2;
                        if (fits(mid, nullptr)) hi = mid; else lo = mid + 1;
                    }
                }
                // the stages start their dealing at different CTAs, so that the CTAs that draw
                // the slightly larger shares change from stage to stage
                int g = (int)((si * 37) % ctas);
                if (cut_fits && hi + 2 < whole_cost) {
                    std::vector<std::vector<std::pair<int, std::pair<int, int>>>> runs;
                    fits(hi, &runs);
                    for (int t = 0; t < ctas; ++t) {
                        for (const auto &r : runs[t]) out[g].push_back(segment(pairs[r.first], r.second.first, r.second.second));
                        g = (g + 1) % ctas;
                    }
                } else {
                    for (int p = 0; p < np; ++p)
                        for (int t = 0; t < share[p]; ++t) {
                            const int da = (int)((long long)pairs[p].duos * t / share[p]);
                            const int db = (int)((long long)pairs[p].duos * (t + 1) / share[p]);
                            if (db > da) out[g].push_back(segment(pairs[p], da, db));
                            g = (g + 1) % ctas;
                        }
                }
            } else {
                long long cum = 0;
                for (int p = 0; p < np; ++p) {
                    const int g = (int)((cum + pairs[p].duos / 2) * ctas / total);
                    out[g < ctas ? g : ctas - 1].push_back(segment(pairs[p], 0, pairs[p].duos));
                    cum += pairs[p].duos;
                }
            }
        }
        for (int g = 0; g < ctas; ++g) {
            if (out[g].size() == before[g]) out[g].push_back(base_item(CH_ITEM_NOTHING));
            out[g].back().last_of_stage = 1;
        }
        prev_target = st.target;
    }
    for (int g = 0; g < ctas; ++g) {
        ChainItem end = {};
        end.kind = CH_ITEM_END;
        end.stage = (int)c->stages.size();
        out[g].push_back(end);
    }
}

int hlq_chain_finish(hlq_chain *c, void *stream_) {
    if (!c || c->finished || c->stages.empty()) return HLQ_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = (cudaStream_t)stream_;
    int prev = -1;
    cudaGetDevice(&prev);
    if (cudaSetDevice(c->device) != cudaSuccess) return HLQ_ERR_NO_DEVICE;
    // state: [status header][done per stage][sum-of-squares cells]
    c->done_off = kWsHeader;
    c->raw_off = c->done_off + ((c->stages.size() * sizeof(unsigned) + 255) & ~(size_t)255);
    c->ss_off = c->raw_off + ((c->stages.size() * sizeof(unsigned) + 255) & ~(size_t)255);
    c->state_bytes = c->ss_off + (((size_t)c->ss_cells * sizeof(float) + 255) & ~(size_t)255);
    // scratch: per job its accumulators
    size_t off = 0;
    std::vector<size_t> aoff(c->jobs.size());
    for (size_t i = 0; i < c->jobs.size(); ++i) {
        aoff[i] = off;
        off += ((size_t)c->jobs[i].np * sizeof(float) + 255) & ~(size_t)255;
    }
    c->scratch_bytes = off;
    int rc = HLQ_OK;
    if (cudaMalloc((void **)&c->d_state, c->state_bytes) != cudaSuccess ||
        cudaMalloc((void **)&c->d_scratch, c->scratch_bytes ? c->scratch_bytes : 256) != cudaSuccess ||
        cudaMalloc((void **)&c->d_first, sizeof(int) * (c->sms + 1)) != cudaSuccess ||
        cudaMalloc((void **)&c->d_jobs, sizeof(ChainJob) * (c->jobs.size() ? c->jobs.size() : 1)) != cudaSuccess ||
        cudaMalloc((void **)&c->d_attn, sizeof(AttnArgs) * (c->attn.size() ? c->attn.size() : 1)) != cudaSuccess)
        rc = note_cuda(cudaErrorMemoryAllocation);
    std::vector<ChainItem> flat;
    std::vector<int> first(c->sms + 1, 0);
    if (!rc) {
        for (size_t i = 0; i < c->jobs.size(); ++i) {
            c->jobs[i].acc = (float *)(c->d_scratch + aoff[i]);
            float *ss = (float *)(c->d_state + c->ss_off);
            c->jobs[i].ss_in = c->job_ss[i].first >= 0 ? ss + c->job_ss[i].first : nullptr;
            c->jobs[i].ss_out = c->job_ss[i].second >= 0 ? ss + c->job_ss[i].second : nullptr;
        }
        std::vector<std::vector<ChainItem>> lists;
        chain_build_items(c, c->sms, c->q, c->gpw, lists);
        for (int g = 0; g < c->sms; ++g) {
            first[g] = (int)flat.size();
            flat.insert(flat.end(), lists[g].begin(), lists[g].end());
        }
        first[c->sms] = (int)flat.size();
        c->items_total = (int)flat.size();
        if (cudaMalloc((void **)&c->d_items, sizeof(ChainItem) * flat.size()) != cudaSuccess)
            rc = note_cuda(cudaErrorMemoryAllocation);
    }
    if (!rc) {
        rc = note_cuda(cudaMemsetAsync(c->d_state, 0, c->state_bytes, stream));
        if (!rc && c->scratch_bytes) rc = note_cuda(cudaMemsetAsync(c->d_scratch, 0, c->scratch_bytes, stream));
        if (!rc) rc = note_cuda(cudaMemcpyAsync(c->d_items, flat.data(), sizeof(ChainItem) * flat.size(),
                                                cudaMemcpyHostToDevice, stream));
        if (!rc) rc = note_cuda(cudaMemcpyAsync(c->d_first, first.data(), sizeof(int) * first.size(),
                                                cudaMemcpyHostToDevice, stream));
        if (!rc && !c->jobs.empty())
            rc = note_cuda(cudaMemcpyAsync(c->d_jobs, c->jobs.data(), sizeof(ChainJob) * c->jobs.size(),
                                           cudaMemcpyHostToDevice, stream));
        if (!rc && !c->attn.empty())
            rc = note_cuda(cudaMemcpyAsync(c->d_attn, c->attn.data(), sizeof(AttnArgs) * c->attn.size(),
                                           cudaMemcpyHostToDevice, stream));
        if (!rc) rc = note_cuda(cudaStreamSynchronize(stream));
    }
    if (prev >= 0) cudaSetDevice(prev);
    if (!rc) c->finished = true;
    return rc;
}

int hlq_chain_forward(hlq_chain *c, void *stream_) {
    if (!c || !c->finished) return HLQ_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = (cudaStream_t)stream_;
    int cur = -1;
    HLQ_CUDA(cudaGetDevice(&cur));
    if (cur != c->device) return HLQ_ERR_INVALID_ARGUMENT;
    // stage counters and sum-of-squares cells start every token at zero; the status word stays
    HLQ_CUDA(cudaMemsetAsync(c->d_state + c->done_off, 0, c->state_bytes - c->done_off, stream));
    ChainArgs a = {};
    a.items = c->d_items;
    a.first = c->d_first;
    a.jobs = c->d_jobs;
    a.attn = c->d_attn;
    a.done = (unsigned *)(c->d_state + c->done_off);
    a.raw = (unsigned *)(c->d_state + c->raw_off);
    a.status = (int *)c->d_state;
    a.tp = c->comm ? c->comm->d_tp : nullptr;
    a.nstages = (int)c->stages.size();
    a.n_tp_stages = c->n_tp_stages;
    a.dyn_smem = kChainDynSmem;
    a.spin_limit = c->comm ? c->comm->spin_limit : kDefaultSpinLimit;
    a.trace = c->d_trace;
    a.trace_items = c->trace_items;
    a.rope_position = c->attn.empty() ? nullptr : c->attn[0].position;
    a.rope_base = c->attn.empty() ? 0.f : c->attn[0].rotary_base;
    a.rope_max_ctx = c->attn.empty() ? 0 : c->attn[0].max_ctx;
    return launch_chain(c->q, c->gpw, a, c->sms, stream);
}

int hlq_chain_status(const hlq_chain *c, void *stream, int *kernel_status) {
    if (!c || !c->finished || !kernel_status) return HLQ_ERR_INVALID_ARGUMENT;
    HLQ_CUDA(cudaMemcpyAsync(kernel_status, c->d_state, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    HLQ_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return *kernel_status ? HLQ_ERR_KERNEL : HLQ_OK;
}

int hlq_chain_trace(hlq_chain *c, void *d_trace, int items_per_cta, int *ctas) {
    if (!c || items_per_cta < 0) return HLQ_ERR_INVALID_ARGUMENT;
    c->d_trace = items_per_cta > 0 ? (unsigned long long *)d_trace : nullptr;
    c->trace_items = c->d_trace ? items_per_cta : 0;
    if (ctas) *ctas = c->sms;
    return HLQ_OK;
}

int hlq_chain_info(const hlq_chain *c, int *stages, int *linears, int *rank_sums, int64_t *scratch_bytes) {
    if (!c) return HLQ_ERR_INVALID_ARGUMENT;
    if (stages) *stages = (int)c->stages.size();
    if (linears) *linears = (int)c->jobs.size();
    if (rank_sums) *rank_sums = c->n_tp_stages;
    if (scratch_bytes)
        *scratch_bytes = (int64_t)(c->state_bytes + c->scratch_bytes + sizeof(ChainItem) * (size_t)c->items_total);
    return HLQ_OK;
}

int hlq_chain_free(hlq_chain *c) {
    if (!c) return HLQ_OK;
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(c->device);
    if (c->d_state) cudaFree(c->d_state);
    if (c->d_scratch) cudaFree(c->d_scratch);
    if (c->d_items) cudaFree(c->d_items);
    if (c->d_first) cudaFree(c->d_first);
    if (c->d_jobs) cudaFree(c->d_jobs);
    if (c->d_attn) cudaFree(c->d_attn);
    if (prev >= 0) cudaSetDevice(prev);
    delete c;
    return HLQ_OK;
}

}  // extern "C"
